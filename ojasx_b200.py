"""Importable alias: ``import ojasx_b200`` gives the package in ``ojasx-vector-24x96_b200/``
(whose directory name is not a valid identifier for the ``import`` statement)."""
import importlib
import os
import sys

_root = os.path.dirname(os.path.abspath(__file__))
if _root not in sys.path:
    sys.path.insert(0, _root)
sys.modules[__name__] = importlib.import_module("ojasx-vector-24x96_b200")
