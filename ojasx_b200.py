"""Importable alias: ``import ojasx_b200`` gives the package in ``ojasx-vector-24x96_b200/``
(whose directory name is not a valid identifier for the ``import`` statement)."""
import importlib
import importlib.abc
import importlib.util
import os
import sys

_REAL = "ojasx-vector-24x96_b200"
_ROOT = os.path.dirname(os.path.abspath(__file__))
if _ROOT not in sys.path:
    sys.path.insert(0, _ROOT)


class _SubmoduleAlias(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    """``import ojasx_b200.x`` / ``from ojasx_b200.x import y`` resolve to the one module object of the real
    package (a second copy of a submodule would duplicate its classes and its library handle)."""

    def find_spec(self, fullname, path=None, target=None):
        if fullname.startswith(__name__ + "."):
            return importlib.util.spec_from_loader(fullname, self)
        return None

    def create_module(self, spec):
        return importlib.import_module(_REAL + spec.name[len(__name__):])

    def exec_module(self, module):
        pass


sys.meta_path.insert(0, _SubmoduleAlias())
sys.modules[__name__] = importlib.import_module(_REAL)
