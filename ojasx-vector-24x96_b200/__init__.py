"""B200 (sm_100a) implementation of OjasX's split-manifold LUT execution path.

The compute lives in ``libojasx_lut_b200.so`` (hand-written CUDA behind a C ABI, see
``include/ojasx_lut_b200.h``).  This package is the Python face of that library: host-array
bindings with the reference's class names (``lut_ctypes``), device-tensor operators
(``ops``) and seeded synthetic workloads (``synth``).  Importing the package does not load the
library; the first call does, and raises if it has not been built.
"""
from . import synth  # noqa: F401
from ._lib import LIB_PATH, OjasxB200Error, launch_count, lib  # noqa: F401

__all__ = ["synth", "lib", "launch_count", "LIB_PATH", "OjasxB200Error"]
