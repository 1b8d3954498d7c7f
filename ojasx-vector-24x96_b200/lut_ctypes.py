"""Host-array bindings with the class names and methods of the reference's
``split_manifold_lut_experiment/native/bindings/ojasx_lut_ctypes.py`` (``:98-241``), bound to
libojasx_lut_b200.so.  Inputs and outputs are numpy arrays in host memory; each forward copies
its activations to the GPU, runs the CUDA kernels and copies the result back.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import check, lib

_vp = C.c_void_p


def _p(a):
    return None if a is None else a.ctypes.data_as(_vp)


def get_engine_info():
    L = lib()
    return {"version": L.ojasx_get_version().decode(), "backend": L.ojasx_get_backend_name().decode()}


class NativeSplitManifoldLinear:
    """ojasx_lut_ctypes.py:98-157."""

    def __init__(self, in_features: int, out_features: int, block_dim: int = 16, codebook_size: int = 256):
        self.in_features = in_features
        self.out_features = out_features
        self.block_dim = block_dim
        self.codebook_size = codebook_size
        self._handle = None

    def initialize_weights(self, codebook, codes, scales, bias=None):
        cb = np.ascontiguousarray(codebook, dtype=np.float32)
        cd = np.ascontiguousarray(codes, dtype=np.uint8)
        sc = None if scales is None else np.ascontiguousarray(scales, dtype=np.float32)
        bi = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        self._handle = lib().ojasx_create_linear(self.in_features, self.out_features, self.block_dim,
                                                 self.codebook_size, _p(cb), _p(cd), _p(sc), _p(bi))
        if not self._handle:
            check(-3, "ojasx_create_linear")

    def set_outliers(self, row_ptrs, col_indices, values):
        assert self._handle is not None
        rp = np.ascontiguousarray(row_ptrs, dtype=np.int32)
        ci = np.ascontiguousarray(col_indices, dtype=np.int32)
        va = np.ascontiguousarray(values, dtype=np.float32)
        check(lib().ojasx_set_linear_outliers(self._handle, len(va), _p(rp), _p(ci), _p(va)),
              "ojasx_set_linear_outliers")

    def forward(self, x, num_threads: int = 0):
        assert self._handle is not None
        batch = x.shape[0] if x.ndim > 1 else 1
        xf = np.ascontiguousarray(x.reshape(batch, self.in_features), dtype=np.float32)
        y = np.zeros((batch, self.out_features), dtype=np.float32)
        ret = lib().ojasx_linear_forward(self._handle, _p(xf), _p(y), batch, num_threads)
        assert ret == 0, f"Forward failed with code {ret}"
        return y.squeeze(0) if x.ndim == 1 else y

    @property
    def handle(self):
        return self._handle

    @property
    def compressed_bytes(self) -> int:
        return lib().ojasx_get_compressed_size(self._handle) if self._handle else 0

    @property
    def compression_ratio(self) -> float:
        return lib().ojasx_get_compression_ratio(self._handle) if self._handle else 0.0

    def __del__(self):
        if getattr(self, "_handle", None):
            lib().ojasx_destroy_linear(self._handle)
            self._handle = None
