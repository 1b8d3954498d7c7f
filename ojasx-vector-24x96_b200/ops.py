"""Device-tensor operators over the ojasx_b200_* entry points (torch supplies memory and streams only)."""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np
import torch

from ._lib import OjasxB200Error, check, lib

_vp = C.c_void_p
F32, BF16 = 0, 1


def _p(a):
    return None if a is None else a.ctypes.data_as(_vp)


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise TypeError(f"activations must be float32 or bfloat16, got {t.dtype}")


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise OjasxB200Error(f"{name} must be a CUDA tensor: this library has no CPU path")


class VQLinear:
    """One split-manifold VQ linear layer resident on the current CUDA device.

    Arrays use the reference layout (``SplitManifoldLinear``, ojasx_lut.h:59-81): ``codebook``
    f32 [256, D], ``codes`` u8 [M, G], optional ``scales``/``bias`` f32 [M], optional CSR
    outliers ``(row_ptrs i32[M+1], cols i32[nnz], vals f32[nnz])``.
    """

    def __init__(self, codebook, codes, scales=None, bias=None, csr=None, *, block_dim: int,
                 in_features: Optional[int] = None, codebook_size: int = 256):
        codes = np.ascontiguousarray(codes, dtype=np.uint8)
        cb = np.ascontiguousarray(codebook, dtype=np.float32)
        self.out_features, self.groups = codes.shape
        self.block_dim = int(block_dim)
        self.in_features = int(in_features) if in_features is not None else self.groups * self.block_dim
        if self.in_features // self.block_dim != self.groups:
            raise ValueError("codes.shape[1] must equal in_features // block_dim")
        sc = None if scales is None else np.ascontiguousarray(scales, dtype=np.float32)
        bi = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        self.device = torch.device("cuda", torch.cuda.current_device())
        self._h = lib().ojasx_create_linear(self.in_features, self.out_features, self.block_dim, codebook_size,
                                            _p(cb), _p(codes), _p(sc), _p(bi))
        if not self._h:
            check(-3, "ojasx_create_linear")
        self.nnz = 0
        if csr is not None:
            rp = np.ascontiguousarray(csr[0], dtype=np.int32)
            ci = np.ascontiguousarray(csr[1], dtype=np.int32)
            va = np.ascontiguousarray(csr[2], dtype=np.float32)
            if rp.shape[0] != self.out_features + 1:
                raise ValueError("row_ptrs must have out_features + 1 entries")
            check(lib().ojasx_set_linear_outliers(self._h, len(va), _p(rp), _p(ci), _p(va)),
                  "ojasx_set_linear_outliers")
            self.nnz = len(va)

    @classmethod
    def from_weights(cls, w) -> "VQLinear":
        return cls(w.codebook, w.codes, w.scales, w.bias, w.csr, block_dim=w.block_dim, in_features=w.in_features)

    @property
    def handle(self):
        return self._h

    def forward(self, x: torch.Tensor, row_start: int = 0, row_stop: Optional[int] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        _require_cuda(x, "x")
        if x.shape[-1] != self.in_features:
            raise ValueError(f"Input feature mismatch: expected {self.in_features}, got {x.shape[-1]}")
        row_stop = self.out_features if row_stop is None else row_stop
        x2 = x.reshape(-1, self.in_features).contiguous()
        rows = row_stop - row_start
        if out is None:
            out = torch.empty((x2.shape[0], rows), device=x.device, dtype=x.dtype)
        check(lib().ojasx_b200_linear_forward(self._h, x2.data_ptr(), out.data_ptr(), x2.shape[0], _dtype_code(x2),
                                              row_start, row_stop, _stream_ptr(x.device)),
              "ojasx_b200_linear_forward")
        return out.reshape(*x.shape[:-1], rows)

    __call__ = forward

    def close(self):
        if getattr(self, "_h", None):
            lib().ojasx_destroy_linear(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class VQLinearGroup:
    """Many independent VQ linear layers evaluated by one kernel launch (same block_dim)."""

    def __init__(self, layers: Sequence[VQLinear]):
        self.layers = list(layers)
        arr = (C.c_void_p * len(self.layers))(*[l.handle for l in self.layers])
        self._g = lib().ojasx_b200_create_linear_group(arr, len(self.layers))
        if not self._g:
            check(-3, "ojasx_b200_create_linear_group")

    def forward(self, x: torch.Tensor, y: torch.Tensor, shared_x: bool = False) -> torch.Tensor:
        """x [P, K] (or [K] with shared_x) and y [P, M_max] rows are used by problem p."""
        _require_cuda(x, "x")
        xs = 0 if shared_x else x.stride(0) * x.element_size()
        ys = y.stride(0) * y.element_size()
        check(lib().ojasx_b200_linear_group_forward(self._g, x.data_ptr(), xs, y.data_ptr(), ys, _dtype_code(x),
                                                    _stream_ptr(x.device)), "ojasx_b200_linear_group_forward")
        return y

    def close(self):
        if getattr(self, "_g", None):
            lib().ojasx_b200_destroy_linear_group(self._g)
            self._g = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
