"""``SplitManifoldLUTLinear`` on the GPU: the module of the reference's Python engine
(``split_manifold_lut_experiment/engine/split_manifold_engine.py:22-250``) with the same constructor, buffer
names and methods, bound to the table kernels instead of ``torch.gather``.

Buffers (``:45-60``): ``codebook [Q, D]``, ``codes u8 [M, G]``, ``scales [M]``, ``outlier_indices i64 [2, nnz]``
(row of the output feature, row of the input feature) and ``outlier_values [nnz]``; optional ``bias``
parameter.  ``forward`` evaluates ``y = (sum_g LUT[g, codes[m, g]]) * scales[m] + outliers . x + bias`` in one
kernel launch; ``build_lut`` returns the table itself.  The outlier entries of a row are added in the order
in which they appear in ``outlier_indices`` (a stable sort by row turns the COO pairs into the CSR arrays the
kernels read).  There is no CPU path: tensors must live on a CUDA device.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch
from torch import nn

from ._lib import check, lib
from .encoder import from_dense as _encode_from_dense
from .ops import VQLinear, _dtype_code, _require_cuda, _stream_ptr


class SplitManifoldLUTLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, block_dim: int = 16, codebook_size: int = 256,
                 outlier_tau: float = 3.5, bias: bool = False, dtype: torch.dtype = torch.float32):
        super().__init__()
        assert in_features % block_dim == 0, f"in_features ({in_features}) must be divisible by block_dim ({block_dim})"
        assert codebook_size <= 256, "codebook_size must fit in uint8 (<= 256)"
        self.in_features, self.out_features, self.block_dim = in_features, out_features, block_dim
        self.num_groups = in_features // block_dim
        self.codebook_size, self.outlier_tau, self.dtype = codebook_size, outlier_tau, dtype
        self.register_buffer("codebook", torch.zeros((codebook_size, block_dim), dtype=dtype))
        self.register_buffer("codes", torch.zeros((out_features, self.num_groups), dtype=torch.uint8))
        self.register_buffer("scales", torch.ones(out_features, dtype=dtype))
        self.register_buffer("outlier_indices", torch.empty((2, 0), dtype=torch.long))
        self.register_buffer("outlier_values", torch.empty((0,), dtype=dtype))
        self.num_outliers = 0
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype))
        else:
            self.register_parameter("bias", None)
        self._layer: Optional[VQLinear] = None

    @property
    def lut_sram_bytes(self) -> int:
        return self.num_groups * self.codebook_size * (4 if self.dtype in (torch.float32, torch.int32) else 2)

    @property
    def compression_ratio(self) -> float:
        """Against dense 16-bit weights, with the reference's byte counts (``:70-80``)."""
        dense = self.out_features * self.in_features * 2
        comp = self.out_features * self.num_groups + self.codebook_size * self.block_dim * 2 + self.out_features * 2 \
            + self.num_outliers * (8 + 2)
        return dense / max(1, comp)

    @classmethod
    def from_dense(cls, dense_weight: torch.Tensor, dense_bias: Optional[torch.Tensor] = None, block_dim: int = 16,
                   codebook_size: int = 256, outlier_tau: float = 3.5, kmeans_iters: int = 5) -> "SplitManifoldLUTLinear":
        """Encodes a dense weight on the GPU (the procedure of ``:90-183``; see ``encoder.from_dense``)."""
        enc = _encode_from_dense(dense_weight, dense_bias, block_dim, codebook_size, outlier_tau, kmeans_iters)
        layer = cls(enc.in_features, enc.out_features, block_dim, codebook_size, outlier_tau, bias=dense_bias is not None)
        layer = layer.to(dense_weight.device)
        layer.codebook.copy_(enc.codebook)
        layer.codes.copy_(enc.codes)
        layer.scales.copy_(enc.scales)
        counts = (enc.csr_row_ptrs[1:] - enc.csr_row_ptrs[:-1]).long()
        rows = torch.repeat_interleave(torch.arange(enc.out_features, device=counts.device), counts)
        layer.outlier_indices = torch.stack([rows, enc.csr_col_indices.long()])
        layer.outlier_values = enc.csr_values.clone()
        layer.num_outliers = enc.num_outliers
        if dense_bias is not None:
            with torch.no_grad():
                layer.bias.copy_(enc.bias)
        return layer

    def refresh(self) -> None:
        """Hands the current buffers to the library again (call after changing them in place)."""
        if self._layer is not None:
            self._layer.close()
        self._layer = None

    def _bound(self) -> VQLinear:
        if self._layer is None:
            _require_cuda(self.codes, "codes")
            nnz = int(self.outlier_values.numel())
            csr = None
            if nnz > 0:
                rows, cols = self.outlier_indices[0], self.outlier_indices[1]
                order = torch.sort(rows, stable=True).indices          # entry order inside a row is kept
                rp = torch.zeros(self.out_features + 1, dtype=torch.int64, device=rows.device)
                rp[1:] = torch.cumsum(torch.bincount(rows, minlength=self.out_features), 0)
                csr = (rp.to(torch.int32).cpu().numpy(), cols[order].to(torch.int32).cpu().numpy(),
                       self.outlier_values[order].float().cpu().numpy())
            with torch.cuda.device(self.codes.device):
                self._layer = VQLinear(self.codebook.float().cpu().numpy(), self.codes.cpu().numpy(),
                                       self.scales.float().cpu().numpy(),
                                       None if self.bias is None else self.bias.detach().float().cpu().numpy(), csr,
                                       block_dim=self.block_dim, in_features=self.in_features,
                                       codebook_size=self.codebook_size)
            self.num_outliers = nnz
        return self._layer

    @torch.no_grad()
    def build_lut(self, x: torch.Tensor) -> torch.Tensor:
        """``LUT[..., g, k] = <x[..., g*D:(g+1)*D], codebook[k]>`` as fp32 ``[..., num_groups, codebook_size]``."""
        _require_cuda(x, "x")
        x2 = x.reshape(-1, self.in_features).contiguous()
        lut = torch.empty((x2.shape[0], self.num_groups, 256), device=x.device, dtype=torch.float32)
        cb = self.codebook.float().contiguous()
        check(lib().ojasx_b200_build_lut(x2.data_ptr(), x2.shape[0], self.in_features, self.block_dim, cb.data_ptr(),
                                         self.codebook_size, lut.data_ptr(), _dtype_code(x2), _stream_ptr(x.device)),
              "ojasx_b200_build_lut")
        return lut[..., : self.codebook_size].reshape(*x.shape[:-1], self.num_groups, self.codebook_size)

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self._bound().forward(x)

    @torch.no_grad()
    def dequantize_weights(self) -> torch.Tensor:
        """Diagnostic only (``:252-270``): the dense matrix the layer stands for."""
        w = (self.codebook[self.codes.long()] * self.scales.view(-1, 1, 1)).reshape(self.out_features, self.in_features)
        if self.outlier_values.numel() > 0:
            w = w.clone()
            w.index_put_((self.outlier_indices[0], self.outlier_indices[1]), self.outlier_values, accumulate=True)
        return w
