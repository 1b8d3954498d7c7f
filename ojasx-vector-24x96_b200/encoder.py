"""Offline encoder of a dense weight into the split-manifold layout, on the GPU.

Same procedure, constants and order of steps as the reference's
``SplitManifoldLUTLinear.from_dense`` (``split_manifold_lut_experiment/engine/split_manifold_engine.py:90-183``):

1. outliers are the cells with ``|W - mean(W)| >= tau * std(W)``; the manifold is ``W`` with those cells zeroed;
2. every row is divided by its largest absolute manifold value (at least 1e-8);
3. the normalised blocks ``[M * G, D]`` are clustered: 256 centroids taken at evenly spaced vector indices
   (``torch.linspace``), five rounds of assign-to-nearest / replace-by-mean (empty clusters keep their centroid),
   then a final assignment gives the uint8 codes;
4. an outlier's stored value is ``W - scale * centroid[code]`` at its cell, so that adding it after the scaled
   table sum restores ``W`` exactly there.

The statistics and masks are torch operations on the weight's device; the assignment step -- the cost of the
procedure, a ``[M*G, 256]`` distance matrix per round in the reference -- is the ``ojasx_b200_vq_assign`` kernel,
which forms no distance matrix and returns the cluster sums of the update with it.  The result carries the
arrays of ``SplitManifoldLinear`` (``ojasx_lut.h:59-81``): codebook, codes, scales, CSR outliers, bias.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np
import torch

from ._lib import check, lib


@dataclass
class SplitManifoldEncoding:
    in_features: int
    out_features: int
    block_dim: int
    codebook: torch.Tensor        # f32 [256, D]
    codes: torch.Tensor           # u8  [M, G]
    scales: torch.Tensor          # f32 [M]
    bias: Optional[torch.Tensor]  # f32 [M]
    csr_row_ptrs: torch.Tensor    # i32 [M + 1]
    csr_col_indices: torch.Tensor  # i32 [nnz], ascending inside a row
    csr_values: torch.Tensor      # f32 [nnz]

    @property
    def num_outliers(self) -> int:
        return int(self.csr_values.numel())

    def csr_numpy(self) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
        return (self.csr_row_ptrs.cpu().numpy(), self.csr_col_indices.cpu().numpy(), self.csr_values.cpu().numpy())

    def to_vq_linear(self):
        """The layer resident on the current device, ready for ``VQLinear.forward``."""
        from .ops import VQLinear
        return VQLinear(self.codebook.cpu().numpy(), self.codes.cpu().numpy(), self.scales.cpu().numpy(),
                        None if self.bias is None else self.bias.cpu().numpy(), self.csr_numpy(),
                        block_dim=self.block_dim, in_features=self.in_features)

    def dequantize(self) -> torch.Tensor:
        """Dense fp32 weight that the layer represents (manifold plus outliers)."""
        M, G, D = self.out_features, self.in_features // self.block_dim, self.block_dim
        w = (self.codebook[self.codes.long()] * self.scales.view(M, 1, 1)).reshape(M, G * D)
        rows = torch.repeat_interleave(torch.arange(M, device=w.device), (self.csr_row_ptrs[1:] - self.csr_row_ptrs[:-1]).long())
        w[rows, self.csr_col_indices.long()] += self.csr_values
        return w


def vq_assign(vectors: torch.Tensor, centroids: torch.Tensor, want_sums: bool = False):
    """codes u8 [n] (and, with ``want_sums``, f64 sums [K, D] and i64 counts [K]) of the nearest centroids."""
    assert vectors.is_cuda and vectors.dtype == torch.float32 and vectors.is_contiguous() and vectors.dim() == 2
    assert centroids.dtype == torch.float32 and centroids.is_contiguous() and centroids.shape[1] == vectors.shape[1]
    n, D = vectors.shape
    K = centroids.shape[0]
    codes = torch.empty(n, dtype=torch.uint8, device=vectors.device)
    sums = torch.zeros((K, D), dtype=torch.float64, device=vectors.device) if want_sums else None
    counts = torch.zeros(K, dtype=torch.int64, device=vectors.device) if want_sums else None
    check(lib().ojasx_b200_vq_assign(vectors.data_ptr(), n, D, centroids.data_ptr(), K, codes.data_ptr(),
                                     0 if sums is None else sums.data_ptr(), 0 if counts is None else counts.data_ptr(),
                                     torch.cuda.current_stream(vectors.device).cuda_stream), "ojasx_b200_vq_assign")
    return (codes, sums, counts) if want_sums else codes


@torch.no_grad()
def from_dense(dense_weight: torch.Tensor, dense_bias: Optional[torch.Tensor] = None, block_dim: int = 16,
               codebook_size: int = 256, outlier_tau: float = 3.5, iterations: int = 5) -> SplitManifoldEncoding:
    if not dense_weight.is_cuda:
        raise ValueError("from_dense needs the weight on a CUDA device: this package has no CPU path")
    M, K = dense_weight.shape
    if K % block_dim != 0:
        raise ValueError("in_features must be a multiple of block_dim")
    W = dense_weight.detach().float()
    std, mean = W.std().item(), W.mean().item()
    mask = (W - mean).abs() >= outlier_tau * std
    manifold = W.masked_fill(mask, 0.0)
    G = K // block_dim
    blocks = manifold.view(M, G, block_dim)
    scales = blocks.abs().amax(dim=(1, 2), keepdim=True).clamp(min=1e-8)
    vectors = (blocks / scales).reshape(-1, block_dim).contiguous()
    pick = torch.linspace(0, vectors.shape[0] - 1, codebook_size, dtype=torch.long, device=W.device)
    centroids = vectors[pick].clone()
    for _ in range(iterations):
        _codes, sums, counts = vq_assign(vectors, centroids, want_sums=True)
        valid = counts > 0
        means = (sums[valid] / counts[valid].unsqueeze(1).double()).float()
        centroids[valid] = means
    codes = vq_assign(vectors, centroids).view(M, G)
    recon = (centroids[codes.long()] * scales).reshape(M, K)
    rows, cols = torch.nonzero(mask, as_tuple=True)            # row-major order: columns ascend inside a row
    values = (W - recon)[mask]
    row_ptrs = torch.zeros(M + 1, dtype=torch.int32, device=W.device)
    row_ptrs[1:] = torch.cumsum(torch.bincount(rows, minlength=M), 0).to(torch.int32)
    return SplitManifoldEncoding(K, M, block_dim, centroids, codes.contiguous(), scales.view(M).contiguous(),
                                 None if dense_bias is None else dense_bias.detach().float().contiguous(),
                                 row_ptrs, cols.to(torch.int32).contiguous(), values.contiguous())
