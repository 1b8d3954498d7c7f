"""The two operators the reference's engines call on this path, as ``torch.nn.Module``s bound to the
CUDA kernels: ``ResidualVQLinear`` (``ojasx_24x96/module.py:171-551``: buffers ``packed_codes``,
``codebooks``, ``row_scales``, ``bias`` -- the OQPack tensor names -- and the two runtime toggles)
and ``ResidualVQFusedExperts`` (``:600-708``: ``forward(hidden_states, top_k_index, top_k_weights)``).
Model surgery, dense caches and the training path of the reference modules are out of scope.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch
from torch import nn

from .codec import QuantizedWeight
from .math_engine import fused_rvq_gemm_native, subspace_lut_rvq_gemm
from .ops import VQMoE


class ResidualVQLinear(nn.Module):
    codec = "adaptive_residual_vq"

    def __init__(self, encoded: QuantizedWeight, bias: Optional[torch.Tensor] = None):
        super().__init__()
        self.out_features, self.in_features = encoded.original_shape
        self.block_size = encoded.block_size
        self.bits_per_stage = encoded.bits_per_stage
        self.register_buffer("packed_codes", encoded.packed_codes)
        self.register_buffer("codebooks", encoded.codebooks)
        self.register_buffer("row_scales", encoded.row_scales)
        self.register_buffer("bias", None if bias is None else bias.to(torch.float32))
        rp, ci, va = encoded.outliers if encoded.outliers is not None else (None, None, None)
        self.register_buffer("csr_row_ptrs", rp)
        self.register_buffer("csr_col_indices", ci)
        self.register_buffer("csr_values", va)
        self.subspace_lut_mode = True
        self.fused_native_gemm = False
        self.cached_weight_bytes = 0  # no dense weight is ever materialised

    def encoded(self) -> QuantizedWeight:
        outliers = None if self.csr_values is None else (self.csr_row_ptrs, self.csr_col_indices, self.csr_values)
        return QuantizedWeight((self.out_features, self.in_features), self.block_size, self.bits_per_stage,
                               self.packed_codes, self.codebooks, self.row_scales, {}, outliers=outliers)

    def set_subspace_lut_mode(self, enabled: bool) -> None:
        self.subspace_lut_mode = bool(enabled)

    def set_fused_native_gemm(self, enabled: bool) -> None:
        self.fused_native_gemm = bool(enabled)

    @torch.no_grad()
    def forward(self, inputs: torch.Tensor) -> torch.Tensor:
        if self.fused_native_gemm and not self.subspace_lut_mode:
            flat = inputs.reshape(-1, self.in_features)
            out = fused_rvq_gemm_native(self.encoded(), flat, 0, self.out_features, bias=self.bias)
            return out.to(inputs.dtype).reshape(*inputs.shape[:-1], self.out_features)
        return subspace_lut_rvq_gemm(inputs, self.encoded(), bias=self.bias)


class ResidualVQFusedExperts(nn.Module):
    """Expert bank of an MoE block in split-manifold code form.  ``weights`` is a
    ``synth.VQMoEWeights``-shaped object (gate rows then up rows per expert, as the reference
    flattens them, ``module.py:620-631, 647``)."""

    def __init__(self, weights, expert_range=None):
        super().__init__()
        self.num_experts = weights.num_experts
        self.hidden_dim, self.intermediate_dim = weights.hidden, weights.inter
        self._moe = VQMoE(weights, expert_range)

    @torch.no_grad()
    def forward(self, hidden_states: torch.Tensor, top_k_index: torch.Tensor, top_k_weights: torch.Tensor) -> torch.Tensor:
        return self._moe.forward(hidden_states, top_k_index, top_k_weights)


def encode_uint8_layout(codes: np.ndarray, codebook: np.ndarray, scales: Optional[np.ndarray], device) -> QuantizedWeight:
    """Wrap split-manifold arrays (codes u8[M,G], codebook f32[256,D]) as the package container (bits 8, one stage)."""
    M, G = codes.shape
    D = codebook.shape[1]
    sc = np.ones(M, np.float32) if scales is None else scales
    return QuantizedWeight((M, G * D), D, 8, torch.from_numpy(np.ascontiguousarray(codes)).reshape(1, -1).to(device),
                           torch.from_numpy(np.ascontiguousarray(codebook, dtype=np.float32))[None].to(device),
                           torch.from_numpy(np.ascontiguousarray(sc, dtype=np.float32)).to(device), {})
