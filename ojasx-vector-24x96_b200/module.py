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
    """Expert bank of an MoE block, with the constructor and call of the reference adapter
    (``ojasx_24x96/module.py:577-708``): ``gate_up_proj`` is ONE ``ResidualVQLinear`` over the flattened
    ``[E * 2I, H]`` matrix (expert ``e`` = rows ``[e * 2I, (e + 1) * 2I)``, gate rows then up rows, ``:620-631, 647``)
    and ``down_proj`` one over ``[E * H, I]``; ``gate_limit`` clamps the gate from above and the up value to
    ``[-limit, limit]`` before ``act_fn(gate) * up`` (``_apply_gate``, ``:646-651``).

    The two projections must be in the split-manifold layout (8-bit codes, one stage: one shared codebook per
    projection, as ``SplitManifoldMoE`` has, ``ojasx_lut.h:156-242``) and ``act_fn`` must be SiLU: that is what the
    expert kernels evaluate.  Their buffers -- ``packed_codes``, ``codebooks``, ``row_scales`` and the optional CSR
    outliers over the flattened rows -- are handed to the library once, at construction.
    ``ResidualVQFusedExperts.from_weights`` builds the same module from a ``synth.VQMoEWeights``-shaped object.
    """

    def __init__(self, num_experts: int, hidden_dim: int, intermediate_dim: int, *, gate_up_proj, down_proj,
                 act_fn: Optional[nn.Module] = None, gate_limit: Optional[float] = None, expert_range=None) -> None:
        super().__init__()
        if min(num_experts, hidden_dim, intermediate_dim) <= 0:
            raise ValueError("Expert-bank dimensions must be positive")
        if gate_limit is not None and (not np.isfinite(gate_limit) or gate_limit <= 0):
            raise ValueError("Expert gate limit must be finite and positive")
        if act_fn is not None and not isinstance(act_fn, nn.SiLU) and getattr(act_fn, "__name__", "") not in ("silu",):
            raise ValueError("the expert kernels evaluate SiLU-gated experts only")
        self.num_experts, self.hidden_dim, self.intermediate_dim = int(num_experts), int(hidden_dim), int(intermediate_dim)
        self.gate_up_proj, self.down_proj = gate_up_proj, down_proj
        self.act_fn = act_fn if act_fn is not None else nn.SiLU()
        self.gate_limit = float(gate_limit) if gate_limit is not None else None
        self.streaming_decode = True     # dense expert weights are never formed here
        self._moe = VQMoE(self._bank_arrays(), expert_range)
        self._moe.set_gate_limit(self.gate_limit)

    def _bank_arrays(self):
        from types import SimpleNamespace
        E, H, I = self.num_experts, self.hidden_dim, self.intermediate_dim
        gu, dn = self.gate_up_proj, self.down_proj
        for name, proj, rows, cols in (("gate_up_proj", gu, E * 2 * I, H), ("down_proj", dn, E * H, I)):
            if not isinstance(proj, ResidualVQLinear):
                raise TypeError(f"{name} must be a ResidualVQLinear over the flattened expert rows")
            if (proj.out_features, proj.in_features) != (rows, cols):
                raise ValueError(f"{name} is {proj.out_features} x {proj.in_features}, expected {rows} x {cols}")
            if proj.bits_per_stage != 8 or proj.codebooks.shape[0] != 1 or proj.bias is not None:
                raise ValueError(f"{name}: the expert kernels need 8-bit codes, one stage and no bias")
        if gu.block_size != dn.block_size:
            raise ValueError("gate_up_proj and down_proj must share block_size")
        D = gu.block_size

        def csr(p):
            return None if p.csr_values is None else tuple(t.detach().cpu().numpy() for t in (p.csr_row_ptrs, p.csr_col_indices, p.csr_values))

        return SimpleNamespace(
            num_experts=E, hidden=H, inter=I, block_dim=D, router=None,
            codebook=gu.codebooks[0].detach().cpu().numpy(), down_codebook=dn.codebooks[0].detach().cpu().numpy(),
            gate_up_codes=gu.packed_codes.detach().cpu().numpy().reshape(E, 2 * I, H // D),
            gate_up_scales=gu.row_scales.detach().cpu().numpy().reshape(E, 2 * I),
            down_codes=dn.packed_codes.detach().cpu().numpy().reshape(E, H, I // D),
            down_scales=dn.row_scales.detach().cpu().numpy().reshape(E, H),
            gate_up_csr=csr(gu), down_csr=csr(dn))

    @classmethod
    def from_weights(cls, weights, expert_range=None, gate_limit: Optional[float] = None) -> "ResidualVQFusedExperts":
        """From arrays in ``SplitManifoldMoE`` layout (``synth.VQMoEWeights``): wraps them as the two flattened
        ``ResidualVQLinear`` projections first, so both construction routes hold the same buffers."""
        E, H, I = weights.num_experts, weights.hidden, weights.inter

        def proj(codes, codebook, scales, csr_arrays):
            enc = encode_uint8_layout(codes.reshape(-1, codes.shape[-1]), codebook, scales.reshape(-1), "cpu")
            if csr_arrays is not None:
                enc.outliers = tuple(torch.from_numpy(np.ascontiguousarray(a)) for a in csr_arrays)
            return ResidualVQLinear(enc)

        return cls(E, H, I, gate_up_proj=proj(weights.gate_up_codes, weights.codebook, weights.gate_up_scales, weights.gate_up_csr),
                   down_proj=proj(weights.down_codes, weights.down_codebook, weights.down_scales, weights.down_csr),
                   act_fn=nn.SiLU(), gate_limit=gate_limit, expert_range=expert_range)

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
