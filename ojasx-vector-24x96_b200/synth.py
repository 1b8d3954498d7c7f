"""Seeded synthetic workloads with the shapes and value distributions of the benchmark configs.

Everything is numpy on the host; callers move the arrays to the device.  The generators are
used by the parity tests, by bench.py and by anybody who wants to time the library without a
real checkpoint.  No dataset or checkpoint is involved: codes are uniform bytes, codebooks
are Gaussian, outliers are a uniform sample of matrix cells.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np

CSR = Tuple[np.ndarray, np.ndarray, np.ndarray]  # row_ptrs int32[M+1], cols int32[nnz], vals f32[nnz]


def make_csr_outliers(rng: np.random.Generator, rows: int, cols: int, frac: float = 0.0038,
                      sigma: float = 0.02) -> CSR:
    """Uniformly placed outliers: round(frac*rows*cols) distinct cells, |value| ~ U(15,36)*sigma, random sign."""
    nnz = int(round(frac * rows * cols))
    total = rows * cols
    if nnz == 0:
        return (np.zeros(rows + 1, np.int32), np.zeros(0, np.int32), np.zeros(0, np.float32))
    # distinct cells without materialising a permutation of rows*cols
    cells = np.unique(rng.integers(0, total, size=int(nnz * 1.05) + 16, dtype=np.int64))
    while cells.shape[0] < nnz:
        cells = np.unique(np.concatenate([cells, rng.integers(0, total, size=nnz, dtype=np.int64)]))
    cells = np.sort(rng.choice(cells, size=nnz, replace=False))
    r = (cells // cols).astype(np.int64)
    c = (cells % cols).astype(np.int32)
    row_ptrs = np.zeros(rows + 1, np.int64)
    np.cumsum(np.bincount(r, minlength=rows), out=row_ptrs[1:])
    mag = rng.uniform(15.0, 36.0, size=nnz) * sigma
    sign = np.where(rng.integers(0, 2, size=nnz) == 0, -1.0, 1.0)
    return (row_ptrs.astype(np.int32), c, (mag * sign).astype(np.float32))


@dataclass
class VQLinearWeights:
    """Layout (A) of the reference: ``SplitManifoldLinear`` fields (ojasx_lut.h:59-81)."""
    in_features: int
    out_features: int
    block_dim: int
    codebook: np.ndarray            # f32 [256, D]
    codes: np.ndarray               # u8  [M, G]
    scales: Optional[np.ndarray]    # f32 [M] or None (= ones)
    bias: Optional[np.ndarray]      # f32 [M] or None
    csr: Optional[CSR]

    @property
    def groups(self) -> int:
        return self.in_features // self.block_dim

    def code_bytes(self) -> int:
        return int(self.codes.size)

    def algorithmic_bytes(self, batch: int = 1, io_bytes: int = 4) -> int:
        """Bytes that must cross HBM once for one forward: codes + codebook + x + CSR + y."""
        n = self.code_bytes() + self.codebook.nbytes
        n += batch * (self.in_features + self.out_features) * io_bytes
        if self.scales is not None:
            n += self.scales.nbytes
        if self.bias is not None:
            n += self.bias.nbytes
        if self.csr is not None:
            n += self.csr[0].nbytes + self.csr[1].nbytes + self.csr[2].nbytes
        return int(n)


def make_vq_linear(seed: int, in_features: int, out_features: int, *, block_dim: int = 8,
                   sigma: float = 0.02, outlier_frac: float = 0.0038, with_scales: bool = False,
                   with_bias: bool = False) -> VQLinearWeights:
    rng = np.random.default_rng(seed)
    G = in_features // block_dim
    codes = rng.integers(0, 256, size=(out_features, G), dtype=np.uint8)
    codebook = (rng.standard_normal((256, block_dim)) * sigma).astype(np.float32)
    csr = make_csr_outliers(rng, out_features, in_features, outlier_frac, sigma) if outlier_frac > 0 else None
    scales = rng.uniform(0.5, 1.5, size=out_features).astype(np.float32) if with_scales else None
    bias = (rng.standard_normal(out_features) * 0.1).astype(np.float32) if with_bias else None
    return VQLinearWeights(in_features, out_features, block_dim, codebook, codes, scales, bias, csr)


@dataclass
class VQMoEWeights:
    """``SplitManifoldMoE`` fields (ojasx_lut.h:156-242) plus router and optional expert CSR."""
    num_experts: int
    hidden: int
    inter: int
    block_dim: int
    codebook: np.ndarray        # f32 [256, D]  shared by every expert's gate/up
    down_codebook: np.ndarray   # f32 [256, D]
    gate_up_codes: np.ndarray   # u8  [E, 2I, H/D]   gate rows [0,I), up rows [I,2I)
    gate_up_scales: np.ndarray  # f32 [E, 2I]
    down_codes: np.ndarray      # u8  [E, H, I/D]
    down_scales: np.ndarray     # f32 [E, H]
    router: Optional[np.ndarray]  # f32 [E, H]
    gate_up_csr: Optional[CSR]    # over the flattened [E*2I, H] matrix
    down_csr: Optional[CSR]       # over the flattened [E*H, I] matrix

    def code_bytes_per_expert(self) -> int:
        return int(self.gate_up_codes[0].size + self.down_codes[0].size)


def make_vq_moe(seed: int, num_experts: int = 512, hidden: int = 2560, inter: int = 640, *,
                block_dim: int = 8, sigma: float = 0.02, outlier_frac: float = 0.0038,
                with_router: bool = True, unit_scales: bool = True) -> VQMoEWeights:
    rng = np.random.default_rng(seed)
    G, Gi = hidden // block_dim, inter // block_dim
    gu = rng.integers(0, 256, size=(num_experts, 2 * inter, G), dtype=np.uint8)
    dn = rng.integers(0, 256, size=(num_experts, hidden, Gi), dtype=np.uint8)
    cb = (rng.standard_normal((256, block_dim)) * sigma).astype(np.float32)
    cbd = (rng.standard_normal((256, block_dim)) * sigma).astype(np.float32)
    if unit_scales:
        gus = np.ones((num_experts, 2 * inter), np.float32)
        dns = np.ones((num_experts, hidden), np.float32)
    else:
        gus = rng.uniform(0.5, 1.5, size=(num_experts, 2 * inter)).astype(np.float32)
        dns = rng.uniform(0.5, 1.5, size=(num_experts, hidden)).astype(np.float32)
    router = (rng.standard_normal((num_experts, hidden)) * sigma).astype(np.float32) if with_router else None
    gcsr = dcsr = None
    if outlier_frac > 0:
        gcsr = make_csr_outliers(rng, num_experts * 2 * inter, hidden, outlier_frac, sigma)
        dcsr = make_csr_outliers(rng, num_experts * hidden, inter, outlier_frac, sigma)
    return VQMoEWeights(num_experts, hidden, inter, block_dim, cb, cbd, gu, gus, dn, dns, router, gcsr, dcsr)


@dataclass
class VQKVCache:
    """Codebook-VQ KV cache of one layer: 16 codes per 128-wide head vector at block_dim 8."""
    batch: int
    kv_heads: int
    q_heads: int
    head_dim: int
    block_dim: int
    k_codes: np.ndarray     # u8 [B, Hkv, T, G]
    v_codes: np.ndarray     # u8 [B, Hkv, T, G]
    k_codebook: np.ndarray  # f32 [Hkv, 256, D]
    v_codebook: np.ndarray  # f32 [Hkv, 256, D]
    q: np.ndarray           # f32 [B, Hq, head_dim]   (round to bf16 for the bf16 path)
    new_k: np.ndarray       # f32 [B, Hkv, head_dim]
    new_v: np.ndarray       # f32 [B, Hkv, head_dim]


def make_vq_kv(seed: int, batch: int, ctx: int, *, kv_heads: int = 8, q_heads: int = 32,
               head_dim: int = 128, block_dim: int = 8) -> VQKVCache:
    rng = np.random.default_rng(seed)
    G = head_dim // block_dim
    sigma = 1.0 / np.sqrt(head_dim)
    kc = rng.integers(0, 256, size=(batch, kv_heads, ctx, G), dtype=np.uint8)
    vc = rng.integers(0, 256, size=(batch, kv_heads, ctx, G), dtype=np.uint8)
    kcb = (rng.standard_normal((kv_heads, 256, block_dim)) * sigma).astype(np.float32)
    vcb = (rng.standard_normal((kv_heads, 256, block_dim)) * sigma).astype(np.float32)
    q = rng.standard_normal((batch, q_heads, head_dim)).astype(np.float32)
    nk = (rng.standard_normal((batch, kv_heads, head_dim)) * sigma).astype(np.float32)
    nv = (rng.standard_normal((batch, kv_heads, head_dim)) * sigma).astype(np.float32)
    return VQKVCache(batch, kv_heads, q_heads, head_dim, block_dim, kc, vc, kcb, vcb, q, nk, nv)


def to_bf16_f32(a: np.ndarray) -> np.ndarray:
    """Round fp32 values to bf16 (nearest even) and return them as fp32."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).reshape(a.shape)
