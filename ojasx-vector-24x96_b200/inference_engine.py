"""Decode driver over the split-manifold kernels: a random-initialised decoder stack whose every linear
(q, k, v, o, the 512-expert MoE, lm_head) is VQ-coded and whose KV cache is codebook-quantised, with the
method names of the reference engines (``OjasXInferenceEngine.prefill / decode_step / generate``,
``ojasx_24x96/engine.py:153-369``; greedy = arg-max of the logits, ``:213-214``; entry class
``UniversalInferenceEngine``, ``ojasx_24x96/inference_engine.py:149-389``).

The reference drives HuggingFace model classes; here the stack is spelled out (RMSNorm, RoPE, GQA
attention, top-k MoE, residuals) because no checkpoint is involved: weights are seeded synthetic
tensors with the shapes and distributions of the benchmark configuration.  Norms, rotary embedding,
residual adds and the arg-max are plain torch ops; everything that touches VQ codes goes through
libojasx_lut_b200.so.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import numpy as np
import torch

from . import synth
from .ops import VQKVCache, VQLinear, VQMoE


@dataclass
class StackConfig:
    layers: int = 24
    hidden: int = 2560
    q_heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    experts: int = 512
    top_k: int = 10
    inter: int = 640
    vocab: int = 151936
    rope_theta: float = 1e6
    rms_eps: float = 1e-6
    block_dim: int = 8
    outlier_frac: float = 0.0038
    max_seq_len: int = 1024
    distinct_layers: int = 1     # host weight sets generated; device copies cycle through them


@dataclass
class LayerWeights:
    """Host arrays of one decoder layer (numpy), so that a CPU restatement can use the very same numbers."""
    q: synth.VQLinearWeights
    k: synth.VQLinearWeights
    v: synth.VQLinearWeights
    o: synth.VQLinearWeights
    moe: synth.VQMoEWeights
    norm1: np.ndarray
    norm2: np.ndarray
    k_codebook: np.ndarray
    v_codebook: np.ndarray


def make_layer_weights(seed: int, cfg: StackConfig) -> LayerWeights:
    rng = np.random.default_rng(seed)
    H, hd, D = cfg.hidden, cfg.head_dim, cfg.block_dim
    lin = lambda s, i, o: synth.make_vq_linear(seed * 16 + s, i, o, block_dim=D, outlier_frac=cfg.outlier_frac)
    sig = 1.0 / np.sqrt(hd)
    return LayerWeights(
        q=lin(1, H, cfg.q_heads * hd), k=lin(2, H, cfg.kv_heads * hd), v=lin(3, H, cfg.kv_heads * hd),
        o=lin(4, cfg.q_heads * hd, H),
        moe=synth.make_vq_moe(seed * 16 + 5, cfg.experts, H, cfg.inter, block_dim=D, outlier_frac=cfg.outlier_frac),
        norm1=(1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32),
        norm2=(1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32),
        k_codebook=(rng.standard_normal((cfg.kv_heads, 256, D)) * sig).astype(np.float32),
        v_codebook=(rng.standard_normal((cfg.kv_heads, 256, D)) * sig).astype(np.float32))


@dataclass
class StackWeights:
    layers: List[LayerWeights]
    embed: np.ndarray            # f32 [vocab, hidden]
    final_norm: np.ndarray
    lm_head: synth.VQLinearWeights


def make_stack_weights(seed: int, cfg: StackConfig) -> StackWeights:
    rng = np.random.default_rng(seed)
    n = max(1, min(cfg.distinct_layers, cfg.layers))
    return StackWeights(
        layers=[make_layer_weights(seed + 1 + i, cfg) for i in range(n)],
        embed=rng.standard_normal((cfg.vocab, cfg.hidden)).astype(np.float32),
        final_norm=(1.0 + 0.1 * rng.standard_normal(cfg.hidden)).astype(np.float32),
        lm_head=synth.make_vq_linear(seed + 999, cfg.hidden, cfg.vocab, block_dim=cfg.block_dim,
                                     outlier_frac=cfg.outlier_frac))


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w).to(x.dtype)


def rope(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotate-half rotary embedding; x [B, heads, head_dim], pos [B] (absolute positions)."""
    hd = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, hd, 2, device=x.device, dtype=torch.float32) / hd))
    ang = pos.float()[:, None] * inv[None, :]                       # [B, hd/2]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    xf = x.float()
    x1, x2 = xf[..., : hd // 2], xf[..., hd // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


class _Layer:
    def __init__(self, w: LayerWeights, cfg: StackConfig, batch: int, device):
        self.q, self.k, self.v, self.o = (VQLinear.from_weights(a) for a in (w.q, w.k, w.v, w.o))
        self.moe = VQMoE(w.moe)
        self.moe.reserve(batch, cfg.top_k)
        self.norm1 = torch.from_numpy(w.norm1).to(device)
        self.norm2 = torch.from_numpy(w.norm2).to(device)
        self.cache = VQKVCache(batch, cfg.kv_heads, cfg.q_heads, cfg.head_dim, cfg.block_dim, cfg.max_seq_len,
                               w.k_codebook, w.v_codebook)


class VQDecoderStack:
    """``batch`` independent sequences decoded in lock step (all at the same position)."""

    def __init__(self, weights: StackWeights, cfg: StackConfig, batch: int = 1, dtype: torch.dtype = torch.float32,
                 device: Optional[torch.device] = None):
        self.cfg, self.batch, self.dtype = cfg, batch, dtype
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.embed = torch.from_numpy(weights.embed).to(self.device)
        self.final_norm = torch.from_numpy(weights.final_norm).to(self.device)
        self.lm_head = VQLinear.from_weights(weights.lm_head)
        n = len(weights.layers)
        self.layers = [_Layer(weights.layers[i % n], cfg, batch, self.device) for i in range(cfg.layers)]
        self.position = 0

    def reset(self) -> None:
        for l in self.layers:
            l.cache.reset()
        self.position = 0

    @torch.no_grad()
    def decode_step(self, token_ids: torch.Tensor) -> torch.Tensor:
        """One token per sequence in, fp32 logits ``[batch, vocab]`` out; the KV caches grow by one."""
        cfg = self.cfg
        B = token_ids.shape[0]
        pos = torch.full((B,), self.position, device=self.device, dtype=torch.int64)
        h = self.embed[token_ids.to(self.device)].to(self.dtype)
        for l in self.layers:
            a = rms_norm(h, l.norm1, cfg.rms_eps)
            q = rope(l.q(a).view(B, cfg.q_heads, cfg.head_dim), pos, cfg.rope_theta)
            k = rope(l.k(a).view(B, cfg.kv_heads, cfg.head_dim), pos, cfg.rope_theta)
            v = l.v(a).view(B, cfg.kv_heads, cfg.head_dim)
            l.cache.append(k.contiguous(), v.contiguous())
            att = l.cache.decode(q.contiguous())
            h = h + l.o(att.view(B, cfg.q_heads * cfg.head_dim))
            m = rms_norm(h, l.norm2, cfg.rms_eps)
            h = h + l.moe.forward_routed(m, cfg.top_k)
        self.position += 1
        return self.lm_head(rms_norm(h, self.final_norm, cfg.rms_eps)).float()

    @torch.no_grad()
    def prefill(self, prompt_ids: torch.Tensor) -> torch.Tensor:
        """Feeds the prompt ``[batch, S]`` token by token (the quantised cache is append-only); returns the last logits."""
        logits = None
        for s in range(prompt_ids.shape[1]):
            logits = self.decode_step(prompt_ids[:, s])
        return logits

    @torch.no_grad()
    def generate(self, prompt_ids: torch.Tensor, max_new_tokens: int) -> torch.Tensor:
        """Greedy decoding: arg-max of the fp32 logits each step.  Returns ``[batch, max_new_tokens]`` ids."""
        logits = self.prefill(prompt_ids)
        out = []
        for _ in range(max_new_tokens):
            nxt = torch.argmax(logits, dim=-1)
            out.append(nxt)
            logits = self.decode_step(nxt)
        return torch.stack(out, dim=1)


class UniversalInferenceEngine:
    """Thin entry class with the reference's call shape: ``engine.generate(prompt_ids, max_new_tokens=...)``."""

    def __init__(self, model: VQDecoderStack, tokenizer=None, *, device=None, max_context_length: Optional[int] = None,
                 subspace_lut_mode: bool = True, fused_native_gemm: bool = False):
        self.model, self.tokenizer = model, tokenizer
        self.max_context_length = max_context_length or model.cfg.max_seq_len

    @classmethod
    def from_synthetic(cls, seed: int, cfg: StackConfig, batch: int = 1, dtype: torch.dtype = torch.float32):
        return cls(VQDecoderStack(make_stack_weights(seed, cfg), cfg, batch, dtype))

    def generate(self, prompt_ids: torch.Tensor, max_new_tokens: int = 16) -> torch.Tensor:
        if prompt_ids.shape[1] + max_new_tokens > self.max_context_length:
            raise ValueError("prompt plus generated tokens exceed max_context_length")
        self.model.reset()
        return self.model.generate(prompt_ids, max_new_tokens)
