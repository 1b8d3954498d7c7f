"""Decode driver over the split-manifold kernels: a random-initialised decoder stack whose every linear
(q, k, v, o, the 512-expert MoE, lm_head) is VQ-coded and whose KV cache is codebook-quantised, with the
method names of the reference engines (``OjasXInferenceEngine.prefill / decode_step / generate``,
``ojasx_24x96/engine.py:153-369``; greedy = arg-max of the logits, ``:213-214``; entry class
``UniversalInferenceEngine``, ``ojasx_24x96/inference_engine.py:149-389``).

The reference drives HuggingFace model classes; here the stack is spelled out (RMSNorm, RoPE, GQA
attention, top-k MoE, residuals) because no checkpoint is involved: weights are seeded synthetic
tensors with the shapes and distributions of the benchmark configuration.  The embedding lookup and the
arg-max are torch ops; norms (with the residual adds folded in), rotary embedding and everything that
touches VQ codes are kernels of libojasx_lut_b200.so, so one decode step is a fixed launch sequence.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import numpy as np
import torch

from . import synth
from .ops import VQKVCache, VQLinear, VQLinearGroup, VQMoE, add_int_, rmsnorm, rope_qk_


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


class _Layer:
    def __init__(self, w: LayerWeights, cfg: StackConfig, batch: int, device):
        self.q, self.k, self.v, self.o = (VQLinear.from_weights(a) for a in (w.q, w.k, w.v, w.o))
        # one sequence: q, k and v read the same vector and run as one grouped launch into a fixed buffer
        self.qkv = VQLinearGroup([self.q, self.k, self.v]) if batch == 1 else None
        self.qkv_out = None
        self.moe = VQMoE(w.moe)
        self.moe.reserve(batch, cfg.top_k)
        self.norm1 = torch.from_numpy(w.norm1).to(device)
        self.norm2 = torch.from_numpy(w.norm2).to(device)
        self.cache = VQKVCache(batch, cfg.kv_heads, cfg.q_heads, cfg.head_dim, cfg.block_dim, cfg.max_seq_len,
                               w.k_codebook, w.v_codebook)


class VQDecoderStack:
    """``batch`` independent sequences decoded in lock step (all at the same position).

    ``use_graph=True`` captures one decode step in a CUDA graph after a warm-up step and replays it for
    every token: the step is a fixed sequence of launches (positions and cache lengths live on the device,
    the KV kernels are planned for the cache capacity), so per-token host work is one graph launch.
    """

    def __init__(self, weights: StackWeights, cfg: StackConfig, batch: int = 1, dtype: torch.dtype = torch.float32,
                 device: Optional[torch.device] = None, use_graph: bool = False):
        self.cfg, self.batch, self.dtype, self.use_graph = cfg, batch, dtype, use_graph
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.embed = torch.from_numpy(weights.embed).to(self.device)
        self.final_norm = torch.from_numpy(weights.final_norm).to(self.device)
        self.lm_head = VQLinear.from_weights(weights.lm_head)
        n = len(weights.layers)
        self.layers = [_Layer(weights.layers[i % n], cfg, batch, self.device) for i in range(cfg.layers)]
        self.pos = torch.zeros(batch, dtype=torch.int32, device=self.device)
        self.position = 0
        self._graph = None
        self._ids = torch.zeros(batch, dtype=torch.int64, device=self.device)
        self._logits = None
        if use_graph:
            for l in self.layers:
                l.cache.set_static_plan(True)

    def reset(self) -> None:
        for l in self.layers:
            l.cache.reset()
        self.pos.zero_()
        self.position = 0

    def _enqueue_step(self, ids: torch.Tensor) -> torch.Tensor:
        cfg, B = self.cfg, self.batch
        h = self.embed[ids].to(self.dtype)
        pending = None                       # residual branch not yet added to h (added inside the next norm)
        for l in self.layers:
            a = rmsnorm(h, l.norm1, cfg.rms_eps, add=pending)
            if l.qkv is not None:
                if l.qkv_out is None or l.qkv_out.dtype != a.dtype:
                    l.qkv_out = torch.empty((3, cfg.q_heads * cfg.head_dim), dtype=a.dtype, device=self.device)
                l.qkv.forward(a.view(-1), l.qkv_out, shared_x=True)
                q = l.qkv_out[0].view(B, cfg.q_heads, cfg.head_dim)
                k = l.qkv_out[1, : cfg.kv_heads * cfg.head_dim].view(B, cfg.kv_heads, cfg.head_dim)
                v = l.qkv_out[2, : cfg.kv_heads * cfg.head_dim].view(B, cfg.kv_heads, cfg.head_dim)
            else:
                q = l.q(a).view(B, cfg.q_heads, cfg.head_dim)
                k = l.k(a).view(B, cfg.kv_heads, cfg.head_dim)
                v = l.v(a).view(B, cfg.kv_heads, cfg.head_dim)
            rope_qk_(q, k, self.pos, cfg.rope_theta)
            l.cache.append(k, v)
            att = l.cache.decode(q)
            o = l.o(att.view(B, cfg.q_heads * cfg.head_dim))
            m = rmsnorm(h, l.norm2, cfg.rms_eps, add=o)
            pending = l.moe.forward_routed(m, cfg.top_k)
        a = rmsnorm(h, self.final_norm, cfg.rms_eps, add=pending)
        add_int_(self.pos, 1)
        return self.lm_head(a).float()

    @torch.no_grad()
    def decode_step(self, token_ids: torch.Tensor) -> torch.Tensor:
        """One token per sequence in, fp32 logits ``[batch, vocab]`` out; the KV caches grow by one."""
        ids = token_ids.to(self.device).to(torch.int64)
        if self.position >= self.cfg.max_seq_len:
            raise ValueError(f"the KV caches hold max_seq_len = {self.cfg.max_seq_len} tokens; reset() before decoding further")
        self.position += 1
        if not self.use_graph:
            return self._enqueue_step(ids)
        if self._graph is None:
            if self.position != 1:
                raise RuntimeError("the first graph-mode step must come right after reset(): capture starts on empty caches")
            # warm-up on a side stream (lazy kernel attributes, occupancy queries, scratch growth) ...
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self._ids.copy_(ids)
                self._enqueue_step(self._ids)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            # ... whose token is dropped again before the capture; a capture records launches, it runs nothing
            self.reset()
            self.position = 1
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph):
                self._logits = self._enqueue_step(self._ids)
        self._ids.copy_(ids)
        self._graph.replay()
        return self._logits

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
