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

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple, Union

import numpy as np
import torch

from torch import nn

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
    def __init__(self, w: LayerWeights, cfg: StackConfig, batch: int, device, segment=None, dtype=torch.float32, shared=None):
        self.q, self.k, self.v, self.o = (VQLinear.from_weights(a) for a in (w.q, w.k, w.v, w.o))
        self.norm1 = torch.from_numpy(w.norm1).to(device)
        self.norm2 = torch.from_numpy(w.norm2).to(device)
        self.qkv_out = None
        if segment is None:
            # one sequence: q, k and v read the same vector and run as one grouped launch into a fixed buffer
            self.qkv = VQLinearGroup([self.q, self.k, self.v]) if batch == 1 else None
            self.moe = VQMoE(w.moe)
            self.moe.reserve(batch, cfg.top_k)
            self.cache = VQKVCache(batch, cfg.kv_heads, cfg.q_heads, cfg.head_dim, cfg.block_dim, cfg.max_seq_len,
                                   w.k_codebook, w.v_codebook)
            return
        # One rank of several: its KV heads with their query heads, its rows of o_proj, its experts.  The three
        # exchanges of a layer (attention outputs, o_proj outputs, expert outputs) are fused into the producing kernels.
        from . import sharding
        world, rank = segment.world, segment.rank
        if cfg.kv_heads % world:
            raise ValueError("the KV heads must divide evenly over the ranks")
        self.qkv = None
        R = cfg.q_heads // cfg.kv_heads
        self.h0, self.h1 = sharding.split_range(cfg.kv_heads, world, rank)
        self.kv_local = self.h1 - self.h0
        self.q_rows = (self.h0 * R * cfg.head_dim, self.h1 * R * cfg.head_dim)
        self.kv_rows = (self.h0 * cfg.head_dim, self.h1 * cfg.head_dim)
        self.cache = VQKVCache(batch, self.kv_local, self.kv_local * R, cfg.head_dim, cfg.block_dim, cfg.max_seq_len,
                               w.k_codebook[self.h0:self.h1], w.v_codebook[self.h0:self.h1])
        # `shared`: exchange buffers of this layer (att, o, expert outputs), handed out by the stack: consecutive layers
        # get different ones, a layer always the same one, so a buffer is written again six exchanges later
        att, o, eo, lg = shared
        self.kv_sharded = sharding.HeadShardedKVCache(self.cache, cfg.q_heads, total_kv_heads=cfg.kv_heads, segment=segment,
                                                      dtype=dtype, buffers=(att, att))
        self.o_sharded = sharding.ShardedVQLinear(self.o, segment=segment, max_batch=batch, dtype=dtype, buffers=(o, o))
        e0, e1 = sharding.split_range(cfg.experts, world, rank)
        self.moe = VQMoE(w.moe, (e0, e1))
        self.moe_ep = sharding.ExpertParallelMoE(self.moe, segment=segment, max_tokens=batch, top_k=cfg.top_k, buffers=(eo, eo),
                                                 logits_buffers=(lg, lg))
        self.moe.reserve(batch, cfg.top_k)


class VQDecoderStack:
    """``batch`` independent sequences decoded in lock step (all at the same position).

    ``use_graph=True`` captures one decode step in a CUDA graph after a warm-up step and replays it for
    every token: the step is a fixed sequence of launches (positions and cache lengths live on the device,
    the KV kernels are planned for the cache capacity), so per-token host work is one graph launch.
    """

    def __init__(self, weights: StackWeights, cfg: StackConfig, batch: int = 1, dtype: torch.dtype = torch.float32,
                 device: Optional[torch.device] = None, use_graph: bool = False, segment=None):
        """``segment``: a ``sharding.PeerSegment`` makes this the stack of ONE rank of several GPUs: KV heads (with the
        q/k/v rows of their heads), o_proj rows, experts and lm_head rows are split over the ranks; hidden states are
        replicated; every exchange goes through the segment.  Every rank must drive its stack with the same calls."""
        self.cfg, self.batch, self.dtype, self.use_graph = cfg, batch, dtype, use_graph
        self.segment = segment
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.embed = torch.from_numpy(weights.embed).to(self.device)
        self.final_norm = torch.from_numpy(weights.final_norm).to(self.device)
        self.lm_head = VQLinear.from_weights(weights.lm_head)
        n = len(weights.layers)
        shared = [None, None]
        if segment is not None:      # two sets of exchange buffers, for even and odd layers
            shared = [(segment.alloc((batch, cfg.q_heads, cfg.head_dim), dtype), segment.alloc((batch, cfg.hidden), dtype),
                       segment.alloc((batch * cfg.top_k, cfg.hidden), torch.float32),
                       segment.alloc((batch, cfg.experts), torch.float32)) for _ in range(2)]
        self.layers = [_Layer(weights.layers[i % n], cfg, batch, self.device, segment, dtype, shared[i & 1]) for i in range(cfg.layers)]
        if segment is not None:
            from . import sharding
            self.lm_sharded = sharding.ShardedVQLinear(self.lm_head, segment=segment, max_batch=batch, dtype=dtype)
            self.vocab_rows = (self.lm_sharded.row_start, self.lm_sharded.row_stop)
            self._best = segment.alloc((segment.world, batch, 2), torch.float32)    # (max, index) of every rank's vocabulary shard
            self._mine = torch.empty((batch, 2), dtype=torch.float32, device=self.device)
            self._next = None
        self.gather_logits = True
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

    def named_quantized_ops(self):
        """(name, operator) of every VQ-coded operator of the stack, for audits."""
        for i, l in enumerate(self.layers):
            for n in ("q", "k", "v", "o"):
                yield f"layers.{i}.attn.{n}_proj", getattr(l, n)
            yield f"layers.{i}.moe", l.moe
        yield "lm_head", self.lm_head

    @torch.no_grad()
    def decode_step_eager(self, token_ids: torch.Tensor) -> torch.Tensor:
        """One decode step launched kernel by kernel (no CUDA-graph replay), q/k/v as separate calls: the form
        an audit can watch.  Advances the caches like ``decode_step``."""
        if self._graph is not None:
            raise RuntimeError("this stack already replays a captured step; audit a stack built with use_graph=False")
        if self.position >= self.cfg.max_seq_len:
            raise ValueError(f"the KV caches hold max_seq_len = {self.cfg.max_seq_len} tokens; reset() before decoding further")
        self.position += 1
        grouped = [l.qkv for l in self.layers]
        for l in self.layers:
            l.qkv = None
        try:
            return self._enqueue_step(token_ids.to(self.device).to(torch.int64))
        finally:
            for l, g in zip(self.layers, grouped):
                l.qkv = g

    def _enqueue_step(self, ids: torch.Tensor) -> torch.Tensor:
        cfg, B = self.cfg, self.batch
        h = self.embed[ids].to(self.dtype)
        pending = None                       # residual branch not yet added to h (added inside the next norm)
        if self.segment is not None:
            return self._enqueue_step_sharded(h)
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

    def _enqueue_step_sharded(self, h: torch.Tensor) -> torch.Tensor:
        """The step of one rank (see ``__init__``); returns the gathered fp32 logits and leaves the greedy next
        token of every sequence, found by an arg-max over the ranks' vocabulary shards, in ``self._next``."""
        cfg, B = self.cfg, self.batch
        R = cfg.q_heads // cfg.kv_heads
        pending = None
        for l in self.layers:
            a = rmsnorm(h, l.norm1, cfg.rms_eps, add=pending)
            q = l.q.forward(a, *l.q_rows).view(B, l.kv_local * R, cfg.head_dim)
            k = l.k.forward(a, *l.kv_rows).view(B, l.kv_local, cfg.head_dim)
            v = l.v.forward(a, *l.kv_rows).view(B, l.kv_local, cfg.head_dim)
            rope_qk_(q, k, self.pos, cfg.rope_theta)
            l.cache.append(k, v)
            att = l.kv_sharded.decode(q)                                         # [B, all query heads, hd] on every rank
            o = l.o_sharded.forward(att.view(B, cfg.q_heads * cfg.head_dim))     # [B, hidden] on every rank
            m = rmsnorm(h, l.norm2, cfg.rms_eps, add=o)
            pending = l.moe_ep.forward_routed(m, cfg.top_k)
        a = rmsnorm(h, self.final_norm, cfg.rms_eps, add=pending)
        add_int_(self.pos, 1)
        # lm_head split over the vocabulary: arg-max of the own shard, (max, index) to every rank, arg-max over ranks
        # (the lowest rank wins a tie, i.e. the lowest index, as torch.argmax does on the full row)
        v0, v1 = self.vocab_rows
        local = self.lm_head.forward(a, v0, v1).float()
        best, where = torch.max(local, dim=-1)
        self._mine[:, 0] = best
        self._mine[:, 1] = (where + v0).float()            # exact: vocabulary indices are below 2^24
        self.segment.put(self._best[self.segment.rank], self._mine)
        self.segment.wait()
        pick = torch.argmax(self._best[:, :, 0], dim=0)
        self._next = self._best[pick, torch.arange(B, device=self.device), 1].long()
        # the full logits on every rank cost one more gather (vocab * 4 bytes per sequence): greedy decoding does
        # not need them, so `gather_logits = False` returns this rank's shard [B, v1 - v0] instead
        return self.lm_sharded.forward(a).float() if self.gather_logits else local

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
            cached = self.position - 1      # tokens in the caches before this step (a prefill may have put some there)
            # warm-up on a side stream (lazy kernel attributes, occupancy queries, scratch growth) ...
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self._ids.copy_(ids)
                self._enqueue_step(self._ids)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            # ... whose token is dropped again before the capture; a capture records launches, it runs nothing
            for l in self.layers:
                l.cache.crop(cached)
            self.pos.fill_(cached)
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph):
                self._logits = self._enqueue_step(self._ids)
        self._ids.copy_(ids)
        self._graph.replay()
        return self._logits

    @torch.no_grad()
    def prefill(self, prompt_ids: torch.Tensor, batched: Optional[bool] = None, max_rows: int = 1024) -> torch.Tensor:
        """The prompt ``[batch, S]`` into the caches; returns the logits after its last token (one model call over the
        prompt, ``ojasx_24x96/engine.py:153-175``).

        ``batched`` (default on one device): all positions of a chunk of the prompt go through the linears and the MoE
        as ONE batch -- the regime of the batched kernels: persistent table kernel in fp32, tensor-core dequant GEMM
        for bf16 -- while attention, whose quantised cache grows a token at a time, appends and decodes position by
        position.  Results are those of the token-by-token form (every kernel keeps its summation order whatever the
        batch).  ``max_rows`` bounds batch * positions per chunk (scratch of the MoE grows with it).  Otherwise, and on
        a stack split over several ranks, the prompt is fed through ``decode_step`` token by token."""
        if batched is None:
            batched = self.segment is None
        if not batched or self.segment is not None:
            logits = None
            for s in range(prompt_ids.shape[1]):
                logits = self.decode_step(prompt_ids[:, s])
            return logits
        ids = prompt_ids.to(self.device).to(torch.int64)
        S = ids.shape[1]
        if self.position + S > self.cfg.max_seq_len:
            raise ValueError(f"the KV caches hold max_seq_len = {self.cfg.max_seq_len} tokens")
        step = max(1, max_rows // self.batch)
        logits = None
        for s0 in range(0, S, step):
            logits = self._prefill_chunk(ids[:, s0:s0 + step])
        return logits

    def _prefill_chunk(self, ids: torch.Tensor) -> torch.Tensor:
        """``ids [batch, Sc]``: rows are ordered position-major (row = s * batch + b), so that the q, k, v and attention
        rows of one position are contiguous ``[batch, heads, head_dim]`` blocks for the cache calls."""
        cfg, B = self.cfg, self.batch
        Sc = ids.shape[1]
        rows = B * Sc
        h = self.embed[ids.t().reshape(-1)].to(self.dtype)
        pos_rows = (self.pos.view(1, B) + torch.arange(Sc, device=self.device, dtype=torch.int32).view(Sc, 1)).reshape(-1).contiguous()
        pending = None
        for l in self.layers:
            l.moe.reserve(rows, cfg.top_k)
            a = rmsnorm(h, l.norm1, cfg.rms_eps, add=pending)
            q = l.q(a).view(rows, cfg.q_heads, cfg.head_dim)
            k = l.k(a).view(rows, cfg.kv_heads, cfg.head_dim)
            v = l.v(a).view(rows, cfg.kv_heads, cfg.head_dim)
            rope_qk_(q, k, pos_rows, cfg.rope_theta)
            q4, k4, v4 = (t.view(Sc, B, t.shape[1], cfg.head_dim) for t in (q, k, v))
            att = torch.empty_like(q4)
            for s in range(Sc):
                l.cache.append(k4[s], v4[s])
                l.cache.decode(q4[s], out=att[s])
            o = l.o(att.view(rows, cfg.q_heads * cfg.head_dim))
            m = rmsnorm(h, l.norm2, cfg.rms_eps, add=o)
            pending = l.moe.forward_routed(m, cfg.top_k)
        a = rmsnorm(h, self.final_norm, cfg.rms_eps, add=pending)
        add_int_(self.pos, Sc)
        self.position += Sc
        return self.lm_head(a[(Sc - 1) * B:].contiguous()).float()

    @torch.no_grad()
    def generate(self, prompt_ids: torch.Tensor, max_new_tokens: int) -> torch.Tensor:
        """Greedy decoding: arg-max of the fp32 logits each step.  Returns ``[batch, max_new_tokens]`` ids."""
        logits = self.prefill(prompt_ids)
        out = []
        for _ in range(max_new_tokens):
            # several ranks: the arg-max over the vocabulary shards that the step left behind (same token on every rank)
            nxt = torch.argmax(logits, dim=-1) if self.segment is None else self._next.clone()
            out.append(nxt)
            logits = self.decode_step(nxt)
        return torch.stack(out, dim=1)


@dataclass
class LayerExecutionTrace:
    """What one quantised layer did during an audited forward pass (``ojasx_24x96/inference_engine.py:39-65``)."""
    layer_name: str
    module_type: str
    codec: str
    call_count: int = 0
    input_shape: Tuple[int, ...] = ()
    output_shape: Tuple[int, ...] = ()
    output_l2_norm: float = 0.0
    all_finite: bool = True
    active_experts: List[int] = field(default_factory=list)

    def to_dict(self) -> Dict[str, object]:
        return {"layer_name": self.layer_name, "module_type": self.module_type, "codec": self.codec,
                "call_count": self.call_count, "input_shape": list(self.input_shape),
                "output_shape": list(self.output_shape), "output_l2_norm": round(self.output_l2_norm, 6),
                "all_finite": self.all_finite, "active_experts": self.active_experts}


@dataclass
class ForwardGraphAuditReport:
    """Summary over every quantised layer of the model (``ojasx_24x96/inference_engine.py:68-95``)."""
    total_quantized_modules: int
    executed_quantized_modules: int
    all_outputs_finite: bool
    total_forward_calls: int
    active_moe_experts_union: List[int]
    traces: Dict[str, LayerExecutionTrace]

    @property
    def execution_coverage_ratio(self) -> float:
        return 1.0 if self.total_quantized_modules == 0 else self.executed_quantized_modules / self.total_quantized_modules

    def to_dict(self) -> Dict[str, object]:
        return {"total_quantized_modules": self.total_quantized_modules,
                "executed_quantized_modules": self.executed_quantized_modules,
                "execution_coverage_ratio": round(self.execution_coverage_ratio, 4),
                "all_outputs_finite": self.all_outputs_finite, "total_forward_calls": self.total_forward_calls,
                "active_moe_experts_union": self.active_moe_experts_union,
                "traces": {k: v.to_dict() for k, v in self.traces.items()}}


def _set_submodule(model: nn.Module, path: str, new: nn.Module) -> None:
    parent = model
    parts = path.split(".")
    for p in parts[:-1]:
        parent = getattr(parent, p)
    setattr(parent, parts[-1], new)


class UniversalInferenceEngine:
    """Entry class with the reference's call shape (``ojasx_24x96/inference_engine.py:149-389``).

    ``model`` is either a ``VQDecoderStack`` of this module (the decode driver of the benchmark configuration)
    or any ``torch.nn.Module`` whose quantised layers are this package's ``ResidualVQLinear`` /
    ``ResidualVQFusedExperts`` (what ``from_oqpack`` produces from a skeleton and a package)."""

    def __init__(self, model, tokenizer=None, *, device=None, max_context_length: Optional[int] = None,
                 subspace_lut_mode: bool = True, fused_native_gemm: bool = False):
        from .module import ResidualVQLinear
        self.model, self.tokenizer = model, tokenizer
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        if isinstance(model, nn.Module):
            model.eval()
            for _, mod in model.named_modules():
                if isinstance(mod, ResidualVQLinear):
                    mod.set_subspace_lut_mode(subspace_lut_mode)
                    mod.set_fused_native_gemm(fused_native_gemm)
            self.max_context_length = int(max_context_length or 4096)
        else:
            self.max_context_length = int(max_context_length or model.cfg.max_seq_len)

    @classmethod
    def from_synthetic(cls, seed: int, cfg: StackConfig, batch: int = 1, dtype: torch.dtype = torch.float32):
        return cls(VQDecoderStack(make_stack_weights(seed, cfg), cfg, batch, dtype))

    @classmethod
    def from_oqpack(cls, skeleton_or_factory: Union[nn.Module, Callable[[], nn.Module]], package_dir, *, tokenizer=None,
                    device="cuda", verify_checksums: bool = True, streaming_decode: bool = True,
                    subspace_lut_mode: bool = True) -> Tuple["UniversalInferenceEngine", Dict[str, object]]:
        """``(engine, manifest)`` from an ``.oqpack`` directory (``ojasx_24x96/inference_engine.py:190-232``): the
        package's quantised linears replace the same-named sub-modules of the skeleton (a module, or a factory
        that builds one), their tensors going from the shard files straight to ``device``; everything else of
        the skeleton (norms, embeddings) is moved to ``device`` as it is.  Layers the kernels do not cover
        are left as the skeleton has them and listed under ``manifest["skipped_layers"]``."""
        from . import oqpack
        skeleton = skeleton_or_factory() if callable(skeleton_or_factory) and not isinstance(skeleton_or_factory, nn.Module) \
            else skeleton_or_factory
        layers, skipped = oqpack.load_quantized_layers(str(package_dir), device=device, verify_checksums=verify_checksums)
        known = dict(skeleton.named_modules())
        for name, layer in layers.items():
            if name not in known:
                raise oqpack.OQPackValidationError(f"Package layer {name} has no counterpart in the skeleton")
            _set_submodule(skeleton, name, layer)
        model = skeleton.to(device)
        manifest = dict(oqpack.read_manifest(str(package_dir)))
        manifest["skipped_layers"] = skipped
        return cls(model, tokenizer=tokenizer, device=device, subspace_lut_mode=subspace_lut_mode), manifest

    def forward_any(self, *args, **kwargs) -> Any:
        """The model's own forward on whatever inputs it takes."""
        return self.model(*args, **kwargs)

    # ------------------------------------------------------------------ audit
    def _quantized_ops(self) -> Dict[str, Tuple[Any, str, str]]:
        """name -> (object, module type, codec) of every top-level quantised operator of the model."""
        from .module import ResidualVQFusedExperts, ResidualVQLinear
        found: Dict[str, Tuple[Any, str, str]] = {}
        if isinstance(self.model, nn.Module):
            inside: List[str] = []
            for name, mod in self.model.named_modules():
                if any(name.startswith(p) for p in inside):
                    continue
                if isinstance(mod, ResidualVQFusedExperts):
                    inside.append(name + ".")     # its two projections are not called on their own
                    found[name] = (mod, "ResidualVQFusedExperts", mod.gate_up_proj.codec)
                elif isinstance(mod, ResidualVQLinear):
                    found[name] = (mod, "ResidualVQLinear", mod.codec)
        else:
            for name, op in self.model.named_quantized_ops():
                found[name] = (op, type(op).__name__, "split_manifold_vq")
        return found

    def audit_forward_graph(self, *forward_args, **forward_kwargs) -> Tuple[Any, ForwardGraphAuditReport]:
        """One real forward pass with every quantised linear and expert bank watched
        (``ojasx_24x96/inference_engine.py:268-357``): call counts, shapes, output norms, finiteness and the
        experts that were routed to.  A ``VQDecoderStack`` is stepped eagerly for this (a replayed CUDA graph runs
        no Python), with ``forward_args`` = the token ids of one decode step."""
        traces: Dict[str, LayerExecutionTrace] = {}
        undo: List[Callable[[], None]] = []

        def record(key: str, inputs, output) -> None:
            tr = traces[key]
            tr.call_count += 1
            if inputs and isinstance(inputs[0], torch.Tensor):
                tr.input_shape = tuple(inputs[0].shape)
            if tr.module_type in ("ResidualVQFusedExperts", "VQMoE") and len(inputs) >= 2 and isinstance(inputs[1], torch.Tensor) \
                    and not inputs[1].is_floating_point():
                tr.active_experts = sorted(set(tr.active_experts).union(int(v) for v in torch.unique(inputs[1].detach()).cpu().tolist()))
            out = output[0] if isinstance(output, tuple) else output
            if isinstance(out, torch.Tensor):
                tr.output_shape = tuple(out.shape)
                tr.output_l2_norm = float(out.detach().float().norm().item())
                tr.all_finite = tr.all_finite and bool(torch.isfinite(out).all().item())

        for name, (op, mtype, codec) in self._quantized_ops().items():
            traces[name] = LayerExecutionTrace(layer_name=name, module_type=mtype, codec=codec)
            if isinstance(op, nn.Module):
                h = op.register_forward_hook(lambda m, i, o, key=name: record(key, i, o))
                undo.append(h.remove)
            else:   # plain operator objects of the decode driver: wrap their bound methods for the duration
                for meth in ("forward", "forward_routed"):
                    if hasattr(op, meth):
                        orig = getattr(op, meth)

                        def wrapped(*a, _orig=orig, _key=name, _meth=meth, _op=op, **kw):
                            out = _orig(*a, **kw)
                            ins = a
                            if _meth == "forward_routed":     # report the experts the layer's router chose
                                ins = (a[0], _op.route(a[0], a[1] if len(a) > 1 else kw.get("top_k", 10))[0])
                            record(_key, ins, out)
                            return out
                        setattr(op, meth, wrapped)
                        undo.append(lambda _op=op, _meth=meth: delattr(_op, _meth))
        try:
            with torch.no_grad():
                if isinstance(self.model, nn.Module):
                    output = self.model(*forward_args, **forward_kwargs)
                else:
                    output = self.model.decode_step_eager(*forward_args, **forward_kwargs)
        finally:
            for u in undo:
                u()
        ran = [t for t in traces.values() if t.call_count > 0]
        report = ForwardGraphAuditReport(
            total_quantized_modules=len(traces), executed_quantized_modules=len(ran),
            all_outputs_finite=all(t.all_finite for t in ran), total_forward_calls=sum(t.call_count for t in traces.values()),
            active_moe_experts_union=sorted({e for t in traces.values() for e in t.active_experts}), traces=traces)
        return output, report

    def generate(self, prompt_ids: torch.Tensor, max_new_tokens: int = 16) -> torch.Tensor:
        if prompt_ids.shape[1] + max_new_tokens > self.max_context_length:
            raise ValueError("prompt plus generated tokens exceed max_context_length")
        if isinstance(self.model, nn.Module):
            # generic module: logits [B, S, V] from token ids, greedy arg-max (engine.py:213-214), no cache
            ids = prompt_ids.to(self.device)
            out = []
            with torch.no_grad():
                for _ in range(max_new_tokens):
                    logits = self.model(ids)
                    nxt = torch.argmax(logits[:, -1].float(), dim=-1)
                    out.append(nxt)
                    ids = torch.cat([ids, nxt[:, None]], dim=1)
            return torch.stack(out, dim=1)
        self.model.reset()
        return self.model.generate(prompt_ids, max_new_tokens)
