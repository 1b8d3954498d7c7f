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

    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)

    def forward_tensor(self, x: torch.Tensor, row_start: int = 0, row_stop: Optional[int] = None) -> torch.Tensor:
        """bf16 batch on the tensor cores (tcgen05 dequant GEMM); tolerance of the bf16 path, not bit-exact."""
        _require_cuda(x, "x")
        if x.dtype != torch.bfloat16:
            raise TypeError("forward_tensor needs bfloat16 activations")
        row_stop = self.out_features if row_stop is None else row_stop
        x2 = x.reshape(-1, self.in_features).contiguous()
        out = torch.empty((x2.shape[0], row_stop - row_start), device=x.device, dtype=torch.bfloat16)
        check(lib().ojasx_b200_linear_forward_tensor(self._h, x2.data_ptr(), out.data_ptr(), x2.shape[0], row_start,
                                                     row_stop, _stream_ptr(x.device)), "ojasx_b200_linear_forward_tensor")
        return out.reshape(*x.shape[:-1], row_stop - row_start)

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

    def set_rows(self, row_start: int, row_stop: int) -> None:
        """Restrict every member to output rows ``[row_start, row_stop)`` (a rank's share of a row-split group)."""
        check(lib().ojasx_b200_linear_group_set_rows(self._g, row_start, row_stop), "ojasx_b200_linear_group_set_rows")

    def forward_gather(self, x: torch.Tensor, y_full: torch.Tensor, link, shared_x: bool = False) -> torch.Tensor:
        """The members' rows into the gathered layout ``y_full [P, out_features]`` on every rank of ``link``
        (``y_full`` inside the link's shared segment), then the link's flag; wait on the link before reading."""
        _require_cuda(x, "x")
        xs = 0 if shared_x else x.stride(0) * x.element_size()
        ys = y_full.stride(0) * y_full.element_size()
        check(lib().ojasx_b200_linear_group_forward_gather(self._g, x.data_ptr(), xs, y_full.data_ptr(), ys, _dtype_code(x),
                                                           link, _stream_ptr(x.device)), "ojasx_b200_linear_group_forward_gather")
        return y_full

    def close(self):
        if getattr(self, "_g", None):
            lib().ojasx_b200_destroy_linear_group(self._g)
            self._g = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def silu_mul(gate: torch.Tensor, up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _require_cuda(gate, "gate")
    g, u = gate.contiguous(), up.contiguous()
    o = torch.empty_like(g) if out is None else out
    check(lib().ojasx_b200_silu_mul(g.data_ptr(), u.data_ptr(), o.data_ptr(), g.numel(), _dtype_code(g),
                                    _stream_ptr(g.device)), "ojasx_b200_silu_mul")
    return o


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, add: Optional[torch.Tensor] = None,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x += add`` (in place, when given) then ``out = x * rsqrt(mean(x^2) + eps) * weight``; x is [rows, hidden]."""
    _require_cuda(x, "x")
    assert x.is_contiguous() and x.dim() == 2 and weight.dtype == torch.float32
    o = torch.empty_like(x) if out is None else out
    check(lib().ojasx_b200_rmsnorm(x.data_ptr(), 0 if add is None else add.data_ptr(), weight.data_ptr(), o.data_ptr(),
                                   x.shape[0], x.shape[1], eps, _dtype_code(x), _stream_ptr(x.device)), "ojasx_b200_rmsnorm")
    return o


def rope_qk_(q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor, theta: float) -> None:
    """In-place rotary embedding of q [B, Hq, hd] and k [B, Hkv, hd] at int32 device positions [B]."""
    assert q.is_contiguous() and k.is_contiguous() and positions.dtype == torch.int32 and q.dtype == k.dtype
    check(lib().ojasx_b200_rope_qk(q.data_ptr(), k.data_ptr(), positions.data_ptr(), q.shape[0], q.shape[1], k.shape[1],
                                   q.shape[2], theta, _dtype_code(q), _stream_ptr(q.device)), "ojasx_b200_rope_qk")


def add_int_(values: torch.Tensor, delta: int) -> None:
    assert values.dtype == torch.int32 and values.is_contiguous()
    check(lib().ojasx_b200_add_int(values.data_ptr(), values.numel(), delta, _stream_ptr(values.device)), "ojasx_b200_add_int")


class VQMLP:
    """Dense SwiGLU block of three VQ linears: ``down(silu(gate(x)) * up(x))`` (config 1 of the benchmark set).
    Every linear keeps its own codebook and outliers; intermediate activations are of the input dtype."""

    def __init__(self, gate: VQLinear, up: VQLinear, down: VQLinear):
        assert gate.in_features == up.in_features and gate.out_features == up.out_features == down.in_features
        self.gate, self.up, self.down = gate, up, down
        self._pair = VQLinearGroup([gate, up])   # one launch for gate and up when there is a single token

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.numel() == self.gate.in_features:   # one token: gate and up share x and run as one grouped launch
            gu = torch.empty((2, self.gate.out_features), dtype=x.dtype, device=x.device)
            self._pair.forward(x.reshape(-1), gu, shared_x=True)
            h = silu_mul(gu[0], gu[1], out=gu[0])
            return self.down(h.view(*x.shape[:-1], -1))
        g = self.gate(x)
        u = self.up(x)
        return self.down(silu_mul(g, u, out=g))

    __call__ = forward


class VQMoE:
    """512-expert style top-k MoE layer over VQ-coded experts, resident on the current device.

    ``expert_range=(first, stop)`` keeps only those experts on this device (expert-parallel
    shard); routed ids outside the range contribute nothing here.
    """

    def __init__(self, w, expert_range=None):
        self.hidden, self.inter, self.block_dim = w.hidden, w.inter, w.block_dim
        self.num_experts_total = w.num_experts
        e0, e1 = (0, w.num_experts) if expert_range is None else expert_range
        self.expert_range = (e0, e1)
        n = e1 - e0
        args = [np.ascontiguousarray(w.codebook, dtype=np.float32), np.ascontiguousarray(w.down_codebook, dtype=np.float32),
                np.ascontiguousarray(w.gate_up_codes[e0:e1], dtype=np.uint8),
                np.ascontiguousarray(w.gate_up_scales[e0:e1], dtype=np.float32),
                np.ascontiguousarray(w.down_codes[e0:e1], dtype=np.uint8),
                np.ascontiguousarray(w.down_scales[e0:e1], dtype=np.float32)]
        self._h = lib().ojasx_create_moe(n, w.hidden, w.inter, 10, w.block_dim, *[_p(a) for a in args])
        if not self._h:
            check(-3, "ojasx_create_moe")
        check(lib().ojasx_b200_moe_set_expert_offset(self._h, e0), "ojasx_b200_moe_set_expert_offset")
        for which, csr, rows_per in ((0, w.gate_up_csr, 2 * w.inter), (1, w.down_csr, w.hidden)):
            if csr is None:
                continue
            rp, ci, va = csr
            r0, r1 = e0 * rows_per, e1 * rows_per
            lo, hi = int(rp[r0]), int(rp[r1])
            srp = np.ascontiguousarray(rp[r0:r1 + 1] - lo, dtype=np.int32)
            sci = np.ascontiguousarray(ci[lo:hi], dtype=np.int32)
            sva = np.ascontiguousarray(va[lo:hi], dtype=np.float32)
            check(lib().ojasx_b200_moe_set_outliers(self._h, which, hi - lo, _p(srp), _p(sci), _p(sva)),
                  "ojasx_b200_moe_set_outliers")
        self.has_router = w.router is not None
        if self.has_router:
            r = np.ascontiguousarray(w.router, dtype=np.float32)
            check(lib().ojasx_b200_moe_set_router(self._h, _p(r), w.num_experts), "ojasx_b200_moe_set_router")

    @property
    def handle(self):
        return self._h

    def reserve(self, max_tokens: int, k: int = 10):
        check(lib().ojasx_b200_moe_reserve(self._h, max_tokens, k), "ojasx_b200_moe_reserve")

    def set_gate_limit(self, limit: Optional[float]):
        """Clamp of ``ResidualVQFusedExperts._apply_gate`` (module.py:646-651); ``None`` or ``<= 0`` removes it."""
        check(lib().ojasx_b200_moe_set_gate_limit(self._h, float(limit or 0.0)), "ojasx_b200_moe_set_gate_limit")

    def forward(self, x: torch.Tensor, top_k_index: torch.Tensor, top_k_weights: torch.Tensor) -> torch.Tensor:
        """Argument order of ``ResidualVQFusedExperts.forward`` (ojasx_24x96/module.py:653-658)."""
        _require_cuda(x, "hidden_states")
        x2 = x.reshape(-1, self.hidden).contiguous()
        idx = top_k_index.reshape(x2.shape[0], -1).to(torch.int32).contiguous()
        wts = top_k_weights.reshape(x2.shape[0], -1).to(torch.float32).contiguous()
        y = torch.empty_like(x2)
        check(lib().ojasx_b200_moe_forward(self._h, x2.data_ptr(), idx.data_ptr(), wts.data_ptr(), y.data_ptr(),
                                           x2.shape[0], idx.shape[1], _dtype_code(x2), _stream_ptr(x.device)),
              "ojasx_b200_moe_forward")
        return y.reshape(x.shape)

    def route(self, x: torch.Tensor, top_k: int = 10):
        _require_cuda(x, "x")
        x2 = x.reshape(-1, self.hidden).contiguous()
        idx = torch.empty((x2.shape[0], top_k), device=x.device, dtype=torch.int32)
        wts = torch.empty((x2.shape[0], top_k), device=x.device, dtype=torch.float32)
        check(lib().ojasx_b200_moe_route(self._h, x2.data_ptr(), x2.shape[0], top_k, idx.data_ptr(), wts.data_ptr(),
                                         _dtype_code(x2), _stream_ptr(x.device)), "ojasx_b200_moe_route")
        return idx, wts

    def forward_routed(self, x: torch.Tensor, top_k: int = 10, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        _require_cuda(x, "x")
        x2 = x.reshape(-1, self.hidden).contiguous()
        y = torch.empty_like(x2) if out is None else out
        check(lib().ojasx_b200_moe_forward_routed(self._h, x2.data_ptr(), y.data_ptr(), x2.shape[0], top_k,
                                                  _dtype_code(x2), _stream_ptr(x.device)),
              "ojasx_b200_moe_forward_routed")
        return y.reshape(x.shape)

    def close(self):
        if getattr(self, "_h", None):
            lib().ojasx_destroy_moe(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class VQKVCache:
    """Codebook-VQ KV cache of one layer: append one token per sequence, one decode query per sequence.

    ``head_range=(first, stop)`` keeps only those KV heads (and their query heads) on this
    device: the KV-head shard of a multi-GPU run.
    """

    def __init__(self, batch: int, kv_heads: int, q_heads: int, head_dim: int, block_dim: int, max_seq_len: int,
                 k_codebook, v_codebook):
        kcb = np.ascontiguousarray(k_codebook, dtype=np.float32)
        vcb = np.ascontiguousarray(v_codebook, dtype=np.float32)
        assert kcb.shape == (kv_heads, 256, block_dim) and vcb.shape == kcb.shape
        self.batch, self.kv_heads, self.q_heads = batch, kv_heads, q_heads
        self.head_dim, self.block_dim, self.max_seq_len = head_dim, block_dim, max_seq_len
        self.groups = head_dim // block_dim
        self._h = lib().ojasx_b200_kvq_create(batch, kv_heads, q_heads, head_dim, block_dim, max_seq_len, _p(kcb), _p(vcb))
        if not self._h:
            check(-3, "ojasx_b200_kvq_create")

    @property
    def handle(self):
        return self._h

    def load(self, k_codes, v_codes):
        kc = np.ascontiguousarray(k_codes, dtype=np.uint8)
        vc = np.ascontiguousarray(v_codes, dtype=np.uint8)
        assert kc.shape[:2] == (self.batch, self.kv_heads) and kc.shape[3] == self.groups and vc.shape == kc.shape
        check(lib().ojasx_b200_kvq_load(self._h, _p(kc), _p(vc), kc.shape[2]), "ojasx_b200_kvq_load")

    def read(self, t_begin: int, t_end: int):
        kc = np.empty((self.batch, self.kv_heads, t_end - t_begin, self.groups), np.uint8)
        vc = np.empty_like(kc)
        check(lib().ojasx_b200_kvq_read(self._h, _p(kc), _p(vc), t_begin, t_end), "ojasx_b200_kvq_read")
        return kc, vc

    @property
    def seq_len(self) -> int:
        return lib().ojasx_b200_kvq_seq_len(self._h)

    def reset(self):
        check(lib().ojasx_b200_kvq_reset(self._h), "ojasx_b200_kvq_reset")

    def set_static_plan(self, enabled: bool = True):
        """Plan launches for the capacity and consult only device-side lengths (needed under CUDA-graph replay)."""
        check(lib().ojasx_b200_kvq_set_static_plan(self._h, int(enabled)), "ojasx_b200_kvq_set_static_plan")

    def sync_len(self) -> int:
        return lib().ojasx_b200_kvq_sync_len(self._h)

    def crop(self, max_length: int) -> int:
        """Forget the tokens beyond ``max_length`` of every sequence; returns the new length."""
        n = lib().ojasx_b200_kvq_crop(self._h, int(max_length))
        if n < 0:
            check(n, "ojasx_b200_kvq_crop")
        return n

    @property
    def memory_bytes(self) -> int:
        return int(lib().ojasx_b200_kvq_get_memory_size(self._h))

    def append(self, k: torch.Tensor, v: torch.Tensor):
        _require_cuda(k, "k")
        k2, v2 = k.contiguous(), v.contiguous()
        assert k2.shape == (self.batch, self.kv_heads, self.head_dim) and v2.shape == k2.shape and v2.dtype == k2.dtype
        check(lib().ojasx_b200_kvq_append(self._h, k2.data_ptr(), v2.data_ptr(), _dtype_code(k2), _stream_ptr(k.device)),
              "ojasx_b200_kvq_append")

    def decode(self, q: torch.Tensor, scale: float = -1.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        _require_cuda(q, "q")
        q2 = q.contiguous()
        assert q2.shape == (self.batch, self.q_heads, self.head_dim)
        o = torch.empty_like(q2) if out is None else out
        check(lib().ojasx_b200_kvq_decode(self._h, q2.data_ptr(), o.data_ptr(), scale, _dtype_code(q2),
                                          _stream_ptr(q.device)), "ojasx_b200_kvq_decode")
        return o

    def close(self):
        if getattr(self, "_h", None):
            lib().ojasx_b200_kvq_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
