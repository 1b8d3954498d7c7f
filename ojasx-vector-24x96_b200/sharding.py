"""Multi-GPU sharding of the path inside one box (one process per GPU, ``torch.distributed``).

The three pieces shard independently and each needs at most one exchange:

* VQ linear: output rows are split across ranks (the ``row_start/row_stop`` contract of
  ``rvq_fused_gemm``, ``ojasx_24x96/native/ojasx_backend_abi.h:97-111``), ``x`` is replicated, the
  row shards of ``y`` are all-gathered;
* MoE: experts are split across ranks, tokens are replicated, every rank evaluates the routed
  experts it holds and the partial outputs are all-reduced;
* KV cache: KV heads (with their query heads) are split across ranks; head outputs are all-gathered.

The partition arithmetic is plain Python so that it can be tested on CPU ranks (gloo); the
compute classes hold one shard each.

Two ways to exchange.  With ``segment=None`` the classes call ``torch.distributed`` collectives after the
kernel.  With a ``PeerSegment`` (GPU ranks of one box) the exchange is fused into the kernel that produces the
shard: its epilogue stores the shard at the same offset in every rank's segment over NVLink and raises a flag,
and the consumer waits for all flags -- no collective launch between producer and consumer.
"""
from __future__ import annotations

from typing import List, Tuple

import ctypes as C

import numpy as np
import torch
import torch.distributed as dist


def split_range(total: int, world: int, rank: int, multiple: int = 1) -> Tuple[int, int]:
    """Contiguous shard ``[start, stop)`` of ``range(total)``; shard sizes are multiples of ``multiple`` except the last."""
    units = (total + multiple - 1) // multiple
    base, extra = divmod(units, world)
    start_u = rank * base + min(rank, extra)
    stop_u = start_u + base + (1 if rank < extra else 0)
    return min(total, start_u * multiple), min(total, stop_u * multiple)


def all_ranges(total: int, world: int, multiple: int = 1) -> List[Tuple[int, int]]:
    return [split_range(total, world, r, multiple) for r in range(world)]


def gather_rows(y_local: torch.Tensor, total_rows: int, group=None) -> torch.Tensor:
    """All-gather row shards ``[B, rows_r]`` (ragged allowed) into ``[B, total_rows]``."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    ranges = all_ranges(total_rows, world, 32)
    width = max(b - a for a, b in ranges)
    pad = torch.zeros((y_local.shape[0], width), device=y_local.device, dtype=y_local.dtype)
    a, b = ranges[rank]
    pad[:, : b - a] = y_local
    parts = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad, group=group)
    return torch.cat([p[:, : hi - lo] for p, (lo, hi) in zip(parts, ranges)], dim=1)


class _DeviceView:
    """Minimal ``__cuda_array_interface__`` carrier: lets torch wrap device memory this package allocated."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False), "version": 2}


_TYPESTR = {torch.float32: "<f4", torch.int32: "<i4", torch.uint8: "|u1", torch.float16: "<f2"}


class PeerSegment:
    """This rank's shared segment, the other ranks' mappings of theirs, and the link the kernels use.

    Every rank must create its segment with the same size and carve the same buffers from it in the same order
    (``alloc``): a buffer then has the same offset everywhere, which is what the kernels rely on.  The first 256
    bytes hold the link's flags.  bf16 buffers are carved as int16-sized views and reinterpreted."""

    def __init__(self, nbytes: int, group=None):
        from ._lib import check, lib
        self._lib, self._check = lib(), check
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.nbytes = int(nbytes) + 256
        self.base = self._lib.ojasx_b200_peer_alloc(self.nbytes)
        if not self.base:
            check(-3, "ojasx_b200_peer_alloc")
        handle = (C.c_ubyte * 64)()
        check(self._lib.ojasx_b200_peer_export(self.base, C.cast(handle, C.c_void_p)), "ojasx_b200_peer_export")
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.mapped = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.mapped.append(self.base)
                continue
            buf = (C.c_ubyte * 64).from_buffer_copy(h)
            ptr = self._lib.ojasx_b200_peer_open(C.cast(buf, C.c_void_p))
            if not ptr:
                check(-3, f"ojasx_b200_peer_open (rank {r})")
            self.mapped.append(ptr)
        arr = (C.c_void_p * self.world)(*self.mapped)
        self.link = self._lib.ojasx_b200_peer_link_create(arr, self.world, self.rank, 0)
        if not self.link:
            check(-3, "ojasx_b200_peer_link_create")
        self._cursor = 256
        self.device = torch.device("cuda", torch.cuda.current_device())
        dist.barrier(group=group)      # nobody stores into a segment that is not mapped everywhere yet

    def alloc(self, shape, dtype=torch.float32) -> torch.Tensor:
        esz = torch.empty((), dtype=dtype).element_size()
        n = int(np.prod(shape)) * esz
        off = (self._cursor + 255) // 256 * 256
        if off + n > self.nbytes:
            raise MemoryError(f"shared segment of {self.nbytes} bytes is full")
        self._cursor = off + n
        if dtype == torch.bfloat16:
            t = torch.as_tensor(_DeviceView(self.base + off, shape, "<i2"), device=self.device).view(torch.bfloat16)
        else:
            t = torch.as_tensor(_DeviceView(self.base + off, shape, _TYPESTR[dtype]), device=self.device)
        return t

    def put(self, dst_shared: torch.Tensor, src: torch.Tensor) -> None:
        """``src`` into ``dst_shared`` (a view of a buffer from ``alloc``) on every rank, then the flag."""
        src = src.contiguous()
        n = src.numel() * src.element_size()
        assert n == dst_shared.numel() * dst_shared.element_size() and n % 4 == 0
        self._check(self._lib.ojasx_b200_peer_put(self.link, dst_shared.data_ptr(), src.data_ptr(), n,
                                                  torch.cuda.current_stream().cuda_stream), "ojasx_b200_peer_put")

    def signal(self) -> None:
        self._check(self._lib.ojasx_b200_peer_signal(self.link, torch.cuda.current_stream().cuda_stream), "ojasx_b200_peer_signal")

    def wait(self) -> None:
        self._check(self._lib.ojasx_b200_peer_wait(self.link, torch.cuda.current_stream().cuda_stream), "ojasx_b200_peer_wait")

    def take_status(self) -> int:
        return int(self._lib.ojasx_b200_peer_take_status(self.link))

    def close(self) -> None:
        if getattr(self, "link", None):
            torch.cuda.synchronize()
            dist.barrier(group=self.group)     # no rank unmaps while another may still store
            self._lib.ojasx_b200_peer_link_destroy(self.link)
            for r, p in enumerate(self.mapped):
                if r != self.rank:
                    self._lib.ojasx_b200_peer_close(p)
            dist.barrier(group=self.group)
            self._lib.ojasx_b200_peer_free(self.base)
            self.link = None


class ShardedVQLinear:
    """Row-split linear: this rank evaluates rows ``split_range(M, world, rank, 32)`` of a full ``ops.VQLinear``."""

    def __init__(self, layer, group=None, segment: "PeerSegment" = None, max_batch: int = 1, dtype=torch.float32, buffers=None):
        """``buffers``: two gathered-output tensors from ``segment.alloc`` to use instead of allocating a pair (callers
        that run many sharded layers in a fixed order can share buffers between layers that are at least two
        exchanges apart; pass the same tensor twice to pin a layer to one buffer)."""
        self.layer, self.group, self.segment = layer, group, segment
        self.row_start, self.row_stop = split_range(layer.out_features, dist.get_world_size(group), dist.get_rank(group), 32)
        self._turn = 0
        if segment is not None:     # two gathered outputs, used in turn (see PeerSegment)
            self._y = list(buffers) if buffers is not None else [segment.alloc((max_batch, layer.out_features), dtype) for _ in range(2)]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x2 = x.reshape(-1, x.shape[-1])
        if self.segment is not None:
            from ._lib import check, lib
            from .ops import _dtype_code, _stream_ptr
            x2 = x2.contiguous()
            y = self._y[self._turn][: x2.shape[0]]
            self._turn ^= 1
            assert y.dtype == x2.dtype and x2.shape[0] <= self._y[0].shape[0]
            check(lib().ojasx_b200_linear_forward_gather(self.layer.handle, x2.data_ptr(), y.data_ptr(), x2.shape[0],
                                                         _dtype_code(x2), self.row_start, self.row_stop, self.segment.link,
                                                         _stream_ptr(x.device)), "ojasx_b200_linear_forward_gather")
            self.segment.wait()
            return y.reshape(*x.shape[:-1], self.layer.out_features)
        if self.row_stop > self.row_start:
            y = self.layer.forward(x2, self.row_start, self.row_stop)
        else:
            y = x2.new_zeros((x2.shape[0], 0))
        return gather_rows(y, self.layer.out_features, self.group).reshape(*x.shape[:-1], self.layer.out_features)


class ExpertParallelMoE:
    """Expert-parallel MoE: ``moe`` is an ``ops.VQMoE`` built with ``expert_range=split_range(E, world, rank)``."""

    def __init__(self, moe, group=None, segment: "PeerSegment" = None, max_tokens: int = 1, top_k: int = 10, buffers=None,
                 logits_buffers=None, shard_router: bool = True):
        """``shard_router``: every rank scores only its own experts and the logits are exchanged too (``logits_buffers``:
        two ``[max_tokens, experts]`` tensors from the segment to use instead of allocating a pair)."""
        self.moe, self.group, self.segment = moe, group, segment
        self._turn = 0
        self._lg = None
        self.shard_router_min_tokens = 64
        if segment is not None and shard_router and moe.has_router:
            self._lg = list(logits_buffers) if logits_buffers is not None else \
                [segment.alloc((max_tokens, moe.num_experts_total), torch.float32) for _ in range(2)]
        if segment is not None:     # per-pair expert outputs of every rank, two buffers used in turn
            self._eo = list(buffers) if buffers is not None else \
                [segment.alloc((max_tokens * top_k, moe.hidden), torch.float32) for _ in range(2)]
            self.moe.reserve(max_tokens, top_k)

    def _gathered(self, x, call, *args):
        from ._lib import check
        from .ops import _dtype_code, _stream_ptr
        x2 = x.reshape(-1, self.moe.hidden).contiguous()
        y = torch.empty_like(x2)
        eo = self._eo[self._turn]
        self._turn ^= 1
        check(call(x2, y, eo, _dtype_code(x2), _stream_ptr(x.device), *args), "expert-parallel MoE forward")
        return y.reshape(x.shape)

    def forward(self, x: torch.Tensor, top_k_index: torch.Tensor, top_k_weights: torch.Tensor) -> torch.Tensor:
        if self.segment is not None:
            from ._lib import lib
            n = x.reshape(-1, self.moe.hidden).shape[0]
            idx = top_k_index.reshape(n, -1).to(torch.int32).contiguous()
            wts = top_k_weights.reshape(n, -1).to(torch.float32).contiguous()
            assert idx.shape[0] * idx.shape[1] <= self._eo[0].shape[0]
            return self._gathered(x, lambda x2, y, eo, dt, st: lib().ojasx_b200_moe_forward_gather(
                self.moe.handle, x2.data_ptr(), idx.data_ptr(), wts.data_ptr(), y.data_ptr(), n, idx.shape[1], dt,
                self.segment.link, eo.data_ptr(), st))
        y = self.moe.forward(x, top_k_index, top_k_weights)
        if y.dtype == torch.float32:
            dist.all_reduce(y, group=self.group)
            return y
        y32 = y.float()
        dist.all_reduce(y32, group=self.group)
        return y32.to(y.dtype)

    def forward_routed(self, x: torch.Tensor, top_k: int = 10) -> torch.Tensor:
        if self.segment is not None:
            from ._lib import lib
            n = x.reshape(-1, self.moe.hidden).shape[0]
            assert n * top_k <= self._eo[0].shape[0]
            # the logits exchange costs about ten microseconds of signalling: it pays once scoring all experts on every
            # rank takes longer than that (measured: from a few dozen tokens)
            lg = self._lg[self._turn].data_ptr() if (self._lg is not None and n >= self.shard_router_min_tokens) else None
            return self._gathered(x, lambda x2, y, eo, dt, st: lib().ojasx_b200_moe_forward_routed_gather(
                self.moe.handle, x2.data_ptr(), y.data_ptr(), n, top_k, dt, self.segment.link, eo.data_ptr(), lg, st))
        idx, wts = self.moe.route(x, top_k)   # router weights are replicated: same routing on every rank
        return self.forward(x, idx, wts)


class HeadShardedKVCache:
    """KV-head split: ``cache`` is an ``ops.VQKVCache`` holding KV heads ``split_range(Hkv, world, rank)`` only."""

    def __init__(self, cache, total_q_heads: int, group=None, total_kv_heads: int = 0, segment: "PeerSegment" = None,
                 dtype=torch.float32, buffers=None):
        self.cache, self.total_q_heads, self.group, self.segment = cache, total_q_heads, group, segment
        world = dist.get_world_size(group)
        self._turn = 0
        if segment is not None:
            self._o = list(buffers) if buffers is not None else \
                [segment.alloc((cache.batch, total_q_heads, cache.head_dim), dtype) for _ in range(2)]
        # query heads held by every rank (ragged when the KV heads do not divide evenly)
        kv = total_kv_heads or world * cache.kv_heads
        per_kv = total_q_heads // kv
        self.q_ranges = [(a * per_kv, b * per_kv) for a, b in all_ranges(kv, world)]

    def decode(self, q_local: torch.Tensor, scale: float = -1.0) -> torch.Tensor:
        if self.segment is not None:
            from ._lib import check, lib
            from .ops import _dtype_code, _stream_ptr
            q2 = q_local.contiguous()
            o = self._o[self._turn]
            self._turn ^= 1
            first = self.q_ranges[dist.get_rank(self.group)][0]
            check(lib().ojasx_b200_kvq_decode_gather(self.cache.handle, q2.data_ptr(), o.data_ptr(), scale, _dtype_code(q2),
                                                     self.total_q_heads, first, self.segment.link, _stream_ptr(q2.device)),
                  "ojasx_b200_kvq_decode_gather")
            self.segment.wait()
            return o
        o = self.cache.decode(q_local, scale)                      # [B, Hq_local, hd]
        width = max(b - a for a, b in self.q_ranges)
        pad = o.new_zeros((o.shape[0], width, o.shape[2]))         # equal-sized pieces: ragged shards are padded
        pad[:, : o.shape[1]] = o
        parts = [torch.empty_like(pad) for _ in self.q_ranges]
        dist.all_gather(parts, pad, group=self.group)
        return torch.cat([p[:, : b - a] for p, (a, b) in zip(parts, self.q_ranges)], dim=1)
