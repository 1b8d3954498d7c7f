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
"""
from __future__ import annotations

from typing import List, Tuple

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


class ShardedVQLinear:
    """Row-split linear: this rank evaluates rows ``split_range(M, world, rank, 32)`` of a full ``ops.VQLinear``."""

    def __init__(self, layer, group=None):
        self.layer, self.group = layer, group
        self.row_start, self.row_stop = split_range(layer.out_features, dist.get_world_size(group), dist.get_rank(group), 32)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x2 = x.reshape(-1, x.shape[-1])
        if self.row_stop > self.row_start:
            y = self.layer.forward(x2, self.row_start, self.row_stop)
        else:
            y = x2.new_zeros((x2.shape[0], 0))
        return gather_rows(y, self.layer.out_features, self.group).reshape(*x.shape[:-1], self.layer.out_features)


class ExpertParallelMoE:
    """Expert-parallel MoE: ``moe`` is an ``ops.VQMoE`` built with ``expert_range=split_range(E, world, rank)``."""

    def __init__(self, moe, group=None):
        self.moe, self.group = moe, group

    def forward(self, x: torch.Tensor, top_k_index: torch.Tensor, top_k_weights: torch.Tensor) -> torch.Tensor:
        y = self.moe.forward(x, top_k_index, top_k_weights)
        if y.dtype == torch.float32:
            dist.all_reduce(y, group=self.group)
            return y
        y32 = y.float()
        dist.all_reduce(y32, group=self.group)
        return y32.to(y.dtype)

    def forward_routed(self, x: torch.Tensor, top_k: int = 10) -> torch.Tensor:
        idx, wts = self.moe.route(x, top_k)   # router weights are replicated: same routing on every rank
        return self.forward(x, idx, wts)


class HeadShardedKVCache:
    """KV-head split: ``cache`` is an ``ops.VQKVCache`` holding KV heads ``split_range(Hkv, world, rank)`` only."""

    def __init__(self, cache, total_q_heads: int, group=None, total_kv_heads: int = 0):
        self.cache, self.total_q_heads, self.group = cache, total_q_heads, group
        world = dist.get_world_size(group)
        # query heads held by every rank (ragged when the KV heads do not divide evenly)
        kv = total_kv_heads or world * cache.kv_heads
        per_kv = total_q_heads // kv
        self.q_ranges = [(a * per_kv, b * per_kv) for a, b in all_ranges(kv, world)]

    def decode(self, q_local: torch.Tensor, scale: float = -1.0) -> torch.Tensor:
        o = self.cache.decode(q_local, scale)                      # [B, Hq_local, hd]
        width = max(b - a for a, b in self.q_ranges)
        pad = o.new_zeros((o.shape[0], width, o.shape[2]))         # equal-sized pieces: ragged shards are padded
        pad[:, : o.shape[1]] = o
        parts = [torch.empty_like(pad) for _ in self.q_ranges]
        dist.all_gather(parts, pad, group=self.group)
        return torch.cat([p[:, : b - a] for p, (a, b) in zip(parts, self.q_ranges)], dim=1)
