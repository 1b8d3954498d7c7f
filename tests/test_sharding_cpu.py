"""World-size-2 gloo tests (CPU ranks) of the multi-GPU plumbing: partition arithmetic, ragged row
all-gather, expert-parallel reduction and KV-head gather.  The compute on each rank is the CPU oracle
standing in for the shard's kernels, so what is tested is exactly the host-side sharding logic."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ojasx_b200 import sharding, synth


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ret[rank] = fn(rank, world)
    finally:
        dist.destroy_process_group()


def _run(fn, world=2):
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), fn, ret), nprocs=world, join=True)
    return [ret[r] for r in range(world)]


def test_split_range_covers_everything():
    for total, world, mult in ((6912, 8, 32), (2560, 8, 32), (151936, 8, 32), (512, 8, 1), (8, 8, 1), (5, 8, 1), (70, 4, 32)):
        rs = sharding.all_ranges(total, world, mult)
        assert rs[0][0] == 0 and rs[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(rs, rs[1:]))
        assert all((hi - lo) % mult == 0 for lo, hi in rs[:-1] if hi < total)


def _rows_job(rank, world):
    from oracle import oracle as O
    w = synth.make_vq_linear(3, 256, 200, block_dim=8, with_scales=True, with_bias=True)
    x = np.random.default_rng(1).standard_normal((3, 256)).astype(np.float32)
    a, b = sharding.split_range(200, world, rank, 32)
    y = O.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, x, block_dim=8, row_start=a, row_stop=b)
    full = sharding.gather_rows(torch.from_numpy(y), 200)
    want = O.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, x, block_dim=8)
    return bool(np.array_equal(full.numpy(), want))


def test_row_split_linear_all_gather():
    assert _run(_rows_job) == [True, True]


class _OracleMoEShard:
    """Stands in for ops.VQMoE(w, expert_range): routed ids outside the shard contribute nothing."""

    def __init__(self, w, e0, e1):
        self.w, self.e0, self.e1 = w, e0, e1

    def forward(self, x, idx, wts):
        from oracle import oracle as O
        w = self.w
        out = []
        for t in range(x.shape[0]):
            local = idx[t].numpy().astype(np.int32) - self.e0
            out.append(O.moe_forward(w.codebook, w.down_codebook, w.gate_up_codes[self.e0:self.e1],
                                     w.gate_up_scales[self.e0:self.e1], w.down_codes[self.e0:self.e1],
                                     w.down_scales[self.e0:self.e1], x[t].numpy(), local, wts[t].numpy(), block_dim=8))
        return torch.from_numpy(np.stack(out))


def _ep_job(rank, world):
    from oracle import oracle as O
    w = synth.make_vq_moe(5, 8, 128, 32, block_dim=8, outlier_frac=0.0, unit_scales=False)
    rng = np.random.default_rng(2)
    x = torch.from_numpy(rng.standard_normal((4, 128)).astype(np.float32))
    idx = torch.from_numpy(np.stack([rng.choice(8, 3, replace=False) for _ in range(4)]).astype(np.int32))
    wts = torch.from_numpy(rng.uniform(0.1, 0.5, (4, 3)).astype(np.float32))
    e0, e1 = sharding.split_range(8, world, rank)
    y = sharding.ExpertParallelMoE(_OracleMoEShard(w, e0, e1)).forward(x, idx, wts)
    want = np.stack([O.moe_forward(w.codebook, w.down_codebook, w.gate_up_codes, w.gate_up_scales, w.down_codes,
                                   w.down_scales, x[t].numpy(), idx[t].numpy(), wts[t].numpy(), block_dim=8)
                     for t in range(4)])
    return bool(np.allclose(y.numpy(), want, rtol=1e-5, atol=1e-6))


def test_expert_parallel_all_reduce():
    assert _run(_ep_job) == [True, True]


class _OracleKVShard:
    def __init__(self, kv, h0, h1):
        self.kv, self.h0, self.h1 = kv, h0, h1

    def decode(self, q_local, scale=-1.0):
        from oracle import oracle as O
        kv, R = self.kv, self.kv.q_heads // self.kv.kv_heads
        B = q_local.shape[0]
        out = np.zeros((B, (self.h1 - self.h0) * R, kv.head_dim), np.float32)
        for b in range(B):
            for i, h in enumerate(range(self.h0, self.h1)):
                out[b, i * R:(i + 1) * R] = O.kvq_decode(q_local[b, i * R:(i + 1) * R].numpy(), kv.k_codes[b, h],
                                                        kv.v_codes[b, h], kv.k_codebook[h], kv.v_codebook[h], block_dim=8)
        return torch.from_numpy(out)


def _kv_job(rank, world, heads=4):
    R = 2
    kv = synth.make_vq_kv(7, 2, 40, kv_heads=heads, q_heads=heads * R, head_dim=32)
    h0, h1 = sharding.split_range(heads, world, rank)
    q = torch.from_numpy(kv.q)
    full = sharding.HeadShardedKVCache(_OracleKVShard(kv, h0, h1), heads * R, total_kv_heads=heads).decode(q[:, h0 * R:h1 * R])
    want = _OracleKVShard(kv, 0, heads).decode(q)
    return bool(np.array_equal(full.numpy(), want.numpy()))


def _kv_job_ragged(rank, world):
    return _kv_job(rank, world, heads=3)     # 2 + 1 heads: the shards' outputs differ in size


def test_kv_head_shards_all_gather():
    assert _run(_kv_job) == [True, True]


def test_kv_head_shards_ragged():
    assert _run(_kv_job_ragged) == [True, True]
