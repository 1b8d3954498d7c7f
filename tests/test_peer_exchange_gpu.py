"""Two GPU ranks of one box: the sharded operators with the exchange fused into the producing kernel (stores into
every rank's shared segment plus a flag, sharding.PeerSegment) against the unsharded operator on the same device.
Skipped where fewer than two GPUs are visible; the partition arithmetic itself is covered on CPU ranks in
tests/test_sharding_cpu.py."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from ojasx_b200 import ops, sharding, synth
        seg = sharding.PeerSegment(64 << 20)
        out = {}
        # ---- row-split linear + gather, twice in a row (alternating buffers), fp32 and a batch
        w = synth.make_vq_linear(3, 2560, 6912, block_dim=8)
        full = ops.VQLinear.from_weights(w)
        sh = sharding.ShardedVQLinear(full, segment=seg, max_batch=3)
        x = torch.randn(3, 2560, device=dev, generator=torch.Generator(device=dev).manual_seed(1))
        want = full(x)
        out["linear"] = all(torch.equal(sh.forward(x * s), full(x * s)) for s in (1.0, 0.5, 2.0))
        out["linear_b1"] = bool(torch.equal(sh.forward(x[:1]), want[:1]))
        # ---- expert-parallel MoE: outputs of all ranks' experts gathered per pair, combined in caller order
        mw = synth.make_vq_moe(5, 16, 512, 256, block_dim=8, outlier_frac=0.01)
        whole = ops.VQMoE(mw)
        e0, e1 = sharding.split_range(16, world, rank)
        ep = sharding.ExpertParallelMoE(ops.VQMoE(mw, (e0, e1)), segment=seg, max_tokens=40, top_k=4)
        xm = torch.randn(40, 512, device=dev, generator=torch.Generator(device=dev).manual_seed(2))
        idx, wts = whole.route(xm, 4)
        want_m = whole.forward(xm, idx, wts)
        out["moe"] = bool(torch.equal(ep.forward(xm, idx, wts), want_m)) and bool(torch.equal(ep.forward_routed(xm, 4), want_m))
        ep.shard_router_min_tokens = 1       # every rank scores its own experts only; the logits are exchanged as well
        out["moe"] = out["moe"] and bool(torch.equal(ep.forward_routed(xm, 4), want_m))
        ep.shard_router_min_tokens = 64
        out["moe_b1"] = bool(torch.equal(ep.forward_routed(xm[:1], 4), whole.forward_routed(xm[:1], 4)))
        os.environ["OJASX_B200_MOE_FUSED_MIN_PAIRS"] = "1"      # the whole-expert kernel takes the same route
        out["moe_fused"] = bool(torch.equal(ep.forward(xm, idx, wts), whole.forward(xm, idx, wts)))
        os.environ.pop("OJASX_B200_MOE_FUSED_MIN_PAIRS")
        # ---- KV cache split by KV head
        kv = synth.make_vq_kv(7, 2, 3000)
        allc = ops.VQKVCache(2, 8, 32, 128, 8, 3008, kv.k_codebook, kv.v_codebook)
        allc.load(kv.k_codes, kv.v_codes)
        h0, h1 = sharding.split_range(8, world, rank)
        mine = ops.VQKVCache(2, h1 - h0, 4 * (h1 - h0), 128, 8, 3008, kv.k_codebook[h0:h1], kv.v_codebook[h0:h1])
        mine.load(kv.k_codes[:, h0:h1], kv.v_codes[:, h0:h1])
        q = torch.from_numpy(kv.q).to(dev)
        hs = sharding.HeadShardedKVCache(mine, 32, total_kv_heads=8, segment=seg)
        # (a shard plans its context splits for its own head count, so the partial sums are merged in another
        # order than in the unsharded cache: same values within fp32 rounding, not the same bits)
        out["kv"] = bool(torch.allclose(hs.decode(q[:, 4 * h0:4 * h1].contiguous()), allc.decode(q), rtol=1e-5, atol=1e-7))
        out["status"] = seg.take_status()
        torch.cuda.synchronize()
        seg.close()
        ret[rank] = out
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_exchange_matches_unsharded_operators():
    world = 2
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    for r in range(world):
        assert ret[r] == {"linear": True, "linear_b1": True, "moe": True, "moe_b1": True, "moe_fused": True, "kv": True,
                          "status": 0}, (r, ret[r])


def _stack_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from ojasx_b200 import inference_engine as ie
        from ojasx_b200 import sharding
        cfg = ie.StackConfig(layers=2, hidden=256, q_heads=8, kv_heads=4, head_dim=32, experts=8, top_k=2, inter=128, vocab=1000,
                             max_seq_len=24, distinct_layers=2, outlier_frac=0.01)
        W = ie.make_stack_weights(11, cfg)
        seg = sharding.PeerSegment(32 << 20)
        whole = ie.VQDecoderStack(W, cfg, batch=2)                       # the unsharded stack on this device
        ids = torch.randint(0, cfg.vocab, (2, 5), device=dev, generator=torch.Generator(device=dev).manual_seed(4))
        want = whole.generate(ids, 6)
        out = {}
        for graph in (False, True):
            part = ie.VQDecoderStack(W, cfg, batch=2, segment=seg, use_graph=graph)
            got = part.generate(ids, 6)
            out[f"tokens_graph{int(graph)}"] = bool(torch.equal(got, want))
            part.reset()
            whole.reset()
            la, lb = part.decode_step(ids[:, 0]), whole.decode_step(ids[:, 0])
            out[f"logits_graph{int(graph)}"] = bool(torch.allclose(la, lb, rtol=1e-4, atol=1e-5))
            del part
        out["status"] = seg.take_status()
        torch.cuda.synchronize()
        seg.close()
        ret[rank] = out
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_decoder_stack_matches_one_device():
    """KV heads, o_proj rows, experts and the vocabulary split over two ranks: same greedy tokens as one device (the
    expert outputs are combined in caller order on every rank, the arg-max runs over the ranks' vocabulary shards)."""
    world = 2
    ret = mp.Manager().dict()
    mp.spawn(_stack_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    for r in range(world):
        assert ret[r] == {"tokens_graph0": True, "logits_graph0": True, "tokens_graph1": True, "logits_graph1": True,
                          "status": 0}, (r, ret[r])
