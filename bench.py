#!/usr/bin/env python
"""Benchmark of the split-manifold LUT path on B200.

Headline workload (N=1): the VQ-LUT GEMV the reference quotes its numbers on -- one VQ linear
2560 -> 6912, batch 1, block_dim 8, 256 centroids, 0.38 % CSR outliers, fp32 activations.
One layer is 2.8 MB, far below a launch latency and the L2 size, so a "step" is one pass over a
rotation of P independent layers (distinct device copies, P x 2.8 MB >> 126 MB of L2, i.e. every
byte comes from HBM) evaluated by ONE grouped kernel launch.  `value` is algorithmic bytes per
second over that pass (codes + codebook + x + CSR + y, each counted once per layer).

`e2e` drives the same layers one by one through the reference-facing host-pointer call
ojasx_linear_forward (x from pinned host memory, y back to pinned host memory, inside the timed
region): one synchronous call per layer, issued by --e2e-threads caller threads that take the layers
round-robin (each layer handle has its own stream and staging, so the calls of different threads
overlap on the GPU the way the reference's calls spread over host cores); `e2e.single_caller` is the
same with one caller thread.  `cpu_baseline` times the reference's own CPU library on this box's host cores on a
bounded sample.  With --impl reference the whole line is that CPU measurement.

N > 1: layers are independent objects, so each rank owns its own rotation (weak scaling, no
data-path collective); the extra `moe` block shards the 512 experts expert-parallel and
all-reduces the partial outputs over NCCL.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

K_IN, M_OUT, BLOCK = 2560, 6912, 8
N_DISTINCT = 8          # distinct host weight sets; device copies cycle through them
WORKLOAD = "config1-gate: VQ linear 2560->6912, B=1, block_dim 8, 256 centroids, CSR 0.38%, fp32"


def env_int(name, default):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


class ClockSampler:
    """Polls NVML (read-only) for SM clock and throttle reasons while the timed region runs."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int, period_s: float = 0.004):
        self.index, self.period, self.samples, self.reasons = index, period_s, [], set()
        self.max_mhz, self._stop, self._thr, self.ok = None, threading.Event(), None, False
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.ok = False

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self.ok:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()

    def stop(self):
        if self._thr:
            self._stop.set()
            self._thr.join()
        med = int(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def make_host_layers(n):
    from ojasx_b200 import synth
    return [synth.make_vq_linear(1000 + i, K_IN, M_OUT, block_dim=BLOCK) for i in range(n)]


def measured_peak_hbm():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return 6650.0, "fallback 6.65 TB/s"


# ------------------------------------------------------------------------------------------
def cpu_reference_run(seconds: float, threads: int):
    """Reference CPU library (or the port when it is not built) on a bounded sample; GB/s of algorithmic bytes."""
    from oracle import oracle as O
    ws = make_host_layers(4)
    x = np.random.default_rng(7).standard_normal((len(ws), K_IN)).astype(np.float32)
    alg = ws[0].algorithmic_bytes()
    if O.ref_available():
        ref = O.RefLib()
        hs = [ref.make_linear(w.codebook, w.codes, w.scales, w.bias, w.csr, block_dim=BLOCK) for w in ws]

        def run(i):
            ref.linear_forward_handle(hs[i], x[i], M_OUT, threads)
        kind, cores = "reference", (os.cpu_count() if threads <= 0 else threads)
    else:
        def run(i):
            w = ws[i]
            O.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, x[i], block_dim=BLOCK)
        kind, cores = "port", 1
    for i in range(len(ws)):
        run(i)
    n, t0 = 0, time.perf_counter()
    while time.perf_counter() - t0 < seconds:
        run(n % len(ws))
        n += 1
    dt = time.perf_counter() - t0
    return {"value": round(alg * n / dt / 1e9, 4), "unit": "GB/s", "cores": cores, "kind": kind,
            "us_per_layer": round(dt / n * 1e6, 1),
            "sample": f"{n} forwards of {WORKLOAD} over {len(ws)} seeded layers in {dt:.1f} s, "
                      f"num_threads={'all' if threads <= 0 else threads}"}


def run_reference_arm(args):
    rank = env_int("RANK", 0)
    if rank != 0:
        return
    per_step = max(0.5, min(10.0, 60.0 / max(1, args.steps + args.warmup)))
    for _ in range(args.warmup):
        cpu_reference_run(min(per_step, 0.5), 0)
    vals = [cpu_reference_run(per_step, 0) for _ in range(args.steps)]
    v = float(np.mean([r["value"] for r in vals]))
    cb = dict(vals[-1])
    cb["value"] = round(v, 4)
    line = {"impl": "reference", "metric": "vq_lut_gemv_2560x6912_hbm_gbs", "value": round(v, 4), "unit": "GB/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(per_step * 1e3, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": {"workload": WORKLOAD, "layers": 4, "step": "bounded CPU sample"},
            "cpu_baseline": cb, "e2e": {"value": round(v, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist
    import ojasx_b200
    from ojasx_b200 import ops

    rank, world, local = env_int("RANK", 0), env_int("WORLD_SIZE", 1), env_int("LOCAL_RANK", 0)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    P = args.layers
    host = make_host_layers(N_DISTINCT)
    alg = host[0].algorithmic_bytes()
    code_bytes = host[0].code_bytes()
    layers = [ops.VQLinear.from_weights(host[i % N_DISTINCT]) for i in range(P)]
    group = ops.VQLinearGroup(layers)
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    x = torch.randn(P, K_IN, device=dev, generator=gen)
    y = torch.zeros(P, M_OUT, device=dev)

    for _ in range(args.warmup):
        group.forward(x, y)
    barrier()
    sampler = ClockSampler(local)
    n0 = ojasx_b200.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.start()
    e0.record()
    for _ in range(args.steps):
        group.forward(x, y)
    e1.record()
    barrier()
    clocks = sampler.stop()
    launches = ojasx_b200.launch_count() - n0
    ms = e0.elapsed_time(e1)
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    ms_step = ms / args.steps
    value = world * P * alg / (ms_step * 1e-3) / 1e9

    # spot-check the last pass against the oracle (outside the timed region)
    parity = None
    if rank == 0:
        from oracle import oracle as O
        xs = x[:2].cpu().numpy()
        ok = True
        for i in range(2):
            w = host[i % N_DISTINCT]
            want = O.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, xs[i], block_dim=BLOCK)
            ok &= bool(np.array_equal(y[i].cpu().numpy(), want))
        parity = "bit-exact vs oracle on 2 sampled layers" if ok else "MISMATCH vs oracle"

    # ---- e2e: the reference-facing host-pointer call, layer by layer, pinned host buffers
    L = ojasx_b200.lib()
    xh = torch.randn(P, K_IN).pin_memory()
    yh = torch.zeros(P, M_OUT).pin_memory()
    xp, yp = xh.data_ptr(), yh.data_ptr()
    e2e_layers = min(P, args.e2e_layers)
    handles = [l.handle for l in layers[:e2e_layers]]

    def e2e_slice(first, stride):
        for i in range(first, e2e_layers, stride):
            rc = L.ojasx_linear_forward(handles[i], xp + i * K_IN * 4, yp + i * M_OUT * 4, 1, 0)
            if rc != 0:
                raise RuntimeError(f"ojasx_linear_forward rc={rc}")

    def e2e_pass(threads):
        """Every layer once, each through its own synchronous host-pointer call; `threads` caller threads take
        the layers round-robin (the call releases the GIL; each handle has its own stream and staging)."""
        if threads <= 1:
            return e2e_slice(0, 1)
        import threading
        errs = []

        def run(t):
            try:
                e2e_slice(t, threads)
            except Exception as ex:   # surfaced after the join
                errs.append(ex)
        ts = [threading.Thread(target=run, args=(t,)) for t in range(threads)]
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        if errs:
            raise errs[0]

    def e2e_time(threads):
        for _ in range(min(3, args.warmup)):
            e2e_pass(threads)
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_pass(threads)
        torch.cuda.synchronize()
        tt = torch.tensor([time.perf_counter() - t0], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item())

    if args.e2e_threads <= 0:
        args.e2e_threads = min(4, max(1, (os.cpu_count() or 4) // max(1, world)))
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    dt1 = e2e_time(1)
    n1 = ojasx_b200.launch_count()
    dt = e2e_time(args.e2e_threads) if args.e2e_threads > 1 else dt1
    e2e_launches = (ojasx_b200.launch_count() - n1) if args.e2e_threads > 1 else e2e_layers * e2e_steps
    if args.e2e_threads > 1:
        e2e_launches -= e2e_layers * min(3, args.warmup)   # the warm-up passes of e2e_time
    if rank == 0:   # what the callers got back, against the oracle (not timed)
        from oracle import oracle as O
        ok_e2e = True
        for i in (0, e2e_layers - 1):
            w = host[i % N_DISTINCT]
            want = O.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, xh[i].numpy(), block_dim=BLOCK)
            ok_e2e &= bool(np.array_equal(yh[i].numpy(), want))
        parity += "; host-pointer outputs bit-exact on 2 layers" if ok_e2e else "; host-pointer outputs MISMATCH"
    e2e_value = world * e2e_layers * e2e_steps * alg / dt / 1e9
    e2e = {"value": round(e2e_value, 3), "unit": "GB/s", "h2d_bytes_per_step": e2e_layers * K_IN * 4,
           "d2h_bytes_per_step": e2e_layers * M_OUT * 4, "caller_threads": args.e2e_threads,
           "us_per_layer": round(dt / (e2e_layers * e2e_steps) * 1e6, 2),
           "single_caller": {"value": round(world * e2e_layers * e2e_steps * alg / dt1 / 1e9, 3),
                             "us_per_layer_call": round(dt1 / (e2e_layers * e2e_steps) * 1e6, 2)},
           "layers_per_step": e2e_layers, "steps": e2e_steps,
           "call": "ojasx_linear_forward (host pointers in and out, one synchronous call per layer)"}

    # single hot launch latency (same layer, hot L2), for the record
    x1 = x[0:1].contiguous()
    for _ in range(5):
        layers[0](x1)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(100):
        layers[0](x1)
    e1.record()
    torch.cuda.synchronize()
    single_us = e0.elapsed_time(e1) / 100 * 1e3

    extras = {}
    if args.moe:
        try:
            extras["moe"] = bench_moe(args, dev, rank, world)
        except Exception as ex:  # the headline must still print
            extras["moe"] = {"error": repr(ex)}
    if args.kv and rank == 0:
        try:
            extras["kv"] = bench_kv(args, dev)
        except Exception as ex:
            extras["kv"] = {"error": repr(ex)}

    if args.stack and rank == 0 and world == 1:
        try:
            extras["stack"] = bench_stack(args, dev)
        except Exception as ex:
            extras["stack"] = {"error": repr(ex)}

    if rank == 0:
        peak, which = measured_peak_hbm()
        achieved = P * alg / (ms_step * 1e-3) / 1e9   # per GPU: the launch processes this rank's P layers
        line = {
            "metric": "vq_lut_gemv_2560x6912_hbm_gbs", "value": round(value, 2), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 5), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "layers_per_gpu": P, "step": "one grouped launch over all layers",
                       "cold_cache": f"inputs larger than L2: {P * alg / 1e6:.0f} MB of distinct layers per pass",
                       "distinct_host_weight_sets": N_DISTINCT,
                       "row_walk": "rows" if os.environ.get("OJASX_B200_LINEAR_WALK", "").startswith("r") else "lanes of a warp share a row"},
            "us_per_layer": round(ms_step * 1e3 / P, 4),
            "code_gbs": round(world * P * code_bytes / (ms_step * 1e-3) / 1e9, 2),
            "single_launch_hot_us": round(single_us, 2),
            "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4), "traffic": TRAFFIC_PER_LAYER * P if TRAFFIC_PER_LAYER else None,
                         "peak_source": which, "algorithmic_bytes_per_launch": P * alg},
            "e2e": e2e, "gpu_launches": int(launches), "e2e_gpu_launches": int(e2e_launches),
            "clocks": clocks, "parity": parity,
        }
        if world == 1 and args.cpu_seconds > 0:
            line["cpu_baseline"] = cpu_reference_run(args.cpu_seconds, 0)
            line["cpu_baseline_1thread"] = cpu_reference_run(min(3.0, args.cpu_seconds), 1)
        line.update(extras)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# DRAM bytes (read + write) per 2560->6912 layer of lut_linear_kernel<8> from the ncu capture
# summarised in profiles/; None until a capture exists.
TRAFFIC_PER_LAYER = 4142938   # 613.2 MB per 148-layer launch (profiles/lut_linear_kernel_gemv_2560x6912.md)


def bench_moe(args, dev, rank, world):
    """Config 2: 512 experts, hidden 2560, inter 640, top-10, router included; tokens/s at B = 1, 32, 256.
    N > 1: experts sharded expert-parallel, activations replicated, partial outputs all-reduced."""
    import torch
    import torch.distributed as dist
    from ojasx_b200 import ops, synth
    E = 512
    w = synth.make_vq_moe(77, E, 2560, 640, block_dim=8, outlier_frac=0.0038 if args.moe_csr else 0.0)
    per = E // world
    moe = ops.VQMoE(w, (rank * per, (rank + 1) * per))
    out = {"experts_per_gpu": per, "csr": bool(args.moe_csr)}
    peak, _ = measured_peak_hbm()
    for B in (1, 32, 256):
        x = torch.randn(B, 2560, device=dev, generator=torch.Generator(device=dev).manual_seed(5))
        y = torch.empty_like(x)
        moe.reserve(B, 10)

        def step():
            moe.forward_routed(x, 10, out=y)
            if world > 1:
                dist.all_reduce(y)
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 20 if B < 256 else 5
        e0.record()
        for _ in range(reps):
            step()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / reps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        # algorithmic code bytes: every distinct routed expert's 614,400 code bytes once, plus the router
        idx, _w = moe.route(x, 10)
        distinct = int(torch.unique(idx).numel())
        code_bytes = distinct * w.code_bytes_per_expert() + w.router.nbytes
        out[f"B{B}"] = {"ms_per_layer": round(ms, 4), "tokens_per_s": round(B / ms * 1e3, 1),
                        "distinct_experts": distinct, "code_gbs": round(code_bytes / ms / 1e6, 1),
                        "hbm_frac_of_measured": round(code_bytes / ms / 1e6 / peak / world, 4)}
    if rank == 0 and world == 1 and args.cpu_seconds > 0:
        # the reference's own CPU MoE (single token, single thread by construction, no outliers) beside it
        try:
            from oracle import oracle as O
            if O.ref_available():
                ref = O.RefLib()
                h = ref.make_moe(w.codebook, w.down_codebook, w.gate_up_codes, w.gate_up_scales, w.down_codes,
                                 w.down_scales, block_dim=8)
                xi = np.random.default_rng(1).standard_normal(2560).astype(np.float32)
                ii = np.arange(0, 500, 50, dtype=np.int32)
                wi = np.full(10, 0.1, np.float32)
                ref.moe_forward_handle(h, xi, ii, wi, 2560)
                n, t0 = 0, time.perf_counter()
                while time.perf_counter() - t0 < min(3.0, args.cpu_seconds):
                    ref.moe_forward_handle(h, xi, ii, wi, 2560)
                    n += 1
                us = (time.perf_counter() - t0) / n * 1e6
                out["cpu_reference"] = {"us_per_token": round(us, 1), "tokens_per_s": round(1e6 / us, 1), "cores": 1,
                                        "kind": "reference", "sample": f"{n} calls of ojasx_moe_forward, top-10 of 512, no outliers"}
        except Exception as ex:
            out["cpu_reference"] = {"error": repr(ex)}
    return out


def bench_stack(args, dev):
    """Config 4: 24-layer decoder stack (hidden 2560, 32/8 heads of 128, RoPE 1e6, RMSNorm, 512-expert top-10
    MoE per layer, VQ lm_head over 151936 tokens, quantised KV), 512 random prompt ids then 256 greedy steps.
    One host weight set, 24 distinct device copies (every layer streams its own HBM bytes)."""
    import torch
    from ojasx_b200 import inference_engine as ie
    out = {}
    cfg = ie.StackConfig(max_seq_len=args.stack_prompt + args.stack_new + 8)
    t0 = time.perf_counter()
    W = ie.make_stack_weights(2024, cfg)
    out["host_weight_seconds"] = round(time.perf_counter() - t0, 1)
    for B in args.stack_batches:
        stack = ie.VQDecoderStack(W, cfg, batch=B, use_graph=not args.stack_eager,
                                  dtype=torch.bfloat16 if args.stack_dtype == "bf16" else torch.float32)
        ids = torch.randint(0, cfg.vocab, (B, args.stack_prompt), device=dev, generator=torch.Generator(device=dev).manual_seed(3))
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        logits = stack.prefill(ids)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        for _ in range(args.stack_new):
            logits = stack.decode_step(torch.argmax(logits, dim=-1))
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        out[f"B{B}"] = {"prefill_tokens_per_s": round(B * args.stack_prompt / (t1 - t0), 1),
                        "decode_tokens_per_s": round(B * args.stack_new / (t2 - t1), 1),
                        "ms_per_decode_step": round((t2 - t1) / args.stack_new * 1e3, 3),
                        "prompt": args.stack_prompt, "new_tokens": args.stack_new, "dtype": args.stack_dtype}
        del stack
        torch.cuda.empty_cache()
    return out


def bench_kv(args, dev):
    """Config 3: append one token + one decode query, 32 q heads / 8 kv heads, head_dim 128, bf16 q."""
    import torch
    from ojasx_b200 import ops, synth
    out = {}
    for B, ctx in ((1, 2048), (1, 32768), (16, 32768)):
        kv = synth.make_vq_kv(3, 1, 8)
        cache = ops.VQKVCache(B, 8, 32, 128, 8, ctx + 64, kv.k_codebook, kv.v_codebook)
        rng = np.random.default_rng(9)
        codes = rng.integers(0, 256, size=(B, 8, ctx, 16), dtype=np.uint8)
        cache.load(codes, codes[:, :, ::-1].copy())
        q = torch.randn(B, 32, 128, device=dev).to(torch.bfloat16)
        nk = (torch.randn(B, 8, 128, device=dev) / 11.3).to(torch.bfloat16)
        o = torch.empty_like(q)
        for _ in range(3):
            cache.decode(q, out=o)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 20
        e0.record()
        for _ in range(reps):
            cache.append(nk, nk)
            cache.decode(q, out=o)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        bytes_ = B * ctx * 256
        out[f"B{B}_ctx{ctx}"] = {"us_append_plus_decode": round(ms * 1e3, 2), "code_gbs": round(bytes_ / ms / 1e6, 1),
                                 "hbm_frac_of_measured": round(bytes_ / ms / 1e6 / measured_peak_hbm()[0], 4)}
        cache.close()
    if args.cpu_seconds > 0:
        # CPU restatement (fp64 port; the reference has no codebook-VQ cache) on one KV head of ctx 2048, scaled to 8 heads
        from oracle import oracle as O
        kv = synth.make_vq_kv(3, 1, 2048)
        t0 = time.perf_counter()
        O.kvq_decode(kv.q[0, :4], kv.k_codes[0, 0], kv.v_codes[0, 0], kv.k_codebook[0], kv.v_codebook[0], block_dim=8)
        out["cpu_port_B1_ctx2048"] = {"us": round((time.perf_counter() - t0) * 8e6, 1), "cores": 1, "kind": "port",
                                      "sample": "one KV head (4 query heads) x 8"}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--layers", type=int, default=1480, help="independent layers per GPU per step (10 per SM)")
    ap.add_argument("--e2e-layers", type=int, default=148)
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--e2e-threads", type=int, default=0,
                    help="host threads that issue the synchronous per-layer calls of the e2e leg (0 = up to 4, as many as the "
                         "host cores allow each rank, since every caller polls for completion)")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--no-moe", dest="moe", action="store_false")
    ap.add_argument("--no-moe-csr", dest="moe_csr", action="store_false")
    ap.add_argument("--no-kv", dest="kv", action="store_false")
    ap.add_argument("--stack", action="store_true", help="also time the 24-layer decoder stack (adds about a minute)")
    ap.add_argument("--stack-eager", action="store_true", help="launch the decode step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--stack-prompt", type=int, default=512)
    ap.add_argument("--stack-new", type=int, default=256)
    ap.add_argument("--stack-batches", type=int, nargs="+", default=[1, 32])
    ap.add_argument("--stack-dtype", default="f32", choices=["f32", "bf16"],
                    help="activation dtype of the stack; bf16 batches >= 32 take the tensor-core linears")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
