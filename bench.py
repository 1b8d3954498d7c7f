#!/usr/bin/env python
"""Benchmark of the split-manifold LUT path on B200.

Headline workload: the VQ-LUT GEMV the reference quotes its numbers on -- one VQ linear 2560 -> 6912, batch 1,
block_dim 8, 256 centroids, 0.38 % CSR outliers, fp32 activations.  One layer is 2.8 MB, far below a launch
latency and the L2 size, so a "step" is one pass over a rotation of P independent layers (distinct device
copies, P x 2.8 MB >> 126 MB of L2, i.e. every byte comes from HBM) evaluated by ONE grouped kernel launch.
`value` is algorithmic bytes per second over that pass (codes + codebook + x + CSR + y, each counted once per
layer).

N = 1: every layer whole on the one GPU.  N > 1 (one process per GPU under torchrun): the SAME P layers, each
split by output rows over the N ranks (the row_start / row_stop contract); a rank's kernel stores its rows of
every layer into the gathered output of every rank over NVLink from its epilogue and raises a flag, and the
step ends when every rank has seen every flag.  Total work is fixed, so this is strong scaling; what does not
shrink with N is the lookup table of a layer, which every rank builds for its rows.

`e2e` drives the same layers one by one through the reference-facing host-pointer call ojasx_linear_forward
(x from pinned host memory, y back to pinned host memory, inside the timed region).  `cpu_baseline` times the
reference's own CPU library on this box's host cores on a bounded sample; with --impl reference the whole line
is that CPU measurement.

Further blocks of the same line, one per benchmark configuration: `mlp_sweep` (configuration 1: SwiGLU block of
three VQ linears, bf16, batch 1..256, table kernels against the tensor-core path), `moe` (configuration 2,
expert-parallel at N > 1), `kv` (configuration 3, split by KV head at N > 1), `stack` (configuration 4, all of it
split at N > 1), `row_split` (single 2560 -> 6912 and 6912 -> 2560 layers split by rows, N > 1).  Each entry
carries a `roofline` object and, where a CPU twin exists, the CPU time beside it.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
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
METRIC = "vq_lut_gemv_2560x6912_hbm_gbs"

# DRAM bytes (read + write) of one 2560->6912 layer inside lut_linear_kernel<8>, from an ncu capture of a
# 148-layer launch of this kernel (dram__bytes_read.sum + dram__bytes_write.sum over the launch / 148); every
# layer of a launch does the same work, so a launch's traffic is this figure times its layer count.
TRAFFIC_PER_LAYER = 4074776
TRAFFIC_SOURCE = ("ncu capture of lut_linear_kernel<8> as benched (outlier entries streamed by the copy engine in the epilogue), "
                  "148 layers per launch: 602,837,760 B read + 229,120 B written; profiles/lut_linear_kernel_gemv_2560x6912.md")


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


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = {"hbm": 6650.0, "tf": 1590.0, "tf_sustained": 1400.0, "src": "fallback 6.65 TB/s / 1.59 PFLOP/s"}
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            out = {"hbm": float(d["hbm_gbs"]), "tf": float(d["bf16_tflops"]), "tf_sustained": float(d["bf16_tflops_sustained"]),
                   "src": "measured (MEASURED_PEAKS.json)"}
        except Exception:
            pass
    return out


def hbm_roofline(alg_bytes: float, seconds: float, n_gpus: int = 1, traffic=None, note=None):
    pk = peaks()
    achieved = alg_bytes / seconds / 1e9 / max(1, n_gpus)
    r = {"bound": "hbm", "achieved": round(achieved, 2), "peak": pk["hbm"], "unit": "GB/s", "frac": round(achieved / pk["hbm"], 4),
         "traffic": traffic, "algorithmic_bytes": int(alg_bytes), "peak_source": pk["src"]}
    if n_gpus > 1:
        r["per_gpu_of"] = n_gpus
    if note:
        r["note"] = note
    return r


# ------------------------------------------------------------------------------------------ CPU reference legs
def cpu_reference_run(seconds: float, threads: int, lib_path=None):
    """Reference CPU library (or the port when it is not built) on a bounded sample; GB/s of algorithmic bytes."""
    from oracle import oracle as O
    ws = make_host_layers(4)
    x = np.random.default_rng(7).standard_normal((len(ws), K_IN)).astype(np.float32)
    alg = ws[0].algorithmic_bytes()
    extra = {}
    if O.ref_available() or lib_path:
        ref = O.RefLib(lib_path) if lib_path else O.RefLib()
        hs = [ref.make_linear(w.codebook, w.codes, w.scales, w.bias, w.csr, block_dim=BLOCK) for w in ws]

        def run(i):
            ref.linear_forward_handle(hs[i], x[i], M_OUT, threads)
        kind, cores = "reference", (os.cpu_count() if threads <= 0 else threads)
        extra = {"backend": ref.backend(), "library": os.path.basename(ref.path)}
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
    out = {"value": round(alg * n / dt / 1e9, 4), "unit": "GB/s", "cores": cores, "kind": kind,
           "us_per_layer": round(dt / n * 1e6, 1),
           "sample": f"{n} forwards of {WORKLOAD} over {len(ws)} seeded layers in {dt:.1f} s, "
                     f"num_threads={'all' if threads <= 0 else threads}"}
    out.update(extra)
    return out


def cpu_native_build_run(seconds: float):
    """The reference library compiled with -march=native (oracle/_ref/libojasx_lut_native.so), timed in a child
    process: it was built for the CPU of the build machine and may use instructions this host lacks."""
    path = os.path.join(ROOT, "oracle", "_ref", "libojasx_lut_native.so")
    flags = "g++ -O3 -std=c++20 -fPIC -march=native (FMA contraction on; table values differ from the default build in the last bit)"
    if not os.path.exists(path):
        return {"unavailable": "oracle/_ref/libojasx_lut_native.so is not built", "flags": flags}
    code = ("import json,sys; sys.path.insert(0, %r); import bench; "
            "print(json.dumps(bench.cpu_reference_run(%f, 0, %r)))" % (ROOT, seconds, path))
    try:
        r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=seconds * 4 + 60)
        if r.returncode != 0:
            return {"unavailable": f"child exited with {r.returncode} (built for another CPU?)", "flags": flags}
        out = json.loads(r.stdout.strip().splitlines()[-1])
        out["flags"] = flags
        return out
    except Exception as ex:
        return {"unavailable": repr(ex), "flags": flags}


def headline_config(P, step):
    return {"workload": WORKLOAD, "layers": P, "step": step}


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
    cb["flags"] = "g++ -O3 -std=c++20 -fPIC (the reference Makefile's defaults, no -march)"
    line = {"impl": "reference", "metric": METRIC, "value": round(v, 4), "unit": "GB/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(per_step * 1e3, 3), "higher_is_better": True,
            "scaling": "weak" if args.gpus == 1 else "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": headline_config(args.layers, "one pass over all layers"),
            "cpu_baseline": cb, "e2e": {"value": round(v, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0, "sample": "each step is a bounded CPU sample of the workload: " + cb["sample"]}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------ our arm
class Env:
    """Rank bookkeeping, timing helpers and (N > 1) the shared segment of this rank."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.args = torch, dist, args
        self.rank, self.world, self.local = env_int("RANK", 0), env_int("WORLD_SIZE", 1), env_int("LOCAL_RANK", 0)
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.seg = None
        if self.world > 1:
            os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
            dist.init_process_group("nccl", device_id=self.dev)
            from ojasx_b200 import sharding
            self.seg = sharding.PeerSegment(args.segment_mb << 20)

    def barrier(self, solo: bool = False):
        """`solo`: a section that only one rank runs must not enter a collective."""
        if self.world > 1 and not solo:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, v: float) -> float:
        if self.world == 1:
            return float(v)
        t = self.torch.tensor([v], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def time_ms(self, fn, reps: int, warmup: int = 3, solo: bool = False) -> float:
        """CUDA-event time of `reps` calls on the current stream, barrier + synchronize on both sides, max over ranks
        (`solo`: this rank alone runs the section: no collective, its own time)."""
        torch = self.torch
        for _ in range(warmup):
            fn()
        self.barrier(solo)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        self.barrier(solo)
        ms = e0.elapsed_time(e1)
        return (ms if solo else self.max_over_ranks(ms)) / reps

    def graph_of(self, fn, solo: bool = False):
        """`fn` recorded once into a CUDA graph (after an eager warm-up on a side stream); returns the replay callable."""
        torch = self.torch
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        self.barrier(solo)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        return g.replay

    def close(self):
        if self.seg is not None:
            self.seg.close()
        if self.world > 1:
            self.dist.destroy_process_group()


def run_ours(args):
    import torch
    import ojasx_b200
    from ojasx_b200 import ops, sharding
    E = Env(args)
    rank, world, dev = E.rank, E.world, E.dev
    pk = peaks()

    P = args.layers
    host = make_host_layers(N_DISTINCT)
    alg = host[0].algorithmic_bytes()
    code_bytes = host[0].code_bytes()
    layers = [ops.VQLinear.from_weights(host[i % N_DISTINCT]) for i in range(P)]
    group = ops.VQLinearGroup(layers)
    gen = torch.Generator(device=dev).manual_seed(1234)      # the same activations on every rank: x is replicated
    x = torch.randn(P, K_IN, device=dev, generator=gen)
    if world == 1:
        ys = [torch.zeros(P, M_OUT, device=dev)]

        def step(i=[0]):
            group.forward(x, ys[0])
        step_desc = "one grouped launch over all layers"
    else:
        r0, r1 = sharding.split_range(M_OUT, world, rank, 32)
        group.set_rows(r0, r1)
        ys = [E.seg.alloc((P, M_OUT), torch.float32) for _ in range(2)]     # gathered outputs, used in turn
        turn = [0]

        def step():
            group.forward_gather(x, ys[turn[0]], E.seg.link)
            E.seg.wait()
            turn[0] ^= 1
        step_desc = (f"one grouped launch per rank over rows [{r0},{r1}) of all layers, rows stored into every rank's "
                     f"gathered output from the kernel epilogue, then a wait for all ranks' flags")

    for _ in range(args.warmup):
        step()
    sampler = ClockSampler(E.local)
    sampler.start()          # before the barrier: a rank that is late into the timed loop holds every other rank up
    n0 = ojasx_b200.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    E.barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    E.barrier()
    clocks = sampler.stop()
    launches = ojasx_b200.launch_count() - n0
    my_ms = e0.elapsed_time(e1)
    ms_step = E.max_over_ranks(my_ms) / args.steps
    if world > 1:
        # every rank sampled its own GPU: the line carries the slowest median clock and every reason seen on any of them
        # (a run in which ANY GPU of the job was slowed down is to be read as such)
        clocks["min_sm_mhz_over_ranks"] = int(-E.max_over_ranks(-float(clocks["sm_mhz"] or 0)))
        for name in ClockSampler.REASONS.values():
            if E.max_over_ranks(1.0 if name in clocks["reasons"] else 0.0) > 0 and name not in clocks["reasons"]:
                clocks["reasons"].append(name)
        clocks["reasons"] = sorted(clocks["reasons"])
        clocks["ms_per_step_fastest_rank"] = round(-E.max_over_ranks(-my_ms) / args.steps, 5)
    value = P * alg / (ms_step * 1e-3) / 1e9          # whole job: the P layers, whoever computed them

    # spot-check the last pass against the oracle (outside the timed region): full rows on every rank
    parity = None
    if rank == 0:
        from oracle import oracle as O
        xs = x[:2].cpu().numpy()
        last = ys[0] if world == 1 else ys[turn[0] ^ 1]
        ok = True
        for i in range(2):
            w = host[i % N_DISTINCT]
            want = O.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, xs[i], block_dim=BLOCK)
            ok &= bool(np.array_equal(last[i].cpu().numpy(), want))
        parity = ("bit-exact vs oracle on 2 sampled layers" + (" (rows of all ranks, gathered)" if world > 1 else "")) if ok \
            else "MISMATCH vs oracle"

    # ---- e2e: the reference-facing host-pointer call, layer by layer, pinned host buffers (whole layers per call;
    # at N > 1 every rank drives its own share of the layers)
    L = ojasx_b200.lib()
    xh = torch.randn(P, K_IN).pin_memory()
    yh = torch.zeros(P, M_OUT).pin_memory()
    xp, yp = xh.data_ptr(), yh.data_ptr()
    e2e_layers = min(P, args.e2e_layers)
    handles = [l.handle for l in layers[:e2e_layers]]
    mine = list(range(rank, e2e_layers, world))

    def e2e_slice(first, stride):
        for i in mine[first::stride]:
            rc = L.ojasx_linear_forward(handles[i], xp + i * K_IN * 4, yp + i * M_OUT * 4, 1, 0)
            if rc != 0:
                raise RuntimeError(f"ojasx_linear_forward rc={rc}")

    def e2e_pass(threads):
        if threads <= 1:
            return e2e_slice(0, 1)
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
        E.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_pass(threads)
        torch.cuda.synchronize()
        return E.max_over_ranks(time.perf_counter() - t0)

    if args.e2e_threads <= 0:
        args.e2e_threads = min(4, max(1, (os.cpu_count() or 4) // max(1, world)))
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    dt1 = e2e_time(1)
    n1 = ojasx_b200.launch_count()
    dt = e2e_time(args.e2e_threads) if args.e2e_threads > 1 else dt1
    e2e_launches = (ojasx_b200.launch_count() - n1) if args.e2e_threads > 1 else len(mine) * e2e_steps
    if args.e2e_threads > 1:
        e2e_launches -= len(mine) * min(3, args.warmup)
    if rank == 0:
        from oracle import oracle as O
        ok_e2e = True
        for i in (mine[0], mine[-1]):
            w = host[i % N_DISTINCT]
            want = O.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, xh[i].numpy(), block_dim=BLOCK)
            ok_e2e &= bool(np.array_equal(yh[i].numpy(), want))
        parity += "; host-pointer outputs bit-exact on 2 layers" if ok_e2e else "; host-pointer outputs MISMATCH"
    e2e_value = e2e_layers * e2e_steps * alg / dt / 1e9
    e2e = {"value": round(e2e_value, 3), "unit": "GB/s", "h2d_bytes_per_step": e2e_layers * K_IN * 4,
           "d2h_bytes_per_step": e2e_layers * M_OUT * 4, "caller_threads": args.e2e_threads,
           "us_per_layer": round(dt / (e2e_layers * e2e_steps) * 1e6, 2),
           "single_caller": {"value": round(e2e_layers * e2e_steps * alg / dt1 / 1e9, 3),
                             "us_per_layer_call": round(dt1 / (len(mine) * e2e_steps) * 1e6, 2)},
           "layers_per_step": e2e_layers, "steps": e2e_steps,
           "call": "ojasx_linear_forward (host pointers in and out, one synchronous call per layer)"
                   + ("" if world == 1 else f"; the layers are shared out over the {world} ranks")}

    # single hot launch latency (same layer, hot L2), for the record
    x1 = x[0:1].contiguous()
    single_us = E.time_ms(lambda: layers[0](x1), 100, 5) * 1e3

    extras = {}
    broken = False
    del group, ys
    for name, fn in (("mlp_sweep", bench_mlp_sweep), ("row_split", bench_row_split), ("moe", bench_moe), ("kv", bench_kv),
                     ("stack", bench_stack)):
        if not getattr(args, name):
            continue
        if name == "row_split" and world == 1:
            continue
        try:
            t0 = time.perf_counter()
            extras[name] = fn(args, E)
            if isinstance(extras[name], dict):
                extras[name]["bench_seconds"] = round(time.perf_counter() - t0, 1)
        except Exception as ex:  # the headline must still print
            import traceback
            extras[name] = {"error": repr(ex), "trace": traceback.format_exc()[-600:]}
        torch.cuda.empty_cache()
        E.barrier()     # rank-0-only sections end here for everybody
        if E.seg is not None:
            bad = E.max_over_ranks(float(E.seg.take_status()))
            if bad:     # a wait for a peer's flag ran out: the ranks are out of step, nothing after this would be valid
                extras[name] = {"error": "a bounded wait for another rank's flag ran out in this section", "partial": extras.get(name)}
                broken = True
                break

    status = 1 if broken else (E.seg.take_status() if E.seg is not None else 0)
    dev_err = ojasx_b200.lib().ojasx_b200_take_device_error()
    if rank == 0:
        achieved = value / world       # per GPU
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 5), "higher_is_better": True,
            "scaling": "weak" if world == 1 else "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": headline_config(P, "one pass over all layers"),
            "execution": {"step": step_desc,
                          "cold_cache": f"inputs larger than L2: {P * alg / 1e6:.0f} MB of distinct layers per pass",
                          "distinct_host_weight_sets": N_DISTINCT,
                          "row_walk": "rows" if os.environ.get("OJASX_B200_LINEAR_WALK", "").startswith("r") else "lanes of a warp share a row"},
            "us_per_layer": round(ms_step * 1e3 / P, 4),
            "code_gbs": round(P * code_bytes / (ms_step * 1e-3) / 1e9, 2),
            "single_launch_hot_us": round(single_us, 2),
            "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": pk["hbm"], "unit": "GB/s",
                         "frac": round(achieved / pk["hbm"], 4),
                         "code_bytes_frac": round(P * code_bytes / (ms_step * 1e-3) / 1e9 / world / pk["hbm"], 4),
                         "traffic": TRAFFIC_PER_LAYER * P if (TRAFFIC_PER_LAYER and world == 1) else None,
                         "traffic_source": TRAFFIC_SOURCE if world == 1 else None,
                         "peak_source": pk["src"], "algorithmic_bytes_per_launch": P * alg,
                         "note": None if world == 1 else "per GPU: the job's algorithmic bytes / N; every rank also rebuilds each layer's table"},
            "e2e": e2e, "gpu_launches": int(launches), "e2e_gpu_launches": int(e2e_launches),
            "clocks": clocks, "parity": parity, "peer_wait_timeouts": int(status), "device_error_flags": int(dev_err),
        }
        if world == 1 and args.cpu_seconds > 0:
            cb = cpu_reference_run(args.cpu_seconds, 0)
            cb["flags"] = "g++ -O3 -std=c++20 -fPIC (the reference Makefile's defaults, no -march)"
            line["cpu_baseline"] = cb
            line["cpu_baseline_1thread"] = cpu_reference_run(min(3.0, args.cpu_seconds), 1)
            line["cpu_baseline_native_build"] = cpu_native_build_run(min(4.0, args.cpu_seconds))
        line.update(extras)
        print(json.dumps(line), flush=True)
    E.close()


# ------------------------------------------------------------------------------------------ configuration 1
def bench_mlp_sweep(args, E):
    """Configuration 1: SwiGLU block gate/up 2560->6912, down 6912->2560 (each its own codes, codebook and 0.38 % CSR
    outliers), bf16 activations, batch 1..256: the table kernels against the tensor-core dequant-GEMM, every
    batch on a rotation of blocks larger than L2.  Rank 0 only (a block is not sharded here)."""
    if E.rank != 0:
        return None
    import torch
    from ojasx_b200 import ops, synth
    from oracle import oracle as O
    pk = peaks()
    R = args.mlp_blocks
    hw = [(synth.make_vq_linear(300 + 3 * i, 2560, 6912), synth.make_vq_linear(301 + 3 * i, 2560, 6912),
           synth.make_vq_linear(302 + 3 * i, 6912, 2560)) for i in range(2)]
    blocks = [ops.VQMLP(*(ops.VQLinear.from_weights(w) for w in hw[i % 2])) for i in range(R)]
    alg_w = sum(w.algorithmic_bytes(0) for w in hw[0])
    out = {"blocks_in_rotation": R, "rotation_mb": round(R * alg_w / 1e6, 1), "dtype": "bf16", "batches": {}}
    switch = None
    for B in (1, 4, 16, 64, 256):
        x = (torch.randn(B, 2560, device=E.dev, generator=torch.Generator(device=E.dev).manual_seed(B))).to(torch.bfloat16)
        alg = alg_w + B * (2560 * 2 + 6912 * 2 * 3 + 2560 * 2)       # + activations in and out of every linear
        flop = 2.0 * B * 3 * 2560 * 6912
        res = {}
        def separately(blk):      # three launches + the gate, so that a single token can take the tensor path too
            g, u = blk.gate(x), blk.up(x)
            return blk.down(ops.silu_mul(g, u, out=g))
        for path, env in (("table", "0"), ("tensor", "1")):
            os.environ["OJASX_B200_TENSOR_MIN_BATCH"] = env
            try:
                run = E.graph_of((lambda: [blk(x) for blk in blocks]) if path == "table" else (lambda: [separately(blk) for blk in blocks]), solo=True)
                ms = E.time_ms(run, 5 if B <= 64 else 3, 2, solo=True) / R
            except Exception as ex:
                res[path] = {"error": repr(ex)[:200]}
                continue
            if path == "table":
                res[path] = {"us_per_block": round(ms * 1e3, 2), "roofline": hbm_roofline(alg, ms * 1e-3)}
            else:
                tf = flop / (ms * 1e-3) / 1e12
                res[path] = {"us_per_block": round(ms * 1e3, 2),
                             "roofline": {"bound": "tensor", "achieved": round(tf, 2), "peak": pk["tf"], "unit": "TFLOP/s",
                                          "frac": round(tf / pk["tf"], 4), "traffic": None, "dense_equivalent_flop": flop,
                                          "hbm_gbs": round(alg / (ms * 1e-3) / 1e9, 1), "peak_source": pk["src"]}}
        os.environ.pop("OJASX_B200_TENSOR_MIN_BATCH", None)
        if "us_per_block" in res.get("table", {}) and "us_per_block" in res.get("tensor", {}):
            res["faster"] = "tensor" if res["tensor"]["us_per_block"] < res["table"]["us_per_block"] else "table"
            if switch is None and res["faster"] == "tensor":
                switch = B
        out["batches"][f"B{B}"] = res
    out["measured_switch_over_batch"] = switch
    out["automatic_switch"] = "bf16 batches >= 32 take the tensor path (OJASX_B200_TENSOR_MIN_BATCH overrides)"
    # parity of both paths on one block against the oracle (bf16 tolerance of the path: rel 2e-2)
    xb = synth.to_bf16_f32(np.random.default_rng(0).standard_normal((4, 2560)).astype(np.float32))
    g, u, d = hw[0]
    lin = lambda w, v: O.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, v, block_dim=8)
    gate, up = synth.to_bf16_f32(lin(g, xb)), synth.to_bf16_f32(lin(u, xb))
    h = synth.to_bf16_f32(gate / (1 + np.exp(-gate.astype(np.float64))).astype(np.float32) * up)
    want = lin(d, h)
    xt = torch.from_numpy(xb).to(E.dev).to(torch.bfloat16)
    os.environ["OJASX_B200_TENSOR_MIN_BATCH"] = "0"
    got = blocks[0](xt).float().cpu().numpy()
    ok_table = bool(np.all(np.abs(got - want) <= 2e-2 * np.abs(want) + 2e-2))
    os.environ.pop("OJASX_B200_TENSOR_MIN_BATCH", None)
    # the tensor path rounds the weights to bf16 as well: checked per layer, with the absolute term its tests use
    got_g = blocks[0].gate.forward_tensor(xt).float().cpu().numpy()
    ok_tensor = bool(np.all(np.abs(got_g - lin(g, xb)) <= 2e-2 * np.abs(lin(g, xb)) + 3e-2))
    out["parity"] = (f"table path: block {'within' if ok_table else 'OUTSIDE'} rel 2e-2 of the oracle on 4 tokens; tensor path: "
                     f"gate layer {'within' if ok_tensor else 'OUTSIDE'} rel 2e-2 + 3e-2 (weights rounded to bf16)")
    if args.cpu_seconds > 0 and O.ref_available():
        ref = O.RefLib()
        hs = [ref.make_linear(w.codebook, w.codes, w.scales, w.bias, w.csr, block_dim=8) for w in hw[0]]
        xi = xb[:1]
        t0, n = time.perf_counter(), 0
        while time.perf_counter() - t0 < min(3.0, args.cpu_seconds):
            a = ref.linear_forward_handle(hs[0], xi, 6912, 0)
            b = ref.linear_forward_handle(hs[1], xi, 6912, 0)
            ref.linear_forward_handle(hs[2], (a / (1 + np.exp(-a)) * b).astype(np.float32), 2560, 0)
            n += 1
        out["cpu_reference_B1"] = {"us_per_block": round((time.perf_counter() - t0) / n * 1e6, 1), "cores": os.cpu_count(),
                                   "kind": "reference", "sample": f"{n} blocks, fp32, three ojasx_linear_forward calls each"}
    return out


# ------------------------------------------------------------------------------------------ row split (N > 1)
def bench_row_split(args, E):
    """Single layers split by output rows over the ranks, gather fused into the kernel: latency of one 2560->6912 and
    one 6912->2560 layer at batch 1, replayed from a CUDA graph over a rotation of layers (cold weights)."""
    import torch
    from ojasx_b200 import ops, sharding, synth
    out = {}
    for K, M in ((2560, 6912), (6912, 2560)):
        R = 48
        hw = [synth.make_vq_linear(500 + i, K, M) for i in range(2)]
        full = [ops.VQLinear.from_weights(hw[i % 2]) for i in range(R)]
        sh = [sharding.ShardedVQLinear(l, segment=E.seg, max_batch=1) for l in full]
        x = torch.randn(1, K, device=E.dev, generator=torch.Generator(device=E.dev).manual_seed(K))
        run = E.graph_of(lambda: [s.forward(x) for s in sh])
        ms = E.time_ms(run, 10, 2) / R
        one = E.graph_of(lambda: [l(x) for l in full])
        ms1 = E.time_ms(one, 10, 2) / R
        ok = bool(torch.equal(sh[0].forward(x), full[0](x)))
        alg = hw[0].algorithmic_bytes()
        out[f"{K}x{M}"] = {"us_per_layer_sharded": round(ms * 1e3, 2), "us_per_layer_one_gpu_here": round(ms1 * 1e3, 2),
                           "rows_per_rank": sh[0].row_stop - sh[0].row_start,
                           "roofline": hbm_roofline(alg, ms * 1e-3, E.world),
                           "parity": "gathered rows bit-identical to the unsharded layer" if ok else "MISMATCH"}
        del sh, full
    return out


# ------------------------------------------------------------------------------------------ configuration 2
def bench_moe(args, E):
    """Configuration 2: 512 experts, hidden 2560, inter 640, top-10, router included; tokens/s at B = 1, 32, 256.
    N > 1: experts split over the ranks, activations replicated, every (token, expert) output row stored into
    every rank's buffer from the down kernel and combined in caller order on every rank (same bits as one GPU).
    A step is one routed layer on fresh activations: 16 different token batches are recorded into one CUDA graph,
    so the routed experts change from layer to layer and their code blocks come from HBM."""
    import torch
    from ojasx_b200 import ops, sharding, synth
    rank, world, dev = E.rank, E.world, E.dev
    NE = 512
    w = synth.make_vq_moe(77, NE, 2560, 640, block_dim=8, outlier_frac=0.0038 if args.moe_csr else 0.0)
    per = NE // world
    moe = ops.VQMoE(w, (rank * per, (rank + 1) * per))
    ep = sharding.ExpertParallelMoE(moe, segment=E.seg, max_tokens=256, top_k=10) if world > 1 else None
    out = {"experts_per_gpu": per, "csr": bool(args.moe_csr)}
    csr_per_expert = 0
    if w.gate_up_csr is not None:
        csr_per_expert = (len(w.gate_up_csr[2]) + len(w.down_csr[2])) * 8 // NE + (2 * 640 + 2560) * 4
    NX = 16
    for B in (1, 32, 256):
        xs = [torch.randn(B, 2560, device=dev, generator=torch.Generator(device=dev).manual_seed(50 + i)) for i in range(NX)]
        y = torch.empty_like(xs[0])
        moe.reserve(B, 10)
        if world == 1:
            layer = lambda xx: moe.forward_routed(xx, 10, out=y)
        else:
            layer = lambda xx: ep.forward_routed(xx, 10)
        run = E.graph_of(lambda: [layer(xx) for xx in xs])
        ms = E.time_ms(run, 10 if B < 256 else 4, 2) / NX
        # algorithmic bytes of a layer: every distinct routed expert's code blocks and outliers once, the router,
        # both codebooks, activations in and out
        idx, wts = moe.route(xs[0], 10)
        distinct = float(np.mean([int(torch.unique(moe.route(xx, 10)[0]).numel()) for xx in xs[:4]]))
        code = distinct * w.code_bytes_per_expert()
        alg = code + distinct * csr_per_expert + w.router.nbytes + 2 * 256 * 8 * 4 + 2 * B * 2560 * 4
        ent = {"ms_per_layer": round(ms, 4), "tokens_per_s": round(B / ms * 1e3, 1), "distinct_experts": round(distinct, 1),
               "code_gbs": round(code / ms / 1e6, 1),
               "roofline": hbm_roofline(alg, ms * 1e-3, world,
                                        note="every code byte is gathered from a shared-memory table once per token routed to its "
                                             "expert, so large batches are bound by the shared-memory gather rate, not by HBM"),
               "code_bytes_frac": round(code / ms / 1e6 / peaks()["hbm"] / world, 4)}
        # parity spot-check against the oracle: two tokens of the first batch
        if rank == 0:
            from oracle import oracle as O
            got = layer(xs[0])
            got = (got if got is not None else y).clone()
            torch.cuda.synchronize()
            oi, ow = O.router_topk(xs[0][:2].cpu().numpy(), w.router, 10)
            ok = bool(np.array_equal(idx[:2].cpu().numpy(), oi))
            for t in range(min(2, B)):
                ref = O.moe_forward(w.codebook, w.down_codebook, w.gate_up_codes, w.gate_up_scales, w.down_codes, w.down_scales,
                                    xs[0][t].cpu().numpy(), oi[t], ow[t], block_dim=8, gu_csr=w.gate_up_csr, dn_csr=w.down_csr)
                ok &= bool(np.all(np.abs(got[t].cpu().numpy() - ref) <= 1e-6 + 1e-5 * np.abs(ref)))
            ent["parity"] = "router index-exact, outputs within rel 1e-5 / abs 1e-6 of the oracle on sampled tokens" if ok else "MISMATCH"
        elif world > 1:
            layer(xs[0])      # the other ranks take part in rank 0's check call
        out[f"B{B}"] = ent
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


# ------------------------------------------------------------------------------------------ configuration 3
def bench_kv(args, E):
    """Configuration 3: append one token + one decode query, 32 q heads / 8 kv heads, head_dim 128, bf16 q, contexts
    2048 / 32768 / 131072 at batch 1 and 16.  N > 1: KV heads split over the ranks, the heads' outputs stored into
    every rank's gathered output by the decode kernel."""
    import torch
    from ojasx_b200 import ops, sharding, synth
    rank, world, dev = E.rank, E.world, E.dev
    out = {}
    h0, h1 = sharding.split_range(8, world, rank)
    hl = h1 - h0
    if hl == 0:
        return {"skipped": "more ranks than KV heads"}
    kvw = synth.make_vq_kv(3, 1, 8)
    for B, ctx in ((1, 2048), (16, 2048), (1, 32768), (16, 32768), (1, 131072), (16, 131072)):
        cache = ops.VQKVCache(B, hl, 4 * hl, 128, 8, ctx + 64, kvw.k_codebook[h0:h1], kvw.v_codebook[h0:h1])
        rng = np.random.default_rng(9 + rank)
        codes = rng.integers(0, 256, size=(B, hl, ctx, 16), dtype=np.uint8)
        cache.load(codes, codes[:, :, ::-1].copy())
        cache.set_static_plan(True)      # launch shape fixed by the capacity: the pair can be replayed from a graph
        q = torch.randn(B, 4 * hl, 128, device=dev).to(torch.bfloat16)
        nk = (torch.randn(B, hl, 128, device=dev) / 11.3).to(torch.bfloat16)
        hs = sharding.HeadShardedKVCache(cache, 32, total_kv_heads=8, segment=E.seg, dtype=torch.bfloat16) if world > 1 else None
        o = torch.empty_like(q)

        def pair():
            cache.append(nk, nk)
            if world == 1:
                cache.decode(q, out=o)
            else:
                hs.decode(q)
        reps = 20
        ms = E.time_ms(pair, reps, 3)
        assert cache.sync_len() >= 0
        bytes_code = B * ctx * 256
        alg = bytes_code + 2 * 8 * 256 * 8 * 4 + B * 32 * 128 * 2 * 2 + B * 8 * 128 * 2 * 2
        ent = {"us_append_plus_decode": round(ms * 1e3, 2), "code_gbs": round(bytes_code / ms / 1e6, 1),
               "roofline": hbm_roofline(alg, ms * 1e-3, world), "kv_heads_per_gpu": hl}
        if rank == 0 and ctx <= 32768:
            # parity spot-check: one (sequence, KV head) of this rank against the fp64 oracle on the codes now cached
            from oracle import oracle as O
            n = cache.sync_len()
            gk, gv = cache.read(0, n)
            got = cache.decode(q)      # this rank's heads, decoded locally (no exchange): every rank's shard is the same kernel
            if got is not None:
                b = B - 1
                qf = q[b, 0:4].float().cpu().numpy()
                want = O.kvq_decode(qf, gk[b, 0], gv[b, 0], kvw.k_codebook[h0], kvw.v_codebook[h0], block_dim=8)
                ok = bool(np.allclose(got[b, 0:4].float().cpu().numpy(), want, rtol=2e-2, atol=2e-3))
                ent["parity"] = "within rel 2e-2 (bf16 path) of the fp64 oracle on a sampled (sequence, KV head)" if ok else "MISMATCH"
        out[f"B{B}_ctx{ctx}"] = ent
        cache.close()
        del cache
    if rank == 0 and args.cpu_seconds > 0:
        # CPU restatement (fp64 port; the reference has no codebook-VQ cache) on one KV head of ctx 2048, scaled to 8 heads
        from oracle import oracle as O
        kv = synth.make_vq_kv(3, 1, 2048)
        t0 = time.perf_counter()
        O.kvq_decode(kv.q[0, :4], kv.k_codes[0, 0], kv.v_codes[0, 0], kv.k_codebook[0], kv.v_codebook[0], block_dim=8)
        out["cpu_port_B1_ctx2048"] = {"us": round((time.perf_counter() - t0) * 8e6, 1), "cores": 1, "kind": "port",
                                      "sample": "one KV head (4 query heads) x 8"}
    return out


# ------------------------------------------------------------------------------------------ configuration 4
def bench_stack(args, E):
    """Configuration 4: 24-layer decoder stack (hidden 2560, 32/8 heads of 128, RoPE 1e6, RMSNorm, 512-expert top-10
    MoE per layer, VQ lm_head over 151936 tokens, quantised KV), 512 random prompt ids then 256 greedy steps at
    batch 1 and 32.  One host weight set, 24 distinct device copies (every layer streams its own HBM bytes).
    N > 1: KV heads, o_proj rows, experts and the vocabulary split over the ranks."""
    import torch
    from ojasx_b200 import inference_engine as ie
    out = {}
    cfg = ie.StackConfig(max_seq_len=args.stack_prompt + args.stack_new + 8)
    t0 = time.perf_counter()
    W = ie.make_stack_weights(2024, cfg)
    out["host_weight_seconds"] = round(time.perf_counter() - t0, 1)
    lw = W.layers[0]
    per_layer = sum(a.algorithmic_bytes(0) for a in (lw.q, lw.k, lw.v, lw.o)) + lw.moe.router.nbytes
    exp_bytes = lw.moe.code_bytes_per_expert() + (len(lw.moe.gate_up_csr[2]) + len(lw.moe.down_csr[2])) * 8 // cfg.experts
    for B in args.stack_batches:
        stack = ie.VQDecoderStack(W, cfg, batch=B, use_graph=not args.stack_eager, segment=E.seg,
                                  dtype=torch.bfloat16 if args.stack_dtype == "bf16" else torch.float32)
        stack.gather_logits = False
        ids = torch.randint(0, cfg.vocab, (B, args.stack_prompt), device=E.dev, generator=torch.Generator(device=E.dev).manual_seed(3))
        stack.prefill(ids)          # untimed: first use of every kernel at these shapes, scratch growth, graph capture
        stack.reset()
        E.barrier()
        t0 = time.perf_counter()
        logits = stack.prefill(ids)
        E.barrier()
        dt_pre = E.max_over_ranks(time.perf_counter() - t0)
        # one untimed step: it records the decode step into a CUDA graph (warm-up launch + capture), which is not decoding
        nxt = torch.argmax(logits, dim=-1) if E.seg is None else stack._next.clone()
        logits = stack.decode_step(nxt)
        E.barrier()
        t1 = time.perf_counter()
        for _ in range(args.stack_new):
            nxt = torch.argmax(logits, dim=-1) if E.seg is None else stack._next.clone()
            logits = stack.decode_step(nxt)
        E.barrier()
        t2 = time.perf_counter()
        dt_dec = E.max_over_ranks(t2 - t1)
        ctx = args.stack_prompt + args.stack_new // 2
        experts_hit = cfg.experts * (1 - (1 - cfg.top_k / cfg.experts) ** B)
        step_bytes = cfg.layers * (per_layer + experts_hit * exp_bytes + B * ctx * 256) + W.lm_head.algorithmic_bytes(0)
        out[f"B{B}"] = {"prefill_tokens_per_s": round(B * args.stack_prompt / dt_pre, 1),
                        "decode_tokens_per_s": round(B * args.stack_new / dt_dec, 1),
                        "ms_per_decode_step": round(dt_dec / args.stack_new * 1e3, 3),
                        "prompt": args.stack_prompt, "new_tokens": args.stack_new, "dtype": args.stack_dtype,
                        "prefill": "positions batched through linears and MoE, attention position by position" if E.seg is None
                                   else "token by token through the sharded decode step",
                        "bytes_per_step_estimate": int(step_bytes),
                        "roofline": hbm_roofline(step_bytes, dt_dec / args.stack_new, E.world,
                                                 note="a decode step is a chain of about 290 small launches per rank; latency, not bandwidth, bounds it"),
                        "all_finite": bool(torch.isfinite(logits).all().item())}
        del stack
        torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--layers", type=int, default=1480, help="independent layers per step (10 per SM of one GPU)")
    ap.add_argument("--e2e-layers", type=int, default=148)
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--e2e-threads", type=int, default=0,
                    help="host threads that issue the synchronous per-layer calls of the e2e leg (0 = up to 4, as many as the "
                         "host cores allow each rank, since every caller polls for completion)")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--segment-mb", type=int, default=320, help="shared segment of a rank for the exchanges (N > 1)")
    ap.add_argument("--no-mlp-sweep", dest="mlp_sweep", action="store_false")
    ap.add_argument("--mlp-blocks", type=int, default=24)
    ap.add_argument("--no-row-split", dest="row_split", action="store_false")
    ap.add_argument("--no-moe", dest="moe", action="store_false")
    ap.add_argument("--no-moe-csr", dest="moe_csr", action="store_false")
    ap.add_argument("--no-kv", dest="kv", action="store_false")
    ap.add_argument("--no-stack", dest="stack", action="store_false", help="skip the 24-layer decoder stack (about a minute)")
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
