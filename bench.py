#!/usr/bin/env python
"""Benchmark of the quantized-weight matmul path on B200.

Headline (BASELINE.json metric): Q4_K-model decode GEMV packed-weight GB/s at M=1. One "step" is one
Qwen2-0.5B-shaped Q4_K_M decode step, matmul only: 24 layers x {Q,K,V,O,gate,up in Q4_K, down in Q6_K}
plus the Q6_K lm_head = 169 fused dequant+matmul products streaming 339,916,416 bytes of GGUF-layout
packed weights (more than the 126 MB L2, so every step re-reads HBM). Inputs are seeded synthetic tensors
(rocmforge_b200.synth); no model file is used.

  python bench.py [--gpus N --steps K --warmup W]          this library (one process per GPU under torchrun)
  python bench.py --impl reference [...]                   the reference's CPU algorithm (oracle port) on host cores

Prints ONE JSON line (rank 0). N > 1: every rank runs the same step on its own replica of the weights
(independent decode streams; the path has no exchange step at M=1), "scaling": "weak"; the column-split +
all-gather of the large projections is measured separately in the "shard" object.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from rocmforge_b200 import synth  # noqa: E402

STEP_BYTES = 339_916_416


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], bf16_tflops_sustained=d.get("bf16_tflops_sustained"),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if not self.proc:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            f = [t.strip() for t in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=float(np.median(sm)) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


def build_step(m, seed=synth.CONFIG_SEEDS[3]):
    """Packed weights (GGUF layout) and fp32 activations of one decode step."""
    ops = synth.qwen2_0p5b_step()
    rng = synth.rng_for(seed)
    weights, acts = [], []
    for name, qt, n, k in ops:
        weights.append(synth.gen_packed(qt, synth.GGUF, n * k, rng))
        acts.append(synth.gen_activations(m, k, rng))
    return ops, weights, acts


def run_reference(args, rank, world):
    """The reference's CPU path (oracle port: dequantise to fp32, then cpu_matmul_f32) on all host threads."""
    if rank != 0:
        return
    from oracle import cpu_oracle as orc
    threads = orc.max_threads()
    ops = synth.qwen2_0p5b_step()[:7]          # bounded sample: layer 0 (7 products, 9.5 MB packed)
    rng = synth.rng_for(synth.CONFIG_SEEDS[3])
    ws = [synth.gen_packed(qt, synth.GGUF, n * k, rng) for _, qt, n, k in ops]
    xs = [synth.gen_activations(args.m, k, rng) for _, _, _, k in ops]
    nbytes = sum(w.size for w in ws)

    def step():
        for (_, qt, n, k), w, x in zip(ops, ws, xs):
            wf = orc.dequantize(qt, synth.GGUF, w, n * k, threads=threads).reshape(n, k)
            orc.matmul_f32(x, wf, nk=True, threads=threads)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    gbs = nbytes / dt / 1e9
    sample = f"layer 0 of the step (7 products, {nbytes} packed bytes) per step"
    print(json.dumps({
        "impl": "reference", "metric": "Q4_K-model decode GEMV packed-weight GB/s at M=%d" % args.m, "value": gbs,
        "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "qwen2-0.5b-q4_k_m-decode-step-matmul-only", "m": args.m, "layout": "GGUF",
                   "l2": "inputs larger than L2"},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


def run_matrix(args, be, peaks):
    """One packed tensor, m activation rows, timed launch by launch (a small case for profiler captures)."""
    from rocmforge_b200.backend import QuantizedWeight
    qt = synth.QNAMES.index(args.qtype)
    rng = synth.rng_for(4242)
    data = synth.gen_packed(qt, synth.GGUF, args.n * args.k, rng)
    x = synth.gen_activations(args.m, args.k, rng)
    w = QuantizedWeight(be, data, qt, synth.GGUF, args.n, args.k)
    xb = be.allocate_buffer(x.nbytes); xb.copy_from_host(x)
    yb = be.allocate_buffer(args.m * args.n * 4)
    for _ in range(max(args.warmup, 1)):
        w.matmul(xb, yb, args.m)
    be.synchronize()
    be.timer_start()
    for _ in range(args.steps):
        w.matmul(xb, yb, args.m)
    ms = be.timer_stop_ms() / args.steps
    gbs = w.packed_bytes / (ms * 1e-3) / 1e9
    print(json.dumps({"workload": "matrix", "qtype": args.qtype, "n": args.n, "k": args.k, "m": args.m,
                      "packed_bytes": w.packed_bytes, "ms_per_launch": ms, "GB/s": gbs, "frac_of_hbm": gbs / peaks["hbm_gbs"],
                      "tflops": 2.0 * args.m * args.n * args.k / (ms * 1e-3) / 1e12}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200q", choices=["b200q", "reference"])
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--skip-extras", action="store_true", help="headline only (no e2e / cpu baseline / gemm / shard legs)")
    ap.add_argument("--workload", default="step", choices=["step", "matrix"],
                    help="step: the decode step (headline); matrix: one [--n, --k] tensor of --qtype (profiling aid)")
    ap.add_argument("--qtype", default="Q4_K")
    ap.add_argument("--n", type=int, default=65536)
    ap.add_argument("--k", type=int, default=4096)
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist
    from rocmforge_b200 import _lib
    from rocmforge_b200.backend import B200Backend, QuantizedWeight

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    peaks = load_peaks()
    be = B200Backend(local_rank)
    lib = be.lib
    m = args.m
    if args.workload == "matrix":
        run_matrix(args, be, peaks)
        return
    ops, weights, acts = build_step(m)
    W = [QuantizedWeight(be, w, qt, synth.GGUF, n, k) for (_, qt, n, k), w in zip(ops, weights)]
    assert sum(w.packed_bytes for w in W) == STEP_BYTES
    X, Y = [], []
    for (_, _, n, k), a in zip(ops, acts):
        xb = be.allocate_buffer(a.nbytes); xb.copy_from_host(a); X.append(xb)
        Y.append(be.allocate_buffer(m * n * 4))
    cnt = len(W)
    arr_w = (ctypes.c_void_p * cnt)(*[w.handle.value for w in W])
    arr_x = (ctypes.c_void_p * cnt)(*[x.ptr for x in X])
    arr_y = (ctypes.c_void_p * cnt)(*[y.ptr for y in Y])
    batch = ctypes.c_void_p()
    _lib.check(lib.b200q_batch_create(be.ctx, cnt, arr_w, arr_x, arr_y, m, ctypes.byref(batch)))
    launches_per_step = int(lib.b200q_batch_launches(batch)) if hasattr(lib, "b200q_batch_launches") else cnt

    def barrier():
        be.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        _lib.check(lib.b200q_batch_run(be.ctx, batch, None))
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    be.timer_start()
    for _ in range(args.steps):
        _lib.check(lib.b200q_batch_run(be.ctx, batch, None))
    ms = be.timer_stop_ms()
    barrier()
    # keep the GPU busy long enough for a few clock samples
    t_end = time.time() + 1.0
    while time.time() < t_end:
        _lib.check(lib.b200q_batch_run(be.ctx, batch, None))
        be.synchronize()
    clocks = sampler.stop()
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_step = ms / args.steps
    value = world * STEP_BYTES / (ms_step * 1e-3) / 1e9
    per_gpu = STEP_BYTES / (ms_step * 1e-3) / 1e9

    out = {
        "metric": "Q4_K-model decode GEMV packed-weight GB/s at M=%d" % m, "value": value, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "qwen2-0.5b-q4_k_m-decode-step-matmul-only", "products": cnt, "m": m, "layout": "GGUF",
                   "packed_bytes_per_step": STEP_BYTES, "parallelism": "replicas" if world > 1 else "single",
                   "l2": "inputs larger than L2 (340 MB streamed per step)"},
        "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": per_gpu / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["source"],
                     "kernel": "decode step (all launches of one step)", "launches_per_step": launches_per_step},
        "clocks": clocks, "gpu_launches": launches_per_step * args.steps,
    }

    if not args.skip_extras:
        # ---- end to end: host activations in, host results out, through the C ABI, every step -----------------
        hx = [torch.from_numpy(a).pin_memory() for a in acts]
        hy = [torch.empty((m, n), dtype=torch.float32).pin_memory() for (_, _, n, _) in ops]
        h2d = sum(a.nbytes for a in acts)
        d2h = sum(m * n * 4 for (_, _, n, _) in ops)

        def e2e_step():
            for w, x, y in zip(W, hx, hy):
                _lib.check(lib.b200q_matmul_host(be.ctx, w.handle, x.data_ptr(), y.data_ptr(), m, 0))

        for _ in range(3):
            e2e_step()
        barrier()
        e2e_steps = max(3, min(args.steps, 20))
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        be.synchronize()
        dt = (time.perf_counter() - t0) / e2e_steps
        if world > 1:
            t = torch.tensor([dt], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        out["e2e"] = {"value": world * STEP_BYTES / dt / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                      "d2h_bytes_per_step": d2h, "ms_per_step": dt * 1e3,
                      "api": "b200q_matmul_host per product (pinned host activations in, host outputs out; weights resident)"}
        # ---- CPU baseline (oracle port of the reference path) on rank 0 at N = 1 ---------------------------------
        if rank == 0 and world == 1:
            from oracle import cpu_oracle as orc
            threads = orc.max_threads()
            sub = list(range(7))
            nb = sum(weights[i].size for i in sub)
            t0 = time.perf_counter()
            reps = 0
            while reps < 3 or (time.perf_counter() - t0 < 10.0 and reps < 200):
                for i in sub:
                    _, qt, n, k = ops[i]
                    wf = orc.dequantize(qt, synth.GGUF, weights[i], n * k, threads=threads).reshape(n, k)
                    orc.matmul_f32(acts[i], wf, nk=True, threads=threads)
                reps += 1
            dt = (time.perf_counter() - t0) / reps
            out["cpu_baseline"] = {"value": nb / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                                   "sample": f"layer 0 of the step (7 products, {nb} packed bytes), {reps} repetitions"}
    if rank == 0:
        print(json.dumps(out))
    _lib.check(lib.b200q_batch_free(batch))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
