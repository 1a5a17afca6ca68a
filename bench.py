#!/usr/bin/env python
"""Benchmark of the quantized-weight matmul path on B200.

Headline (BASELINE.json metric, first half): Q4_K-model decode GEMV packed-weight GB/s at M=1. One "step" is one
Qwen2-0.5B-shaped Q4_K_M decode step, matmul only: 24 layers x {Q,K,V,O,gate,up in Q4_K, down in Q6_K} plus the
Q6_K lm_head = 169 fused dequant+matmul products streaming 339,916,416 bytes of GGUF-layout packed weights per
step (more than the 126 MB L2, so every step re-reads HBM), issued as ONE grouped launch through the batch
front end. The second half of the metric (prefill GEMM TFLOP/s at M=512, Llama-2-7B-shaped Q4_K) is reported in
the "gemm" object of the same line. Inputs are seeded synthetic tensors (rocmforge_b200.synth); no model file or
public dataset is used.

  python bench.py [--gpus N --steps K --warmup W]      this library (one process per GPU under torchrun)
  python bench.py --impl reference [...]               the reference's CPU algorithm (oracle port) on the host cores
  python bench.py --workload matrix --qtype Q4_K --n 65536 --k 4096 [--m M]   one tensor (profiling aid)

Prints ONE JSON line (rank 0). N > 1: every rank runs the step on its own replica of the weights (independent
decode streams; a decode step has no exchange between GPUs), "scaling": "weak". The column split of a large
projection across the ranks followed by an NCCL all-gather of the output slices is measured in the "shard"
object of the same line.
"""
import argparse
import ctypes
import json
import re
import os
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from rocmforge_b200 import _lib, synth  # noqa: E402

STEP_BYTES = 339_916_416
METRIC = "Q4_K-model decode GEMV packed-weight GB/s at M=%d"


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


def host_threads():
    """Host cores this process may run on. The launcher for N > 1 exports OMP_NUM_THREADS=1, which would turn the
    CPU legs into single-thread runs; the oracle's OpenMP loops take an explicit thread count instead."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def step_config(m, gpus):
    """The `config` object, identical in both arms (this library and --impl reference)."""
    return {"workload": "qwen2-0.5b-q4_k_m-decode-step-matmul-only", "products": 169, "m": m, "layout": "GGUF",
            "packed_bytes_per_step": STEP_BYTES, "parallelism": "replicas" if gpus > 1 else "single",
            "l2": "inputs larger than L2 (340 MB streamed per step)"}


def cpu_step(m, threads, products=None):
    """The step (or its first `products` products) on the CPU oracle, the composition the reference's own bench
    times (benches/matmul_bench.rs:360-365): dequantise the tensor to fp32, then cpu_matmul_f32."""
    from oracle import cpu_oracle as orc
    ops = synth.qwen2_0p5b_step()
    if products:
        ops = ops[:products]
    rng = synth.rng_for(synth.CONFIG_SEEDS[3])
    ws = [synth.gen_packed(qt, synth.GGUF, n * k, rng) for _, qt, n, k in ops]
    xs = [synth.gen_activations(m, k, rng) for _, _, _, k in ops]
    nbytes = sum(w.size for w in ws)

    def step():
        for (_, qt, n, k), w, x in zip(ops, ws, xs):
            wf = orc.dequantize(qt, synth.GGUF, w, n * k, threads=threads).reshape(n, k)
            orc.matmul_f32(x, wf, nk=True, threads=threads)

    return step, nbytes


def run_reference(args, rank, world):
    """The reference's CPU path (oracle port of its dequant + cpu_matmul_f32 composition) on all host threads, one whole
    step (all 169 products) per timed step."""
    if rank != 0:
        return
    threads = host_threads()
    step, nbytes = cpu_step(args.m, threads)
    assert nbytes == STEP_BYTES
    for _ in range(max(args.warmup, 1)):      # also warms the OpenMP pool and the page cache of the temporaries
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    gbs = nbytes / dt / 1e9
    sample = f"the whole step (169 products, {nbytes} packed bytes) per timed step, all {threads} host threads"
    print(json.dumps({
        "impl": "reference", "metric": METRIC % args.m, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": step_config(args.m, args.gpus),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


def step_traffic(m):
    """DRAM bytes one launch of the step kernel moves (dram__bytes_read.sum + dram__bytes_write.sum of the ncu capture
    summarised under profiles/), or None when the kernel source has changed since that capture was taken."""
    import hashlib
    tp = os.path.join(ROOT, "profiles", "gemv_i8_kernel_qwen2_decode_step.md")
    src = os.path.join(ROOT, "rocmforge_b200", "csrc", "gemv_i8.cu")
    if not (os.path.exists(tp) and os.path.exists(src)):
        return None
    text = open(tp).read()
    want = re.search(r"source_sha256\(gemv_i8\.cu\)\s*=\s*([0-9a-f]{64})", text)
    hit = re.search(r"dram_bytes_per_launch\(m=%d\)\s*=\s*([0-9]+)" % m, text)
    if not want or not hit or hashlib.sha256(open(src, "rb").read()).hexdigest() != want.group(1):
        return None
    return int(hit.group(1))


def time_matmul(be, w, m, steps, warmup, x_dtype=0, flags=0):
    """Device time per launch of one fused dequant+matmul (CUDA events on the library's stream)."""
    rng = synth.rng_for(4243)
    x = synth.gen_activations(m, w.k, rng)
    xb = be.allocate_buffer(x.nbytes); xb.copy_from_host(x)
    yb = be.allocate_buffer(m * w.n_local * 4)
    for _ in range(max(warmup, 1)):
        w.matmul(xb, yb, m, flags=flags)
    be.synchronize()
    be.timer_start()
    for _ in range(steps):
        w.matmul(xb, yb, m, flags=flags)
    ms = be.timer_stop_ms() / steps
    be.synchronize()
    xb.free(); yb.free()
    return ms


def run_matrix(args, be, peaks):
    """One packed tensor, m activation rows, timed launch by launch (a small case for profiler captures)."""
    from rocmforge_b200.backend import QuantizedWeight
    qt = synth.QNAMES.index(args.qtype)
    rng = synth.rng_for(4242)
    data = synth.gen_packed(qt, synth.GGUF, args.n * args.k, rng)
    w = QuantizedWeight(be, data, qt, synth.GGUF, args.n, args.k)
    ms = time_matmul(be, w, args.m, args.steps, args.warmup, flags=_lib.MM_MX_NATIVE if args.native_mx else 0)
    gbs = w.packed_bytes / (ms * 1e-3) / 1e9
    print(json.dumps({"workload": "matrix", "qtype": args.qtype, "n": args.n, "k": args.k, "m": args.m, "native_mx": bool(args.native_mx),
                      "packed_bytes": w.packed_bytes, "ms_per_launch": ms, "GB/s": gbs, "frac_of_hbm": gbs / peaks["hbm_gbs"],
                      "tflops": 2.0 * args.m * args.n * args.k / (ms * 1e-3) / 1e12}))


def gemm_leg(be, peaks, steps):
    """Second half of the metric: Llama-2-7B-shaped Q4_K prefill GEMM at M=512 (device-resident operands)."""
    from rocmforge_b200.backend import QuantizedWeight
    rows = []
    rng = synth.rng_for(synth.CONFIG_SEEDS[4])
    for n, k in synth.LLAMA7B_SHAPES:
        data = synth.gen_packed(synth.Q4_K, synth.GGUF, n * k, rng)
        w = QuantizedWeight(be, data, synth.Q4_K, synth.GGUF, n, k)
        for m in (256, 512, 2048):
            ms = time_matmul(be, w, m, steps, 3)
            rows.append({"n": n, "k": k, "m": m, "ms": ms, "tflops": 2.0 * m * n * k / (ms * 1e-3) / 1e12})
        w.free()
    head = rows[1]
    return {"metric": "Q4_K prefill GEMM TFLOP/s at M=512", "workload": "llama-2-7b ffn_up Q4_K [11008,4096], M=512",
            "value": head["tflops"], "unit": "TFLOP/s", "peak": peaks["bf16_tflops"], "frac": head["tflops"] / peaks["bf16_tflops"],
            "peak_source": peaks["source"], "operands": "f16 x f16 -> fp32 (tcgen05, TMEM accumulators)", "shapes": rows}


def mlp_leg(be, peaks, steps):
    """The SwiGLU MLP block of a Llama-2-7B-shaped layer on packed weights (gate/up Q4_K [11008,4096], down Q6_K
    [4096,11008]): gate+up grouped launch, activation kernel, down projection; device-resident operands."""
    from rocmforge_b200 import projections
    from rocmforge_b200.backend import QuantizedWeight
    hidden, n_ff = 4096, 11008
    rng = synth.rng_for(synth.CONFIG_SEEDS[4] + 50)
    wg = QuantizedWeight(be, synth.gen_packed(synth.Q4_K, synth.GGUF, n_ff * hidden, rng), synth.Q4_K, synth.GGUF, n_ff, hidden)
    wu = QuantizedWeight(be, synth.gen_packed(synth.Q4_K, synth.GGUF, n_ff * hidden, rng), synth.Q4_K, synth.GGUF, n_ff, hidden)
    wd = QuantizedWeight(be, synth.gen_packed(synth.Q6_K, synth.GGUF, hidden * n_ff, rng), synth.Q6_K, synth.GGUF, hidden, n_ff)
    packed = wg.packed_bytes + wu.packed_bytes + wd.packed_bytes
    rows = []
    for m in (1, 512):
        x = synth.gen_activations(m, hidden, synth.rng_for(60 + m))
        xb = be.allocate_buffer(x.nbytes); xb.copy_from_host(x)
        ob = be.allocate_buffer(m * hidden * 4)
        plan = projections.MlpSwiglu(be, xb, wg, wu, wd, ob, m)
        for _ in range(3):
            plan.run()
        be.synchronize()
        be.timer_start()
        for _ in range(steps):
            plan.run()
        ms = be.timer_stop_ms() / steps
        be.synchronize()
        rows.append({"m": m, "ms": ms, "packed_GB/s": packed / (ms * 1e-3) / 1e9,
                     "tflops": 2.0 * m * 3 * n_ff * hidden / (ms * 1e-3) / 1e12})
        plan.free(); xb.free(); ob.free()
    for w in (wg, wu, wd):
        w.free()
    return {"workload": "llama-2-7b SwiGLU MLP block, gate/up Q4_K + down Q6_K (87.7 MB packed), b200q_mlp_run",
            "launches_per_run": {"m=1": 3, "m=512": 5}, "shapes": rows}


def formats_leg(be, peaks, steps):
    """Every GGUF format with a tensor-core decode kernel and a tensor-memory prefill kernel on one [8192, 8192]
    tensor: decode (m = 1) in packed GB/s and prefill (m = 512) in TFLOP/s, device-resident operands."""
    from rocmforge_b200.backend import QuantizedWeight
    n = k = 8192
    rows = []
    for qname in ("Q4_0", "Q8_0", "Q4_K", "Q5_K", "Q6_K", "MXFP4", "MXFP6_E2M3", "MXFP6_E3M2", "Q2_K", "Q3_K"):
        qt = synth.QNAMES.index(qname)
        w = QuantizedWeight(be, synth.gen_packed(qt, synth.GGUF, n * k, synth.rng_for(9000 + qt)), qt, synth.GGUF, n, k)
        ms1 = time_matmul(be, w, 1, steps * 2, 3)
        ms512 = time_matmul(be, w, 512, steps, 3)
        rows.append({"qtype": qname, "decode_GB/s": w.packed_bytes / (ms1 * 1e-3) / 1e9,
                     "decode_frac_of_hbm": w.packed_bytes / (ms1 * 1e-3) / 1e9 / peaks["hbm_gbs"],
                     "prefill_tflops": 2.0 * 512 * n * k / (ms512 * 1e-3) / 1e12,
                     "prefill_frac_of_peak": 2.0 * 512 * n * k / (ms512 * 1e-3) / 1e12 / peaks["bf16_tflops"]})
        w.free()
    return {"workload": "[8192, 8192] GGUF tensor per format, single launches (m = 1 and m = 512)",
            "note": "MXFP6_E3M2 and Q2_K have no tensor-core decode kernel (CUDA-core kernel at m = 1); Q3_K decodes re-encoded in "
                    "Q6_K's item form (6.6 bit per weight streamed for 3.4 in the file) and prefills on Q6_K planes; MXFP6_E3M2 prefills through an image of E2M3's form "
                    "(f16 high bytes); Q2_K prefills on the shared-memory-operand tensor-core kernel", "rows": rows}


def config5_leg(be, peaks, steps):
    """BASELINE config 5: MXFP4 and MXFP6 at the Llama-70B FFN shape [28672, 8192], m = 1 (packed GB/s) and m = 64, 512
    (TFLOP/s), single launches, device-resident operands. Fractions use the FORMAT's bytes (17 / 25 bytes per 32
    weights), not the bytes of the decode image."""
    from rocmforge_b200.backend import QuantizedWeight
    n, k = synth.LLAMA70B_FFN_SHAPES[0]
    rows = []
    for qname in ("MXFP4", "MXFP6_E2M3", "MXFP6_E3M2"):
        qt = synth.QNAMES.index(qname)
        w = QuantizedWeight(be, synth.gen_packed(qt, synth.GGUF, n * k, synth.rng_for(synth.CONFIG_SEEDS[5] + qt)), qt, synth.GGUF, n, k)
        ms1 = time_matmul(be, w, 1, steps * 2, 3)
        row = {"qtype": qname, "m1_ms": ms1, "m1_GB/s": w.packed_bytes / (ms1 * 1e-3) / 1e9,
               "m1_frac_of_hbm": w.packed_bytes / (ms1 * 1e-3) / 1e9 / peaks["hbm_gbs"]}
        for m in (64, 512):
            ms = time_matmul(be, w, m, steps, 3)
            row[f"m{m}_ms"] = ms
            row[f"m{m}_tflops"] = 2.0 * m * n * k / (ms * 1e-3) / 1e12
            row[f"m{m}_frac_of_peak"] = row[f"m{m}_tflops"] / peaks["bf16_tflops"]
        if True:
            # opt-in: the 4- or 6-bit codes and E8M0 scales straight into the block-scaled MMA, activations quantised to
            # MXFP8 (a lower-precision mode: a few 1e-2 against 2e-3); the fraction is still taken of the measured bf16 peak
            for m in (64, 512, 2048):
                ms = time_matmul(be, w, m, steps, 3, flags=_lib.MM_MX_NATIVE)
                row[f"m{m}_native_mx_ms"] = ms
                row[f"m{m}_native_mx_tflops"] = 2.0 * m * n * k / (ms * 1e-3) / 1e12
                row[f"m{m}_native_mx_vs_bf16_peak"] = row[f"m{m}_native_mx_tflops"] / peaks["bf16_tflops"]
        rows.append(row)
        w.free()
    return {"workload": "llama-70b ffn [28672, 8192], MXFP4 and MXFP6 (E2M3, E3M2), single launches; native_mx = B200Q_MM_MX_NATIVE "
                        "(tcgen05.mma.kind::mxf8f6f4.block_scale on the packed codes, MXFP8 activations)", "rows": rows}


def config2_leg(be, steps):
    """BASELINE config 2: Q8_0 [896, 896] and [4864, 896], m = 1, 16, 128, 512. These products are launch-bound (0.85 and
    4.6 MB of weights): the figure is the time of one launch in a back-to-back series."""
    from rocmforge_b200.backend import QuantizedWeight
    rows = []
    for n in (896, 4864):
        w = QuantizedWeight(be, synth.gen_packed(synth.Q8_0, synth.GGUF, n * 896, synth.rng_for(synth.CONFIG_SEEDS[2] + n)),
                            synth.Q8_0, synth.GGUF, n, 896)
        for m in (1, 16, 128, 512):
            ms = time_matmul(be, w, m, steps * 2, 3)
            rows.append({"n": n, "k": 896, "m": m, "us": ms * 1e3, "packed_GB/s": w.packed_bytes / (ms * 1e-3) / 1e9,
                         "tflops": 2.0 * m * n * 896 / (ms * 1e-3) / 1e12})
        w.free()
    return {"workload": "Q8_0 [896, 896] and [4864, 896] (qwen2-0.5b attention / FFN shapes), single launches", "rows": rows}


def shard_leg(be, rank, world, steps):
    """Column split of the Llama-70B-shaped FFN projection [28672, 8192] over the ranks + NCCL all-gather."""
    import torch
    import torch.distributed as dist
    from rocmforge_b200.backend import QuantizedWeight
    n, k = synth.LLAMA70B_FFN_SHAPES[0]
    out = {"workload": "llama-70b ffn [28672,8192], output features split over the ranks, all-gather of the slices",
           "cases": []}
    for qname in ("Q4_K", "MXFP4"):
        qt = synth.QNAMES.index(qname)
        rng = synth.rng_for(synth.CONFIG_SEEDS[5] + qt)
        data = synth.gen_packed(qt, synth.GGUF, n * k, rng)
        w = QuantizedWeight(be, data, qt, synth.GGUF, n, k, shard_rank=rank, shard_count=world)
        full = QuantizedWeight(be, data, qt, synth.GGUF, n, k) if rank == 0 else None
        for m in (1, 512):
            x = synth.gen_activations(m, k, synth.rng_for(77 + m))
            xt = torch.from_numpy(x).cuda()
            y_slice = torch.empty((m, n // world), dtype=torch.float32, device="cuda")
            y_all = torch.empty((world, m, n // world), dtype=torch.float32, device="cuda")
            cur = torch.cuda.current_stream()

            def kernel():
                w.matmul(xt.data_ptr(), y_slice.data_ptr(), m)

            def timed(fn, reps):
                torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(cur)
                for _ in range(reps):
                    fn()
                e1.record(cur)
                torch.cuda.synchronize()
                t = torch.tensor([e0.elapsed_time(e1) / reps], device="cuda", dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                return float(t.item())

            def with_gather():
                kernel()
                dist.all_gather_into_tensor(y_all.view(world * m, -1), y_slice)

            # fused form: the kernels' epilogues store this rank's slice into every rank's full output through
            # peer-mapped pointers (b200q_matmul_scatter); then every rank raises a flag in every other rank's
            # memory (b200q_peer_signal) and holds its stream until the others' flags are in (b200q_peer_wait,
            # bounded). Outputs and flags live in library allocations so that they can be exported.
            y_full = be.allocate_buffer(m * n * 4)
            flags = be.allocate_buffer(64); flags.fill(0)
            handles = [None] * world
            dist.all_gather_object(handles, (be.ipc_handle(y_full), be.ipc_handle(flags)))
            peers = [y_full.as_ptr() if r == rank else be.ipc_open(handles[r][0]) for r in range(world)]
            peer_flags = [flags.as_ptr() if r == rank else be.ipc_open(handles[r][1]) for r in range(world)]
            epoch = [0]

            def fused():
                epoch[0] += 1
                w.matmul_scatter_signal(xt.data_ptr(), peers, m, n, peer_flags, rank, epoch[0])
                be.peer_wait(flags, world, rank, epoch[0])

            # the same with bf16 outputs (B200Q_MM_SCATTER_BF16, prefill only): half the bytes over NVLink
            t_fused16 = None
            if m > 8:
                y16 = be.allocate_buffer(m * n * 2)
                h16 = [None] * world
                dist.all_gather_object(h16, be.ipc_handle(y16))
                peers16 = [y16.as_ptr() if r == rank else be.ipc_open(h16[r]) for r in range(world)]

                def fused16():
                    epoch[0] += 1
                    w.matmul_scatter_signal(xt.data_ptr(), peers16, m, n, peer_flags, rank, epoch[0], flags=_lib.MM_SCATTER_BF16)
                    be.peer_wait(flags, world, rank, epoch[0])

            for _ in range(3):
                with_gather()
                fused()
                if m > 8:
                    fused16()
            t_kernel = timed(kernel, steps)
            t_total = timed(with_gather, steps)
            t_fused = timed(fused, steps)
            if m > 8:
                t_fused16 = timed(fused16, steps)
            gathered = int(m * n * 4 * (world - 1) / world)
            case = {"qtype": qname, "m": m, "ranks": world, "ms_kernel": t_kernel, "ms_kernel_plus_allgather": t_total,
                    "ms_fused_peer_stores_plus_flags": t_fused,
                    "gathered_bytes_per_rank": gathered,
                    # what the bytes every rank must receive cost at the measured peer-copy rate of this pool
                    "nvlink_floor_ms": gathered / 770e9 * 1e3, "nvlink_GBps_assumed": 770}
            if t_fused16 is not None:
                case["ms_fused_bf16_outputs"] = t_fused16
                case["nvlink_floor_ms_bf16"] = gathered / 2 / 770e9 * 1e3
            if rank == 0:
                yb = torch.empty((m, n), dtype=torch.float32, device="cuda")
                for _ in range(3):
                    full.matmul(xt.data_ptr(), yb.data_ptr(), m)
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(cur)
                for _ in range(steps):
                    full.matmul(xt.data_ptr(), yb.data_ptr(), m)
                e1.record(cur)
                torch.cuda.synchronize()
                t1 = e0.elapsed_time(e1) / steps
                case["ms_one_gpu_unsharded"] = t1
                # strong scaling on the fixed problem: t(1 GPU) / (ranks x t(ranks))
                case["efficiency_kernel"] = t1 / (world * t_kernel)
                case["efficiency_with_allgather"] = t1 / (world * t_total)
                case["efficiency_fused"] = t1 / (world * t_fused)
                if t_fused16 is not None:
                    case["efficiency_fused_bf16"] = t1 / (world * t_fused16)
                # the gathered result equals the unsharded one (same kernel, same per-row arithmetic)
                got = y_all.permute(1, 0, 2).reshape(m, n)
                case["max_abs_diff_vs_unsharded"] = float((got - yb).abs().max().item())
                fused_host = torch.from_numpy(y_full.to_numpy(np.float32, m * n).reshape(m, n)).cuda()
                case["fused_max_abs_diff_vs_unsharded"] = float((fused_host - yb).abs().max().item())
            dist.barrier()
            for r in range(world):
                if r != rank:
                    be.ipc_close(peers[r])
                    be.ipc_close(peer_flags[r])
                    if m > 8:
                        be.ipc_close(peers16[r])
            dist.barrier()
            if m > 8:
                y16.free()
            y_full.free()
            flags.free()
            out["cases"].append(case)
        w.free()
        if full is not None:
            full.free()
    return out


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
    ap.add_argument("--native-mx", action="store_true", help="matrix workload: B200Q_MM_MX_NATIVE (MXFP4 / MXFP6, m > 8)")
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
    from rocmforge_b200.backend import B200Backend, QuantizedWeight
    from rocmforge_b200.batch import DeviceBatch

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    peaks = load_peaks()
    # the library works on torch's current stream so that torch.cuda events and NCCL see its kernels
    be = B200Backend(local_rank, stream=torch.cuda.current_stream().cuda_stream)
    m = args.m
    if args.workload == "matrix":
        run_matrix(args, be, peaks)
        return
    ops, weights, acts = build_step(m)
    W = [QuantizedWeight(be, w, qt, synth.GGUF, n, k) for (_, qt, n, k), w in zip(ops, weights)]
    assert sum(w.packed_bytes for w in W) == STEP_BYTES
    batch = DeviceBatch(be, W, m)
    batch.set_inputs(acts)

    def barrier():
        be.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        batch.run()
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    be.timer_start()
    for _ in range(args.steps):
        batch.run()
    ms = be.timer_stop_ms()
    barrier()
    t_end = time.time() + 1.0          # keep the GPU busy long enough for a few clock samples
    while time.time() < t_end:
        for _ in range(50):
            batch.run()
        be.synchronize()
    clocks = sampler.stop()
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_step = ms / args.steps
    per_gpu = STEP_BYTES / (ms_step * 1e-3) / 1e9
    value = world * per_gpu
    traffic = step_traffic(m)

    out = {
        "metric": METRIC % m, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": step_config(m, world),
        "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": per_gpu / peaks["hbm_gbs"], "traffic": traffic, "peak_source": peaks["source"],
                     "kernel": "gemv_i8_kernel (one grouped launch = one step; back-to-back launches overlap their prologues through programmatic dependent launch)",
                     "launches_per_step": batch.launches},
        "clocks": clocks, "gpu_launches": batch.launches * args.steps,
    }

    if not args.skip_extras:
        # ---- end to end through the C ABI: pinned host activations in, host results out, every step ------------
        hx = torch.from_numpy(np.concatenate([a.reshape(-1) for a in acts])).pin_memory()
        hy = torch.empty(sum(batch.ysizes), dtype=torch.float32).pin_memory()
        for _ in range(3):
            batch.run_host(hx.data_ptr(), hy.data_ptr())
        barrier()
        e2e_steps = max(3, args.steps)
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            batch.run_host(hx.data_ptr(), hy.data_ptr())
        dt = (time.perf_counter() - t0) / e2e_steps
        if world > 1:
            t = torch.tensor([dt], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        out["e2e"] = {"value": world * STEP_BYTES / dt / 1e9, "unit": "GB/s", "h2d_bytes_per_step": int(hx.numel() * 4),
                      "d2h_bytes_per_step": int(hy.numel() * 4), "ms_per_step": dt * 1e3,
                      "api": "b200q_batch_run_host: pinned host activations in (one H2D copy), outputs stored by the kernel straight into the pinned host buffer, weights resident (uploaded once)"}
        if world == 1:
            # ---- the same step with 8 activation rows (config 3 is m = 1 and m = 8) --------------------------------
            rng8 = synth.rng_for(synth.CONFIG_SEEDS[3] + 8)
            batch8 = DeviceBatch(be, W, 8)
            batch8.set_inputs([synth.gen_activations(8, k, rng8) for _, _, _, k in ops])
            for _ in range(3):
                batch8.run()
            be.synchronize()
            be.timer_start()
            for _ in range(args.steps):
                batch8.run()
            ms8 = be.timer_stop_ms() / args.steps
            out["decode_m8"] = {"workload": "the same 169-product step with m = 8", "ms_per_step": ms8,
                                "GB/s": STEP_BYTES / (ms8 * 1e-3) / 1e9, "frac": STEP_BYTES / (ms8 * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                "traffic": step_traffic(8), "launches_per_step": batch8.launches}
            batch8.free()
            # ---- prefill GEMM (second half of the metric) and a single large Q4_K GEMV --------------------------
            out["gemm"] = gemm_leg(be, peaks, 10)
            out["mlp"] = mlp_leg(be, peaks, 10)
            out["formats"] = formats_leg(be, peaks, 10)
            out["config5"] = config5_leg(be, peaks, 10)
            out["config2"] = config2_leg(be, 10)
            rng = synth.rng_for(4242)
            big = QuantizedWeight(be, synth.gen_packed(synth.Q4_K, synth.GGUF, 65536 * 4096, rng), synth.Q4_K, synth.GGUF, 65536, 4096)
            msb = time_matmul(be, big, 1, 20, 3)
            out["gemv_single"] = {"workload": "Q4_K [65536,4096], M=1, one launch", "GB/s": big.packed_bytes / (msb * 1e-3) / 1e9,
                                  "frac_of_hbm": big.packed_bytes / (msb * 1e-3) / 1e9 / peaks["hbm_gbs"]}
            big.free()
            # ---- CPU baseline (oracle port of the reference path) on the host cores ---------------------------
            threads = host_threads()
            step, nb = cpu_step(m, threads)
            step()                              # warms the OpenMP pool
            t0 = time.perf_counter()
            reps = 0
            while reps < 3 or (time.perf_counter() - t0 < 12.0 and reps < 200):
                step()
                reps += 1
            dtc = (time.perf_counter() - t0) / reps
            # the "faithful" figure: the reference's matmul is single-threaded (src/tensor/matmul.rs:219-233)
            step1, nb1 = cpu_step(m, 1, products=7)
            step1()
            t0 = time.perf_counter()
            reps1 = 0
            while reps1 < 2 or (time.perf_counter() - t0 < 6.0 and reps1 < 50):
                step1()
                reps1 += 1
            dt1 = (time.perf_counter() - t0) / reps1
            out["cpu_baseline"] = {"value": nb / dtc / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                                   "sample": f"the whole step (169 products, {nb} packed bytes), {reps} repetitions",
                                   "single_thread": {"value": nb1 / dt1 / 1e9, "unit": "GB/s", "cores": 1,
                                                     "sample": f"layer 0 of the step (7 products, {nb1} packed bytes), {reps1} repetitions"}}
        else:
            out["shard"] = shard_leg(be, rank, world, 10)
    if rank == 0:
        print(json.dumps(out))
    batch.free()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
