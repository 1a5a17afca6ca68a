"""Prefill path (m > 8): the tcgen05 tensor-core kernel against the CPU oracle.

Tolerance 2e-3 (max |y - ref| / max |ref|) against the fp32 oracle on the same activation values. Inside the
kernel weights and activations are rounded once to f16 (activations with a power-of-two scale per row);
accumulation is fp32 in tensor memory. bf16 activations convert to f16 exactly, so for them the oracle runs
on the bf16 values widened to fp32.
"""
import numpy as np
import pytest
import torch

from rocmforge_b200 import _lib, synth

pytestmark = pytest.mark.gpu
TOL = 2e-3

from gpu_util import ALL_FMTS, FMT_IDS, QuantizedWeight, backend, gpu_matmul, rel_err  # noqa: E402


def bf16_round(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(torch.bfloat16).float().numpy()


def reference(oracle, qt, lay, data, n, k, x, rows=None):
    w = oracle.dequantize(qt, lay, data, n * k, threads=8).reshape(n, k)
    if rows is not None:
        w = np.ascontiguousarray(w[rows])
    return oracle.matmul_f32(x, w, nk=True, threads=8)


def test_smallest_tile_first(oracle):
    """One CTA, four k-blocks: the first thing to run on a new build."""
    be = backend()
    rng = synth.rng_for(3100)
    n, k, m = 128, 256, 64
    data = synth.gen_packed(synth.Q8_0, synth.GGUF, n * k, rng)
    x = synth.gen_activations(m, k, rng)
    w = QuantizedWeight(be, data, synth.Q8_0, synth.GGUF, n, k)
    y = gpu_matmul(be, w, x, m)
    assert rel_err(y, reference(oracle, synth.Q8_0, synth.GGUF, data, n, k, x)) <= TOL
    w.free()


@pytest.mark.parametrize("k", [256, 512, 2048])
def test_q4k_weights_in_tensor_memory_smallest(oracle, k):
    """GGUF Q4_K with k % 256 == 0 takes the kernel whose weight operand lives in tensor memory: one CTA,
    1 / 2 / 8 super-blocks per row (fewer, as many and more k-blocks than pipeline stages)."""
    be = backend()
    rng = synth.rng_for(3150 + k)
    n, m = 128, 64
    data = synth.gen_packed(synth.Q4_K, synth.GGUF, n * k, rng)
    x = synth.gen_activations(m, k, rng)
    w = QuantizedWeight(be, data, synth.Q4_K, synth.GGUF, n, k)
    y = gpu_matmul(be, w, x, m)
    assert rel_err(y, reference(oracle, synth.Q4_K, synth.GGUF, data, n, k, x)) <= TOL
    w.free()


@pytest.mark.parametrize("qt,lay", ALL_FMTS, ids=FMT_IDS)
def test_every_format_ragged_tiles(oracle, qt, lay):
    """n and m are not tile multiples; k = 5 super-blocks."""
    be = backend()
    rng = synth.rng_for(3200 + qt * 2 + lay)
    n, k, m = 300, 1280, 100
    data = synth.gen_packed(qt, lay, n * k, rng)
    x = synth.gen_activations(m, k, rng)
    w = QuantizedWeight(be, data, qt, lay, n, k)
    y = gpu_matmul(be, w, x, m)
    assert rel_err(y, reference(oracle, qt, lay, data, n, k, x)) <= TOL
    # CUDA-core path on the same input agrees with the fp32 oracle much more tightly
    y2 = gpu_matmul(be, w, x, m, flags=_lib.MM_NO_TENSOR)
    wf = oracle.dequantize(qt, lay, data, n * k).reshape(n, k)
    assert rel_err(y2, oracle.matmul_f32(x, wf, nk=True, threads=8)) <= 1e-4
    w.free()


@pytest.mark.parametrize("k", [896, 1024])
@pytest.mark.parametrize("m", [9, 16, 17, 255, 256, 257, 512])
def test_token_counts_around_the_tile_edges(oracle, m, k):
    """k = 896 runs the shared-memory-operand kernel, k = 1024 the tensor-memory-operand one."""
    be = backend()
    rng = synth.rng_for(3300 + m + k)
    n = 256
    data = synth.gen_packed(synth.Q4_K, synth.GGUF, n * k, rng)
    x = synth.gen_activations(m, k, rng)
    w = QuantizedWeight(be, data, synth.Q4_K, synth.GGUF, n, k)
    y = gpu_matmul(be, w, x, m)
    assert rel_err(y, reference(oracle, synth.Q4_K, synth.GGUF, data, n, k, x)) <= TOL
    w.free()


@pytest.mark.parametrize("k,bf16,pitch", [(4096, False, 0), (4096, True, 0), (8192, False, 0), (8192, True, 0),
                                          (12032, False, 0), (12288, False, 0), (14336, True, 0),
                                          (2048, False, 2049), (8192, False, 8195)],
                         ids=["regs", "regs-bf16", "smem", "smem-bf16", "smem-max", "two-pass", "two-pass-bf16",
                              "scalar-odd-pitch", "scalar-odd-pitch-long"])
def test_every_form_of_the_activation_conversion(oracle, k, bf16, pitch):
    """The f16 copy of the activations is made by one of four kernels, chosen by row length and alignment: rows kept
    in registers (k <= 4096), in shared memory (k <= 12032), the two-pass form beyond, and the scalar form for a row
    pitch that is not a multiple of four elements. One row carries a single large value, one is all zero."""
    be = backend()
    rng = synth.rng_for(3450 + k + (1 if bf16 else 0) + pitch)
    n, m = 128, 40
    data = synth.gen_packed(synth.Q4_K, synth.GGUF, n * k, rng)
    x = synth.gen_activations(m, k, rng)
    x[3, :] = 0.0
    x[5, k - 1] = 3.0e4
    if bf16:
        x = bf16_round(x)
    ld = pitch or k
    xp = np.zeros((m, ld), dtype=np.float32)
    xp[:, :k] = x
    w = QuantizedWeight(be, data, synth.Q4_K, synth.GGUF, n, k)
    if bf16:
        xb = be.allocate_buffer(m * ld * 2)
        xb.copy_from_host(torch.from_numpy(xp).to(torch.bfloat16).view(torch.int16).numpy())
    else:
        xb = be.allocate_buffer(m * ld * 4); xb.copy_from_host(xp)
    yb = be.allocate_buffer(m * n * 4)
    w.matmul(xb, yb, m, x_dtype=_lib.BF16 if bf16 else _lib.F32, ldx=pitch)
    be.synchronize()
    y = yb.to_numpy(np.float32, m * n).reshape(m, n)
    ref = reference(oracle, synth.Q4_K, synth.GGUF, data, n, k, x)
    for r in range(m):                      # per row: the large value of row 5 must not hide the others
        scale = np.max(np.abs(ref[r]))
        assert np.max(np.abs(y[r] - ref[r])) <= TOL * scale if scale > 0 else np.all(y[r] == 0), r
    xb.free(); yb.free(); w.free()


def test_bf16_activations_and_outputs(oracle):
    be = backend()
    rng = synth.rng_for(3400)
    n, k, m = 384, 1024, 128
    data = synth.gen_packed(synth.Q6_K, synth.GGUF, n * k, rng)
    x = synth.gen_activations(m, k, rng)
    xbf = torch.from_numpy(x).to(torch.bfloat16)
    w = QuantizedWeight(be, data, synth.Q6_K, synth.GGUF, n, k)
    xb = be.allocate_buffer(m * k * 2); xb.copy_from_host(xbf.view(torch.int16).numpy())
    yb = be.allocate_buffer(m * n * 4)
    w.matmul(xb, yb, m, x_dtype=_lib.BF16)
    be.synchronize()
    y = yb.to_numpy(np.float32, m * n).reshape(m, n)
    ref = reference(oracle, synth.Q6_K, synth.GGUF, data, n, k, bf16_round(x))
    assert rel_err(y, ref) <= TOL
    y16 = be.allocate_buffer(m * n * 2)
    w.matmul(xb, y16, m, x_dtype=_lib.BF16, y_dtype=_lib.BF16)
    be.synchronize()
    got = torch.from_numpy(y16.to_numpy(np.int16, m * n)).view(torch.bfloat16).float().numpy().reshape(m, n)
    assert rel_err(got, ref) <= 8e-3
    for b in (xb, yb, y16):
        b.free()
    w.free()


@pytest.mark.parametrize("n,k", [(4096, 4096), (11008, 4096), (4096, 11008)])
@pytest.mark.parametrize("m", [256, 512])
def test_config4_llama7b_q4k_prefill(oracle, n, k, m):
    """Full-size Llama-2-7B-shaped Q4_K projections; 96 sampled weight rows (plus the last) against the oracle."""
    be = backend()
    rng = synth.rng_for(synth.CONFIG_SEEDS[4] + n + m)
    data = synth.gen_packed(synth.Q4_K, synth.GGUF, n * k, rng)
    x = synth.gen_activations(m, k, rng)
    w = QuantizedWeight(be, data, synth.Q4_K, synth.GGUF, n, k)
    y = gpu_matmul(be, w, x, m)
    rows = np.unique(np.concatenate([rng.integers(0, n, size=96), [0, n - 1]]))
    blocks = data.reshape(-1, 144)
    sel = np.concatenate([blocks[r * k // 256:(r + 1) * k // 256] for r in rows]).reshape(-1)
    wsel = oracle.dequantize(synth.Q4_K, synth.GGUF, sel, rows.size * k, threads=8).reshape(rows.size, k)
    ref = oracle.matmul_f32(x, wsel, nk=True, threads=8)
    scale = float(np.max(np.abs(y)))
    assert float(np.max(np.abs(y[:, rows] - ref))) / scale <= TOL
    assert np.all(np.isfinite(y))
    w.free()


@pytest.mark.parametrize("qt,m", [(synth.MXFP4, 64), (synth.MXFP4, 512), (synth.Q6_K, 300), (synth.Q4_0, 512), (synth.MXFP6_E3M2, 512),
                                  (synth.MXFP6_E3M2, 40)],
                         ids=["mxfp4-m64", "mxfp4-m512", "q6k-m300", "q4_0-m512", "e3m2-m512", "e3m2-m40"])
def test_config5_llama70b_shapes_on_the_tensor_memory_kernel(oracle, qt, m):
    """[28672 x 8192] (config 5; Q6_K and Q4_0 on the same shape): MXFP4, Q6_K and Q4_0 take the persistent kernel whose weight
    operand lives in tensor memory; with 448+ tiles on 148 SMs most tiles are split between CTAs. 64 sampled
    weight rows plus the first and last against the oracle."""
    be = backend()
    n, k = synth.LLAMA70B_FFN_SHAPES[0]
    rng = synth.rng_for(synth.CONFIG_SEEDS[5] + qt + m)
    data = synth.gen_packed(qt, synth.GGUF, n * k, rng)
    x = synth.gen_activations(m, k, rng)
    w = QuantizedWeight(be, data, qt, synth.GGUF, n, k)
    y = gpu_matmul(be, w, x, m)
    rows = np.unique(np.concatenate([rng.integers(0, n, size=64), [0, n - 1]]))
    bb = synth.block_bytes(qt, synth.GGUF)
    be_ = synth.block_elems(qt)
    blocks = np.frombuffer(bytes(data), dtype=np.uint8).reshape(-1, bb)
    sel = np.concatenate([blocks[r * k // be_:(r + 1) * k // be_] for r in rows]).reshape(-1)
    wsel = oracle.dequantize(qt, synth.GGUF, sel, rows.size * k, threads=8).reshape(rows.size, k)
    ref = oracle.matmul_f32(x, wsel, nk=True, threads=8)
    scale = float(np.max(np.abs(y)))
    assert float(np.max(np.abs(y[:, rows] - ref))) / scale <= TOL
    assert np.all(np.isfinite(y))
    w.free()


@pytest.mark.parametrize("case", ["mxfp4-huge", "mxfp4-tiny", "mxfp4-nan-free-mix", "q4k-big-d", "q8_0-big-d",
                                  "mxfp6-huge", "mxfp6-tiny", "mxfp6-mixed-exponents", "mxfp6-ordinary",
                                  "e3m2-huge", "e3m2-tiny", "e3m2-mixed-exponents", "e3m2-edge-exponents", "e3m2-ordinary",
                                  "q3k-big-d", "q3k-huge-d", "q2k-huge-d", "rf-q4_0-huge", "rf-q4_0-tiny", "rf-q8_0-huge",
                                  "rf-q4_0-ordinary"])
def test_prefill_with_block_scales_outside_the_f16_range(oracle, case):
    """The tensor-memory prefill kernels form block scales in f16. The upload scans the scale bytes: a tensor whose
    scales (or weights) leave the f16 range takes the next more careful kernel, down to the fp32 decode kernels, so
    that m > 8 gives what m <= 8 gives. Exponent bytes 0x00, 0x40, 0x90 and 0xF0; f16 d of 2000 and 30000. The layouts
    with f32 scales (RF) have their weights scanned on the device the first time a prefill product asks."""
    be = backend()
    n, k, m = 256, 512, 64
    rng = synth.rng_for(8800 + len(case))
    lay = synth.GGUF
    if case.startswith("rf-"):
        # RF blocks start with an f32 scale: 20 bytes (Q4_0) or 36 bytes (Q8_0) per 32 weights
        lay = synth.RF
        qt = synth.Q4_0 if "q4_0" in case else synth.Q8_0
        data = synth.gen_packed(qt, lay, n * k, rng).copy()
        blocks = data.reshape(-1, 20 if qt == synth.Q4_0 else 36)
        if case.endswith("huge"):
            blocks[:, 0:4] = np.frombuffer(np.float32(1.0e6).tobytes(), dtype=np.uint8)   # weights up to 8e6 / 1.3e8
        elif case.endswith("tiny"):
            blocks[:, 0:4] = np.frombuffer(np.float32(1.0e-9).tobytes(), dtype=np.uint8)  # every weight below the smallest f16
    elif case.startswith("q3k"):
        qt = synth.Q3_K
        data = synth.gen_packed(qt, lay, n * k, rng).copy()
        blocks = data.reshape(-1, 110)
        d = 3000.0 if case == "q3k-big-d" else 30000.0     # d * 32 overflows f16 / weights up to 3.8e6 do
        blocks[:, 108:110] = np.frombuffer(np.float16(d).tobytes(), dtype=np.uint8)
    elif case.startswith("q2k"):
        qt = synth.Q2_K
        data = synth.gen_packed(qt, lay, n * k, rng).copy()
        blocks = data.reshape(-1, 84)
        blocks[:, 80:82] = np.frombuffer(np.float16(30000.0).tobytes(), dtype=np.uint8)   # weights up to 1.35e6
    elif case.startswith("mxfp4"):
        qt = synth.MXFP4
        data = synth.gen_packed(qt, synth.GGUF, n * k, rng).copy()
        blocks = data.reshape(-1, 17)
        if case == "mxfp4-huge":
            blocks[:, 0] = 0x90          # 2^17: weights up to 7.9e5, beyond f16
        elif case == "mxfp4-tiny":
            blocks[:, 0] = 0x40          # 2^-63: every weight below the smallest f16
        else:
            blocks[::7, 0] = 0x00        # a few vanishing blocks among ordinary ones
            blocks[3::11, 0] = 0x40
    elif case.startswith("e3m2"):
        # E3M2 reaches the tensor-memory kernel as f16 (value / 4096) times 2^(e-115): exact for e in 107..130
        qt = synth.MXFP6_E3M2
        data = synth.gen_packed(qt, synth.GGUF, n * k, rng).copy()
        blocks = data.reshape(-1, 25)
        if case == "e3m2-huge":
            blocks[:, 0] = 0x90
        elif case == "e3m2-tiny":
            blocks[:, 0] = 0x40
        elif case == "e3m2-mixed-exponents":
            blocks[::5, 0] = 0x00        # vanishing blocks with codes among ordinary ones: not the f16 path
            blocks[1::9, 0] = 107
            blocks[2::9, 0] = 130
        elif case == "e3m2-edge-exponents":
            blocks[0::2, 0] = 107        # both ends of the exact range, every code (subnormals and 28 included)
            blocks[1::2, 0] = 130
            every = np.packbits(((np.arange(64)[:, None] >> np.arange(6)) & 1).astype(np.uint8).ravel(), bitorder="little")
            blocks[0::4, 1:] = every[:24]    # codes 0..31 at either exponent ...
            blocks[1::4, 1:] = every[:24]
            blocks[2::4, 1:] = every[24:]    # ... and 32..63
            blocks[3::4, 1:] = every[24:]
    elif case.startswith("mxfp6"):
        # E2M3 reaches the tensor-memory kernel as int8 codes times 2^(e-130) in f16: exact for e in 106..140
        qt = synth.MXFP6_E2M3
        data = synth.gen_packed(qt, synth.GGUF, n * k, rng).copy()
        blocks = data.reshape(-1, 25)
        if case == "mxfp6-huge":
            blocks[:, 0] = 0x90
        elif case == "mxfp6-tiny":
            blocks[:, 0] = 0x40
        elif case == "mxfp6-mixed-exponents":
            blocks[::5, 0] = 0x00        # vanishing blocks with codes among ordinary ones: not the f16 path
            blocks[1::9, 0] = 106
            blocks[2::9, 0] = 139
    elif case == "q4k-big-d":
        qt = synth.Q4_K
        data = synth.gen_packed(qt, synth.GGUF, n * k, rng).copy()
        blocks = data.reshape(-1, 144)
        blocks[:, 0:2] = np.frombuffer(np.float16(2000.0).tobytes(), dtype=np.uint8)      # d * 63 overflows f16
    else:
        qt = synth.Q8_0
        data = synth.gen_packed(qt, synth.GGUF, n * k, rng).copy()
        blocks = data.reshape(-1, 34)
        blocks[:, 0:2] = np.frombuffer(np.float16(30000.0).tobytes(), dtype=np.uint8)     # weights up to 3.8e6
    x = synth.gen_activations(m, k, rng)
    w = QuantizedWeight(be, data, qt, lay, n, k)
    y = gpu_matmul(be, w, x, m)
    ref = reference(oracle, qt, lay, data, n, k, x)
    assert np.all(np.isfinite(ref)) and np.all(np.isfinite(y))
    assert rel_err(y, ref) <= TOL
    assert np.array_equal(gpu_matmul(be, w, x, m), y)     # the answer of the scan is kept with the tensor
    w.free()


@pytest.mark.parametrize("n,k,m", [(4096, 4096, 512), (1000, 1280, 300), (4096, 11008, 64)],
                         ids=["4096x4096-m512", "ragged", "k11008-m64"])
def test_q3k_prefill_on_q6k_planes(oracle, n, k, m):
    """A GGUF Q3_K tensor with k % 256 == 0 runs the Q6_K tensor-memory kernel on planes that hold the same weights
    re-encoded (q6 = q3 + 28, int8 scale sc6 - 32): sampled weight rows against the oracle, twice (the planes are
    built by the first product and kept)."""
    be = backend()
    rng = synth.rng_for(8900 + m)
    data = synth.gen_packed(synth.Q3_K, synth.GGUF, n * k, rng)
    x = synth.gen_activations(m, k, rng)
    w = QuantizedWeight(be, data, synth.Q3_K, synth.GGUF, n, k)
    y = gpu_matmul(be, w, x, m)
    rows = np.unique(np.concatenate([rng.integers(0, n, size=96), [0, n - 1]]))
    bb = 110 * (k // 256)
    sub = np.concatenate([data[r * bb:(r + 1) * bb] for r in rows])
    ref = reference(oracle, synth.Q3_K, synth.GGUF, sub, len(rows), k, x)
    scale = float(np.max(np.abs(ref)))
    assert float(np.max(np.abs(y[:, rows] - ref))) / scale <= TOL
    assert np.array_equal(gpu_matmul(be, w, x, m), y)
    y1 = gpu_matmul(be, w, x[:1], 1)                       # the decode kernel still reads the tensor's own image
    assert float(np.max(np.abs(y1[0, rows] - ref[0]))) / float(np.max(np.abs(ref[0]))) <= 1e-4
    w.free()
