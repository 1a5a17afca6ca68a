"""Fused dequant + matmul on the GPU against the CPU oracle (dequantise, then cpu_matmul_f32).

Tolerances (max |y - ref| / max |ref|): 1e-4 for the fp32-accumulate decode kernels, 2e-3 for the
bf16 tensor-core kernel; the sequential kernel must match the fp32 oracle bit for bit.
"""
import json
import os

import numpy as np
import pytest

from rocmforge_b200 import _lib, ops, synth

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
TOL_GEMV = 1e-4
TOL_GEMM = 2e-3

from gpu_util import ALL_FMTS, FMT_IDS, QuantizedWeight, backend, gpu_matmul, rel_err  # noqa: E402


@pytest.fixture(scope="module")
def be():
    return backend()


def oracle_y(oracle, qt, lay, data, n, k, x, threads=8):
    w = oracle.dequantize(qt, lay, data, n * k, threads=threads).reshape(n, k)
    return oracle.matmul_f32(x, w, nk=True, threads=threads), w


@pytest.mark.parametrize("qt,lay", ALL_FMTS, ids=FMT_IDS)
@pytest.mark.parametrize("m", [1, 3, 8])
def test_decode_gemv_every_format(be, oracle, qt, lay, m):
    rng = synth.rng_for(2000 + qt * 2 + lay)
    n, k = 300, 1280          # 300 rows: partial last warp; k = 5 super-blocks
    data = synth.gen_packed(qt, lay, n * k, rng)
    x = synth.gen_activations(m, k, rng)
    ref, wf = oracle_y(oracle, qt, lay, data, n, k, x)
    w = QuantizedWeight(be, data, qt, lay, n, k)
    y = gpu_matmul(be, w, x, m)
    assert rel_err(y, ref) <= TOL_GEMV
    # nearer to the exact (fp64) sum than the tolerance as well
    assert rel_err(y, oracle.matmul_f64(x, wf, nk=True)) <= TOL_GEMV
    w.free()


@pytest.mark.parametrize("qt,lay", ALL_FMTS, ids=FMT_IDS)
def test_sequential_kernel_is_bit_exact_in_both_orientations(be, oracle, qt, lay):
    rng = synth.rng_for(2100 + qt * 2 + lay)
    n, k = 24, 256 if synth.block_elems(qt) == 256 else 96
    data = synth.gen_packed(qt, lay, n * k, rng)
    x = synth.gen_activations(2, k, rng)
    flat = oracle.dequantize(qt, lay, data, n * k)
    for orient, wmat, nk in ((_lib.ORIENT_NK, flat.reshape(n, k), True), (_lib.ORIENT_KN, flat.reshape(k, n), False)):
        ref = oracle.matmul_f32(x, wmat, nk=nk)
        w = QuantizedWeight(be, data, qt, lay, n, k, orient=orient)
        y = gpu_matmul(be, w, x, 2, flags=_lib.MM_SEQUENTIAL)
        assert np.array_equal(y.view(np.uint32), ref.view(np.uint32)), orient
        w.free()


def test_reference_fused_matmul_cases(be):
    """The 4x4 inputs of tests/q_dequant_tests.rs through the operator entry points."""
    gold = json.load(open(os.path.join(HERE, "golden", "reference_vectors.json")))
    fn = {synth.Q4_0: ops.matmul_q4_0, synth.Q4_K: ops.matmul_q4_k, synth.Q6_K: ops.matmul_q6_k}
    for case in gold["matmul"]:
        x = np.array(case["input"], dtype=np.float32)
        xb, yb = be.allocate_buffer(16), be.allocate_buffer(16)
        xb.copy_from_host(x)
        fn[case["qtype"]](be, bytes.fromhex(case["data"]), xb, case["n_rows"], case["n_cols"], yb)
        y = yb.to_numpy(np.float32, 4)
        assert np.all(np.abs(y - np.array(case["expect"])) <= case["tol"]), case["name"]
        xb.free(); yb.free()


@pytest.mark.parametrize("lay", [0, 1], ids=["RF", "GGUF"])
def test_config1_q4_0_ffn_up_gemv(be, oracle, lay):
    """Q4_0 [4864, 896] x fp32 [1, 896], seeded; the CPU-runnable configuration, full size."""
    rng = synth.rng_for(synth.CONFIG_SEEDS[1])
    n, k = 4864, 896
    data = synth.gen_packed(synth.Q4_0, lay, n * k, rng)
    x = synth.gen_activations(1, k, rng)
    ref, _ = oracle_y(oracle, synth.Q4_0, lay, data, n, k, x)
    w = QuantizedWeight(be, data, synth.Q4_0, lay, n, k)
    assert rel_err(gpu_matmul(be, w, x, 1), ref) <= TOL_GEMV
    y = w.matmul_host(x)                      # host buffers in and out
    assert rel_err(y, ref) <= TOL_GEMV
    yseq = gpu_matmul(be, w, x, 1, flags=_lib.MM_SEQUENTIAL)
    assert np.array_equal(yseq.view(np.uint32), ref.view(np.uint32))
    w.free()


@pytest.mark.parametrize("n", [896, 4864])
@pytest.mark.parametrize("m", [1, 16, 128, 512])
def test_config2_q8_0_gemm(be, oracle, n, m):
    rng = synth.rng_for(synth.CONFIG_SEEDS[2] + n)
    k = 896
    data = synth.gen_packed(synth.Q8_0, synth.GGUF, n * k, rng)
    x = synth.gen_activations(m, k, rng)
    ref, _ = oracle_y(oracle, synth.Q8_0, synth.GGUF, data, n, k, x)
    w = QuantizedWeight(be, data, synth.Q8_0, synth.GGUF, n, k)
    y = gpu_matmul(be, w, x, m)
    assert rel_err(y, ref) <= (TOL_GEMV if m <= 8 else TOL_GEMM)
    w.free()


@pytest.mark.parametrize("name,qt,n,k", [("attn_q", synth.Q4_K, 896, 896), ("attn_k", synth.Q4_K, 128, 896),
                                         ("ffn_up", synth.Q4_K, 4864, 896), ("ffn_down", synth.Q6_K, 896, 4864)])
@pytest.mark.parametrize("m", [1, 8])
def test_config3_qwen_step_matrices(be, oracle, name, qt, n, k, m):
    """K = 896 is 3.5 super-blocks: odd rows start in the middle of a super-block."""
    rng = synth.rng_for(synth.CONFIG_SEEDS[3] + n + k)
    data = synth.gen_packed(qt, synth.GGUF, n * k, rng)
    x = synth.gen_activations(m, k, rng)
    ref, _ = oracle_y(oracle, qt, synth.GGUF, data, n, k, x)
    w = QuantizedWeight(be, data, qt, synth.GGUF, n, k)
    assert rel_err(gpu_matmul(be, w, x, m), ref) <= TOL_GEMV
    w.free()


def test_shards_concatenate_to_the_whole(be, oracle):
    """Output-feature shards of one tensor give, side by side, the unsharded result: to rounding, not bit for bit,
    because a launch cuts a row's k-range where its work split falls, and the pieces are added in that order."""
    rng = synth.rng_for(77)
    n, k, m = 1024, 2048, 4
    for qt in (synth.Q4_K, synth.MXFP4, synth.MXFP6_E2M3):
        data = synth.gen_packed(qt, synth.GGUF, n * k, rng)
        x = synth.gen_activations(m, k, rng)
        whole = QuantizedWeight(be, data, qt, synth.GGUF, n, k)
        y = gpu_matmul(be, whole, x, m)
        for g in (2, 4, 8):
            parts = []
            for r in range(g):
                w = QuantizedWeight(be, data, qt, synth.GGUF, n, k, shard_rank=r, shard_count=g)
                assert w.n_local == n // g and w.row0 == r * n // g
                parts.append(gpu_matmul(be, w, x, m))
                w.free()
            assert rel_err(np.concatenate(parts, axis=1), y) <= 2e-6
        whole.free()


def test_strided_output_and_bf16_io(be, oracle):
    rng = synth.rng_for(78)
    n, k, m = 256, 512, 4
    data = synth.gen_packed(synth.Q4_K, synth.GGUF, n * k, rng)
    x = synth.gen_activations(m, k, rng)
    ref, _ = oracle_y(oracle, synth.Q4_K, synth.GGUF, data, n, k, x)
    w = QuantizedWeight(be, data, synth.Q4_K, synth.GGUF, n, k)
    xb = be.allocate_buffer(x.nbytes); xb.copy_from_host(x)
    ld = 3 * n
    yb = be.allocate_buffer(m * ld * 4); yb.fill(0)
    w.matmul(xb, yb.ptr + n * 4, m, ldy=ld)          # write into the middle column block of a wider matrix
    be.synchronize()
    full = yb.to_numpy(np.float32, m * ld).reshape(m, ld)
    assert rel_err(full[:, n:2 * n], ref) <= TOL_GEMV
    assert np.all(full[:, :n] == 0) and np.all(full[:, 2 * n:] == 0)
    # bf16 activations and outputs
    import torch
    xbf = torch.from_numpy(x).to(torch.bfloat16)
    xb16 = be.allocate_buffer(m * k * 2); xb16.copy_from_host(xbf.view(torch.int16).numpy())
    yb16 = be.allocate_buffer(m * n * 2)
    w.matmul(xb16, yb16, m, x_dtype=_lib.BF16, y_dtype=_lib.BF16)
    be.synchronize()
    y16 = torch.from_numpy(yb16.to_numpy(np.int16, m * n)).view(torch.bfloat16).float().numpy().reshape(m, n)
    ref16, _ = oracle_y(oracle, synth.Q4_K, synth.GGUF, data, n, k, xbf.float().numpy())
    assert rel_err(y16, ref16) <= 8e-3           # one bf16 rounding of the output
    for b in (xb, yb, xb16, yb16):
        b.free()
    w.free()


def test_linearity_at_full_size(be):
    """[28672, 8192] MXFP4 (124.8 MB packed): y(x1 + x2) = y(x1) + y(x2) within fp32 rounding; rows are independent."""
    rng = synth.rng_for(synth.CONFIG_SEEDS[5])
    n, k = 28672, 8192
    data = synth.gen_packed(synth.MXFP4, synth.GGUF, n * k, rng)
    w = QuantizedWeight(be, data, synth.MXFP4, synth.GGUF, n, k)
    x = synth.gen_activations(2, k, rng)
    y12 = gpu_matmul(be, w, x, 2)
    ysum = gpu_matmul(be, w, (x[0] + x[1]).reshape(1, k), 1)
    assert rel_err(ysum, y12[0] + y12[1]) <= TOL_GEMV
    y1 = gpu_matmul(be, w, x[:1], 1)
    assert rel_err(y1, y12[:1]) <= 1e-6
    w.free()


def test_matmul_argument_errors(be):
    rng = synth.rng_for(3)
    data = synth.gen_packed(synth.Q4_0, synth.RF, 64 * 64, rng)
    w = QuantizedWeight(be, data, synth.Q4_0, synth.RF, 64, 64)
    buf = be.allocate_buffer(64 * 8 * 4)
    for bad in (dict(m=-1), dict(m=1, x_dtype=7), dict(m=1, ldx=8), dict(m=1, ldy=3)):
        with pytest.raises(_lib.B200QError) as e:
            w.matmul(buf, buf, **bad)
        assert e.value.status == _lib.ERR_INVALID
    with pytest.raises(_lib.B200QError):
        _lib.check(be.lib.b200q_matmul(be.ctx, None, buf.ptr, 0, buf.ptr, 0, 1, 0))
    with pytest.raises(_lib.B200QError) as e:
        ops.matmul_q4_0(be, data[:-1], buf, 64, 64, buf)
    assert e.value.status == _lib.ERR_INVALID
    w.matmul(buf, buf, 0)          # m = 0 is a no-op
    buf.free(); w.free()
