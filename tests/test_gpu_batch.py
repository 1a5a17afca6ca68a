"""The batch front end (one grouped launch for many products) against the CPU oracle."""
import ctypes

import numpy as np
import pytest

from rocmforge_b200 import _lib, synth

pytestmark = pytest.mark.gpu
from gpu_util import QuantizedWeight, backend, rel_err  # noqa: E402


def run_batch(be, ops, datas, xs, m):
    W = [QuantizedWeight(be, d, qt, synth.GGUF, n, k) for (qt, n, k), d in zip(ops, datas)]
    X, Y = [], []
    for (qt, n, k), x in zip(ops, xs):
        xb = be.allocate_buffer(x.nbytes); xb.copy_from_host(x); X.append(xb)
        yb = be.allocate_buffer(m * n * 4 + 64); yb.fill(0xCD); Y.append(yb)
    cnt = len(W)
    aw = (ctypes.c_void_p * cnt)(*[w.handle.value for w in W])
    ax = (ctypes.c_void_p * cnt)(*[x.ptr for x in X])
    ay = (ctypes.c_void_p * cnt)(*[y.ptr for y in Y])
    b = ctypes.c_void_p()
    _lib.check(be.lib.b200q_batch_create(be.ctx, cnt, aw, ax, ay, m, ctypes.byref(b)))
    ms = ctypes.c_float()
    _lib.check(be.lib.b200q_batch_run(be.ctx, b, ctypes.byref(ms)))
    be.synchronize()
    outs = []
    for (qt, n, k), yb in zip(ops, Y):
        raw = yb.to_numpy(np.uint32, m * n + 16)
        assert np.all(raw[m * n:] == 0xCDCDCDCD)
        outs.append(raw[:m * n].view(np.float32).reshape(m, n).copy())
    nb = be.lib.b200q_batch_weight_bytes(b)
    nl = be.lib.b200q_batch_launches(b)
    _lib.check(be.lib.b200q_batch_free(b))
    for t in W + X + Y:
        t.free()
    return outs, ms.value, nb, nl


@pytest.mark.parametrize("m", [1, 2, 5, 8])
def test_grouped_launch_of_mixed_products(oracle, m):
    be = backend()
    rng = synth.rng_for(500 + m)
    ops = [(synth.Q4_K, 896, 896), (synth.Q4_K, 128, 896), (synth.Q4_K, 100, 896), (synth.Q6_K, 896, 4864),
           (synth.Q4_K, 4864, 896), (synth.Q6_K, 1000, 896), (synth.Q4_K, 48, 4096), (synth.Q6_K, 17, 128),
           (synth.Q4_K, 1, 128)]
    datas = [synth.gen_packed(qt, synth.GGUF, n * k, rng) for qt, n, k in ops]
    xs = [synth.gen_activations(m, k, rng) for _, _, k in ops]
    outs, ms, nb, nl = run_batch(be, ops, datas, xs, m)
    assert nb == sum(d.size for d in datas) and nl == 1 and ms > 0
    for (qt, n, k), d, x, y in zip(ops, datas, xs, outs):
        w = oracle.dequantize(qt, synth.GGUF, d, n * k, threads=8).reshape(n, k)
        ref = oracle.matmul_f32(x, w, nk=True, threads=8)
        assert rel_err(y, ref) <= 1e-4, (qt, n, k, rel_err(y, ref))
        assert rel_err(y, oracle.matmul_f64(x, w, nk=True)) <= 1e-4


def test_batch_of_other_formats_falls_back_to_per_product_launches(oracle):
    be = backend()
    rng = synth.rng_for(600)
    ops = [(synth.MXFP6_E3M2, 256, 512), (synth.Q2_K, 300, 1024), (synth.Q4_K, 128, 256)]
    datas = [synth.gen_packed(qt, synth.GGUF, n * k, rng) for qt, n, k in ops]
    xs = [synth.gen_activations(2, k, rng) for _, _, k in ops]
    outs, ms, nb, nl = run_batch(be, ops, datas, xs, 2)
    assert nl == 3
    for (qt, n, k), d, x, y in zip(ops, datas, xs, outs):
        w = oracle.dequantize(qt, synth.GGUF, d, n * k).reshape(n, k)
        assert rel_err(y, oracle.matmul_f32(x, w, nk=True)) <= 1e-4


@pytest.mark.parametrize("m", [1, 3, 8])
def test_q4_0_q8_0_and_q5_k_gguf_ride_the_grouped_tensor_core_launch(oracle, m):
    """GGUF Q4_0 (config 1's format: [4864, 896]), Q8_0 and Q5_K share the grouped decode launch with the K-quants and MXFP4;
    odd row counts exercise the clamped last tile."""
    be = backend()
    rng = synth.rng_for(601 + m)
    ops = [(synth.Q4_0, 4864, 896), (synth.Q8_0, 4864, 896), (synth.Q4_0, 300, 1024), (synth.Q4_K, 128, 256), (synth.Q4_0, 17, 128),
           (synth.Q8_0, 301, 1152), (synth.Q8_0, 9, 128), (synth.Q5_K, 4864, 1024), (synth.Q5_K, 33, 256), (synth.Q5_K, 300, 2304),
           # Q3_K rides the launch re-encoded in Q6_K's item form (an exact integer re-encoding made at upload)
           (synth.Q3_K, 4864, 1024), (synth.Q3_K, 33, 256), (synth.Q3_K, 300, 2304)]
    datas = [synth.gen_packed(qt, synth.GGUF, n * k, rng) for qt, n, k in ops]
    xs = [synth.gen_activations(m, k, rng) for _, _, k in ops]
    outs, ms, nb, nl = run_batch(be, ops, datas, xs, m)
    assert nl == 1
    for (qt, n, k), d, x, y in zip(ops, datas, xs, outs):
        w = oracle.dequantize(qt, synth.GGUF, d, n * k).reshape(n, k)
        assert rel_err(y, oracle.matmul_f32(x, w, nk=True)) <= 1e-4, (qt, n, k)
        assert rel_err(y, oracle.matmul_f64(x, w, nk=True)) <= 1e-4, (qt, n, k)


def test_large_activation_magnitudes_and_zeros(oracle):
    """The f16 hi/lo split is normalised per group: huge, tiny and all-zero activation groups stay accurate."""
    be = backend()
    rng = synth.rng_for(601)
    n, k = 64, 1024
    d = synth.gen_packed(synth.Q4_K, synth.GGUF, n * k, rng)
    x = synth.gen_activations(3, k, rng)
    x[0] *= 1e6
    x[1] *= 1e-12
    x[2, :512] = 0.0
    x[2, 512:544] *= 3e4
    outs, _, _, _ = run_batch(be, [(synth.Q4_K, n, k)], [d], [x], 3)
    w = oracle.dequantize(synth.Q4_K, synth.GGUF, d, n * k).reshape(n, k)
    ref = oracle.matmul_f64(x, w, nk=True)
    for i in range(3):
        assert rel_err(outs[0][i], ref[i]) <= 1e-4, i


def test_batch_argument_errors():
    be = backend()
    b = ctypes.c_void_p()
    assert be.lib.b200q_batch_create(be.ctx, 1, None, None, None, 1, ctypes.byref(b)) == _lib.ERR_INVALID
    assert be.lib.b200q_batch_create(be.ctx, 0, None, None, None, 9, ctypes.byref(b)) == _lib.ERR_INVALID
    assert be.lib.b200q_batch_create(be.ctx, 0, None, None, None, 1, ctypes.byref(b)) == 0
    assert be.lib.b200q_batch_run(be.ctx, b, None) == 0
    assert be.lib.b200q_batch_free(b) == 0
    assert be.lib.b200q_batch_run(be.ctx, None, None) == _lib.ERR_INVALID


def test_run_host_pinned_outputs_equal_pageable_outputs():
    """b200q_batch_run_host: with page-locked, device-addressable outputs the grouped kernel stores straight into
    host memory; the bits must equal the device-buffer + copy path taken for pageable memory."""
    torch = pytest.importorskip("torch")
    from rocmforge_b200.batch import DeviceBatch
    be = backend()
    m = 2
    rng = synth.rng_for(8101)
    shapes = [(synth.Q4_K, 896, 896), (synth.Q4_K, 128, 896), (synth.Q6_K, 896, 4864), (synth.MXFP4, 512, 1024)]
    ws = [QuantizedWeight(be, synth.gen_packed(q, synth.GGUF, n * k, rng), q, synth.GGUF, n, k) for q, n, k in shapes]
    batch = DeviceBatch(be, ws, m)
    assert batch.launches == 1
    xtot, ytot = sum(batch.xsizes), sum(batch.ysizes)
    hx = torch.from_numpy(rng.standard_normal(xtot, dtype=np.float32)).pin_memory()
    hy_pinned = torch.full((ytot + 16,), float("nan"), dtype=torch.float32).pin_memory()
    hy_paged = np.full(ytot, np.nan, dtype=np.float32)
    batch.run_host(hx.data_ptr(), hy_paged.ctypes.data)
    batch.run_host(hx.data_ptr(), hy_pinned.data_ptr())
    batch.run_host(hx.data_ptr(), hy_pinned.data_ptr())          # the host-output plan is cached and reused
    got = hy_pinned.numpy()
    assert np.all(np.isfinite(hy_paged))
    assert np.array_equal(got[:ytot].view(np.uint32), hy_paged.view(np.uint32))
    assert np.all(np.isnan(got[ytot:]))                          # nothing written past the outputs
    batch.free()
    for w in ws:
        w.free()
