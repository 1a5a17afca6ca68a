"""Projection-site operators on the GPU against the oracle: SwiGLU activation, row bias, the SwiGLU MLP block
on packed weights (decode and prefill row counts) and the shared-input projection group (Q, K, V).

Tolerances: activation 2e-6 relative (device expf vs libm expf), bias bit-exact, MLP 1e-4 (m <= 8) and 2e-3
(m > 8) of the output maximum, the tolerances of the products it is built from."""
import numpy as np
import pytest

from rocmforge_b200 import _lib, projections, synth
from rocmforge_b200._lib import B200QError
from rocmforge_b200.backend import QuantizedWeight

from gpu_util import backend

pytestmark = pytest.mark.gpu


def dev(be, a):
    b = be.allocate_buffer(a.nbytes)
    b.copy_from_host(a)
    return b


@pytest.mark.parametrize("shape", [(1, 4864), (7, 1003), (512, 11008)])
def test_swiglu_kernel(oracle, shape):
    be = backend()
    rng = synth.rng_for(900 + shape[0])
    g = rng.standard_normal(shape, dtype=np.float32)
    u = rng.standard_normal(shape, dtype=np.float32) * 3
    u.reshape(-1)[:4] = [0.0, -100.0, 100.0, -20.0]
    gb, ub = dev(be, g), dev(be, u)
    ob = be.allocate_buffer(g.nbytes)
    projections.swiglu_gpu_kernel(be, gb, ub, ob, shape[0], shape[1])
    be.synchronize()
    got = ob.to_numpy(np.float32, g.size).reshape(shape)
    ref = oracle.swiglu(g, u)
    assert np.allclose(got, ref, rtol=2e-6, atol=1e-30)
    projections.swiglu_gpu_kernel(be, gb, ub, gb, shape[0], shape[1])      # in place over gate
    be.synchronize()
    assert np.array_equal(gb.to_numpy(np.float32, g.size).reshape(shape), got)
    for b in (gb, ub, ob):
        b.free()


def test_add_row_bias_bit_exact_and_shape_errors(oracle):
    be = backend()
    rng = synth.rng_for(901)
    y = rng.standard_normal((5, 1001), dtype=np.float32)
    b = rng.standard_normal(1001, dtype=np.float32)
    yb, bb = dev(be, y), dev(be, b)
    projections.add_row_bias(be, yb, (5, 1001), bb, (1001,))
    be.synchronize()
    got = yb.to_numpy(np.float32, y.size).reshape(y.shape)
    assert np.array_equal(got.view(np.uint32), oracle.add_row_bias(y, b).view(np.uint32))
    projections.add_row_bias(be, yb, (0, 1001), bb, (1, 1001))               # empty tensor: a no-op
    with pytest.raises(ValueError, match="Tensor for row bias must be 2D"):
        projections.add_row_bias(be, yb, (5005,), bb, (1001,))
    with pytest.raises(ValueError, match="incompatible with tensor shape"):
        projections.add_row_bias(be, yb, (5, 1001), bb, (1000,))
    yb.free(); bb.free()


@pytest.mark.parametrize("m,tol", [(1, 1e-4), (4, 1e-4), (40, 2e-3), (300, 2e-3)])
def test_mlp_swiglu_qwen2_shaped(oracle, m, tol):
    """Qwen2-0.5B-shaped block: gate/up Q4_K [4864, 896], down Q6_K [896, 4864] (a Q4_K_M file's mix)."""
    be = backend()
    hidden, n_ff = 896, 4864
    rng = synth.rng_for(910 + m)
    gate = synth.gen_packed(synth.Q4_K, synth.GGUF, n_ff * hidden, rng)
    up = synth.gen_packed(synth.Q4_K, synth.GGUF, n_ff * hidden, rng)
    down = synth.gen_packed(synth.Q6_K, synth.GGUF, hidden * n_ff, rng)
    x = synth.gen_activations(m, hidden, rng)
    wg = QuantizedWeight(be, gate, synth.Q4_K, synth.GGUF, n_ff, hidden)
    wu = QuantizedWeight(be, up, synth.Q4_K, synth.GGUF, n_ff, hidden)
    wd = QuantizedWeight(be, down, synth.Q6_K, synth.GGUF, hidden, n_ff)
    xb = dev(be, x)
    ob = be.allocate_buffer(m * hidden * 4)
    plan = projections.MlpSwiglu(be, xb, wg, wu, wd, ob, m)
    plan.run(); plan.run()                                             # a plan is reusable
    be.synchronize()
    got = ob.to_numpy(np.float32, m * hidden).reshape(m, hidden)
    ref, _ = oracle.mlp_swiglu((synth.Q4_K, synth.Q4_K, synth.Q6_K), synth.GGUF, gate, up, down, x, hidden, n_ff)
    assert np.max(np.abs(got - ref)) <= tol * np.max(np.abs(ref))
    plan.free()
    ob.fill(0)
    projections.mlp_swiglu(be, xb, wg, wu, wd, ob, m)                  # the one-call form
    assert np.array_equal(ob.to_numpy(np.float32, m * hidden).reshape(m, hidden), got)
    for w in (wg, wu, wd):
        w.free()
    xb.free(); ob.free()


def test_mlp_swiglu_generic_formats_and_shape_errors(oracle):
    be = backend()
    hidden, n_ff, m = 256, 512, 3
    rng = synth.rng_for(920)
    gate = synth.gen_packed(synth.Q8_0, synth.RF, n_ff * hidden, rng)
    up = synth.gen_packed(synth.Q4_0, synth.RF, n_ff * hidden, rng)
    down = synth.gen_packed(synth.Q5_K, synth.GGUF, hidden * n_ff, rng)
    x = synth.gen_activations(m, hidden, rng)
    wg = QuantizedWeight(be, gate, synth.Q8_0, synth.RF, n_ff, hidden)
    wu = QuantizedWeight(be, up, synth.Q4_0, synth.RF, n_ff, hidden)
    wd = QuantizedWeight(be, down, synth.Q5_K, synth.GGUF, hidden, n_ff)
    xb = dev(be, x)
    ob = be.allocate_buffer(m * hidden * 4)
    projections.mlp_swiglu(be, xb, wg, wu, wd, ob, m)
    got = ob.to_numpy(np.float32, m * hidden).reshape(m, hidden)
    wgf = oracle.dequantize(synth.Q8_0, synth.RF, gate, n_ff * hidden).reshape(n_ff, hidden)
    wuf = oracle.dequantize(synth.Q4_0, synth.RF, up, n_ff * hidden).reshape(n_ff, hidden)
    wdf = oracle.dequantize(synth.Q5_K, synth.GGUF, down, hidden * n_ff).reshape(hidden, n_ff)
    act = oracle.swiglu(oracle.matmul_f32(x, wgf, nk=True), oracle.matmul_f32(x, wuf, nk=True))
    ref = oracle.matmul_f32(act, wdf, nk=True)
    assert np.max(np.abs(got - ref)) <= 1e-4 * np.max(np.abs(ref))
    with pytest.raises(B200QError, match="down_weight must be 2D"):
        projections.MlpSwiglu(be, xb, wg, wu, wg, ob, m)               # "down" stored as [n_ff, hidden]
    sq = synth.gen_packed(synth.Q8_0, synth.RF, hidden * hidden, rng)
    bad = QuantizedWeight(be, sq, synth.Q8_0, synth.RF, hidden, hidden)    # [hidden, hidden]: inner size is not n_ff
    with pytest.raises(B200QError, match="All intermediate dimensions must match"):
        projections.MlpSwiglu(be, xb, wg, wu, bad, ob, m)
    for w in (wg, wu, wd, bad):
        w.free()
    xb.free(); ob.free()


def test_qkv_projections_share_one_launch(oracle):
    """Q [896, 896], K and V [128, 896] of one input: one grouped launch, every output as its own product."""
    be = backend()
    hidden = 896
    rng = synth.rng_for(930)
    shapes = [896, 128, 128]
    packed = [synth.gen_packed(synth.Q4_K, synth.GGUF, n * hidden, rng) for n in shapes]
    ws = [QuantizedWeight(be, p, synth.Q4_K, synth.GGUF, n, hidden) for p, n in zip(packed, shapes)]
    x = synth.gen_activations(1, hidden, rng)
    xb = dev(be, x)
    outs = [be.allocate_buffer(n * 4) for n in shapes]
    grp = projections.SharedInputProjections(be, xb, ws, outs, seq_len=1)
    assert grp.launches == 1
    grp.run()
    be.synchronize()
    for p, n, o in zip(packed, shapes, outs):
        wf = oracle.dequantize(synth.Q4_K, synth.GGUF, p, n * hidden).reshape(n, hidden)
        ref = oracle.matmul_f32(x, wf, nk=True)
        got = o.to_numpy(np.float32, n).reshape(1, n)
        assert np.max(np.abs(got - ref)) <= 1e-4 * np.max(np.abs(ref))
    grp.free()
    for w in ws:
        w.free()
    for o in outs:
        o.free()
    xb.free()
