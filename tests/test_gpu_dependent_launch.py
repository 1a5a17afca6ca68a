"""Chains of dependent products on one stream: every kernel is launched with programmatic stream serialisation
and starts streaming its weights before the kernel ahead of it has finished, so a misplaced dependency wait
would read activations that are not written yet. The chains are run many times; every run must give the same
bits, and the result must match the oracle's chain."""
import numpy as np
import pytest

from rocmforge_b200 import synth
from rocmforge_b200.backend import QuantizedWeight

from gpu_util import backend

pytestmark = pytest.mark.gpu


def test_decode_chain_of_six_products(oracle):
    be = backend()
    n = 1024
    rng = synth.rng_for(7001)
    qts = [synth.Q4_K, synth.Q6_K, synth.MXFP4, synth.Q4_K, synth.Q6_K, synth.Q4_K]
    packed = [synth.gen_packed(q, synth.GGUF, n * n, rng) for q in qts]
    ws = [QuantizedWeight(be, p, q, synth.GGUF, n, n) for p, q in zip(packed, qts)]
    x = synth.gen_activations(1, n, rng)
    bufs = [be.allocate_buffer(n * 4) for _ in range(7)]
    bufs[0].copy_from_host(x)
    first = None
    for rep in range(25):
        for i, w in enumerate(ws):
            w.matmul(bufs[i], bufs[i + 1], 1)
        be.synchronize()
        got = bufs[6].to_numpy(np.float32, n)
        if first is None:
            first = got.copy()
        assert np.array_equal(got.view(np.uint32), first.view(np.uint32)), f"run {rep} differs from run 0"
    # the oracle's dequantised tensors, chained in float64
    r = x.astype(np.float64)
    for p, q in zip(packed, qts):
        wf = oracle.dequantize(q, synth.GGUF, p, n * n).reshape(n, n).astype(np.float64)
        r = r @ wf.T
    assert np.all(np.isfinite(first))
    assert np.max(np.abs(first - r[0])) <= 6e-4 * np.max(np.abs(r))     # six products at 1e-4 each
    for w in ws:
        w.free()
    for b in bufs:
        b.free()


def test_prefill_then_decode_chain(oracle):
    """A prefill product (activation conversion kernel + tensor-core kernel) followed at once by a decode product
    that consumes one row of its output."""
    be = backend()
    n, k, m = 1024, 1024, 64
    rng = synth.rng_for(7002)
    p1 = synth.gen_packed(synth.Q4_K, synth.GGUF, n * k, rng)
    p2 = synth.gen_packed(synth.Q6_K, synth.GGUF, n * n, rng)
    w1 = QuantizedWeight(be, p1, synth.Q4_K, synth.GGUF, n, k)
    w2 = QuantizedWeight(be, p2, synth.Q6_K, synth.GGUF, n, n)
    x = synth.gen_activations(m, k, rng)
    xb = be.allocate_buffer(x.nbytes); xb.copy_from_host(x)
    y1 = be.allocate_buffer(m * n * 4)
    y2 = be.allocate_buffer(n * 4)
    first = None
    for rep in range(15):
        w1.matmul(xb, y1, m)
        w2.matmul(y1, y2, 1)              # row 0 of y1
        be.synchronize()
        got = y2.to_numpy(np.float32, n)
        if first is None:
            first = got.copy()
        assert np.array_equal(got.view(np.uint32), first.view(np.uint32)), f"run {rep} differs from run 0"
    w1f = oracle.dequantize(synth.Q4_K, synth.GGUF, p1, n * k).reshape(n, k).astype(np.float64)
    w2f = oracle.dequantize(synth.Q6_K, synth.GGUF, p2, n * n).reshape(n, n).astype(np.float64)
    r = (x[0].astype(np.float64) @ w1f.T) @ w2f.T
    assert np.max(np.abs(first - r)) <= 2.2e-3 * np.max(np.abs(r))
    for o in (w1, w2, xb, y1, y2):
        o.free()
