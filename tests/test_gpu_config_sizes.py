"""Full-size configurations against the CPU oracle: config 5 (MXFP4 / MXFP6, both orientations of the Llama-70B FFN
shape), the whole 169-product decode step of config 3, and the row-sharded product against the unsharded one.

Weight rows are independent, so at sizes the oracle cannot finish in seconds a sample of weight rows (plus the
first and last) is dequantised and multiplied on the CPU and compared with the same columns of the GPU result.
Tolerances (max |y - ref| / max |y|): 1e-4 for the decode kernels (m <= 8), 2e-3 for the prefill kernels.
"""
import ctypes

import numpy as np
import pytest

from rocmforge_b200 import _lib, synth

pytestmark = pytest.mark.gpu
from gpu_util import QuantizedWeight, backend, gpu_matmul, rel_err  # noqa: E402

TOL_DECODE = 1e-4
TOL_PREFILL = 2e-3


def sampled_reference(oracle, qt, data, n, k, x, rows):
    """x . W[rows]^T on the CPU. A row of k weights may start inside a block (k = 896 is 3.5 super-blocks): the blocks
    that cover the row are dequantised and the row cut out of them."""
    bb, be_ = synth.block_bytes(qt, synth.GGUF), synth.block_elems(qt)
    blocks = np.frombuffer(bytes(data), dtype=np.uint8).reshape(-1, bb)
    wsel = np.empty((rows.size, k), dtype=np.float32)
    for i, r in enumerate(rows):
        e0 = int(r) * k
        b0, b1 = e0 // be_, -(-(e0 + k) // be_)
        part = oracle.dequantize(qt, synth.GGUF, blocks[b0:b1].reshape(-1), (b1 - b0) * be_)
        wsel[i] = part[e0 - b0 * be_: e0 - b0 * be_ + k]
    return oracle.matmul_f32(x, wsel, nk=True, threads=8)


@pytest.mark.parametrize("shape", synth.LLAMA70B_FFN_SHAPES, ids=["28672x8192", "8192x28672"])
@pytest.mark.parametrize("qt", [synth.MXFP4, synth.MXFP6_E2M3], ids=["mxfp4", "mxfp6"])
def test_config5_full_size_against_the_oracle(oracle, qt, shape):
    """MXFP4 and MXFP6 at [28672, 8192] and [8192, 28672], m = 1, 64 and 512, one upload per tensor."""
    be = backend()
    n, k = shape
    rng = synth.rng_for(synth.CONFIG_SEEDS[5] + 100 * qt + n)
    data = synth.gen_packed(qt, synth.GGUF, n * k, rng)
    w = QuantizedWeight(be, data, qt, synth.GGUF, n, k)
    rows = np.unique(np.concatenate([rng.integers(0, n, size=48), [0, n - 1]]))
    for m in (1, 64, 512):
        x = synth.gen_activations(m, k, rng)
        y = gpu_matmul(be, w, x, m)
        ref = sampled_reference(oracle, qt, data, n, k, x, rows)
        scale = float(np.max(np.abs(y)))
        err = float(np.max(np.abs(y[:, rows] - ref))) / scale
        assert err <= (TOL_DECODE if m <= 8 else TOL_PREFILL), (m, err)
        assert np.all(np.isfinite(y))
    w.free()


@pytest.mark.parametrize("m", [1, 8])
def test_whole_decode_step_against_the_oracle(oracle, m):
    """The 169 products of the benchmark's step (24 Qwen2-0.5B-shaped layers + the 151936-row lm_head) as ONE grouped
    launch through b200q_batch_run, every product compared with the oracle (the lm_head on sampled rows)."""
    be = backend()
    ops = synth.qwen2_0p5b_step()
    rng = synth.rng_for(synth.CONFIG_SEEDS[3] + m)
    datas = [synth.gen_packed(qt, synth.GGUF, n * k, rng) for _, qt, n, k in ops]
    xs = [synth.gen_activations(m, k, rng) for _, _, _, k in ops]
    W = [QuantizedWeight(be, d, qt, synth.GGUF, n, k) for (_, qt, n, k), d in zip(ops, datas)]
    assert sum(w.packed_bytes for w in W) == 339_916_416
    X, Y = [], []
    for (_, _, n, k), x in zip(ops, xs):
        xb = be.allocate_buffer(x.nbytes); xb.copy_from_host(x); X.append(xb)
        yb = be.allocate_buffer(m * n * 4 + 64); yb.fill(0xCD); Y.append(yb)
    cnt = len(W)
    aw = (ctypes.c_void_p * cnt)(*[w.handle.value for w in W])
    ax = (ctypes.c_void_p * cnt)(*[x.ptr for x in X])
    ay = (ctypes.c_void_p * cnt)(*[y.ptr for y in Y])
    b = ctypes.c_void_p()
    _lib.check(be.lib.b200q_batch_create(be.ctx, cnt, aw, ax, ay, m, ctypes.byref(b)))
    assert be.lib.b200q_batch_launches(b) == 1
    for _ in range(2):   # the second run must not depend on anything the first left behind
        _lib.check(be.lib.b200q_batch_run(be.ctx, b, None))
    be.synchronize()
    worst = 0.0
    for (name, qt, n, k), d, x, yb in zip(ops, datas, xs, Y):
        raw = yb.to_numpy(np.uint32, m * n + 16)
        assert np.all(raw[m * n:] == 0xCDCDCDCD), name
        y = raw[:m * n].view(np.float32).reshape(m, n)
        if n > 8192:
            rows = np.unique(np.concatenate([rng.integers(0, n, size=160), [0, 15, 16, n - 17, n - 16, n - 1]]))
            ref = sampled_reference(oracle, qt, d, n, k, x, rows)
            err = float(np.max(np.abs(y[:, rows] - ref))) / float(np.max(np.abs(y)))
        else:
            wf = oracle.dequantize(qt, synth.GGUF, d, n * k, threads=8).reshape(n, k)
            err = rel_err(y, oracle.matmul_f32(x, wf, nk=True, threads=8))
        worst = max(worst, err)
        assert err <= TOL_DECODE, (name, err)
    _lib.check(be.lib.b200q_batch_free(b))
    for t in W + X + Y:
        t.free()
    assert worst > 0.0


@pytest.mark.parametrize("qt", [synth.Q4_K, synth.MXFP4], ids=["q4_k", "mxfp4"])
def test_sharded_result_equals_the_unsharded_one_to_tolerance(oracle, qt):
    """[28672, 8192] split by output feature into 2, 4 and 8 shards on one GPU, m = 1 and 512. A shard sums a row's
    k-range in other pieces than the whole tensor does (the pieces follow the launch's work split), so the two
    agree to the tolerance of the path, not bit for bit."""
    be = backend()
    n, k = synth.LLAMA70B_FFN_SHAPES[0]
    rng = synth.rng_for(synth.CONFIG_SEEDS[5] + 7 * qt)
    data = synth.gen_packed(qt, synth.GGUF, n * k, rng)
    whole = QuantizedWeight(be, data, qt, synth.GGUF, n, k)
    xs = {m: synth.gen_activations(m, k, rng) for m in (1, 512)}
    full = {m: gpu_matmul(be, whole, xs[m], m) for m in (1, 512)}
    whole.free()
    for g in (2, 4, 8):
        shards = [QuantizedWeight(be, data, qt, synth.GGUF, n, k, shard_rank=r, shard_count=g) for r in range(g)]
        for m in (1, 512):
            got = np.concatenate([gpu_matmul(be, s, xs[m], m) for s in shards], axis=1)
            err = rel_err(got, full[m])
            assert err <= (2e-5 if m == 1 else TOL_PREFILL), (g, m, err)
        for s in shards:
            s.free()
