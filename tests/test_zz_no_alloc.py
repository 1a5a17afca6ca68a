"""The entry point that allocates nothing (b200q_matmul_noalloc) against the ordinary one.

Some callers of this library cannot allocate device memory at the moment they need a product: their own
memory pool already owns the rest of HBM, or they cannot take the device-wide synchronisation a cudaMalloc
implies. For them the library keeps the scratch of the prefill kernel in a fixed array of its own image.
This file is collected last on purpose: if it fails, every other test has already run. It must also pass
when it is the only test in a fresh process.
"""
import ctypes

import numpy as np
import pytest

from rocmforge_b200 import _lib, synth

pytestmark = pytest.mark.gpu
TOL = 2e-3    # the tolerance of the prefill tests; both entry points run the same kernel


def _run(be, w, x, m, noalloc):
    from gpu_util import rel_err  # noqa: F401
    xb = be.allocate_buffer(x.nbytes)
    xb.copy_from_host(x)
    yb = be.allocate_buffer(m * w.n_local * 4 + 64)
    yb.fill(0xCD)
    if noalloc:
        _lib.check(be.lib.b200q_matmul_noalloc(be.ctx, w.handle, xb.ptr, yb.ptr, m))
    else:
        _lib.check(be.lib.b200q_matmul(be.ctx, w.handle, xb.ptr, _lib.F32, yb.ptr, _lib.F32, m, 0))
    be.synchronize()
    raw = yb.to_numpy(np.uint32, m * w.n_local + 16)
    assert np.all(raw[m * w.n_local:] == 0xCDCDCDCD)
    xb.free(); yb.free()
    return raw[:m * w.n_local].view(np.float32).reshape(m, w.n_local).copy()


def test_noalloc_matches_the_ordinary_entry_point_twice_in_a_row(oracle):
    from gpu_util import QuantizedWeight, backend, rel_err
    be = backend()
    rng = synth.rng_for(9100)
    n, k = 384, 1024
    data = synth.gen_packed(synth.Q4_K, synth.GGUF, n * k, rng)
    w = QuantizedWeight(be, data, synth.Q4_K, synth.GGUF, n, k)
    wf = oracle.dequantize(synth.Q4_K, synth.GGUF, data, n * k).reshape(n, k)
    # second call is smaller and uses other values: leftovers of the first call in the shared scratch must not show
    for m, seed in ((200, 1), (48, 2)):
        x = synth.gen_activations(m, k, synth.rng_for(seed))
        y_new = _run(be, w, x, m, noalloc=True)
        y_old = _run(be, w, x, m, noalloc=False)
        assert rel_err(y_new, y_old) <= TOL
        assert rel_err(y_new, oracle.matmul_f32(x, wf, nk=True, threads=8)) <= TOL
    w.free()


@pytest.mark.parametrize("qt,n,k,m", [(synth.Q8_0, 256, 1024, 96), (synth.MXFP4, 192, 2048, 40), (synth.Q6_K, 128, 512, 130),
                                      (synth.Q4_K, 256, 320, 64), (synth.Q4_K, 128, 8192, 1024)],
                         ids=["q8_0", "mxfp4", "q6_k", "q4_k-k320", "q4_k-at-the-limit"])
def test_noalloc_other_formats_and_the_size_limit(oracle, qt, n, k, m):
    """Formats other than Q4_K (and Q4_K rows that are not whole super-blocks) take the kernel whose weight tile is
    staged in shared memory; the last case sits exactly on m * k = 8,388,608. Free device memory must not move
    across a call: nothing is allocated, not even on the first use of a format."""
    from gpu_util import QuantizedWeight, backend, rel_err
    be = backend()
    rng = synth.rng_for(9200 + qt + k)
    data = synth.gen_packed(qt, synth.GGUF, n * k, rng)
    w = QuantizedWeight(be, data, qt, synth.GGUF, n, k)
    x = synth.gen_activations(m, k, rng)
    wf = oracle.dequantize(qt, synth.GGUF, data, n * k, threads=8).reshape(n, k)
    ref = oracle.matmul_f32(x, wf, nk=True, threads=8)
    y0 = _run(be, w, x, m, noalloc=True)          # warm-up: kernel attributes, the array's address
    info = _lib.DeviceInfo()
    _lib.check(be.lib.b200q_get_device_info(be.ctx, ctypes.byref(info)))
    free_before = info.free_mem
    xb = be.allocate_buffer(x.nbytes); xb.copy_from_host(x)
    yb = be.allocate_buffer(m * n * 4)
    _lib.check(be.lib.b200q_get_device_info(be.ctx, ctypes.byref(info)))
    free_before = info.free_mem
    _lib.check(be.lib.b200q_matmul_noalloc(be.ctx, w.handle, xb.ptr, yb.ptr, m))
    be.synchronize()
    _lib.check(be.lib.b200q_get_device_info(be.ctx, ctypes.byref(info)))
    assert info.free_mem == free_before
    y1 = yb.to_numpy(np.float32, m * n).reshape(m, n)
    assert rel_err(y0, ref) <= TOL and rel_err(y1, ref) <= TOL
    assert rel_err(y1, _run(be, w, x, m, noalloc=False)) <= TOL
    xb.free(); yb.free(); w.free()


def test_noalloc_refuses_what_does_not_fit():
    from gpu_util import QuantizedWeight, backend
    be = backend()
    rng = synth.rng_for(9101)
    n, k = 128, 8192
    w = QuantizedWeight(be, synth.gen_packed(synth.Q8_0, synth.GGUF, n * k, rng), synth.Q8_0, synth.GGUF, n, k)
    buf = be.allocate_buffer(1 << 20)
    rc = be.lib.b200q_matmul_noalloc(be.ctx, w.handle, buf.ptr, buf.ptr, 1025)      # 1025 * 8192 > 8,388,608
    assert rc == _lib.ERR_INVALID and b"built-in scratch" in be.lib.b200q_last_error()
    rc = be.lib.b200q_matmul_noalloc(be.ctx, None, buf.ptr, buf.ptr, 16)
    assert rc == _lib.ERR_INVALID
    wk = QuantizedWeight(be, synth.gen_packed(synth.Q8_0, synth.GGUF, 64 * 96, rng), synth.Q8_0, synth.GGUF, 64, 96)
    assert be.lib.b200q_matmul_noalloc(be.ctx, wk.handle, buf.ptr, buf.ptr, 16) == _lib.ERR_UNSUPPORTED   # k % 64 != 0
    assert be.lib.b200q_matmul_noalloc(be.ctx, w.handle, buf.ptr, buf.ptr, 0) == 0
    buf.free(); w.free(); wk.free()
