"""Fused dequant + RMSNorm on the GPU against the oracle (tolerance 1e-5 of the row maximum: the reduction
order and rsqrt differ between any two implementations; the dequantised inputs are bit-exact)."""
import numpy as np
import pytest

from rocmforge_b200 import _lib, ops, synth
from rocmforge_b200._lib import B200QError
from rocmforge_b200.backend import QuantizedWeight

from gpu_util import backend

pytestmark = pytest.mark.gpu
TOL = 1e-5
ALL = [(q, l) for q in range(10) for l in (synth.RF, synth.GGUF)]
IDS = [f"{synth.QNAMES[q]}-{synth.LAYOUT_NAMES[l]}" for q, l in ALL]


def run(be, qt, lay, data, seq, hidden, g, eps):
    gbuf = be.allocate_buffer(hidden * 4)
    gbuf.copy_from_host(g)
    out = be.allocate_buffer(seq * hidden * 4)
    out.fill(0xFF)
    ops.fused_q4_0_rmsnorm(be, data, gbuf, out, seq, hidden, eps, qtype=qt, layout=lay)
    return out.to_numpy(np.float32, seq * hidden).reshape(seq, hidden)


def test_reference_operator_signature_q4_0_rf(oracle):
    be = backend()
    rng = synth.rng_for(4200)
    seq, hidden = 17, 896
    data = synth.gen_packed(synth.Q4_0, synth.RF, seq * hidden, rng)
    g = rng.standard_normal(hidden).astype(np.float32)
    got = run(be, synth.Q4_0, synth.RF, data, seq, hidden, g, 1e-6)
    ref = oracle.fused_dequant_rmsnorm(synth.Q4_0, synth.RF, data, seq, hidden, g, 1e-6)
    assert np.max(np.abs(got - ref)) <= TOL * np.max(np.abs(ref))


@pytest.mark.parametrize("qt,lay", ALL, ids=IDS)
def test_every_format(oracle, qt, lay):
    be = backend()
    rng = synth.rng_for(4300 + qt * 2 + lay)
    seq, hidden = 9, 2304                      # 2304 / 8 = 288 pieces: more than one pass of the 256 threads
    data = synth.gen_packed(qt, lay, seq * hidden, rng)
    g = rng.standard_normal(hidden).astype(np.float32)
    got = run(be, qt, lay, data, seq, hidden, g, 1e-5)
    ref = oracle.fused_dequant_rmsnorm(qt, lay, data, seq, hidden, g, 1e-5)
    assert np.all(np.isfinite(got))
    assert np.max(np.abs(got - ref)) <= TOL * np.max(np.abs(ref))


def test_zero_rows_single_row_and_large_shape(oracle):
    be = backend()
    hidden = 4096
    zero = bytes(hidden // 32 * 20)
    got = run(be, synth.Q4_0, synth.RF, zero, 1, hidden, np.ones(hidden, np.float32), 1e-6)
    assert np.all(got == 0.0)
    rng = synth.rng_for(4400)
    seq = 512
    data = synth.gen_packed(synth.Q4_0, synth.GGUF, seq * hidden, rng)
    g = rng.standard_normal(hidden).astype(np.float32)
    got = run(be, synth.Q4_0, synth.GGUF, data, seq, hidden, g, 1e-6)
    ref = oracle.fused_dequant_rmsnorm(synth.Q4_0, synth.GGUF, data, seq, hidden, g, 1e-6)
    assert np.max(np.abs(got - ref)) <= TOL * np.max(np.abs(ref))


def test_bad_arguments_are_status_codes():
    be = backend()
    rng = synth.rng_for(4500)
    data = synth.gen_packed(synth.Q4_0, synth.RF, 4 * 64, rng)
    w = QuantizedWeight(be, data, synth.Q4_0, synth.RF, 64, 4, orient=_lib.ORIENT_KN)     # not rows of hidden values
    out = be.allocate_buffer(4 * 64 * 4)
    g = be.allocate_buffer(64 * 4)
    with pytest.raises(B200QError) as e:
        ops.fused_q4_0_rmsnorm(be, w, g, out, 4, 64, 1e-6)
    assert e.value.status == _lib.ERR_UNSUPPORTED
    w.free()
