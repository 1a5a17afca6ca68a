"""The give-up path of the device-side bounded waits, exercised without faulting or hanging anything: a
wait on a barrier nothing arrives on runs out after a short budget, the status reaches the host as a
recoverable error, and the same context keeps working."""
import numpy as np
import pytest

from rocmforge_b200 import _lib, synth
from rocmforge_b200._lib import B200QError, check
from rocmforge_b200.backend import QuantizedWeight

from gpu_util import backend, gpu_matmul, rel_err

pytestmark = pytest.mark.gpu


def test_wait_that_runs_out_reports_timeout_and_context_survives(oracle):
    be = backend()
    check(be.lib.b200q_selftest_bounded_wait(be.ctx, 1 << 21))          # about a millisecond of SM cycles
    with pytest.raises(B200QError) as e:
        be.synchronize()
    assert e.value.status == _lib.ERR_TIMEOUT and e.value.recoverable
    assert be.lib.b200q_is_recoverable(_lib.ERR_TIMEOUT) == 1
    be.synchronize()                                                     # the status word was cleared
    rng = synth.rng_for(5100)
    n, k, m = 256, 512, 64
    data = synth.gen_packed(synth.Q4_K, synth.GGUF, n * k, rng)
    x = synth.gen_activations(m, k, rng)
    w = QuantizedWeight(be, data, synth.Q4_K, synth.GGUF, n, k)
    y = gpu_matmul(be, w, x, m)                                          # a prefill product on the same context
    wf = oracle.dequantize(synth.Q4_K, synth.GGUF, data, n * k).reshape(n, k)
    assert rel_err(y, oracle.matmul_f32(x, wf, nk=True, threads=8)) <= 2e-3
    w.free()


def test_selftest_budget_is_validated():
    be = backend()
    assert be.lib.b200q_selftest_bounded_wait(be.ctx, 0) == _lib.ERR_INVALID
    assert be.lib.b200q_selftest_bounded_wait(be.ctx, 1 << 40) == _lib.ERR_INVALID
