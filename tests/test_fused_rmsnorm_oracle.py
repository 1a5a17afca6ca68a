"""The oracle's restatement of the fused dequant + RMSNorm kernel against a float64 numpy evaluation."""
import numpy as np
import pytest

from rocmforge_b200 import synth


@pytest.mark.parametrize("qt,lay", [(synth.Q4_0, synth.RF), (synth.Q4_0, synth.GGUF), (synth.Q6_K, synth.GGUF)])
def test_oracle_matches_float64(oracle, qt, lay):
    rng = synth.rng_for(4100 + qt * 2 + lay)
    seq, hidden = 5, 768
    data = synth.gen_packed(qt, lay, seq * hidden, rng)
    g = rng.standard_normal(hidden).astype(np.float32)
    got = oracle.fused_dequant_rmsnorm(qt, lay, data, seq, hidden, g, 1e-6)
    w = oracle.dequantize(qt, lay, data, seq * hidden).reshape(seq, hidden).astype(np.float64)
    ref = w / np.sqrt((w * w).mean(axis=1, keepdims=True) + 1e-6) * g.astype(np.float64)
    assert np.max(np.abs(got - ref)) <= 1e-5 * np.max(np.abs(ref))


def test_oracle_zero_row_gives_zero(oracle):
    hidden = 256
    data = bytes(hidden // 32 * 20)                      # RF Q4_0: scale 0.0 everywhere
    got = oracle.fused_dequant_rmsnorm(synth.Q4_0, synth.RF, data, 1, hidden, np.ones(hidden, np.float32), 1e-6)
    assert np.all(got == 0.0)
