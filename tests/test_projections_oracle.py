"""CPU checks of the oracle's projection-site restatements (SwiGLU activation, row bias).

The reference's own cases: swiglu at zeros is 0, at gate = 1 it equals swish(up) (src/mlp/swiglu_tests.rs compares
the kernel with `gate * (up * sigmoid(up))` at 1e-4); add_row_bias adds the bias to every row (backend.rs:924-975)."""
import numpy as np


def test_swiglu_known_values(oracle):
    up = np.array([0.0, 1.0, -1.0, 2.5, -30.0, 30.0, 100.0, -100.0], dtype=np.float32)
    gate = np.ones_like(up)
    got = oracle.swiglu(gate, up)
    want = (up.astype(np.float64) / (1.0 + np.exp(-up.astype(np.float64)))).astype(np.float32)
    assert np.allclose(got, want, rtol=1e-6, atol=1e-30)
    assert got[0] == 0.0 and got[6] == 100.0 and got[7] == 0.0       # expf saturates: sigmoid -> 1 and 0 exactly
    assert not oracle.swiglu(np.zeros(5, np.float32), up[:5]).any()


def test_swiglu_is_gate_times_swish_up_in_that_order(oracle):
    rng = np.random.Generator(np.random.PCG64(11))
    g = rng.standard_normal((3, 37), dtype=np.float32)
    u = rng.standard_normal((3, 37), dtype=np.float32) * 4
    got = oracle.swiglu(g, u)
    sig = np.float32(1.0) / (np.float32(1.0) + np.exp(-u))           # numpy's float32 exp is within an ulp of expf
    want = g * (u * sig)
    assert got.shape == g.shape
    assert np.allclose(got, want, rtol=3e-7, atol=1e-30)


def test_add_row_bias(oracle):
    rng = np.random.Generator(np.random.PCG64(12))
    y = rng.standard_normal((4, 9), dtype=np.float32)
    b = rng.standard_normal(9, dtype=np.float32)
    got = oracle.add_row_bias(y, b)
    assert np.array_equal(got, y + b[None, :])
    assert np.array_equal(oracle.add_row_bias(y, b.reshape(1, 9)), got)
