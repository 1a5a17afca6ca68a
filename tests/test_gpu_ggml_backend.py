"""execute_op(Op.MatMulQ4_0 / MatMulQ8_0) on the GPU against the CPU oracle, with the weights bound as host bytes and
as a device buffer of packed bytes (what the reference's graph binds, src/ggml/hip_backend/op_dispatch.rs:951-1082)."""
import numpy as np
import pytest

from rocmforge_b200 import _lib, synth
from rocmforge_b200.ggml_backend import B200GgmlBackend, DType, Op, TensorDesc

pytestmark = pytest.mark.gpu
from gpu_util import backend, rel_err  # noqa: E402


@pytest.mark.parametrize("op,dtype,qt", [(Op.MatMulQ4_0, DType.Q4_0, synth.Q4_0), (Op.MatMulQ8_0, DType.Q8_0, synth.Q8_0)])
@pytest.mark.parametrize("bound_on_device", [False, True])
def test_execute_op_matches_the_cpu_composition(oracle, op, dtype, qt, bound_on_device):
    be = backend()
    g = B200GgmlBackend(be)                      # weights read as the flat [k, n] stream, as the reference's kernels do
    rng = synth.rng_for(7300 + qt)
    n_rows, n_cols, m = 96, 128, 3
    data = synth.gen_packed(qt, synth.RF, n_rows * n_cols, rng)
    x = synth.gen_activations(m, n_cols, rng)
    wdesc = TensorDesc([n_rows, n_cols], dtype, id=10)
    if bound_on_device:
        wb = be.allocate_buffer(data.size); wb.copy_from_host(data)
        g.bind(wdesc, wb)
    else:
        g.bind(wdesc, data)
    xdesc, ydesc = TensorDesc([m, n_cols], DType.F32, id=11), TensorDesc([m, n_rows], DType.F32, id=12)
    g.alloc(xdesc); g.alloc(ydesc)
    g.buffer(11).copy_from_host(x)
    for _ in range(2):                           # the second op reuses the uploaded weights
        g.execute_op(op, [10, 11], [12])
    g.synchronize()
    y = g.buffer(12).to_numpy(np.float32, m * n_rows).reshape(m, n_rows)
    w = oracle.dequantize(qt, synth.RF, data, n_rows * n_cols).reshape(n_cols, n_rows)   # [k, n]
    ref = oracle.matmul_f32(x, w, nk=False)
    assert rel_err(y, ref) <= 1e-4
    for t in (10, 11, 12):
        g.free(t)
