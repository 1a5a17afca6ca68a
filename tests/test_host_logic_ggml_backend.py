"""The IR-level entry (execute_op with Op.MatMulQ4_0 / MatMulQ8_0) without a GPU: the argument checks of
execute_matmul_q4_0 / execute_matmul_q8_0 (src/ggml/hip_backend/op_dispatch.rs:951-1082) fire, with the reference's
messages, before anything touches the device, and the capability entry answers the way
src/ggml/hip_backend/capability.rs:44-50 does."""
import pytest

from rocmforge_b200.ggml_backend import B200GgmlBackend, DType, GgmlError, Op, OpType, TensorDesc


class NoDevice:          # any use of the library would raise AttributeError instead of GgmlError
    pass


def make(shape_w, shape_x, dtype=DType.Q4_0):
    be = B200GgmlBackend(NoDevice())
    be.bind(TensorDesc(shape_w, dtype, id=1), b"")
    be.bind(TensorDesc(shape_x, DType.F32, id=2), object())
    be.bind(TensorDesc([shape_x[0], shape_w[0]], DType.F32, id=3), object())
    return be


def test_argument_checks_carry_the_reference_messages():
    be = make([4, 64], [1, 64])
    with pytest.raises(GgmlError, match="MatMulQ4_0 expects 2 inputs and 1 output"):
        be.execute_op(Op.MatMulQ4_0, [1], [3])
    with pytest.raises(GgmlError, match="Missing weights desc"):
        be.execute_op(Op.MatMulQ4_0, [9, 2], [3])
    with pytest.raises(GgmlError, match="Missing input desc"):
        be.execute_op(Op.MatMulQ4_0, [1, 9], [3])
    be3 = make([4, 64], [1, 64])
    be3.bind(TensorDesc([1, 4, 16], DType.F32, id=2), object())
    with pytest.raises(GgmlError, match="MatMulQ4_0 expects 2D tensors"):
        be3.execute_op(Op.MatMulQ4_0, [1, 2], [3])
    with pytest.raises(GgmlError, match="MatMulQ8_0 dimension mismatch: k=32 weights_k=64"):
        make([4, 64], [1, 32], DType.Q8_0).execute_op(Op.MatMulQ8_0, [1, 2], [3])
    be4 = make([4, 64], [1, 64])
    be4.free(3)
    with pytest.raises(GgmlError, match="Missing output buffer"):
        be4.execute_op(Op.MatMulQ4_0, [1, 2], [3])


def test_byte_size_rules_and_weight_size_check():
    assert TensorDesc([4, 64], DType.Q4_0).byte_size() == 8 * 20        # ceil(rows * cols / 32) * 20
    assert TensorDesc([4, 64], DType.Q8_0).byte_size() == 8 * 36
    assert TensorDesc([3, 10], DType.Q4_0).byte_size() == 20            # a partial block still takes a whole one
    be = make([4, 64], [1, 64])
    with pytest.raises(GgmlError, match="Failed to read weights: buffer holds 0 bytes, 160 expected"):
        be.execute_op(Op.MatMulQ4_0, [1, 2], [3])                       # bound to empty host bytes


def test_capability_and_refusal_of_other_ops():
    be = B200GgmlBackend(NoDevice())
    assert be.backend_id() == "b200"
    assert be.can_execute(Op.MatMulQ4_0) and be.can_execute(Op.MatMulQ8_0)
    assert not be.can_execute(Op.MatMul) and not be.can_execute(Op.GetRows)
    cap = be.op_capability(Op.MatMulQ8_0)
    assert cap.op_type is OpType.QuantizedMatMul and cap.supported_dtypes == [DType.F32]
    assert OpType.from_op(Op.Add) is None
    with pytest.raises(GgmlError, match="Unimplemented"):
        be.execute_op(Op.MlpSwiglu, [], [])
