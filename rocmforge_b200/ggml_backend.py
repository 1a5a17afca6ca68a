"""The IR-level entry of the quantized-weight path: the counterpart of `impl GgmlBackend for HipGgmlBackend`.

Mirrors, for this path only, the reference's backend plug-in contract (src/ggml/backend.rs:5-23: alloc / bind /
free / tensor_desc / buffer / execute_op / synchronize), its IR types (Op, src/ggml/op.rs:4-30; DType and
TensorDesc, src/ggml/tensor.rs:8-60), the dispatch of the two quantized ops (execute_matmul_q4_0 / execute_matmul_q8_0,
src/ggml/hip_backend/op_dispatch.rs:951-1082: same argument checks, same messages) and the capability entry the hybrid
scheduler reads (OpType::QuantizedMatMul, src/ggml/hip_backend/capability.rs:44-50, src/ggml/hybrid_scheduler.rs:36-91).

Differences that are deliberate: the reference copies the weights device -> host and uploads them again on EVERY
op (op_dispatch.rs:1001-1004); here a weights tensor is uploaded once, when it is bound, and stays packed on the
device. The reference's wrappers hard-wire m = 1; here m is the input's first dimension.
"""
import enum

import numpy as np

from . import _lib
from .backend import DeviceBuffer, QuantizedWeight, as_u8


class GgmlError(Exception):
    """GgmlError::{InvalidShape, Backend, Unimplemented} (src/ggml/mod.rs:30-35)."""

    def __init__(self, kind, message):
        super().__init__(f"{kind}: {message}")
        self.kind, self.message = kind, message


def InvalidShape(msg):
    return GgmlError("InvalidShape", msg)


def BackendError(msg):
    return GgmlError("Backend", msg)


class Op(enum.Enum):
    """The ops of src/ggml/op.rs this backend executes (the quantized products) or names (to refuse them)."""
    GetRows = "GetRows"
    MatMul = "MatMul"
    MatMulQ4_0 = "MatMulQ4_0"
    MatMulQ8_0 = "MatMulQ8_0"
    Add = "Add"
    MlpSwiglu = "MlpSwiglu"


class DType(enum.Enum):
    I32 = "I32"
    U32 = "U32"
    F32 = "F32"
    F16 = "F16"
    Q8_0 = "Q8_0"
    Q4_0 = "Q4_0"
    Mxfp4 = "Mxfp4"
    Mxfp6 = "Mxfp6"


class OpType(enum.Enum):
    MatMul = "MatMul"
    QuantizedMatMul = "QuantizedMatMul"

    @staticmethod
    def from_op(op):
        """OpType::from_op (src/ggml/hybrid_scheduler.rs:56-73)."""
        if op in (Op.MatMulQ4_0, Op.MatMulQ8_0):
            return OpType.QuantizedMatMul
        if op is Op.MatMul:
            return OpType.MatMul
        return None


class OpCapability:
    def __init__(self, op_type, supported_dtypes, max_tensor_size, requires_feature):
        self.op_type, self.supported_dtypes = op_type, supported_dtypes
        self.max_tensor_size, self.requires_feature = max_tensor_size, requires_feature


# bytes per 32-weight block of the reference's own layouts, as its dispatch checks them (op_dispatch.rs:973, 1039)
_BLOCK_BYTES = {DType.Q4_0: 20, DType.Q8_0: 36}
_QTYPE = {DType.Q4_0: _lib.Q4_0, DType.Q8_0: _lib.Q8_0}


class TensorDesc:
    """TensorDesc (src/ggml/tensor.rs:20-60): id, shape, dtype; byte_size follows its rules for the block types."""

    def __init__(self, shape, dtype, id=0):
        self.id, self.shape, self.dtype = id, list(shape), dtype

    def element_count(self):
        n = 1
        for d in self.shape:
            n *= d
        return n

    def byte_size(self):
        n = self.element_count()
        if self.dtype in _BLOCK_BYTES:
            return (n + 31) // 32 * _BLOCK_BYTES[self.dtype]
        return n * (2 if self.dtype is DType.F16 else 4)


class B200GgmlBackend:
    """`impl GgmlBackend` + `impl CapabilityProvider` for the quantized-weight ops, on top of the C ABI."""

    def __init__(self, backend, orient=_lib.ORIENT_KN):
        self.backend = backend
        self.orient = orient            # how bound weight bytes map to [rows, cols]; the reference's kernels read [k, n]
        self._desc, self._buf, self._weights = {}, {}, {}

    # ---- GgmlBackend -------------------------------------------------------------------------------------------
    def alloc(self, desc):
        self._desc[desc.id] = desc
        if desc.dtype not in _BLOCK_BYTES:
            self._buf[desc.id] = self.backend.allocate_buffer(max(16, desc.byte_size()))

    def bind(self, desc, buffer):
        """A weights tensor may be bound to host bytes or to a device buffer holding the packed bytes (what the
        reference binds); either way it is uploaded into the packed device form once, on first use."""
        self._desc[desc.id] = desc
        self._buf[desc.id] = buffer
        self._weights.pop(desc.id, None)

    def free(self, id):
        w = self._weights.pop(id, None)
        if w is not None:
            w.free()
        self._desc.pop(id, None)
        self._buf.pop(id, None)

    def tensor_desc(self, id):
        return self._desc.get(id)

    def buffer(self, id):
        return self._buf.get(id)

    def synchronize(self):
        self.backend.synchronize()

    def execute_op(self, op, inputs, outputs):
        if op is Op.MatMulQ4_0:
            return self._execute_matmul_q(inputs, outputs, DType.Q4_0, "MatMulQ4_0")
        if op is Op.MatMulQ8_0:
            return self._execute_matmul_q(inputs, outputs, DType.Q8_0, "MatMulQ8_0")
        raise GgmlError("Unimplemented", f"{op.value} is outside the quantized-weight path of this backend")

    # ---- CapabilityProvider ------------------------------------------------------------------------------------
    def capabilities(self):
        return [OpCapability(OpType.QuantizedMatMul, [DType.F32], None, "cuda-sm100a")]

    def op_capability(self, op):
        t = OpType.from_op(op)
        for c in self.capabilities():
            if c.op_type is t:
                return c
        return None

    def can_execute(self, op):
        return self.op_capability(op) is not None

    def backend_id(self):
        return "b200"

    # ---- execute_matmul_q4_0 / execute_matmul_q8_0 (op_dispatch.rs:951-1082) -----------------------------------
    def _execute_matmul_q(self, inputs, outputs, dtype, name):
        if len(inputs) != 2 or len(outputs) != 1:
            raise InvalidShape(f"{name} expects 2 inputs and 1 output")
        wd = self.tensor_desc(inputs[0])
        if wd is None:
            raise InvalidShape("Missing weights desc")
        xd = self.tensor_desc(inputs[1])
        if xd is None:
            raise InvalidShape("Missing input desc")
        if len(wd.shape) != 2 or len(xd.shape) != 2:
            raise InvalidShape(f"{name} expects 2D tensors")
        n_rows, n_cols = wd.shape
        expected = (n_rows * n_cols + 31) // 32 * _BLOCK_BYTES[dtype]
        if wd.byte_size() != expected:
            raise InvalidShape(f"{name} weights size mismatch: expected {expected} bytes, got {wd.byte_size()}")
        m, k = xd.shape
        if k != n_cols:
            raise InvalidShape(f"{name} dimension mismatch: k={k} weights_k={n_cols}")
        wbuf = self.buffer(inputs[0])
        if wbuf is None:
            raise BackendError("Missing weights buffer")
        xbuf = self.buffer(inputs[1])
        if xbuf is None:
            raise BackendError("Missing input buffer")
        ybuf = self.buffer(outputs[0])
        if ybuf is None:
            raise BackendError("Missing output buffer")
        w = self._weights.get(inputs[0])
        if w is None:
            if isinstance(wbuf, DeviceBuffer):       # the packed bytes live on the device, as in the reference
                host = wbuf.to_numpy(np.uint8, expected)
            else:
                host = as_u8(wbuf)
            if host.size != expected:
                raise BackendError(f"Failed to read weights: buffer holds {host.size} bytes, {expected} expected")
            try:
                w = QuantizedWeight(self.backend, host, _QTYPE[dtype], _lib.LAYOUT_RF, n_rows, n_cols, orient=self.orient)
            except _lib.B200QError as e:
                raise BackendError(str(e))
            self._weights[inputs[0]] = w
        try:
            w.matmul(xbuf, ybuf, m)
        except _lib.B200QError as e:
            raise BackendError(str(e))
