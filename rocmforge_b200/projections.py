"""Projection-site operators on packed weights: the callers either side of the fused dequant + matmul products.

Mirrors HipBackend::mlp_swiglu (src/backend/hip_backend/backend.rs:1153-1276), HipBackend::add_row_bias
(backend.rs:924-975), swiglu_gpu_kernel (src/mlp/kernels.rs, kernels/swiglu.hip:37-63) and the Q/K/V projection
group of the layer (src/model/execution_plan/execute.rs:456-458) with the same argument meaning and error texts;
the weights are resident QuantizedWeight tensors ([out_features, in_features], rows of in_features values)
instead of fp32 device tensors.
"""
import ctypes

from . import _lib
from ._lib import check
from .backend import QuantizedWeight


def swiglu_gpu_kernel(backend, gate, up, output, seq_len, intermediate_size):
    """output = gate * swish(up), fp32 [seq_len, intermediate_size] DeviceBuffers; output may be gate."""
    check(backend.lib.b200q_swiglu(backend.ctx, gate.as_ptr(), up.as_ptr(), output.as_ptr(), seq_len, intermediate_size))


def add_row_bias(backend, tensor, tensor_shape, bias, bias_shape):
    """tensor[r, :] += bias for every row. Shapes are tuples, checked as the reference checks them."""
    if len(tensor_shape) != 2:
        raise ValueError("Tensor for row bias must be 2D")
    rows, cols = tensor_shape
    bs = tuple(bias_shape)
    if not ((len(bs) == 1 and bs[0] == cols) or (len(bs) == 2 and bs[0] == 1 and bs[1] == cols)):
        raise ValueError(f"Bias shape {list(bs)} incompatible with tensor shape {list(tensor_shape)}")
    if rows == 0 or cols == 0:
        return
    check(backend.lib.b200q_add_row_bias(backend.ctx, tensor.as_ptr(), cols, bias.as_ptr(), rows, cols))


class MlpSwiglu:
    """A bound SwiGLU MLP block: output[seq_len, hidden] = (gate(x) * swish(up(x))) . down, weights packed.

    The plan owns the two [seq_len, intermediate] scratch projections; run() may be called any number of
    times on the bound buffers (decode loop). At seq_len <= 8 gate and up are one grouped launch."""

    def __init__(self, backend, hidden_states, gate_weight, up_weight, down_weight, output, seq_len):
        for w in (gate_weight, up_weight, down_weight):
            if not isinstance(w, QuantizedWeight):
                raise TypeError("weights must be resident QuantizedWeight tensors")
        hidden_size = gate_weight.k
        if hidden_states.size < seq_len * hidden_size * 4:
            raise ValueError("hidden_states must be 2D [seq_len, hidden_size]")
        if output.size < seq_len * hidden_size * 4:
            raise ValueError("output must match hidden_states shape [seq_len, hidden_size]")
        self.backend = backend
        self.seq_len, self.hidden_size, self.intermediate_size = seq_len, hidden_size, gate_weight.n_total
        h = ctypes.c_void_p()
        check(backend.lib.b200q_mlp_create(backend.ctx, gate_weight.handle, up_weight.handle, down_weight.handle,
                                           hidden_states.as_ptr(), output.as_ptr(), seq_len, ctypes.byref(h)))
        self.handle = h
        self._keep = (hidden_states, gate_weight, up_weight, down_weight, output)

    def run(self):
        check(self.backend.lib.b200q_mlp_run(self.backend.ctx, self.handle))

    def free(self):
        if self.handle:
            self.backend.lib.b200q_mlp_free(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def mlp_swiglu(backend, hidden_states, gate_weight, up_weight, down_weight, output, seq_len):
    """One call of HipBackend::mlp_swiglu: builds the plan, runs it, synchronises (the reference's operator
    ends with a synchronise), frees the plan."""
    plan = MlpSwiglu(backend, hidden_states, gate_weight, up_weight, down_weight, output, seq_len)
    try:
        plan.run()
        backend.synchronize()
    finally:
        plan.free()


class SharedInputProjections:
    """Several packed projections of ONE input (Q, K, V of a layer; gate and up): one grouped launch at
    seq_len <= 8, the input read once per CTA tile. outputs[i] is a DeviceBuffer of [seq_len, weights[i].n]."""

    def __init__(self, backend, input, weights, outputs, seq_len=1):
        n = len(weights)
        if n != len(outputs):
            raise ValueError("one output per projection")
        aw = (ctypes.c_void_p * n)(*[w.handle for w in weights])
        ax = (ctypes.c_void_p * n)(*[input.as_ptr() for _ in weights])
        ay = (ctypes.c_void_p * n)(*[o.as_ptr() for o in outputs])
        h = ctypes.c_void_p()
        check(backend.lib.b200q_batch_create(backend.ctx, n, aw, ax, ay, seq_len, ctypes.byref(h)))
        self.backend, self.handle = backend, h
        self.launches = int(backend.lib.b200q_batch_launches(h))
        self._keep = (input, list(weights), list(outputs))

    def run(self):
        check(self.backend.lib.b200q_batch_run(self.backend.ctx, self.handle, None))

    def free(self):
        if self.handle:
            self.backend.lib.b200q_batch_free(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass
