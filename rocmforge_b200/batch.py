"""Batch front end: the counterpart of BatchQuantizedMatmul (src/ggml/hip_backend/ops/batch_quantized.rs:22-412).

QuantFormat / QuantizedMatmulOp / BatchMatmulResult keep the reference's names and meaning (weights are host
bytes, m = 1 by default, n = n_rows, k = n_cols). process_batch shares one device input among the products,
as the reference does; where the reference loops over per-product launches, this issues ONE grouped launch
for the whole batch when every product has a grouped decode kernel. There is no AsyncKernelLauncher: the
reference's launches a kernel against a freshly allocated, never filled weight buffer
(batch_quantized.rs:326-338), which is not a behaviour to keep.
"""
import ctypes
import enum

import numpy as np

from . import _lib
from ._lib import LAYOUT_RF, ORIENT_NK, check
from .backend import QuantizedWeight, _host_ptr


class QuantFormat(enum.Enum):
    Q4_0 = _lib.Q4_0
    Q4_K = _lib.Q4_K
    Q6_K = _lib.Q6_K
    Q8_0 = _lib.Q8_0
    MXFP4 = _lib.MXFP4
    MXFP6_E2M3 = _lib.MXFP6_E2M3
    MXFP6_E3M2 = _lib.MXFP6_E3M2

    def bytes_per_element(self, layout=LAYOUT_RF):
        lib = _lib.load()
        return lib.b200q_block_bytes(self.value, layout) / lib.b200q_block_elems(self.value)


class QuantizedMatmulOp:
    """One product of a batch: weights [n_rows x n_cols] (host bytes), m = 1 unless the batch says otherwise."""

    def __init__(self, weights, n_rows, n_cols, format, layout=LAYOUT_RF):
        self.weights = weights
        self.m, self.n, self.k = 1, n_rows, n_cols
        self.format, self.layout = format, layout

    def weight_bytes(self):
        return len(self.weights)

    def output_elements(self):
        return self.m * self.n


class BatchMatmulResult:
    def __init__(self, outputs, timings_ms, total_time_ms):
        self.outputs, self.timings_ms, self.total_time_ms = outputs, timings_ms, total_time_ms


class DeviceBatch:
    """Weights uploaded once, activations and outputs in two contiguous device arenas, one b200q_batch handle."""

    def __init__(self, backend, weights, m, shared_input=None):
        self.backend, self.m, self.weights = backend, m, weights
        lib = backend.lib
        self.xsizes = [m * w.k for w in weights]
        self.ysizes = [m * w.n_local for w in weights]
        self.shared = shared_input is not None
        if self.shared:
            self.xarena = None
            xptrs = [shared_input.as_ptr()] * len(weights)
        else:
            self.xarena = backend.allocate_buffer(max(16, 4 * sum(self.xsizes)))
            xptrs, off = [], 0
            for s in self.xsizes:
                xptrs.append(self.xarena.ptr + 4 * off)
                off += s
        self.yarena = backend.allocate_buffer(max(16, 4 * sum(self.ysizes)))
        yptrs, off = [], 0
        for s in self.ysizes:
            yptrs.append(self.yarena.ptr + 4 * off)
            off += s
        self.xptrs, self.yptrs = xptrs, yptrs
        cnt = len(weights)
        aw = (ctypes.c_void_p * cnt)(*[w.handle.value for w in weights])
        ax = (ctypes.c_void_p * cnt)(*xptrs)
        ay = (ctypes.c_void_p * cnt)(*yptrs)
        h = ctypes.c_void_p()
        check(lib.b200q_batch_create(backend.ctx, cnt, aw, ax, ay, m, ctypes.byref(h)))
        self.handle = h
        self.weight_bytes = int(lib.b200q_batch_weight_bytes(h))
        self.launches = int(lib.b200q_batch_launches(h))

    def set_inputs(self, xs):
        flat = np.concatenate([np.ascontiguousarray(x, dtype=np.float32).reshape(-1) for x in xs])
        self.xarena.copy_from_host(flat)

    def run(self, timed=False):
        ms = ctypes.c_float()
        check(self.backend.lib.b200q_batch_run(self.backend.ctx, self.handle, ctypes.byref(ms) if timed else None))
        return ms.value if timed else None

    def run_host(self, h_x_ptr, h_y_ptr):
        check(self.backend.lib.b200q_batch_run_host(self.backend.ctx, self.handle, h_x_ptr, h_y_ptr))

    def outputs(self):
        flat = self.yarena.to_numpy(np.float32, sum(self.ysizes))
        out, off = [], 0
        for w, s in zip(self.weights, self.ysizes):
            out.append(flat[off:off + s].reshape(self.m, w.n_local).copy())
            off += s
        return out

    def free(self):
        if self.handle:
            self.backend.lib.b200q_batch_free(self.handle)
            self.handle = None
        for b in (self.xarena, self.yarena):
            if b is not None:
                b.free()


class BatchQuantizedMatmul:
    """process_batch / process_batch_profiled / calculate_throughput with the reference's meaning."""

    def __init__(self, backend, enable_profiling=False):
        self.backend, self.enable_profiling = backend, enable_profiling

    def process_batch(self, input, ops, orient=ORIENT_NK):
        return self.process_batch_profiled(input, ops, orient).outputs

    def process_batch_profiled(self, input, ops, orient=ORIENT_NK):
        if not ops:
            return BatchMatmulResult([], [], 0.0)
        be = self.backend
        ws = [QuantizedWeight(be, op.weights, op.format.value, op.layout, op.n, op.k, orient=orient) for op in ops]
        batch = DeviceBatch(be, ws, ops[0].m, shared_input=input)
        try:
            total = batch.run(timed=True)
            be.synchronize()
            outs = batch.outputs()
        finally:
            batch.free()
            for w in ws:
                w.free()
        share = [total * op.weight_bytes() / max(1, sum(o.weight_bytes() for o in ops)) for op in ops]
        return BatchMatmulResult(outs, share, total)

    @staticmethod
    def calculate_throughput(ops, total_time_ms):
        """(products per second, weight bytes per second), batch_quantized.rs:277-289."""
        if total_time_ms <= 0:
            return 0.0, 0.0
        secs = total_time_ms / 1000.0
        return len(ops) / secs, sum(op.weight_bytes() for op in ops) / secs
