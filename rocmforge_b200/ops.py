"""Operator surface of the quantized-weight path, with the reference's names and argument meaning.

dequantize_*:  src/kernels/quant/q4_0.rs:107 (dequantize_q4_0_kernel_cached), q4_k.rs:99
               (dequantize_q4_k_gpu_kernel), q6_k.rs:102 (dequantize_q6_k_gpu_kernel): host packed bytes in,
               fp32 written to a device buffer. Q8_0 / MXFP4 / MXFP6 have HIP kernels but no Rust wrapper in
               the reference (kernels/q8_0_dequant.hip, mxfp_dequant.hip); they get the same shape here.
matmul_q*:     src/kernels/matmul/quantized/{q4_0.rs:153, q4_k.rs:173, q6_k.rs:163, q8_0.rs:69}: host packed
               weights, device fp32 input and output, M = 1.
There is no *_with_fallback and no *_cpu_fallback: a failing GPU call raises B200QError.

`layout` picks the block byte layout (RF = what the reference parses, the default; GGUF = llama.cpp
blocks). `orient` picks how the flat weight stream maps to [n_rows, n_cols]: the reference's kernels and
its CPU composition index it as a flat [k, n] stream (ORIENT_KN, the default here so results match the
reference on the same bytes); ORIENT_NK is n_rows rows of n_cols weights, as its doc comments describe.
"""
import ctypes

from . import _lib
from ._lib import (F32, LAYOUT_GGUF, LAYOUT_RF, MXFP4, MXFP6_E2M3, MXFP6_E3M2, ORIENT_KN, ORIENT_NK, Q4_0, Q4_K,  # noqa: F401
                   Q6_K, Q8_0, check)
from .backend import QuantizedWeight, _host_ptr, as_u8


def dequantize_gpu(backend, qtype, quantized_data, output, num_elements, layout=LAYOUT_RF):
    a = as_u8(quantized_data)
    if num_elements * 4 > output.size:
        raise _lib.B200QError(_lib.ERR_INVALID, f"output buffer holds {output.size // 4} floats, {num_elements} needed")
    check(backend.lib.b200q_dequantize_bytes(backend.ctx, _host_ptr(a) if a.size else None, a.size, qtype, layout,
                                             output.as_ptr(), num_elements))


def dequantize_q4_0_kernel_cached(backend, quantized_data, output, num_elements, layout=LAYOUT_RF):
    dequantize_gpu(backend, Q4_0, quantized_data, output, num_elements, layout)


def dequantize_q8_0_gpu_kernel(backend, quantized_data, output, num_elements, layout=LAYOUT_RF):
    dequantize_gpu(backend, Q8_0, quantized_data, output, num_elements, layout)


def dequantize_q4_k_gpu_kernel(backend, quantized_data, output, num_elements, layout=LAYOUT_RF):
    dequantize_gpu(backend, Q4_K, quantized_data, output, num_elements, layout)


def dequantize_q6_k_gpu_kernel(backend, quantized_data, output, num_elements, layout=LAYOUT_RF):
    dequantize_gpu(backend, Q6_K, quantized_data, output, num_elements, layout)


def dequantize_mxfp4_gpu_kernel(backend, quantized_data, output, num_elements, layout=LAYOUT_RF):
    dequantize_gpu(backend, MXFP4, quantized_data, output, num_elements, layout)


def dequantize_mxfp6_gpu_kernel(backend, quantized_data, output, num_elements, layout=LAYOUT_RF, e3m2=False):
    dequantize_gpu(backend, MXFP6_E3M2 if e3m2 else MXFP6_E2M3, quantized_data, output, num_elements, layout)


def _matmul_q(backend, qtype, quantized_weights, input, n_rows, n_cols, output, layout, orient, m, flags):
    expect = backend.lib.b200q_tensor_bytes(qtype, layout, n_rows * n_cols)
    a = as_u8(quantized_weights)
    if a.size != expect:
        # same validation as execute_matmul_q4_0, src/ggml/hip_backend/op_dispatch.rs:973-979
        raise _lib.B200QError(_lib.ERR_INVALID, f"weights are {a.size} bytes, [{n_rows} x {n_cols}] needs {expect}")
    if input.size < m * n_cols * 4 or output.size < m * n_rows * 4:
        raise _lib.B200QError(_lib.ERR_INVALID, "input or output buffer too small for the shape")
    w = QuantizedWeight(backend, a, qtype, layout, n_rows, n_cols, orient=orient)
    try:
        w.matmul(input, output, m, flags=flags)
        backend.synchronize()
    finally:
        w.free()


def matmul_q4_0(backend, quantized_weights, input, n_rows, n_cols, output, layout=LAYOUT_RF, orient=ORIENT_KN, m=1, flags=0):
    _matmul_q(backend, Q4_0, quantized_weights, input, n_rows, n_cols, output, layout, orient, m, flags)


def matmul_q8_0(backend, quantized_weights, input, n_rows, n_cols, output, layout=LAYOUT_RF, orient=ORIENT_KN, m=1, flags=0):
    _matmul_q(backend, Q8_0, quantized_weights, input, n_rows, n_cols, output, layout, orient, m, flags)


def matmul_q4_k(backend, quantized_weights, input, n_rows, n_cols, output, layout=LAYOUT_RF, orient=ORIENT_KN, m=1, flags=0):
    _matmul_q(backend, Q4_K, quantized_weights, input, n_rows, n_cols, output, layout, orient, m, flags)


def matmul_q6_k(backend, quantized_weights, input, n_rows, n_cols, output, layout=LAYOUT_RF, orient=ORIENT_KN, m=1, flags=0):
    _matmul_q(backend, Q6_K, quantized_weights, input, n_rows, n_cols, output, layout, orient, m, flags)


def matmul_mxfp4(backend, quantized_weights, input, n_rows, n_cols, output, layout=LAYOUT_RF, orient=ORIENT_KN, m=1, flags=0):
    _matmul_q(backend, MXFP4, quantized_weights, input, n_rows, n_cols, output, layout, orient, m, flags)


def matmul_mxfp6(backend, quantized_weights, input, n_rows, n_cols, output, layout=LAYOUT_RF, orient=ORIENT_KN, m=1,
                 flags=0, e3m2=False):
    _matmul_q(backend, MXFP6_E3M2 if e3m2 else MXFP6_E2M3, quantized_weights, input, n_rows, n_cols, output, layout,
              orient, m, flags)


def fused_q4_0_rmsnorm(backend, q4_0_input, weight, output, seq_len, hidden_size, eps, qtype=Q4_0, layout=LAYOUT_RF):
    """fused_q4_0_rmsnorm (src/ggml/hip_backend/ops/fused_ops.rs:149-215): packed [seq_len, hidden_size] rows ->
    RMSNorm(deq(row)) * weight, fp32, without writing the dequantised rows. q4_0_input: host bytes of the packed
    tensor (uploaded for the call, as the reference's operators re-upload their weights) or a resident
    QuantizedWeight; weight / output: DeviceBuffer."""
    own = not isinstance(q4_0_input, QuantizedWeight)
    w = QuantizedWeight(backend, q4_0_input, qtype, layout, seq_len, hidden_size) if own else q4_0_input
    try:
        _lib.check(backend.lib.b200q_fused_dequant_rmsnorm(backend.ctx, w.handle, weight.as_ptr(), output.as_ptr(),
                                                            ctypes.c_float(eps)))
        backend.synchronize()
    finally:
        if own:
            w.free()


def validate_token_ids(tokens, vocab_size):
    """validate_token_ids (src/ggml/hip_backend/ops/get_rows.rs:84-94): the first id >= vocab_size is an error."""
    for t in tokens:
        if int(t) >= vocab_size:
            raise ValueError(f"Token ID {int(t)} exceeds vocab size {vocab_size}")


def get_rows(backend, weights, tokens, n_embd, n_vocab, output, qtype=None, layout=LAYOUT_GGUF, trim_padding=False):
    """get_rows (src/ggml/hip_backend/ops/get_rows.rs:24-78) on a PACKED embedding table: output[i, :] =
    deq(weights)[tokens[i], :], fp32 [len(tokens), n_embd]. weights: a resident QuantizedWeight uploaded as
    [n_vocab, n_embd], or host bytes of the packed table with qtype/layout (uploaded for the call). tokens: host
    integers, validated before anything is launched. trim_padding=True drops everything from the first 0 id on,
    as execute_get_rows does with its padded token buffer (src/ggml/hip_backend/op_dispatch.rs:71-76).
    Returns the number of rows written."""
    import numpy as np
    toks = np.ascontiguousarray(np.asarray(tokens, dtype=np.uint32).reshape(-1))
    if trim_padding:
        zeros = np.nonzero(toks == 0)[0]
        if zeros.size:
            toks = toks[:int(zeros[0])]
    validate_token_ids(toks, n_vocab)
    own = not isinstance(weights, QuantizedWeight)
    w = QuantizedWeight(backend, weights, qtype, layout, n_vocab, n_embd) if own else weights
    try:
        if w.n_total != n_vocab or w.k != n_embd:
            raise ValueError(f"table is [{w.n_total}, {w.k}], expected [{n_vocab}, {n_embd}]")
        if output.size < toks.size * n_embd * 4:
            raise ValueError("Output size does not match n_embd * actual_n_tokens")
        if toks.size:
            _lib.check(backend.lib.b200q_get_rows_host(backend.ctx, w.handle, toks.ctypes.data_as(ctypes.c_void_p),
                                                        toks.size, output.as_ptr(), n_embd))
    finally:
        if own:
            w.free()
    return int(toks.size)
