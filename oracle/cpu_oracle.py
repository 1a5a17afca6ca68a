"""ctypes front end of liboracle.so (the C restatement of the reference CPU path).

Test infrastructure only: used by tests/, the smoke check and the benchmark's CPU
baseline legs as the checker / the timed CPU baseline, never by the product path.
The reference (Rust) cannot be built here, so there is no oracle/_ref; every rf_*
function is pinned by the reference's own unit-test vectors instead
(tests/golden/reference_vectors.json).
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")

Q4_0, Q8_0, Q4_K, Q6_K, MXFP4, MXFP6_E2M3, MXFP6_E3M2, Q2_K, Q3_K, Q5_K = range(10)
RF, GGUF = 0, 1
QNAMES = ["Q4_0", "Q8_0", "Q4_K", "Q6_K", "MXFP4", "MXFP6_E2M3", "MXFP6_E3M2", "Q2_K", "Q3_K", "Q5_K"]


def build(force=False):
    """Compile liboracle.so with gcc if it is missing or older than its sources."""
    srcs = [os.path.join(_HERE, f) for f in ("oracle.c", "oracle.h", "Makefile")]
    if (not force and os.path.exists(_SO)
            and os.path.getmtime(_SO) >= max(os.path.getmtime(s) for s in srcs)):
        return _SO
    subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True,
                   stdout=subprocess.PIPE, stderr=subprocess.PIPE)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_SO)
        u8p, f32p, f64p = ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p
        sz, ci = ctypes.c_size_t, ctypes.c_int
        L.orc_f16_to_f32.restype = ctypes.c_float
        L.orc_f16_to_f32.argtypes = [ctypes.c_uint16]
        L.orc_pow2i.restype = ctypes.c_float
        L.orc_pow2i.argtypes = [ci]
        L.rf_decode_e2m1.restype = ctypes.c_float
        L.rf_decode_e2m1.argtypes = [ctypes.c_uint8]
        L.rf_decode_e2m3.restype = ctypes.c_float
        L.rf_decode_e2m3.argtypes = [ctypes.c_uint8]
        L.rf_encode_e2m1.restype = ctypes.c_uint8
        L.rf_encode_e2m1.argtypes = [ctypes.c_float]
        L.rf_encode_e2m3.restype = ctypes.c_uint8
        L.rf_encode_e2m3.argtypes = [ctypes.c_float]
        L.rf_e8m0_from_f32.restype = ctypes.c_int8
        L.rf_e8m0_from_f32.argtypes = [ctypes.c_float]
        L.orc_dequantize.restype = ci
        L.orc_dequantize.argtypes = [ci, ci, u8p, sz, sz, f32p]
        L.orc_dequantize_omp.restype = ci
        L.orc_dequantize_omp.argtypes = [ci, ci, u8p, sz, sz, f32p, ci]
        L.rf_dequant_q8_0_i8.restype = None
        L.rf_dequant_q8_0_i8.argtypes = [u8p, sz, sz, f32p]
        L.orc_block_bytes.restype = sz
        L.orc_block_bytes.argtypes = [ci, ci]
        L.orc_block_elems.restype = sz
        L.orc_block_elems.argtypes = [ci]
        for name in ("orc_matmul_f32", "orc_matmul_f32_nk"):
            getattr(L, name).restype = None
            getattr(L, name).argtypes = [f32p, f32p, ci, ci, ci, f32p]
        for name in ("orc_matmul_f64", "orc_matmul_f64_nk"):
            getattr(L, name).restype = None
            getattr(L, name).argtypes = [f32p, f32p, ci, ci, ci, f64p]
        for name in ("orc_matmul_f32_omp", "orc_matmul_f32_nk_omp"):
            getattr(L, name).restype = ci
            getattr(L, name).argtypes = [f32p, f32p, ci, ci, ci, f32p, ci]
        L.orc_max_threads.restype = ci
        L.rf_pack_6bit.argtypes = [u8p, sz, u8p]
        L.rf_unpack_6bit.argtypes = [u8p, sz, sz, u8p]
        L.rf_mxfpblock_pack_mxfp4.argtypes = [f32p, ctypes.POINTER(ctypes.c_int8), u8p]
        L.rf_mxfpblock_unpack_mxfp4.argtypes = [ctypes.c_int8, u8p, f32p]
        L.rf_mxfpblock_pack_mxfp6.argtypes = [f32p, ctypes.POINTER(ctypes.c_int8), u8p]
        L.rf_mxfpblock_unpack_mxfp6.argtypes = [ctypes.c_int8, u8p, f32p]
        _lib = L
    return _lib


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _bytes(data):
    a = np.ascontiguousarray(np.frombuffer(data, dtype=np.uint8) if isinstance(data, (bytes, bytearray))
                             else np.asarray(data, dtype=np.uint8))
    return a


def block_bytes(qtype, layout):
    return int(lib().orc_block_bytes(qtype, layout))


def block_elems(qtype):
    return int(lib().orc_block_elems(qtype))


def tensor_bytes(qtype, layout, n_elements):
    be = block_elems(qtype)
    return (n_elements + be - 1) // be * block_bytes(qtype, layout)


def dequantize(qtype, layout, data, n_elements, threads=1):
    """fp32 values of the first n_elements of a packed stream (reference CPU dequant)."""
    a = _bytes(data)
    out = np.empty(n_elements, dtype=np.float32)
    if threads == 1:
        rc = lib().orc_dequantize(qtype, layout, _ptr(a), a.size, n_elements, _ptr(out))
    else:
        rc = lib().orc_dequantize_omp(qtype, layout, _ptr(a), a.size, n_elements, _ptr(out), threads)
    if rc < 0:
        raise ValueError(f"unknown qtype/layout {qtype}/{layout}")
    return out


def dequant_q8_0_i8_variant(data, n_elements):
    a = _bytes(data)
    out = np.empty(n_elements, dtype=np.float32)
    lib().rf_dequant_q8_0_i8(_ptr(a), a.size, n_elements, _ptr(out))
    return out


def fused_dequant_rmsnorm(qtype, layout, data, seq_len, hidden, weight, eps):
    """Row-wise RMSNorm of the dequantised [seq_len, hidden] tensor times `weight` (fused_q4_0_rmsnorm)."""
    a = _bytes(data)
    w = np.ascontiguousarray(weight, dtype=np.float32)
    assert w.size == hidden
    out = np.empty((seq_len, hidden), dtype=np.float32)
    L = lib()
    L.orc_fused_dequant_rmsnorm.restype = ctypes.c_int
    L.orc_fused_dequant_rmsnorm.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int,
                                            ctypes.c_int, ctypes.c_void_p, ctypes.c_float, ctypes.c_void_p]
    rc = L.orc_fused_dequant_rmsnorm(qtype, layout, _ptr(a), a.size, seq_len, hidden, _ptr(w), eps, _ptr(out))
    if rc < 0:
        raise ValueError(f"unknown qtype/layout {qtype}/{layout}")
    return out


def swiglu(gate, up):
    """gate * swish(up) in fp32, the order of kernels/swiglu.hip."""
    g = np.ascontiguousarray(gate, dtype=np.float32)
    u = np.ascontiguousarray(up, dtype=np.float32)
    assert g.shape == u.shape
    out = np.empty_like(g)
    L = lib()
    L.orc_swiglu.restype = None
    L.orc_swiglu.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]
    L.orc_swiglu(_ptr(g), _ptr(u), _ptr(out), g.size)
    return out


def add_row_bias(y, bias):
    """y[r, :] += bias (saxpy with alpha = 1 per row); returns a new array."""
    out = np.array(y, dtype=np.float32, order="C", copy=True)
    b = np.ascontiguousarray(bias, dtype=np.float32).reshape(-1)
    assert out.ndim == 2 and b.size == out.shape[1]
    L = lib()
    L.orc_add_row_bias.restype = None
    L.orc_add_row_bias.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t]
    L.orc_add_row_bias(_ptr(out), _ptr(b), out.shape[0], out.shape[1])
    return out


def mlp_swiglu(qtypes, layout, gate, up, down, x, hidden, n_ff):
    """HipBackend::mlp_swiglu on packed weights: cpu_matmul_f32 of x with the dequantised gate / up tensors
    ([n_ff, hidden], stored as rows of hidden values), swiglu, cpu_matmul_f32 with the dequantised down tensor
    ([hidden, n_ff]). qtypes = (gate, up, down) quantisation types."""
    xg = np.ascontiguousarray(x, dtype=np.float32)
    wg = dequantize(qtypes[0], layout, gate, n_ff * hidden).reshape(n_ff, hidden)
    wu = dequantize(qtypes[1], layout, up, n_ff * hidden).reshape(n_ff, hidden)
    wd = dequantize(qtypes[2], layout, down, hidden * n_ff).reshape(hidden, n_ff)
    t = max_threads()
    act = swiglu(matmul_f32(xg, wg, nk=True, threads=t), matmul_f32(xg, wu, nk=True, threads=t))
    return matmul_f32(act, wd, nk=True, threads=t), act


def matmul_f32(a, b, nk=False, threads=1):
    """cpu_matmul_f32: fp32, ascending k, multiply then add.

    nk=False: b is [K,N] row-major (the reference's call); nk=True: b is [N,K].
    """
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    m, k = a.shape
    n = b.shape[0] if nk else b.shape[1]
    assert (b.shape[1] if nk else b.shape[0]) == k
    c = np.empty((m, n), dtype=np.float32)
    L = lib()
    if threads == 1:
        (L.orc_matmul_f32_nk if nk else L.orc_matmul_f32)(_ptr(a), _ptr(b), m, n, k, _ptr(c))
    else:
        (L.orc_matmul_f32_nk_omp if nk else L.orc_matmul_f32_omp)(_ptr(a), _ptr(b), m, n, k, _ptr(c), threads)
    return c


def matmul_f64(a, b, nk=False):
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    m, k = a.shape
    n = b.shape[0] if nk else b.shape[1]
    c = np.empty((m, n), dtype=np.float64)
    L = lib()
    (L.orc_matmul_f64_nk if nk else L.orc_matmul_f64)(_ptr(a), _ptr(b), m, n, k, _ptr(c))
    return c


def max_threads():
    return int(lib().orc_max_threads())


def f16_to_f32(bits):
    return float(lib().orc_f16_to_f32(int(bits) & 0xFFFF))


def pow2i(e):
    return float(lib().orc_pow2i(int(e)))
