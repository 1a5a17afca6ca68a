"""ctypes binding of libb200q.so -- exactly the entry points include/b200q.h declares.

The library is the product path: if it is missing this module raises, there is no CPU fallback.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200q.so")

OK = 0
ERR_INIT, ERR_NO_DEVICE, ERR_ALLOC, ERR_COPY, ERR_LAUNCH, ERR_DEVICE, ERR_INVALID, ERR_UNSUPPORTED, ERR_TIMEOUT = \
    -1, -2, -3, -4, -5, -6, -7, -8, -9
Q4_0, Q8_0, Q4_K, Q6_K, MXFP4, MXFP6_E2M3, MXFP6_E3M2, Q2_K, Q3_K, Q5_K = range(10)
LAYOUT_RF, LAYOUT_GGUF = 0, 1
ORIENT_NK, ORIENT_KN = 0, 1
F32, BF16 = 0, 1
MM_DEFAULT, MM_SEQUENTIAL, MM_NO_TENSOR, MM_SCATTER_BF16, MM_MX_NATIVE = 0, 1, 2, 4, 8


class DeviceInfo(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char * 128), ("sm_count", ctypes.c_int), ("cc_major", ctypes.c_int),
                ("cc_minor", ctypes.c_int), ("total_mem", ctypes.c_size_t), ("free_mem", ctypes.c_size_t),
                ("smem_per_block_optin", ctypes.c_size_t), ("l2_bytes", ctypes.c_int)]


GGUF_REFERENCE_FIXTURE = 1


class GgufTensorInfo(ctypes.Structure):
    """b200q_gguf_tensor"""
    _fields_ = [("name", ctypes.c_char_p), ("n_dims", ctypes.c_int), ("dims", ctypes.c_int64 * 4),
                ("ggml_type", ctypes.c_int), ("qtype", ctypes.c_int), ("layout", ctypes.c_int),
                ("n", ctypes.c_int64), ("k", ctypes.c_int64), ("file_offset", ctypes.c_int64),
                ("nbytes", ctypes.c_size_t)]


_vp, _i, _sz, _i64, _u = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_int64, ctypes.c_uint
_pvp = ctypes.POINTER(ctypes.c_void_p)

# name -> (restype, argtypes); one row per declaration in include/b200q.h
SIGNATURES = {
    "b200q_init": (_i, [_i, _pvp]),
    "b200q_init_on_stream": (_i, [_i, _vp, _pvp]),
    "b200q_destroy": (None, [_vp]),
    "b200q_last_error": (ctypes.c_char_p, []),
    "b200q_is_recoverable": (_i, [_i]),
    "b200q_get_device_info": (_i, [_vp, ctypes.POINTER(DeviceInfo)]),
    "b200q_malloc": (_i, [_vp, _sz, _pvp]),
    "b200q_free": (_i, [_vp, _vp]),
    "b200q_memcpy_h2d": (_i, [_vp, _vp, _vp, _sz]),
    "b200q_memcpy_d2h": (_i, [_vp, _vp, _vp, _sz]),
    "b200q_memset": (_i, [_vp, _vp, _i, _sz]),
    "b200q_synchronize": (_i, [_vp]),
    "b200q_stream": (_vp, [_vp]),
    "b200q_timer_start": (_i, [_vp]),
    "b200q_timer_stop_ms": (_i, [_vp, ctypes.POINTER(ctypes.c_float)]),
    "b200q_block_elems": (_i, [_i]),
    "b200q_block_bytes": (_sz, [_i, _i]),
    "b200q_tensor_bytes": (_sz, [_i, _i, _i64]),
    "b200q_weight_upload": (_i, [_vp, _vp, _sz, _i, _i, _i, _i64, _i64, _i, _i, _pvp]),
    "b200q_weight_free": (_i, [_vp]),
    "b200q_weight_info": (_i, [_vp, ctypes.POINTER(_i), ctypes.POINTER(_i), ctypes.POINTER(_i), ctypes.POINTER(_i64),
                               ctypes.POINTER(_i64), ctypes.POINTER(_i64), ctypes.POINTER(_i64), ctypes.POINTER(_sz)]),
    "b200q_dequantize": (_i, [_vp, _vp, _vp, _i64]),
    "b200q_dequantize_bytes": (_i, [_vp, _vp, _sz, _i, _i, _vp, _i64]),
    "b200q_matmul": (_i, [_vp, _vp, _vp, _i, _vp, _i, _i, _u]),
    "b200q_matmul_ex": (_i, [_vp, _vp, _vp, _i, _i64, _vp, _i, _i64, _i, _u]),
    "b200q_matmul_noalloc": (_i, [_vp, _vp, _vp, _vp, _i]),
    "b200q_matmul_host": (_i, [_vp, _vp, _vp, _vp, _i, _u]),
    "b200q_batch_create": (_i, [_vp, _i, _pvp, _pvp, _pvp, _i, _pvp]),
    "b200q_batch_run": (_i, [_vp, _vp, ctypes.POINTER(ctypes.c_float)]),
    "b200q_batch_run_host": (_i, [_vp, _vp, _vp, _vp]),
    "b200q_batch_free": (_i, [_vp]),
    "b200q_batch_weight_bytes": (_sz, [_vp]),
    "b200q_batch_launches": (_i, [_vp]),
    "b200q_matmul_scatter": (_i, [_vp, _vp, _vp, _i, _pvp, _i, _i64, _i, _u]),
    "b200q_peer_signal": (_i, [_vp, _pvp, _i, _i, _i]),
    "b200q_peer_wait": (_i, [_vp, _vp, _i, _i, _i]),
    "b200q_arena_tensor_bytes": (_i, [_i, _i, _i, _i64, _i64, ctypes.POINTER(ctypes.c_size_t)]),
    "b200q_arena_create": (_i, [_vp, ctypes.c_size_t, _pvp]),
    "b200q_arena_upload": (_i, [_vp, _vp, _vp, ctypes.c_size_t, _i, _i, _i, _i64, _i64, _i, _i, _pvp]),
    "b200q_arena_info": (_i, [_vp, ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(_i64), ctypes.POINTER(_i64)]),
    "b200q_arena_free": (_i, [_vp]),
    "b200q_gguf_upload_all": (_i, [_vp, _vp, _i, _i, _pvp, _pvp, _i64]),
    "b200q_matmul_scatter_signal": (_i, [_vp, _vp, _vp, _i, _pvp, _i, _i64, _i, _u, _pvp, _i, _i]),
    "b200q_ipc_get_handle": (_i, [_vp, _vp, _vp]),
    "b200q_ipc_open": (_i, [_vp, _vp, _pvp]),
    "b200q_ipc_close": (_i, [_vp, _vp]),
    "b200q_selftest_bounded_wait": (_i, [_vp, _i64]),
    "b200q_fused_dequant_rmsnorm": (_i, [_vp, _vp, _vp, _vp, ctypes.c_float]),
    "b200q_swiglu": (_i, [_vp, _vp, _vp, _vp, _i64, _i64]),
    "b200q_add_row_bias": (_i, [_vp, _vp, _i64, _vp, _i64, _i64]),
    "b200q_mlp_create": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _pvp]),
    "b200q_mlp_run": (_i, [_vp, _vp]),
    "b200q_mlp_free": (_i, [_vp]),
    "b200q_get_rows": (_i, [_vp, _vp, _vp, _i64, _vp, _i64]),
    "b200q_get_rows_host": (_i, [_vp, _vp, _vp, _i64, _vp, _i64]),
    "b200q_gguf_open": (_i, [ctypes.c_char_p, _i, _pvp]),
    "b200q_gguf_close": (None, [_vp]),
    "b200q_gguf_tensor_count": (_i64, [_vp]),
    "b200q_gguf_kv_count": (_i64, [_vp]),
    "b200q_gguf_find_tensor": (_i64, [_vp, ctypes.c_char_p]),
    "b200q_gguf_tensor_info": (_i, [_vp, _i64, ctypes.POINTER(GgufTensorInfo)]),
    "b200q_gguf_kv_key": (_i, [_vp, _i64, ctypes.POINTER(ctypes.c_char_p), ctypes.POINTER(_i)]),
    "b200q_gguf_meta_string": (_i, [_vp, ctypes.c_char_p, ctypes.c_char_p, _sz, ctypes.POINTER(_sz)]),
    "b200q_gguf_tensor_data": (_i, [_vp, _i64, _pvp, ctypes.POINTER(_sz)]),
    "b200q_gguf_upload_tensor": (_i, [_vp, _vp, _i64, _i, _i, _pvp]),
}

_lib = None


class B200QError(RuntimeError):
    """A non-zero status from the library; .status is the b200q_status code."""

    def __init__(self, status, message):
        super().__init__(f"b200q status {status}: {message}")
        self.status = status
        self.recoverable = status in (ERR_ALLOC, ERR_COPY, ERR_LAUNCH, ERR_DEVICE, ERR_TIMEOUT)


def load():
    """dlopen libb200q.so and set every prototype. Raises if the library was not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m rocmforge_b200.build` "
                              "(there is no CPU fallback)")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)      # AttributeError here means the .so and the header disagree
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status):
    if status != OK:
        raise B200QError(status, load().b200q_last_error().decode("utf-8", "replace"))
