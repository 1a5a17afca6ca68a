"""Helpers shared by the GPU parity tests (all device work goes through the C ABI)."""
import numpy as np

from rocmforge_b200 import _lib, synth
from rocmforge_b200.backend import B200Backend, QuantizedWeight

ALL_FMTS = [(qt, lay) for qt in range(10) for lay in (0, 1)]
FMT_IDS = [f"{synth.QNAMES[q]}-{synth.LAYOUT_NAMES[l]}" for q, l in ALL_FMTS]

_backend = None


def backend():
    global _backend
    if _backend is None:
        _backend = B200Backend(0)
    return _backend


def bits_equal(a, b):
    """Bitwise equality of fp32 arrays, NaNs compare equal to NaNs."""
    a = np.ascontiguousarray(a, dtype=np.float32).reshape(-1)
    b = np.ascontiguousarray(b, dtype=np.float32).reshape(-1)
    return bool(np.all((a.view(np.uint32) == b.view(np.uint32)) | (np.isnan(a) & np.isnan(b))))


def gpu_dequant_bytes(be, qt, lay, data, n, canary=64):
    """b200q_dequantize_bytes into a canary-padded buffer; returns the n floats."""
    buf = be.allocate_buffer((n + 2 * canary) * 4)
    buf.fill(0xCD)
    import ctypes
    a = np.ascontiguousarray(data, dtype=np.uint8)
    _lib.check(be.lib.b200q_dequantize_bytes(be.ctx, a.ctypes.data_as(ctypes.c_void_p) if a.size else None, a.size, qt, lay,
                                             buf.ptr + canary * 4, n))
    be.synchronize()
    out = buf.to_numpy(np.uint32, n + 2 * canary)
    assert np.all(out[:canary] == 0xCDCDCDCD) and np.all(out[canary + n:] == 0xCDCDCDCD), "write outside the output"
    buf.free()
    return out[canary:canary + n].view(np.float32).copy()


def gpu_matmul(be, w, x, m, flags=0, y_canary=32):
    """y[m, n_local] through b200q_matmul with device buffers; checks a canary after y."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    xb = be.allocate_buffer(max(x.nbytes, 16))
    xb.copy_from_host(x)
    n = w.n_local
    yb = be.allocate_buffer((m * n + y_canary) * 4)
    yb.fill(0xCD)
    w.matmul(xb, yb, m, flags=flags)
    be.synchronize()
    out = yb.to_numpy(np.uint32, m * n + y_canary)
    assert np.all(out[m * n:] == 0xCDCDCDCD), "write outside the output"
    xb.free()
    yb.free()
    return out[:m * n].view(np.float32).reshape(m, n).copy()


def rel_err(y, ref):
    """max |y - ref| / max |ref| (the normalisation the tolerance of the path is quoted in)."""
    ref = np.asarray(ref, dtype=np.float64)
    denom = max(float(np.max(np.abs(ref))), 1e-30)
    return float(np.max(np.abs(np.asarray(y, dtype=np.float64) - ref))) / denom


__all__ = ["ALL_FMTS", "FMT_IDS", "backend", "bits_equal", "gpu_dequant_bytes", "gpu_matmul", "rel_err", "QuantizedWeight"]
