"""Device plumbing above the C ABI: the counterpart of ROCmForge's HipBackend / HipBuffer.

Mirrors src/backend/hip_backend/backend.rs (HipBackend: allocate_buffer :704, synchronize :753) and
src/backend/hip_backend/memory.rs:19-31 (HipBuffer: copy_from_host / copy_to_host / as_ptr / size).
Errors surface as B200QError carrying the library's status code and message, the way the reference
returns HipError values (src/backend/hip_backend/error.rs:6-28).
"""
import ctypes

import numpy as np

from . import _lib
from ._lib import B200QError, check  # noqa: F401


def _host_ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def as_u8(data):
    """bytes / bytearray / ndarray -> contiguous uint8 ndarray (no copy when possible)."""
    if isinstance(data, (bytes, bytearray, memoryview)):
        return np.frombuffer(data, dtype=np.uint8)
    a = np.asarray(data)
    if a.dtype != np.uint8:
        a = a.view(np.uint8)
    return np.ascontiguousarray(a).reshape(-1)


class DeviceBuffer:
    """A device allocation owned by a backend (HipBuffer)."""

    def __init__(self, backend, size):
        self.backend = backend
        self.size = int(size)
        p = ctypes.c_void_p()
        check(backend.lib.b200q_malloc(backend.ctx, self.size, ctypes.byref(p)))
        self.ptr = p.value

    def as_ptr(self):
        return self.ptr

    def copy_from_host(self, data):
        a = np.ascontiguousarray(data)
        if a.nbytes > self.size:
            raise B200QError(_lib.ERR_INVALID, f"copy_from_host: {a.nbytes} bytes into a {self.size}-byte buffer")
        check(self.backend.lib.b200q_memcpy_h2d(self.backend.ctx, self.ptr, _host_ptr(a), a.nbytes))

    def copy_to_host(self, out):
        if not out.flags["C_CONTIGUOUS"]:
            raise B200QError(_lib.ERR_INVALID, "copy_to_host: destination must be contiguous")
        if out.nbytes > self.size:
            raise B200QError(_lib.ERR_INVALID, f"copy_to_host: {out.nbytes} bytes from a {self.size}-byte buffer")
        check(self.backend.lib.b200q_memcpy_d2h(self.backend.ctx, _host_ptr(out), self.ptr, out.nbytes))
        return out

    def to_numpy(self, dtype, count):
        out = np.empty(count, dtype=dtype)
        return self.copy_to_host(out)

    def fill(self, byte):
        check(self.backend.lib.b200q_memset(self.backend.ctx, self.ptr, byte, self.size))

    def free(self):
        if self.ptr:
            self.backend.lib.b200q_free(self.backend.ctx, self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            if self.ptr and self.backend.ctx:
                self.free()
        except Exception:
            pass


class B200Backend:
    """One device + one stream (HipBackend). `stream` may be a raw cudaStream_t to share a caller's stream."""

    def __init__(self, device=0, stream=None):
        self.lib = _lib.load()
        p = ctypes.c_void_p()
        if stream is None:
            check(self.lib.b200q_init(device, ctypes.byref(p)))
        else:
            check(self.lib.b200q_init_on_stream(device, ctypes.c_void_p(stream), ctypes.byref(p)))
        self.ctx = p
        self.device = device

    def allocate_buffer(self, size):
        return DeviceBuffer(self, size)

    def ipc_handle(self, buf):
        """64 opaque bytes another process on this node can turn into a pointer to `buf` (ipc_open)."""
        h = (ctypes.c_uint8 * 64)()
        check(self.lib.b200q_ipc_get_handle(self.ctx, buf.as_ptr(), h))
        return bytes(h)

    def ipc_open(self, handle):
        p = ctypes.c_void_p()
        hb = (ctypes.c_uint8 * 64).from_buffer_copy(handle)
        check(self.lib.b200q_ipc_open(self.ctx, hb, ctypes.byref(p)))
        return p

    def ipc_close(self, ptr):
        check(self.lib.b200q_ipc_close(self.ctx, ptr))

    def peer_signal(self, flag_arrays, my_rank, epoch):
        """Behind a scattered product: store `epoch` into slot my_rank of every other rank's flag array
        (DeviceBuffers or raw, peer-mapped pointers, one per rank)."""
        ptrs = [f.as_ptr() if isinstance(f, DeviceBuffer) else f for f in flag_arrays]
        arr = (ctypes.c_void_p * len(ptrs))(*[p.value if isinstance(p, ctypes.c_void_p) else p for p in ptrs])
        check(self.lib.b200q_peer_signal(self.ctx, arr, len(ptrs), my_rank, epoch))

    def peer_wait(self, own_flags, n_ranks, my_rank, epoch):
        """Hold the stream (bounded) until every other rank has signalled `epoch` into this rank's flag array."""
        p = own_flags.as_ptr() if isinstance(own_flags, DeviceBuffer) else own_flags
        check(self.lib.b200q_peer_wait(self.ctx, p, n_ranks, my_rank, epoch))

    def synchronize(self):
        check(self.lib.b200q_synchronize(self.ctx))

    def stream(self):
        return self.lib.b200q_stream(self.ctx)

    def device_info(self):
        info = _lib.DeviceInfo()
        check(self.lib.b200q_get_device_info(self.ctx, ctypes.byref(info)))
        return dict(name=info.name.decode(), sm_count=info.sm_count, cc=(info.cc_major, info.cc_minor),
                    total_mem=info.total_mem, free_mem=info.free_mem, smem_per_block_optin=info.smem_per_block_optin,
                    l2_bytes=info.l2_bytes)

    def timer_start(self):
        check(self.lib.b200q_timer_start(self.ctx))

    def timer_stop_ms(self):
        ms = ctypes.c_float()
        check(self.lib.b200q_timer_stop_ms(self.ctx, ctypes.byref(ms)))
        return ms.value

    def close(self):
        if self.ctx:
            self.lib.b200q_destroy(self.ctx)
            self.ctx = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class WeightArena:
    """ModelWeightArena (src/memory/arena.rs:82,206) for packed tensors: one device allocation, 256-byte aligned
    bump allocation. Uploads are queued on the backend's stream without waiting for one another."""

    def __init__(self, backend, capacity=None, handle=None):
        self.backend = backend
        if handle is None:
            handle = ctypes.c_void_p()
            check(backend.lib.b200q_arena_create(backend.ctx, int(capacity), ctypes.byref(handle)))
        self.handle = handle

    @staticmethod
    def tensor_bytes(backend, qtype, layout, n_local, k, orient=_lib.ORIENT_NK) -> int:
        b = ctypes.c_size_t()
        check(backend.lib.b200q_arena_tensor_bytes(qtype, layout, orient, n_local, k, ctypes.byref(b)))
        return b.value

    def upload(self, data, qtype, layout, n, k, orient=_lib.ORIENT_NK, shard_rank=0, shard_count=1) -> "QuantizedWeight":
        a = as_u8(data)
        h = ctypes.c_void_p()
        check(self.backend.lib.b200q_arena_upload(self.backend.ctx, self.handle, _host_ptr(a), a.size, qtype, layout, orient, n, k,
                                                  shard_rank, shard_count, ctypes.byref(h)))
        return QuantizedWeight.from_handle(self.backend, h)

    def info(self) -> dict:
        cap, used = ctypes.c_size_t(), ctypes.c_size_t()
        t, live = ctypes.c_int64(), ctypes.c_int64()
        check(self.backend.lib.b200q_arena_info(self.handle, ctypes.byref(cap), ctypes.byref(used), ctypes.byref(t), ctypes.byref(live)))
        return {"capacity": cap.value, "used": used.value, "tensors": t.value, "live": live.value}

    def free(self):
        """Refused (B200Error) while weight handles of the arena are alive."""
        if self.handle:
            check(self.backend.lib.b200q_arena_free(self.handle))
            self.handle = None


class QuantizedWeight:
    """A packed tensor resident on the device (what load_tensor_to_gpu hands out for a quantized weight)."""

    def __init__(self, backend, data, qtype, layout, n, k, orient=_lib.ORIENT_NK, shard_rank=0, shard_count=1):
        self.backend = backend
        a = as_u8(data)
        h = ctypes.c_void_p()
        check(backend.lib.b200q_weight_upload(backend.ctx, _host_ptr(a), a.size, qtype, layout, orient, n, k,
                                              shard_rank, shard_count, ctypes.byref(h)))
        self.handle = h
        self.qtype, self.layout, self.orient = qtype, layout, orient
        self.n_total, self.k = n, k
        self.n_local = n // shard_count
        self.row0 = self.n_local * shard_rank
        psz = ctypes.c_size_t()
        check(backend.lib.b200q_weight_info(h, None, None, None, None, None, None, None, ctypes.byref(psz)))
        self.packed_bytes = psz.value

    @classmethod
    def from_handle(cls, backend, handle):
        """Wrap a b200q_weight* another entry point produced (the GGUF loader's upload)."""
        self = cls.__new__(cls)
        self.backend = backend
        self.handle = handle
        q, l, o = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        nl, k, r0, nt = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
        psz = ctypes.c_size_t()
        check(backend.lib.b200q_weight_info(handle, ctypes.byref(q), ctypes.byref(l), ctypes.byref(o), ctypes.byref(nl),
                                            ctypes.byref(k), ctypes.byref(r0), ctypes.byref(nt), ctypes.byref(psz)))
        self.qtype, self.layout, self.orient = q.value, l.value, o.value
        self.n_local, self.k, self.row0, self.n_total = nl.value, k.value, r0.value, nt.value
        self.packed_bytes = psz.value
        return self

    def dequantize(self, out, n_elements=None):
        n = self.n_local * self.k if n_elements is None else n_elements
        check(self.backend.lib.b200q_dequantize(self.backend.ctx, self.handle, out.as_ptr(), n))

    def matmul(self, x, y, m, x_dtype=_lib.F32, y_dtype=_lib.F32, flags=0, ldx=0, ldy=0):
        xp = x.as_ptr() if isinstance(x, DeviceBuffer) else x
        yp = y.as_ptr() if isinstance(y, DeviceBuffer) else y
        check(self.backend.lib.b200q_matmul_ex(self.backend.ctx, self.handle, xp, x_dtype, ldx, yp, y_dtype, ldy, m, flags))

    def matmul_scatter(self, x, outputs, m, ldy, x_dtype=_lib.F32, flags=0):
        """Sharded product with the gather fused in: this shard's columns are stored into every full output
        [m, ldy] listed (DeviceBuffers or raw device pointers, own GPU's or peer-mapped)."""
        xp = x.as_ptr() if isinstance(x, DeviceBuffer) else x
        ptrs = [o.as_ptr() if isinstance(o, DeviceBuffer) else o for o in outputs]
        arr = (ctypes.c_void_p * len(ptrs))(*[p.value if isinstance(p, ctypes.c_void_p) else p for p in ptrs])
        check(self.backend.lib.b200q_matmul_scatter(self.backend.ctx, self.handle, xp, x_dtype, arr, len(ptrs), ldy, m, flags))

    def matmul_scatter_signal(self, x, outputs, m, ldy, flag_arrays, my_rank, epoch, x_dtype=_lib.F32, flags=0):
        """matmul_scatter, then `epoch` into slot my_rank of every other rank's flag array (raised by the decode kernel's
        last CTA itself at m <= 8). outputs[p] and flag_arrays[p] belong to rank p."""
        xp = x.as_ptr() if isinstance(x, DeviceBuffer) else x
        conv = lambda seq: (ctypes.c_void_p * len(seq))(*[(q.as_ptr() if isinstance(q, DeviceBuffer) else q) if not isinstance(q, ctypes.c_void_p) else q.value for q in seq])
        check(self.backend.lib.b200q_matmul_scatter_signal(self.backend.ctx, self.handle, xp, x_dtype, conv(outputs), len(outputs), ldy,
                                                           m, flags, conv(flag_arrays), my_rank, epoch))

    def matmul_host(self, x, m=None, flags=0):
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, self.k)
        m = x.shape[0] if m is None else m
        y = np.empty((m, self.n_local), dtype=np.float32)
        check(self.backend.lib.b200q_matmul_host(self.backend.ctx, self.handle, _host_ptr(x), _host_ptr(y), m, flags))
        return y

    def free(self):
        if self.handle:
            self.backend.lib.b200q_weight_free(self.handle)
            self.handle = None

    def __del__(self):
        try:
            if self.handle and self.backend.ctx:
                self.free()
        except Exception:
            pass
