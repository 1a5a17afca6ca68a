"""CPU-only checks of the C-ABI library: it loads, exports every symbol include/b200q.h declares, answers the
size queries, and reports 'no device' as a status code instead of crashing."""
import ctypes
import os
import re

import pytest

from rocmforge_b200 import _lib, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from rocmforge_b200 import build
    build.build()
    return _lib.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200q.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200q_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(lib):
    names = declared_symbols()
    assert len(names) >= 25
    assert set(names) == set(_lib.SIGNATURES), set(names) ^ set(_lib.SIGNATURES)
    for n in names:
        assert hasattr(lib, n), n


def test_size_queries_match_the_format_tables(lib):
    for qt in range(10):
        assert lib.b200q_block_elems(qt) == synth.block_elems(qt)
        for lay in (0, 1):
            assert lib.b200q_block_bytes(qt, lay) == synth.block_bytes(qt, lay)
            for n in (0, 1, 31, 32, 33, 255, 256, 257, 4864 * 896):
                assert lib.b200q_tensor_bytes(qt, lay, n) == synth.tensor_bytes(qt, lay, n)
    assert lib.b200q_block_bytes(10, 0) == 0 and lib.b200q_block_elems(-1) == 0
    # the byte counts the benchmark configurations are quoted on
    assert lib.b200q_tensor_bytes(_lib.Q4_0, 1, 4864 * 896) == 2_451_456
    assert lib.b200q_tensor_bytes(_lib.Q4_0, 0, 4864 * 896) == 2_723_840
    assert lib.b200q_tensor_bytes(_lib.Q8_0, 1, 896 * 896) == 852_992
    assert lib.b200q_tensor_bytes(_lib.Q4_K, 1, 11008 * 4096) == 25_362_432
    assert lib.b200q_tensor_bytes(_lib.Q6_K, 1, 151936 * 896) == 111_672_960
    assert lib.b200q_tensor_bytes(_lib.MXFP4, 1, 28672 * 8192) == 124_780_544
    assert lib.b200q_tensor_bytes(_lib.MXFP6_E2M3, 1, 28672 * 8192) == 183_500_800
    step = sum(lib.b200q_tensor_bytes(q, 1, n * k) for _, q, n, k in synth.qwen2_0p5b_step())
    assert step == 339_916_416


def test_recoverable_split_follows_the_reference(lib):
    rec = {_lib.ERR_ALLOC, _lib.ERR_COPY, _lib.ERR_LAUNCH, _lib.ERR_DEVICE, _lib.ERR_TIMEOUT}
    for s in range(-9, 1):
        assert bool(lib.b200q_is_recoverable(s)) == (s in rec)


def test_no_device_is_a_status_not_a_crash(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    p = ctypes.c_void_p()
    rc = lib.b200q_init(0, ctypes.byref(p))
    assert rc == _lib.ERR_NO_DEVICE and not p.value
    assert b"no CUDA device" in lib.b200q_last_error()
    assert lib.b200q_synchronize(None) == _lib.ERR_INVALID
    assert lib.b200q_weight_free(None) == 0
    with pytest.raises(_lib.B200QError) as e:
        from rocmforge_b200.backend import B200Backend
        B200Backend(0)
    assert e.value.status == _lib.ERR_NO_DEVICE and not e.value.recoverable


def test_arena_tensor_bytes_is_host_arithmetic():
    """Planes plus the decode image (NK tensors of the decode kernel's formats with k % 128 == 0), each rounded up to
    256 bytes: computed without touching a device."""
    import ctypes
    from rocmforge_b200 import _lib, synth
    lib = _lib.load()
    def nbytes(qt, orient, n, k):
        b = ctypes.c_size_t()
        assert lib.b200q_arena_tensor_bytes(qt, synth.GGUF, orient, n, k, ctypes.byref(b)) == 0
        return b.value
    n, k = 64, 512
    packed = n * k // 256 * 144
    nk, kn = nbytes(synth.Q4_K, _lib.ORIENT_NK, n, k), nbytes(synth.Q4_K, _lib.ORIENT_KN, n, k)
    assert packed <= kn <= packed + 512 and kn % 256 == 0       # the planes (with their tail padding); no image for KN
    items = (n // 16) * (k // 128)
    assert nk == kn + (items * 1216 + 256 + 255) // 256 * 256
    assert nbytes(synth.Q2_K, _lib.ORIENT_NK, n, k) % 256 == 0  # a format without an image
    b = ctypes.c_size_t()
    assert lib.b200q_arena_tensor_bytes(99, synth.GGUF, _lib.ORIENT_NK, n, k, ctypes.byref(b)) != 0
