"""GGUF file -> packed upload -> kernels, end to end on the GPU, against the oracle fed with the file's bytes."""
import numpy as np
import pytest

from rocmforge_b200 import synth
from rocmforge_b200.gguf_loader import GgufLoader

from gpu_util import backend, rel_err
from test_gguf_loader import make_tensors, reference_style_file, write_model

pytestmark = pytest.mark.gpu
gguf = pytest.importorskip("gguf")


def test_file_to_decode_and_prefill_products(oracle, tmp_path):
    tensors = make_tensors(21)
    path = tmp_path / "m.gguf"
    write_model(path, tensors)
    be = backend()
    L = GgufLoader(path)
    weights = L.load_to_gpu(be)
    assert set(weights) == {t[0] for t in tensors}                 # the fp32 norm vector has no packed kernel
    assert L.load_tensor_to_gpu(tensors[0][0], be) is weights[tensors[0][0]]   # second request served from the cache
    rng = synth.rng_for(22)
    for name, qt, n, k, data in tensors:
        w = weights[name]
        assert (w.qtype, w.n_local, w.k) == (qt, n, k)
        wf = oracle.dequantize(qt, synth.GGUF, bytes(data), n * k).reshape(n, k)
        for m, tol in ((1, 1e-4), (64, 2e-3)):
            x = synth.gen_activations(m, k, rng)
            y = w.matmul_host(x)
            assert rel_err(y, oracle.matmul_f32(x, wf, nk=True, threads=8)) <= tol, (name, m)
    L.close()


def test_sharded_upload_from_file(oracle, tmp_path):
    tensors = make_tensors(23)[:1]
    path = tmp_path / "s.gguf"
    write_model(path, tensors)
    be = backend()
    L = GgufLoader(path)
    name, qt, n, k, data = tensors[0]
    x = synth.gen_activations(2, k, synth.rng_for(24))
    full = L.load_tensor_to_gpu(name, be).matmul_host(x)
    parts = [L.load_tensor_to_gpu(name, be, r, 4).matmul_host(x) for r in range(4)]
    assert np.array_equal(np.concatenate(parts, axis=1), full)
    L.close()


def test_reference_fixture_style_dequantises_bit_exactly(oracle, tmp_path):
    path = tmp_path / "ref.gguf"
    data = reference_style_file(path)
    be = backend()
    L = GgufLoader(path, reference_fixture=True)
    w = L.load_tensor_to_gpu("output.weight", be)
    out = be.allocate_buffer(8 * 64 * 4)
    w.dequantize(out)
    be.synchronize()
    got = out.to_numpy(np.float32, 8 * 64)
    assert np.array_equal(got.view(np.uint32), oracle.dequantize(synth.Q4_0, synth.RF, bytes(data), 8 * 64).view(np.uint32))
    L.close()


def test_bulk_upload_into_one_arena_equals_per_tensor_uploads(oracle, tmp_path):
    """load_to_gpu_async: every packed tensor of the file in ONE allocation, uploads queued without waiting for one
    another. Products and dequantised values equal those of tensors uploaded one by one, bit for bit."""
    from rocmforge_b200._lib import B200QError as B200Error
    from rocmforge_b200.backend import WeightArena
    tensors = make_tensors(31)
    path = tmp_path / "bulk.gguf"
    write_model(path, tensors)
    be = backend()
    L = GgufLoader(path)
    weights = L.load_to_gpu_async(be)
    assert set(weights) == {t[0] for t in tensors}
    arena = L.arenas[0]
    info = arena.info()
    want = sum(WeightArena.tensor_bytes(be, qt, synth.GGUF, n, k) for _, qt, n, k, _ in tensors)
    assert info["tensors"] == info["live"] == len(tensors)
    assert info["used"] == want == info["capacity"] and want % 256 == 0
    assert L.load_tensor_to_gpu(tensors[0][0], be) is weights[tensors[0][0]]        # served from the cache afterwards
    with pytest.raises(B200Error):
        arena.free()                                                                # handles are alive
    L2 = GgufLoader(path)
    rng = synth.rng_for(32)
    for name, qt, n, k, data in tensors:
        single = L2.load_tensor_to_gpu(name, be)
        for m in (1, 8, 64):
            x = synth.gen_activations(m, k, rng)
            assert np.array_equal(weights[name].matmul_host(x), single.matmul_host(x)), (name, m)
        a, b = be.allocate_buffer(n * k * 4), be.allocate_buffer(n * k * 4)
        weights[name].dequantize(a)
        single.dequantize(b)
        be.synchronize()
        assert np.array_equal(a.to_numpy(np.uint32, n * k), b.to_numpy(np.uint32, n * k))
        assert np.array_equal(a.to_numpy(np.float32, n * k).view(np.uint32), oracle.dequantize(qt, synth.GGUF, bytes(data), n * k).view(np.uint32))
        a.free(); b.free()
    L2.close()
    L.close()                                                                       # frees the handles, then the arena
    assert L.arenas == []


def test_arena_refuses_what_does_not_fit(tmp_path):
    from rocmforge_b200._lib import B200QError as B200Error
    from rocmforge_b200.backend import WeightArena
    be = backend()
    qt, n, k = synth.Q4_K, 64, 256
    data = synth.gen_packed(qt, synth.GGUF, n * k, synth.rng_for(33))
    need = WeightArena.tensor_bytes(be, qt, synth.GGUF, n, k)
    arena = WeightArena(be, need + 256)
    w = arena.upload(data, qt, synth.GGUF, n, k)
    with pytest.raises(B200Error) as e:
        arena.upload(data, qt, synth.GGUF, n, k)
    assert "arena" in str(e.value)
    x = synth.gen_activations(1, k, synth.rng_for(34))
    y = w.matmul_host(x)
    assert np.all(np.isfinite(y))
    w.free()
    arena.free()


def test_bulk_upload_of_a_rank_s_shards(oracle, tmp_path):
    """load_to_gpu_async with shard_rank / shard_count: every tensor whose rows divide is cut like a per-tensor sharded
    upload; the arena is sized for the shards, not for the whole tensors."""
    from rocmforge_b200.backend import WeightArena
    tensors = make_tensors(41)
    path = tmp_path / "bulk_shards.gguf"
    write_model(path, tensors)
    be = backend()
    rng = synth.rng_for(42)
    loaders = [GgufLoader(path) for _ in range(2)]
    parts = [L.load_to_gpu_async(be, shard_rank=r, shard_count=2) for r, L in enumerate(loaders)]
    whole = GgufLoader(path)
    for name, qt, n, k, data in tensors:
        x = synth.gen_activations(2, k, rng)
        full = whole.load_tensor_to_gpu(name, be).matmul_host(x)
        if n % 2 == 0:
            assert parts[0][name].n_local == n // 2 and parts[1][name].row0 == n // 2
            got = np.concatenate([p[name].matmul_host(x) for p in parts], axis=1)
        else:
            assert parts[0][name].n_local == n
            got = parts[1][name].matmul_host(x)
        assert rel_err(got, full) <= 2e-6, name
    used = loaders[0].arenas[0].info()["used"]
    want = sum(WeightArena.tensor_bytes(be, qt, synth.GGUF, n // 2 if n % 2 == 0 else n, k) for _, qt, n, k, _ in tensors)
    assert used == want
    for L in loaders + [whole]:
        L.close()
