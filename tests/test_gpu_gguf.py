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
