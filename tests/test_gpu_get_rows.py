"""Quantised embedding lookup (GetRows on a packed token_embd) against the oracle's dequantised table.

Follows the reference's own GetRows cases (src/ggml/hip_backend/ops/get_rows.rs tests: ids in range pick their
rows, an id >= vocab_size is an error naming the id and the vocabulary size) on packed tables, bit-exact."""
import ctypes

import numpy as np
import pytest

from rocmforge_b200 import _lib, ops, synth
from rocmforge_b200.backend import QuantizedWeight

from gpu_util import backend

pytestmark = pytest.mark.gpu


@pytest.fixture()
def be():
    return backend()


@pytest.mark.parametrize("qtype,layout", [(synth.Q6_K, synth.GGUF), (synth.Q4_K, synth.GGUF), (synth.Q4_0, synth.RF),
                                          (synth.Q8_0, synth.GGUF), (synth.MXFP4, synth.RF), (synth.Q5_K, synth.GGUF)])
def test_get_rows_matches_dequantised_table(be, oracle, qtype, layout):
    vocab, n_embd = 1000, 768
    data = synth.gen_packed(qtype, layout, vocab * n_embd, synth.rng_for(31 + qtype))
    table = oracle.dequantize(qtype, layout, data, vocab * n_embd).reshape(vocab, n_embd)
    w = QuantizedWeight(be, data, qtype, layout, vocab, n_embd)
    tokens = np.array([5, 999, 0, 17, 17, 123, 998, 1], dtype=np.uint32)
    out = be.allocate_buffer(tokens.size * n_embd * 4)
    n = ops.get_rows(be, w, tokens, n_embd, vocab, out)
    assert n == tokens.size
    got = out.to_numpy(np.float32, tokens.size * n_embd).reshape(tokens.size, n_embd)
    assert np.array_equal(got.view(np.uint32), table[tokens].view(np.uint32))
    # padded token buffer: everything from the first 0 on is dropped, as execute_get_rows does
    n = ops.get_rows(be, w, tokens, n_embd, vocab, out, trim_padding=True)
    assert n == 2
    w.free(); out.free()


def test_get_rows_rejects_an_id_beyond_the_vocabulary_before_launching(be):
    vocab, n_embd = 64, 256
    data = synth.gen_packed(synth.Q6_K, synth.GGUF, vocab * n_embd, synth.rng_for(5))
    w = QuantizedWeight(be, data, synth.Q6_K, synth.GGUF, vocab, n_embd)
    out = be.allocate_buffer(2 * n_embd * 4)
    with pytest.raises(ValueError, match="Token ID 64 exceeds vocab size 64"):
        ops.get_rows(be, w, [3, 64], n_embd, vocab, out)
    ids = (ctypes.c_uint32 * 2)(3, 64)
    rc = be.lib.b200q_get_rows_host(be.ctx, w.handle, ids, 2, out.as_ptr(), n_embd)
    assert rc == _lib.ERR_INVALID
    assert b"Token ID 64 exceeds vocab size 64" in be.lib.b200q_last_error()
    w.free(); out.free()


def test_get_rows_device_ids_out_of_range_zero_fill_and_report(be, oracle):
    vocab, n_embd = 64, 256
    data = synth.gen_packed(synth.Q4_K, synth.GGUF, vocab * n_embd, synth.rng_for(6))
    table = oracle.dequantize(synth.Q4_K, synth.GGUF, data, vocab * n_embd).reshape(vocab, n_embd)
    w = QuantizedWeight(be, data, synth.Q4_K, synth.GGUF, vocab, n_embd)
    ids = np.array([7, -1, 64, 63], dtype=np.int32)
    idb = be.allocate_buffer(ids.nbytes); idb.copy_from_host(ids)
    out = be.allocate_buffer(ids.size * n_embd * 4)
    out.fill(0xFF)
    _lib.check(be.lib.b200q_get_rows(be.ctx, w.handle, idb.as_ptr(), ids.size, out.as_ptr(), n_embd))
    rc = be.lib.b200q_synchronize(be.ctx)
    assert rc == _lib.ERR_INVALID and b"2 token id(s)" in be.lib.b200q_last_error()
    got = out.to_numpy(np.float32, ids.size * n_embd).reshape(ids.size, n_embd)
    assert np.array_equal(got[0], table[7]) and np.array_equal(got[3], table[63])
    assert not got[1].any() and not got[2].any()
    be.synchronize()   # the status words were cleared: the context is usable
    w.free(); idb.free(); out.free()
