"""GGUF container parsing (host-only part of the loader row): files written by the third-party `gguf`
package (an independent writer) and by hand in the style of the reference's own fixtures, parsed by the C
library; error behaviour follows src/loader/gguf/header.rs and metadata.rs."""
import os
import struct

import numpy as np
import pytest

from rocmforge_b200 import _lib, synth
from rocmforge_b200._lib import B200QError
from rocmforge_b200.gguf_loader import GgufLoader, GgufMetadata, layer_tensor_names, update_metadata

gguf = pytest.importorskip("gguf")

ROW_BYTES = {synth.Q4_0: (32, 18), synth.Q8_0: (32, 34), synth.Q4_K: (256, 144), synth.Q6_K: (256, 210)}
GG = {synth.Q4_0: "Q4_0", synth.Q8_0: "Q8_0", synth.Q4_K: "Q4_K", synth.Q6_K: "Q6_K"}


def write_model(path, tensors, arch="qwen2", extra=None):
    w = gguf.GGUFWriter(str(path), arch)
    w.add_uint32(f"{arch}.block_count", 2)
    w.add_uint32(f"{arch}.embedding_length", 512)
    w.add_uint32(f"{arch}.attention.head_count", 8)
    w.add_uint32(f"{arch}.attention.head_count_kv", 2)
    w.add_float32(f"{arch}.attention.layer_norm_rms_epsilon", 1e-5)
    w.add_uint64("some.u64", 2 ** 40 + 3)
    w.add_int32("some.i32", -7)
    w.add_bool("some.flag", True)
    w.add_string("general.name", "synthetic model")
    w.add_array("tokenizer.ggml.tokens", ["<s>", "</s>", "hello", "wörld"])
    w.add_array("tokenizer.ggml.scores", [0.0, -1.5, 2.25])
    for k, v in (extra or {}).items():
        w.add_uint32(k, v)
    for name, qt, n, k, data in tensors:
        be, bb = ROW_BYTES[qt]
        w.add_tensor(name, np.frombuffer(data, dtype=np.uint8).reshape(n, k // be * bb),
                     raw_dtype=getattr(gguf.GGMLQuantizationType, GG[qt]))
    w.add_tensor("output_norm.weight", np.arange(512, dtype=np.float32))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


def make_tensors(seed=7):
    rng = synth.rng_for(seed)
    names = layer_tensor_names(0)
    spec = [(names["attn_q"], synth.Q4_K, 512, 512), (names["attn_k"], synth.Q4_K, 128, 512),
            (names["ffn_down"], synth.Q6_K, 512, 1024), ("blk.0.ffn_up.weight", synth.Q8_0, 96, 512),
            ("token_embd.weight", synth.Q4_0, 64, 512)]
    return [(nm, qt, n, k, synth.gen_packed(qt, synth.GGUF, n * k, rng)) for nm, qt, n, k in spec]


def test_file_from_independent_writer_round_trips(tmp_path):
    tensors = make_tensors()
    path = tmp_path / "m.gguf"
    write_model(path, tensors)
    L = GgufLoader(path)
    md = L.metadata
    assert (md.architecture, md.num_layers, md.hidden_size, md.num_heads, md.num_kv_heads) == ("qwen2", 2, 512, 8, 2)
    assert abs(md.rms_norm_eps - 1e-5) < 1e-11
    assert md.raw["some.u64"] == str(2 ** 40 + 3) and md.raw["some.i32"] == "-7" and md.raw["some.flag"] == "true"
    assert md.raw["general.name"] == "synthetic model"
    assert md.raw["tokenizer.ggml.tokens"] == "" and md.raw["tokenizer.ggml.scores"] == ""   # arrays are skipped
    assert set(L.tensor_names()) == {t[0] for t in tensors} | {"output_norm.weight"}
    for name, qt, n, k, data in tensors:
        lt = L.lazy_tensors[name]
        assert (lt.qtype, lt.n, lt.k, lt.tensor_type) == (qt, n, k, GG[qt])
        assert lt.shape == (k // ROW_BYTES[qt][0] * ROW_BYTES[qt][0], n)      # ggml order: contiguous dimension first
        assert lt.size == len(data) == _lib.load().b200q_tensor_bytes(qt, _lib.LAYOUT_GGUF, n * k)
        assert lt.offset % 32 == 0                                          # default general.alignment
        assert np.array_equal(L.tensor_bytes(name), np.frombuffer(data, dtype=np.uint8))
    norm = L.lazy_tensors["output_norm.weight"]
    assert norm.qtype == -1 and norm.tensor_type == "FP32" and norm.size == 2048
    assert np.array_equal(np.frombuffer(L.tensor_bytes("output_norm.weight").tobytes(), dtype=np.float32),
                          np.arange(512, dtype=np.float32))
    L.close()


def test_alignment_key_moves_the_data_section(tmp_path):
    tensors = make_tensors(8)[:2]
    path = tmp_path / "a.gguf"
    write_model(path, tensors, extra={"general.alignment": 256})
    L = GgufLoader(path)
    for name, qt, n, k, data in tensors:
        assert np.array_equal(L.tensor_bytes(name), np.frombuffer(data, dtype=np.uint8))
    L.close()


def _kv_u32(key, v):
    return struct.pack("<Q", len(key)) + key.encode() + struct.pack("<II", 4, v)


def _tinfo(name, dims, type_id, offset):
    b = struct.pack("<Q", len(name)) + name.encode() + struct.pack("<I", len(dims))
    for d in dims:
        b += struct.pack("<Q", d)
    return b + struct.pack("<IQ", type_id, offset)


def reference_style_file(path, n=8, k=64):
    """A file laid out like the reference's fixture writer: rows first, absolute offsets, RF Q4_0 blocks of 20 bytes."""
    rng = synth.rng_for(11)
    data = synth.gen_packed(synth.Q4_0, synth.RF, n * k, rng)
    head = b"GGUF" + struct.pack("<IQQ", 3, 1, 2) + _kv_u32("llama.block_count", 1) + _kv_u32("llama.vocab_size", n)
    name = "output.weight"
    info_len = 8 + len(name) + 4 + 16 + 4 + 8
    offset = len(head) + info_len + 13                      # deliberately unaligned: offsets are taken as they are
    blob = head + _tinfo(name, [n, k], 2, offset) + b"\0" * 13 + bytes(data)
    path.write_bytes(blob)
    return data


def test_reference_fixture_style(tmp_path):
    path = tmp_path / "ref.gguf"
    data = reference_style_file(path)
    L = GgufLoader(path, reference_fixture=True)
    lt = L.lazy_tensors["output.weight"]
    assert (lt.n, lt.k, lt.qtype, lt.size) == (8, 64, synth.Q4_0, 8 * 64 // 32 * 20)
    assert np.array_equal(L.tensor_bytes("output.weight"), np.frombuffer(data, dtype=np.uint8))
    assert L.metadata.num_layers == 1 and L.metadata.vocab_size == 8
    L.close()


@pytest.mark.parametrize("blob,status,text", [
    (b"GGML" + struct.pack("<IQQ", 3, 0, 0) + b"\0" * 8, _lib.ERR_INVALID, "magic"),
    (b"GGUF" + struct.pack("<IQQ", 2, 0, 0) + b"\0" * 8, _lib.ERR_UNSUPPORTED, "version 2"),
    (b"GGUF" + struct.pack("<IQQ", 3, 0, 1) + struct.pack("<Q", 200000) + b"\0" * 8, _lib.ERR_INVALID, "key_len"),
    (b"GGUF" + struct.pack("<IQQ", 3, 0, 1) + _kv_u32("a.b", 1)[:-2], _lib.ERR_INVALID, "ends inside"),
    (b"GGUF" + struct.pack("<IQQ", 3, 1, 0) + _tinfo("w", [32, 4], 3, 0) + b"\0" * 64, _lib.ERR_UNSUPPORTED, "type 3"),
    (b"GGUF" + struct.pack("<IQQ", 3, 1, 0) + _tinfo("w", [4096, 4096], 12, 0) + b"\0" * 64, _lib.ERR_INVALID, "out of bounds"),
    (b"GGUF" + struct.pack("<IQQ", 3, 1, 0) + _tinfo("w", [32] * 5, 0, 0)[:60], _lib.ERR_INVALID, "4 dimensions"),
], ids=["magic", "version", "key-too-long", "truncated-kv", "q4_1-type", "slice-out-of-bounds", "five-dims"])
def test_malformed_files_are_refused_with_a_status(tmp_path, blob, status, text):
    path = tmp_path / "bad.gguf"
    path.write_bytes(blob)
    with pytest.raises(B200QError) as e:
        GgufLoader(path)
    assert e.value.status == status and text in str(e.value)


def test_missing_file_and_unknown_names(tmp_path):
    with pytest.raises(B200QError):
        GgufLoader(tmp_path / "nope.gguf")
    path = tmp_path / "m.gguf"
    write_model(path, make_tensors()[:1])
    L = GgufLoader(path)
    assert L.lib.b200q_gguf_find_tensor(L.handle, b"does.not.exist") == -1
    with pytest.raises(KeyError):
        L.load_tensor_to_gpu("does.not.exist", backend=None)
    L.close()


def test_metadata_key_table():
    md = GgufMetadata()
    for k, v in [("general.architecture", "llama"), ("llama.block_count", "32"), ("llama.attention.head_count", "32"),
                 ("llama.attention.head_count_kv", "8"), ("llama.embedding_length", "4096"),
                 ("llama.feed_forward_length", "11008"), ("llama.rope.dimension_count", "128"),
                 ("llama.max_position_embeddings", "oops"), ("llama.vocab_size", "32000"),
                 ("llama.attention.layer_norm_rms_epsilon", "1e-5"), ("llama.intermediate_size", "1"),
                 ("model.tokenizer_json", "{}"), ("tokenizer.json", "ignored: first one wins")]:
        update_metadata(md, k, v)
    assert (md.num_layers, md.num_heads, md.num_kv_heads, md.hidden_size, md.intermediate_size, md.head_dim) == \
        (32, 32, 8, 4096, 11008, 128)
    assert md.max_position_embeddings == 2048          # unparsable -> the reference's default
    assert md.vocab_size == 32000 and md.rms_norm_eps == 1e-5 and md.embedded_tokenizer_json == "{}"
    names = layer_tensor_names(3)
    assert names["attn_qkv"] == "blk.3.attn_qkv.weight" and names["ffn_down"] == "blk.3.ffn_down.weight"


def test_type_ids_20_to_22_mean_mxfp_only_in_the_reference_dialect(tmp_path):
    """The reference's enum gives ids 20/21/22 to MXFP4 / MXFP6 (src/loader/tensor_type.rs:31-33); ggml gives them to
    IQ4_NL / IQ3_S / IQ2_S and writes MXFP4 as 39. A file read in the ggml dialect must not decode an IQ tensor
    as MXFP: the open fails with the reference's 'unsupported tensor type' class of error."""
    n, k = 4, 64
    name = "blk.0.ffn_up.weight"
    for type_id in (20, 21, 22):
        head = b"GGUF" + struct.pack("<IQQ", 3, 1, 0)
        blob = head + _tinfo(name, [k, n], type_id, 0) + b"\0" * 64 + b"\0" * (n * k)
        path = tmp_path / f"ggml_{type_id}.gguf"
        path.write_bytes(blob)
        with pytest.raises(B200QError) as e:
            GgufLoader(path)
        assert e.value.status == _lib.ERR_UNSUPPORTED and str(type_id) in str(e.value)
    # the same ids in the reference's dialect: its own byte layouts
    rng = synth.rng_for(12)
    data = synth.gen_packed(synth.MXFP4, synth.RF, n * k, rng)
    head = b"GGUF" + struct.pack("<IQQ", 3, 1, 0)
    info_len = 8 + len(name) + 4 + 16 + 4 + 8
    offset = len(head) + info_len
    path = tmp_path / "ref_20.gguf"
    path.write_bytes(head + _tinfo(name, [n, k], 20, offset) + bytes(data))
    L = GgufLoader(path, reference_fixture=True)
    lt = L.lazy_tensors[name]
    assert (lt.n, lt.k, lt.qtype, lt.size) == (n, k, synth.MXFP4, n * k // 32 * 17)
    L.close()
    # and ggml's MXFP4 id is not part of the reference's enum
    path = tmp_path / "ref_39.gguf"
    path.write_bytes(head + _tinfo(name, [n, k], 39, offset) + bytes(data))
    with pytest.raises(B200QError) as e:
        GgufLoader(path, reference_fixture=True)
    assert e.value.status == _lib.ERR_UNSUPPORTED
