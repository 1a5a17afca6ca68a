"""Dequantise-to-fp32 on the GPU against the CPU oracle: bit-exact, every format, both layout families."""
import json
import os

import numpy as np
import pytest

from rocmforge_b200 import _lib, ops, synth

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def be():
    from gpu_util import backend
    return backend()


from gpu_util import ALL_FMTS, FMT_IDS, QuantizedWeight, bits_equal, gpu_dequant_bytes  # noqa: E402


@pytest.mark.parametrize("qt,lay", ALL_FMTS, ids=FMT_IDS)
def test_synthetic_tensor_bit_exact(be, oracle, qt, lay):
    rng = synth.rng_for(100 + qt * 2 + lay)
    be_ = synth.block_elems(qt)
    n = 1237 * be_
    data = synth.gen_packed(qt, lay, n, rng)
    ref = oracle.dequantize(qt, lay, data, n)
    assert bits_equal(gpu_dequant_bytes(be, qt, lay, data, n), ref)
    # through an uploaded handle, full and stopping inside a block
    w = QuantizedWeight(be, data, qt, lay, 1237, be_)
    for cnt in (n, n - be_ + 5, 8, 3):
        out = be.allocate_buffer(cnt * 4)
        w.dequantize(out, cnt)
        be.synchronize()
        assert bits_equal(out.to_numpy(np.float32, cnt), ref[:cnt]), cnt
        out.free()
    w.free()


@pytest.mark.parametrize("qt,lay", ALL_FMTS, ids=FMT_IDS)
def test_every_header_bit_pattern(be, oracle, qt, lay):
    """Fully random block bytes: every f16 / f32 / E8M0 header pattern class (subnormal, inf, NaN, -128) occurs."""
    rng = synth.rng_for(900 + qt * 2 + lay)
    bb, be_ = synth.block_bytes(qt, lay), synth.block_elems(qt)
    nblk = 70_000 if be_ == 32 else 9_000
    data = rng.integers(0, 256, size=(nblk, bb), dtype=np.uint8)
    if bb in (17, 25):
        data[:256, 0] = np.arange(256)                 # every exponent byte
    elif be_ == 32 and lay == synth.GGUF:
        data[:65536, 0:2] = np.arange(65536, dtype=np.uint16).view(np.uint8).reshape(-1, 2)   # every f16 scale
    elif qt == synth.Q4_K and lay == synth.GGUF:
        data[:, 0:2] = np.arange(nblk, dtype=np.uint16).view(np.uint8).reshape(-1, 2)
    ref = oracle.dequantize(qt, lay, data.reshape(-1), nblk * be_)
    assert bits_equal(gpu_dequant_bytes(be, qt, lay, data.reshape(-1), nblk * be_), ref)


def test_exhaustive_scale_times_code_tables(be, oracle):
    """GGUF Q4_0: every f16 scale x every 4-bit code; MXFP: every exponent byte x every element code."""
    scales = np.arange(65536, dtype=np.uint16)
    blk = np.zeros((65536, 18), dtype=np.uint8)
    blk[:, 0:2] = scales.view(np.uint8).reshape(-1, 2)
    blk[:, 2:18] = np.arange(16, dtype=np.uint8) | (np.arange(15, -1, -1, dtype=np.uint8) << 4)
    ref = oracle.dequantize(synth.Q4_0, synth.GGUF, blk.reshape(-1), 65536 * 32)
    assert bits_equal(gpu_dequant_bytes(be, synth.Q4_0, synth.GGUF, blk.reshape(-1), 65536 * 32), ref)
    for lay in (synth.RF, synth.GGUF):
        blk = np.zeros((256, 17), dtype=np.uint8)
        blk[:, 0] = np.arange(256)
        blk[:, 1:17] = np.arange(16, dtype=np.uint8) | (np.arange(15, -1, -1, dtype=np.uint8) << 4)
        ref = oracle.dequantize(synth.MXFP4, lay, blk.reshape(-1), 256 * 32)
        assert bits_equal(gpu_dequant_bytes(be, synth.MXFP4, lay, blk.reshape(-1), 256 * 32), ref)
        for qt in (synth.MXFP6_E2M3, synth.MXFP6_E3M2):
            blk = np.zeros((512, 25), dtype=np.uint8)
            blk[:, 0] = np.repeat(np.arange(256), 2)
            codes = np.concatenate([np.arange(32), np.arange(32, 64)]).astype(np.uint32).reshape(2, 8, 4)
            word = codes[..., 0] | (codes[..., 1] << 6) | (codes[..., 2] << 12) | (codes[..., 3] << 18)
            by = np.stack([word & 255, (word >> 8) & 255, (word >> 16) & 255], axis=-1).astype(np.uint8).reshape(2, 24)
            blk[:, 1:] = np.tile(by, (256, 1))
            ref = oracle.dequantize(qt, lay, blk.reshape(-1), 512 * 32)
            assert bits_equal(gpu_dequant_bytes(be, qt, lay, blk.reshape(-1), 512 * 32), ref)


@pytest.mark.parametrize("qt,lay", ALL_FMTS, ids=FMT_IDS)
def test_short_and_ragged_streams(be, oracle, qt, lay):
    """A byte stream that ends early leaves the uncovered outputs 0.0, exactly where the CPU code does."""
    rng = synth.rng_for(40 + qt * 2 + lay)
    bb, be_ = synth.block_bytes(qt, lay), synth.block_elems(qt)
    n = 5 * be_
    data = synth.gen_packed(qt, lay, n, rng)
    for cut in (data.size, data.size - 1, data.size - bb // 2, 3 * bb + 5, 3 * bb + 1, 3 * bb, 2, 0):
        for cnt in (n, n - 3, 2 * be_ + 9):
            ref = oracle.dequantize(qt, lay, data[:cut], cnt)
            got = gpu_dequant_bytes(be, qt, lay, data[:cut], cnt)
            assert bits_equal(got, ref), (cut, cnt)


def test_reference_known_answer_vectors_on_gpu(be):
    gold = json.load(open(os.path.join(HERE, "golden", "reference_vectors.json")))
    fn = {"rf_q4_0": ops.dequantize_q4_0_kernel_cached, "rf_q8_0": ops.dequantize_q8_0_gpu_kernel,
          "rf_q4_k": ops.dequantize_q4_k_gpu_kernel, "rf_q6_k": ops.dequantize_q6_k_gpu_kernel}
    generic = {"rf_q5_k": synth.Q5_K, "rf_q3_k": synth.Q3_K, "rf_q2_k": synth.Q2_K}   # src/loader/dequant.rs:439-665
    for case in gold["dequant"]:
        if case["fn"] not in fn and case["fn"] not in generic:
            continue
        data, n = bytes.fromhex(case["data"]), case["n"]
        out = be.allocate_buffer(n * 4)
        if case["fn"] in generic:   # the reference has no GPU wrapper for these: host bytes -> device fp32
            got = gpu_dequant_bytes(be, generic[case["fn"]], synth.RF, np.frombuffer(data, dtype=np.uint8), n)
        else:
            fn[case["fn"]](be, data, out, n)
            got = out.to_numpy(np.float32, n)
        if case.get("finite"):
            assert np.all(np.isfinite(got))
        for k, v in case["expect"].items():
            for i in (range(n) if k == "all" else [int(k)]):
                assert abs(got[i] - v) <= case["tol"], (case["cite"], i)
        out.free()


def test_committed_gguf_fixtures_on_gpu(be):
    fx = np.load(os.path.join(HERE, "golden", "gguf_fixtures.npz"))
    for qt in (synth.Q4_0, synth.Q8_0, synth.Q4_K, synth.Q6_K, synth.MXFP4):
        name = synth.QNAMES[qt]
        data, ref = fx[f"in_{name}"], fx[f"out_{name}"]
        assert bits_equal(gpu_dequant_bytes(be, qt, synth.GGUF, data, ref.size), ref), name


def test_full_size_lm_head_dequant_properties(be, oracle):
    """151936 x 896 Q6_K (111.7 MB packed -> 545 MB fp32): sampled rows bit-exact, whole-tensor checksum stable."""
    rng = synth.rng_for(synth.CONFIG_SEEDS[3])
    n, k = 151936, 896
    data = synth.gen_packed(synth.Q6_K, synth.GGUF, n * k, rng)
    w = QuantizedWeight(be, data, synth.Q6_K, synth.GGUF, n, k)
    out = be.allocate_buffer(n * k * 4)
    w.dequantize(out)
    be.synchronize()
    got = out.to_numpy(np.float32, n * k)
    for blk0 in (0, 12345, 531776 - 64):
        ref = oracle.dequantize(synth.Q6_K, synth.GGUF, data[blk0 * 210:(blk0 + 64) * 210], 64 * 256)
        assert bits_equal(got[blk0 * 256:(blk0 + 64) * 256], ref)
    w.dequantize(out)          # idempotent: a second run gives the same words
    be.synchronize()
    assert np.array_equal(out.to_numpy(np.uint32, n * k), got.view(np.uint32))
    out.free()
    w.free()


def test_argument_errors_are_status_codes(be):
    out = be.allocate_buffer(1024)
    with pytest.raises(_lib.B200QError) as e:
        ops.dequantize_gpu(be, 10, b"\0" * 20, out, 32)      # no such tensor type
    assert e.value.status == _lib.ERR_INVALID
    with pytest.raises(_lib.B200QError) as e:
        ops.dequantize_gpu(be, synth.Q4_0, b"\0" * 20, out, 4096)       # output buffer too small
    assert e.value.status == _lib.ERR_INVALID
    with pytest.raises(_lib.B200QError) as e:
        QuantizedWeight(be, b"\0" * 19, synth.Q4_0, synth.RF, 1, 32)   # byte count does not match the shape
    assert e.value.status == _lib.ERR_INVALID
    with pytest.raises(_lib.B200QError) as e:
        QuantizedWeight(be, b"\0" * 20 * 3, synth.Q4_0, synth.RF, 3, 32, shard_rank=0, shard_count=2)
    assert e.value.status == _lib.ERR_INVALID
    # the context is still usable afterwards
    ops.dequantize_q4_0_kernel_cached(be, b"\0" * 20, out, 32)
    out.free()
