"""The CPU oracle against the reference's own known-answer vectors and against gguf.quants.

CPU-only. These tests pin the restatement in oracle/oracle.c before anything else trusts it.
"""
import ctypes
import json
import os

import numpy as np
import pytest

from rocmforge_b200 import synth

HERE = os.path.dirname(os.path.abspath(__file__))
with open(os.path.join(HERE, "golden", "reference_vectors.json")) as f:
    GOLD = json.load(f)

FN = {"rf_q4_0": (synth.Q4_0, synth.RF), "rf_q8_0": (synth.Q8_0, synth.RF), "rf_q4_k": (synth.Q4_K, synth.RF),
      "rf_q6_k": (synth.Q6_K, synth.RF), "rf_q5_k": (synth.Q5_K, synth.RF), "rf_q3_k": (synth.Q3_K, synth.RF),
      "rf_q2_k": (synth.Q2_K, synth.RF)}


@pytest.mark.parametrize("case", GOLD["dequant"], ids=[c["name"] for c in GOLD["dequant"]])
def test_reference_dequant_vectors(oracle, case):
    data = bytes.fromhex(case["data"])
    n = case["n"]
    if case["fn"] == "rf_q8_0_i8":
        out = oracle.dequant_q8_0_i8_variant(data, n)
    else:
        qt, lay = FN[case["fn"]]
        out = oracle.dequantize(qt, lay, data, n)
    assert out.shape == (n,)
    if case.get("finite"):
        assert np.all(np.isfinite(out))
    for k, v in case["expect"].items():
        idx = range(n) if k == "all" else [int(k)]
        for i in idx:
            assert abs(out[i] - v) <= case["tol"], (case["cite"], i, out[i], v)


def test_e8m0_vectors(oracle):
    for e, v in GOLD["e8m0_to_f32"]["cases"]:
        assert oracle.pow2i(e) == v
    L = oracle.lib()
    for v in GOLD["e8m0_from_f32_roundtrip"]["values"]:
        rec = oracle.pow2i(L.rf_e8m0_from_f32(v))
        assert abs(rec - v) / v * 100 < GOLD["e8m0_from_f32_roundtrip"]["tol_pct"]
    assert L.rf_e8m0_from_f32(float("inf")) == GOLD["e8m0_from_inf"]["expect"]
    assert -127 <= L.rf_e8m0_from_f32(0.0) <= 127
    # exact powers of two over the whole int8 range except the documented -128 edge
    for e in range(-127, 128):
        assert oracle.pow2i(e) == float(np.ldexp(np.float32(1.0), e))
    assert oracle.pow2i(-128) == 0.0


def test_e2m1_e2m3_vectors(oracle):
    L = oracle.lib()
    g = GOLD["e2m1"]
    assert L.rf_encode_e2m1(0.0) == g["encode_zero"]
    assert L.rf_encode_e2m1(0.5) & 0x08 == 0 and L.rf_encode_e2m1(-0.5) & 0x08 != 0
    assert L.rf_decode_e2m1(0) == g["decode_zero"]
    p, n = L.rf_decode_e2m1(g["pos_code"]), L.rf_decode_e2m1(g["neg_code"])
    assert p > 0 and n < 0 and abs(p) == abs(n)
    g = GOLD["e2m3"]
    assert L.rf_encode_e2m3(0.0) == g["encode_zero"]
    assert L.rf_encode_e2m3(0.5) & 0x20 == 0 and L.rf_encode_e2m3(-0.5) & 0x20 != 0
    assert L.rf_decode_e2m3(0) == g["decode_zero"]
    p, n = L.rf_decode_e2m3(g["pos_code"]), L.rf_decode_e2m3(g["neg_code"])
    assert p > 0 and n < 0 and abs(p) == abs(n)
    # the full code tables as the reference's formula gives them
    assert [L.rf_decode_e2m1(c) for c in range(16)] == [0, 1, 1, 2, 2, 4, 4, 8, -.5, -1, -1, -2, -2, -4, -4, -8]
    for c in range(1, 64):
        s = -1.0 if c & 0x20 else 1.0
        assert L.rf_decode_e2m3(c) == s * (1 + (c & 7) / 8) * 2.0 ** (((c >> 3) & 3) - 1)


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def test_pack6_and_block_roundtrips(oracle):
    L = oracle.lib()
    vals = np.array(GOLD["pack6_roundtrip"]["values"], dtype=np.uint8)
    packed = np.zeros(24, dtype=np.uint8)
    L.rf_pack_6bit(_p(vals), 32, _p(packed))
    back = np.zeros(32, dtype=np.uint8)
    L.rf_unpack_6bit(_p(packed), 24, 32, _p(back))
    assert np.array_equal(vals, back)
    tol = GOLD["mxfp_block_roundtrip"]["tol"]
    for v in GOLD["mxfp_block_roundtrip"]["values"]:
        x = np.full(32, v, dtype=np.float32)
        for pack, unpack, nb in ((L.rf_mxfpblock_pack_mxfp4, L.rf_mxfpblock_unpack_mxfp4, 16),
                                 (L.rf_mxfpblock_pack_mxfp6, L.rf_mxfpblock_unpack_mxfp6, 24)):
            e = ctypes.c_int8(0)
            el = np.zeros(nb, dtype=np.uint8)
            out = np.zeros(32, dtype=np.float32)
            pack(_p(x), ctypes.byref(e), _p(el))
            unpack(e, _p(el), _p(out))
            assert np.all(np.abs(out - x) < tol)
    g = GOLD["mxfp_clamp"]
    x = np.zeros(32, dtype=np.float32)
    x[:4] = g["values"]
    for pack, unpack, nb, rng in ((L.rf_mxfpblock_pack_mxfp4, L.rf_mxfpblock_unpack_mxfp4, 16, g["mxfp4_range"]),
                                  (L.rf_mxfpblock_pack_mxfp6, L.rf_mxfpblock_unpack_mxfp6, 24, g["mxfp6_range"])):
        e = ctypes.c_int8(0)
        el = np.zeros(nb, dtype=np.uint8)
        out = np.zeros(32, dtype=np.float32)
        pack(_p(x), ctypes.byref(e), _p(el))
        unpack(e, _p(el), _p(out))
        assert np.all(out >= -rng) and np.all(out <= rng)
    x = np.array(GOLD["mxfp6_better_than_mxfp4"]["values"], dtype=np.float32)
    mse = []
    for pack, unpack, nb in ((L.rf_mxfpblock_pack_mxfp4, L.rf_mxfpblock_unpack_mxfp4, 16),
                             (L.rf_mxfpblock_pack_mxfp6, L.rf_mxfpblock_unpack_mxfp6, 24)):
        e = ctypes.c_int8(0)
        el = np.zeros(nb, dtype=np.uint8)
        out = np.zeros(32, dtype=np.float32)
        pack(_p(x), ctypes.byref(e), _p(el))
        unpack(e, _p(el), _p(out))
        mse.append(float(np.sum((x - out) ** 2)))
    assert mse[1] < mse[0]


def test_rf_mxfp_streams_follow_the_dispatcher_rules(oracle):
    """dequant_mxfp4/6 on raw byte streams (src/loader/dequant.rs:41-132): properties the code fixes."""
    rng = synth.rng_for(11)
    d4 = synth.gen_packed(synth.MXFP4, synth.RF, 64 * 32, rng)
    o4 = oracle.dequantize(synth.MXFP4, synth.RF, d4, 64 * 32)
    blk = d4.reshape(64, 17)
    tbl = np.array([0, 1, 1, 2, 2, 4, 4, 8, -.5, -1, -1, -2, -2, -4, -4, -8], dtype=np.float32)
    exp = np.empty((64, 32), dtype=np.float32)
    sc = np.ldexp(np.float32(1), blk[:, 0].view(np.int8).astype(np.int32)).astype(np.float32)
    exp[:, 0::2] = tbl[blk[:, 1:] >> 4] * sc[:, None]      # high nibble first
    exp[:, 1::2] = tbl[blk[:, 1:] & 15] * sc[:, None]
    assert np.array_equal(o4, np.clip(exp, -8, 8).reshape(-1))
    d6 = synth.gen_packed(synth.MXFP6_E2M3, synth.RF, 64 * 32, rng)
    o6 = oracle.dequantize(synth.MXFP6_E2M3, synth.RF, d6, 64 * 32).reshape(64, 32)
    assert np.all(o6[:, 31] == 0.0)                       # element 31 of every block is never written
    assert np.all(np.abs(o6) <= 7.5)
    o6b = oracle.dequantize(synth.MXFP6_E3M2, synth.RF, d6, 64 * 32).reshape(64, 32)
    assert np.array_equal(o6, o6b)                        # both tensor types decode as E2M3
    # clamp engages for large exponents
    one = np.zeros(17, dtype=np.uint8)
    one[0] = 5
    one[1:] = 0x7F
    assert np.all(np.abs(oracle.dequantize(synth.MXFP4, synth.RF, one, 32)) <= 8.0)


def test_partial_and_truncated_streams(oracle):
    """Tail rules: n may stop inside a block; a stream that ends early leaves zeros."""
    rng = synth.rng_for(5)
    for qt in range(10):
        for lay in (synth.RF, synth.GGUF):
            be = synth.block_elems(qt)
            data = synth.gen_packed(qt, lay, 3 * be, rng)
            full = oracle.dequantize(qt, lay, data, 3 * be)
            part = oracle.dequantize(qt, lay, data, 2 * be + 7)
            assert np.array_equal(full[:2 * be + 7].view(np.uint32), part.view(np.uint32))
            short = oracle.dequantize(qt, lay, data[:2 * synth.block_bytes(qt, lay)], 3 * be)
            assert np.all(short[2 * be:] == 0.0)
    assert oracle.dequantize(synth.Q4_0, synth.RF, np.zeros(0, np.uint8), 0).size == 0


def test_gguf_layout_against_committed_fixtures(oracle):
    fx = np.load(os.path.join(HERE, "golden", "gguf_fixtures.npz"))
    for qt in (synth.Q4_0, synth.Q8_0, synth.Q4_K, synth.Q6_K, synth.MXFP4):
        name = synth.QNAMES[qt]
        data, ref = fx[f"in_{name}"], fx[f"out_{name}"]
        out = oracle.dequantize(qt, synth.GGUF, data, ref.size)
        assert np.array_equal(out.view(np.uint32), ref.view(np.uint32)), name


def test_gguf_layout_against_gguf_package_live(oracle):
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    types = {synth.Q4_0: gguf.GGMLQuantizationType.Q4_0, synth.Q8_0: gguf.GGMLQuantizationType.Q8_0,
             synth.Q4_K: gguf.GGMLQuantizationType.Q4_K, synth.Q6_K: gguf.GGMLQuantizationType.Q6_K,
             synth.MXFP4: gguf.GGMLQuantizationType.MXFP4, synth.Q2_K: gguf.GGMLQuantizationType.Q2_K,
             synth.Q3_K: gguf.GGMLQuantizationType.Q3_K, synth.Q5_K: gguf.GGMLQuantizationType.Q5_K}
    for qt, gt in types.items():
        rng = synth.rng_for(300 + qt)
        nblk = 100_000 if synth.block_elems(qt) == 32 else 12_500
        bb = synth.block_bytes(qt, synth.GGUF)
        data = rng.integers(0, 256, size=(nblk, bb), dtype=np.uint8)   # every header bit pattern can occur
        with np.errstate(all="ignore"):
            ref = quants.dequantize(data, gt).astype(np.float32).reshape(-1)
        out = oracle.dequantize(qt, synth.GGUF, data.reshape(-1), ref.size)
        same = (out.view(np.uint32) == ref.view(np.uint32)) | (np.isnan(out) & np.isnan(ref))
        assert np.all(same), synth.QNAMES[qt]


def test_gguf_mxfp6_tables(oracle):
    """OCP FP6 element tables under a biased E8M0 header (no third-party implementation: unpinned)."""
    codes = np.arange(32, dtype=np.uint8)
    for hi in (0, 32):
        c = codes + hi
        w = c.astype(np.uint32).reshape(8, 4)
        word = w[:, 0] | (w[:, 1] << 6) | (w[:, 2] << 12) | (w[:, 3] << 18)
        blk = np.zeros(25, dtype=np.uint8)
        blk[0] = 127
        blk[1:] = np.stack([word & 255, (word >> 8) & 255, (word >> 16) & 255], axis=-1).reshape(-1)
        e2m3 = oracle.dequantize(synth.MXFP6_E2M3, synth.GGUF, blk, 32)
        e3m2 = oracle.dequantize(synth.MXFP6_E3M2, synth.GGUF, blk, 32)
        for i, ci in enumerate(int(v) for v in c):
            s = -1.0 if ci & 32 else 1.0
            e, m = (ci >> 3) & 3, ci & 7
            assert e2m3[i] == s * (m / 8 if e == 0 else (1 + m / 8) * 2.0 ** (e - 1))
            e, m = (ci >> 2) & 7, ci & 3
            assert e3m2[i] == s * (m / 16 if e == 0 else (1 + m / 4) * 2.0 ** (e - 3))
    assert np.max(np.abs(e2m3)) == 7.5 and np.max(np.abs(e3m2)) == 28.0


def test_f16_widening_is_exact(oracle):
    bits = np.arange(65536, dtype=np.uint16)
    ref = bits.view(np.float16).astype(np.float32)
    got = np.array([oracle.f16_to_f32(int(b)) for b in bits[::7]], dtype=np.float32)
    r = ref[::7]
    assert np.all((got.view(np.uint32) == r.view(np.uint32)) | (np.isnan(got) & np.isnan(r)))


@pytest.mark.parametrize("case", GOLD["matmul"], ids=[c["name"] for c in GOLD["matmul"]])
def test_reference_fused_matmul_cases(oracle, case):
    """tests/q_dequant_tests.rs fused-matmul inputs: dequant, then cpu_matmul_f32 on the flat [K,N] stream."""
    data = bytes.fromhex(case["data"])
    n, k = case["n_rows"], case["n_cols"]
    w = oracle.dequantize(case["qtype"], synth.RF, data, n * k).reshape(k, n)
    x = np.array(case["input"], dtype=np.float32).reshape(1, k)
    y = oracle.matmul_f32(x, w)
    assert np.all(np.abs(y.reshape(-1) - np.array(case["expect"])) <= case["tol"])


def test_matmul_orders_and_threads(oracle):
    rng = synth.rng_for(9)
    a = rng.standard_normal((3, 160), dtype=np.float32)
    w = rng.standard_normal((37, 160), dtype=np.float32)
    y_nk = oracle.matmul_f32(a, w, nk=True)
    y_kn = oracle.matmul_f32(a, np.ascontiguousarray(w.T))
    assert np.array_equal(y_nk, y_kn)
    assert np.array_equal(y_nk, oracle.matmul_f32(a, w, nk=True, threads=4))
    # sequential fp32 accumulation, multiply then add, in python for one output
    acc = np.float32(0)
    for l in range(160):
        acc = np.float32(acc + np.float32(a[1, l] * w[5, l]))
    assert y_nk[1, 5] == acc
    y64 = oracle.matmul_f64(a, w, nk=True)
    assert np.allclose(y64, a.astype(np.float64) @ w.astype(np.float64).T, rtol=1e-12)
    # threaded dequant equals single-thread dequant
    data = synth.gen_packed(synth.Q4_K, synth.GGUF, 256 * 50, rng)
    assert np.array_equal(oracle.dequantize(synth.Q4_K, synth.GGUF, data, 256 * 50),
                          oracle.dequantize(synth.Q4_K, synth.GGUF, data, 256 * 50, threads=3))


def test_rf_k_quants_follow_the_reference_loops(oracle):
    """Q5_K / Q3_K / Q2_K in the reference's 256-byte layouts (src/loader/dequant.rs:150-419), evaluated here
    element by element in Python from the same formulas on random bytes. The reference's own known-answer
    vectors for these formats (src/loader/dequant.rs:439-665) are checked in test_reference_dequant_vectors;
    this test widens them to non-trivial scales, minima and high bits."""
    rng = synth.rng_for(77)
    for qt in (synth.Q5_K, synth.Q3_K, synth.Q2_K):
        data = synth.gen_packed(qt, synth.RF, 3 * 256, rng)
        got = oracle.dequantize(qt, synth.RF, data, 3 * 256 - 5)
        blk = data.reshape(3, 256).astype(np.int64)
        want = np.zeros(3 * 256, np.float32)
        for b in range(3):
            for sb in range(16):
                scale = np.float32(blk[b, 2 * sb:2 * sb + 2].astype(np.uint8).view(np.float16)[0])
                for i in range(16):
                    bits = {synth.Q5_K: 5, synth.Q3_K: 3, synth.Q2_K: 2}[qt]
                    qoff = {synth.Q5_K: 48, synth.Q3_K: 36, synth.Q2_K: 68}[qt] + sb * 2 * bits + (i * bits) // 8
                    comb = int(blk[b, qoff]) | (int(blk[b, qoff + 1]) << 8)
                    low = (comb >> ((i * bits) % 8)) & ((1 << bits) - 1)
                    if qt == synth.Q5_K:
                        mn = np.float32(np.int8(np.uint8(blk[b, 32 + sb])))
                        v = mn + np.float32(low) * scale
                    elif qt == synth.Q3_K:
                        qh = (int(blk[b, 32 + sb // 4]) >> ((sb % 4) * 2)) & 3
                        high = (qh >> i) & 1 if i < 8 else 0
                        v = (np.float32(low | (high << 3)) - np.float32(4.0)) * scale
                    else:
                        mn = np.float32(blk[b, 32 + 2 * sb:34 + 2 * sb].astype(np.uint8).view(np.float16)[0])
                        qh = (int(blk[b, 64 + sb // 8]) >> (sb % 8)) & 1
                        high = (qh >> i) & 1 if i < 8 else 0
                        v = mn + np.float32(low | (high << 2)) * scale
                    want[b * 256 + sb * 16 + i] = v
        assert np.array_equal(got.view(np.uint32), want[:got.size].view(np.uint32)), synth.QNAMES[qt]
        # a block that is not completely inside the stream is skipped
        short = oracle.dequantize(qt, synth.RF, data[:2 * 256 + 100], 3 * 256)
        assert np.all(short[512:] == 0.0) and np.array_equal(short[:512].view(np.uint32), want[:512].view(np.uint32))
