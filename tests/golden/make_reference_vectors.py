"""Re-express the known-answer vectors of the reference's own unit tests as data.

Every case below rebuilds the INPUT bytes the way one reference test builds them and
records the EXPECTATION that test asserts (value + tolerance), citing the test by its
path inside the ROCmForge tree. Nothing is computed with the oracle here: where a
reference test recomputes its expectation with a formula, the same formula is
evaluated in plain Python.

Run:  python tests/golden/make_reference_vectors.py   (writes reference_vectors.json)
"""
import json
import os
import struct

import numpy as np

Q4_0, Q8_0, Q4_K, Q6_K, MXFP4, MXFP6 = 0, 1, 2, 3, 4, 5
cases = []


def f32le(v):
    return struct.pack("<f", v)


def f16le(v):
    return np.float16(v).tobytes()


def add(name, cite, fn, data, n, expect, tol, **kw):
    """expect: dict index -> value, or {"all": v} for every element < n."""
    cases.append(dict(name=name, cite=cite, fn=fn, data=bytes(data).hex(), n=n,
                      expect={str(k): float(v) for k, v in expect.items()}, tol=tol, **kw))


# ---- Q4_0: src/kernels/quant/q4_0.rs:316-437 ---------------------------------
d = bytearray(20); d[0:4] = f32le(1.0); d[4:20] = b"\x88" * 16
add("q4_0_zeros", "src/kernels/quant/q4_0.rs:317-335", "rf_q4_0", d, 32, {"all": 0.0}, 0.01)
d = bytearray(20); d[0:4] = f32le(2.0)
for i in range(16):
    d[4 + i] = ((i + 1) << 4 | i) & 0xFF
add("q4_0_positive", "src/kernels/quant/q4_0.rs:338-362", "rf_q4_0", d, 32,
    {0: -16.0, 1: -14.0, 31: -16.0, 30: 14.0}, 0.01)
d = bytearray(20); d[0:4] = f32le(-1.5); d[4:20] = b"\x88" * 16
add("q4_0_negative_scale", "src/kernels/quant/q4_0.rs:365-383", "rf_q4_0", d, 32, {"all": 0.0}, 0.01)
d = bytearray(20); d[0:4] = f32le(1.0); d[4:20] = b"\x88" * 16
add("q4_0_partial_block", "src/kernels/quant/q4_0.rs:386-404", "rf_q4_0", d, 10, {"all": 0.0}, 0.01)
d = bytearray(40); d[0:4] = f32le(1.0); d[4:20] = b"\x88" * 16; d[20:24] = f32le(2.0); d[24:40] = b"\xCC" * 16
e = {i: 0.0 for i in range(32)}; e.update({i: 8.0 for i in range(32, 64)})
add("q4_0_multiple_blocks", "src/kernels/quant/q4_0.rs:407-437", "rf_q4_0", d, 64, e, 0.01)
d = bytearray(20); d[0:4] = f32le(1.0)
for i in range(16):
    d[4 + i] = (i % 16) | (((i + 1) % 16) << 4)
add("q4_0_loader_single_block", "src/loader/gguf/tensor_data.rs:508-531", "rf_q4_0", d, 32, {0: -8.0, 1: -7.0}, 0.0)
d = bytearray(20); d[0:4] = f32le(1.0); d[4:20] = b"\x88" * 16
add("q4_0_matmul_copy_simple", "src/kernels/matmul/quantized/q4_0.rs:317-338", "rf_q4_0", d, 32, {"all": 0.0}, 0.01)

# ---- Q8_0: src/kernels/quant/q8_0.rs:77-173 ----------------------------------
d = bytearray(36); d[0:4] = f32le(1.0); d[4:36] = bytes([128] * 32)
add("q8_0_zeros", "src/kernels/quant/q8_0.rs:78-96", "rf_q8_0", d, 32, {"all": 0.0}, 0.01)
d = bytearray(36); d[0:4] = f32le(2.0); d[4:36] = bytes([120 + i for i in range(32)])
add("q8_0_positive", "src/kernels/quant/q8_0.rs:99-120", "rf_q8_0", d, 32, {0: -16.0, 15: 14.0, 31: 46.0}, 0.01)
d = bytearray(36); d[0:4] = f32le(1.0); d[4:36] = bytes([128] * 32)
add("q8_0_partial_block", "src/kernels/quant/q8_0.rs:123-141", "rf_q8_0", d, 10, {"all": 0.0}, 0.01)
d = bytearray(72); d[0:4] = f32le(1.0); d[4:36] = bytes([128] * 32); d[36:40] = f32le(0.5); d[40:72] = bytes([138] * 32)
e = {i: 0.0 for i in range(32)}; e.update({i: 5.0 for i in range(32, 64)})
add("q8_0_multiple_blocks", "src/kernels/quant/q8_0.rs:144-173", "rf_q8_0", d, 64, e, 0.01)
d = bytearray(36); d[0:4] = f32le(1.0); d[4:36] = bytes([128 + i for i in range(32)])
add("q8_0_loader_single_block", "src/loader/gguf/tensor_data.rs:483-505", "rf_q8_0", d, 32, {0: 0.0, 1: 1.0, 31: 31.0}, 0.0)
d = bytearray(36); d[0:4] = f32le(1.0); d[4:36] = bytes([(i - 16) & 0xFF for i in range(32)])
add("q8_0_i8_variant_simple", "src/kernels/matmul/quantized/q8_0.rs:113-130", "rf_q8_0_i8", d, 32,
    {i: float(i - 16) for i in range(32)}, 0.01)

# ---- Q4_K: src/kernels/quant/q4_k.rs:279-368 (expectation = the test's own formula) ----
def q4k_expect(data, n):
    out = {}
    for i in range(n):
        sb, el = i // 32, i % 32
        byte_idx, bit_off = (el * 4) // 8, (el * 4) % 8
        qo = sb * 28 + byte_idx
        comb = (data[32 + qo + 1] << 8) | data[32 + qo]
        out[i] = float((comb >> bit_off) & 0x0F)
    return out

d = bytearray(256)
for i in range(8):
    d[2 * i:2 * i + 2] = f16le(1.0)
for i in range(224):
    d[32 + i] = ((i % 16) << 4) | (i % 16)
add("q4_k_single_block", "src/kernels/quant/q4_k.rs:280-323", "rf_q4_k", d, 256, q4k_expect(d, 256), 0.01)
d = bytearray(256)
for i in range(8):
    d[2 * i:2 * i + 2] = f16le(1.0)
d[32:256] = b"\x88" * 224
add("q4_k_partial_block", "src/kernels/quant/q4_k.rs:326-368", "rf_q4_k", d, 100, q4k_expect(d, 100), 0.01)

# ---- Q6_K: src/kernels/quant/q6_k.rs:272-399 -----------------------------------
d = bytearray(256)
for i in range(16):
    d[2 * i:2 * i + 2] = f16le(1.0)
for i in range(192):
    d[32 + i] = ((i % 64) * 4) & 0xFF
add("q6_k_single_block_finite", "src/kernels/quant/q6_k.rs:273-306", "rf_q6_k", d, 256, {}, 0.0, finite=True)
d = bytearray(256)
for i in range(16):
    d[2 * i:2 * i + 2] = f16le(2.0)
add("q6_k_partial_block_zero", "src/kernels/quant/q6_k.rs:309-337", "rf_q6_k", d, 100, {"all": 0.0}, 1.0)
d = bytearray(256)
for i in range(16):
    d[2 * i:2 * i + 2] = f16le(1.0)
d[32:224] = b"\xFF" * 192
add("q6_k_negative_values", "src/kernels/quant/q6_k.rs:340-399", "rf_q6_k", d, 256, {"all": -1.0}, 1.0)

# ---- GPU-vs-CPU test inputs, tests/q_dequant_tests.rs (Q4_K: 0x3C00 scales, Q6_K: f16 2.0) ----
d = bytearray(256)
for i in range(8):
    d[2 * i:2 * i + 2] = struct.pack("<H", 0x3C00)
d[32:256] = b"\x88" * 224
add("q4_k_gpu_test_input", "tests/q_dequant_tests.rs:257-273", "rf_q4_k", d, 256, q4k_expect(d, 256), 1e-3)

# ---- Q5_K / Q3_K / Q2_K in the reference's 256-byte layouts: src/loader/dequant.rs:439-665 -------------------
# (the tests set only the first sub-block's f16 scale; every other scale, min and code byte is zero)
def kblock(scale=1.0):
    b = bytearray(256); b[0:2] = f16le(scale)
    return b

d = kblock()
add("q5_k_zeros", "src/loader/dequant.rs:440-461", "rf_q5_k", d, 256, {"all": 0.0}, 1e-6)
d = kblock(); d[48] = 0x01
e = {0: 1.0}; e.update({i: 0.0 for i in range(1, 16)})
add("q5_k_positive", "src/loader/dequant.rs:464-495", "rf_q5_k", d, 256, e, 0.1)
d = kblock()
add("q5_k_partial_block", "src/loader/dequant.rs:498-515", "rf_q5_k", d, 100, {"all": 0.0}, 1e-6)
d = kblock() + kblock(2.0); d[256 + 48] = 0xFF; d[256 + 49] = 0x80
add("q5_k_multiple_blocks_first", "src/loader/dequant.rs:518-546", "rf_q5_k", d, 512, {i: 0.0 for i in range(256)}, 1e-5)
add("q5_k_multiple_blocks_second", "src/loader/dequant.rs:518-546", "rf_q5_k", d, 512, {256: 62.0}, 1.0)
d = kblock()
add("q3_k_zeros", "src/loader/dequant.rs:549-566", "rf_q3_k", d, 256, {i: -4.0 for i in range(16)}, 0.1)
d = kblock(); d[36] = 0x01
e = {0: -3.0}; e.update({i: -4.0 for i in range(1, 16)})
add("q3_k_positive", "src/loader/dequant.rs:569-592", "rf_q3_k", d, 256, e, 0.1)
d = kblock()
add("q3_k_partial_block", "src/loader/dequant.rs:595-613", "rf_q3_k", d, 100, {i: -4.0 for i in range(16)}, 0.1)
d = kblock()
add("q2_k_zeros", "src/loader/dequant.rs:616-635", "rf_q2_k", d, 256, {i: 0.0 for i in range(16)}, 1e-5)
d = kblock(); d[68] = 0x01
add("q2_k_positive", "src/loader/dequant.rs:638-657", "rf_q2_k", d, 256, {0: 1.0}, 0.1)
d = kblock()
add("q2_k_partial_block", "src/loader/dequant.rs:660-678", "rf_q2_k", d, 100, {i: 0.0 for i in range(16)}, 1e-5)

json_cases = dict(dequant=cases)

# ---- scalar codecs, src/loader/mxfp_tests.rs ------------------------------------
json_cases["e8m0_to_f32"] = dict(cite="src/loader/mxfp_tests.rs:21-51",
                                 cases=[[0, 1.0], [1, 2.0], [2, 4.0], [10, 1024.0], [-1, 0.5], [-2, 0.25]])
json_cases["e8m0_from_f32_roundtrip"] = dict(cite="src/loader/mxfp_tests.rs:54-72",
                                             values=[1.0, 2.0, 4.0, 8.0, 0.5, 0.25, 0.125, 256.0, 1024.0], tol_pct=0.1)
json_cases["e8m0_from_inf"] = dict(cite="src/loader/mxfp_tests.rs:75-78", expect=127)
json_cases["e2m1"] = dict(cite="src/loader/mxfp_tests.rs:142-172",
                          encode_zero=0, decode_zero=0.0, pos_code=0b0101, neg_code=0b1101)
json_cases["e2m3"] = dict(cite="src/loader/mxfp_tests.rs:246-276",
                          encode_zero=0, decode_zero=0.0, pos_code=0b001010, neg_code=0b101010)
json_cases["pack6_roundtrip"] = dict(cite="src/loader/mxfp_tests.rs:294-309", values=list(range(32)), packed_len=24)
json_cases["mxfp_block_roundtrip"] = dict(cite="src/loader/mxfp_tests.rs:320-383", values=[1.0, 2.0, 4.0],
                                          tol=float(np.finfo(np.float32).eps))
json_cases["mxfp_clamp"] = dict(cite="src/loader/mxfp_tests.rs:176-190,280-291", values=[10.0, -10.0, 100.0, -100.0],
                                mxfp4_range=8.0, mxfp6_range=7.5)
json_cases["mxfp6_better_than_mxfp4"] = dict(cite="src/loader/mxfp_tests.rs:386-420",
                                             values=[i * 0.1 + 0.01 for i in range(32)])

# ---- fused matmul 4x4 cases, tests/q_dequant_tests.rs:396-806 --------------------
mm = []
d = bytearray(20); d[0:4] = f32le(1.0); d[4:20] = b"\x88" * 16
mm.append(dict(name="matmul_q4_0_zero_weights", cite="tests/q_dequant_tests.rs:396-500", qtype=Q4_0,
               data=bytes(d).hex(), n_rows=4, n_cols=4, input=[1.0, 2.0, 3.0, 4.0], expect=[0.0, 0.0, 0.0, 0.0], tol=1e-2))
# Q4_0 with varying codes, all-ones input (tests/q_dequant_tests.rs:735-806). The reference compares its GPU
# kernel with "CPU dequant, then [K,N] matmul"; the expectation here is that composition in plain Python.
d = bytearray(20); d[0:4] = f32le(2.0)
for i in range(16):
    d[4 + i] = ((((i + 1) % 16) << 4) | (i % 16)) & 0xFF
w = []
for i in range(16):
    w += [2.0 * ((d[4 + i] & 15) - 8), 2.0 * ((d[4 + i] >> 4) - 8)]
exp = [sum(1.0 * w[k * 4 + n] for k in range(4)) for n in range(4)]
mm.append(dict(name="matmul_q4_0_varying", cite="tests/q_dequant_tests.rs:735-806", qtype=Q4_0,
               data=bytes(d).hex(), n_rows=4, n_cols=4, input=[1.0, 1.0, 1.0, 1.0], expect=exp, tol=1e-2))
# Q4_K: scales 1.0h, mins 0, every nibble 8 -> every weight 8.0 (tests/q_dequant_tests.rs:500-610)
d = bytearray(256)
for i in range(8):
    d[2 * i:2 * i + 2] = struct.pack("<H", 0x3C00)
d[32:256] = b"\x88" * 224
mm.append(dict(name="matmul_q4_k_eights", cite="tests/q_dequant_tests.rs:500-610", qtype=Q4_K,
               data=bytes(d).hex(), n_rows=4, n_cols=4, input=[1.0, 2.0, 3.0, 4.0], expect=[80.0] * 4, tol=1e-2))
# Q6_K: scales 1.0h, every code byte 32 (tests/q_dequant_tests.rs:625-730); weights by the 6-bit formula of
# src/kernels/quant/q6_k.rs:241-260 evaluated in plain Python.
d = bytearray(256)
for i in range(16):
    d[2 * i:2 * i + 2] = struct.pack("<H", 0x3C00)
d[32:224] = bytes([32] * 192)
w = []
for i in range(16):
    bo, bi = (i * 6) % 8, (i * 6) // 8
    c = (((d[32 + bi + 1] << 8) | d[32 + bi]) >> bo) & 63
    w.append(float(c - 64 if c >= 32 else c))
x = [1.0, 2.0, 3.0, 4.0]
exp = [sum(x[k] * w[k * 4 + n] for k in range(4)) for n in range(4)]
mm.append(dict(name="matmul_q6_k_32s", cite="tests/q_dequant_tests.rs:625-730", qtype=Q6_K,
               data=bytes(d).hex(), n_rows=4, n_cols=4, input=x, expect=exp, tol=1e-2))
json_cases["matmul"] = mm

here = os.path.dirname(os.path.abspath(__file__))
with open(os.path.join(here, "reference_vectors.json"), "w") as f:
    json.dump(json_cases, f, indent=1)
print("wrote", len(cases), "dequant cases")
