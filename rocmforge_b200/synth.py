"""Seeded synthetic packed-weight tensors with the block contents of the benchmark configurations.

No model file or public dataset is used anywhere: every tensor is drawn from
numpy.random.Generator(PCG64(seed)) with the value laws below, in either layout family:

  RF    the byte layouts ROCmForge's own CPU dequant parses
        (src/kernels/quant/{q4_0,q8_0,q4_k,q6_k}.rs, src/loader/dequant.rs:41-132)
  GGUF  the llama.cpp/GGUF block layouts

Value laws: f16 scales d = f16(|N(0,1)| * s) with s = 0.02 (0.01 for Q8_0); 4/6-bit
codes uniform over all codes; Q8_0 codes uniform in [-127, 127]; K-quant 6-bit
scales/mins uniform bytes; MXFP block exponents uniform integers in [-8, 0].
"""
import numpy as np

Q4_0, Q8_0, Q4_K, Q6_K, MXFP4, MXFP6_E2M3, MXFP6_E3M2, Q2_K, Q3_K, Q5_K = range(10)
RF, GGUF = 0, 1
QNAMES = ["Q4_0", "Q8_0", "Q4_K", "Q6_K", "MXFP4", "MXFP6_E2M3", "MXFP6_E3M2", "Q2_K", "Q3_K", "Q5_K"]
LAYOUT_NAMES = ["RF", "GGUF"]

_BLOCK_ELEMS = [32, 32, 256, 256, 32, 32, 32, 256, 256, 256]
_BLOCK_BYTES = {RF: [20, 36, 256, 256, 17, 25, 25, 256, 256, 256], GGUF: [18, 34, 144, 210, 17, 25, 25, 84, 110, 176]}


def block_elems(qtype):
    return _BLOCK_ELEMS[qtype]


def block_bytes(qtype, layout):
    return _BLOCK_BYTES[layout][qtype]


def tensor_bytes(qtype, layout, n_elements):
    be = _BLOCK_ELEMS[qtype]
    return (n_elements + be - 1) // be * _BLOCK_BYTES[layout][qtype]


def rng_for(seed):
    return np.random.Generator(np.random.PCG64(seed))


def _f16_scales(rng, shape, s):
    return (np.abs(rng.standard_normal(shape, dtype=np.float32)) * np.float32(s)).astype(np.float16)


def _pack6_le(codes):
    """codes [..., 32] (0..63) -> bytes [..., 24], code i at bits [6i, 6i+6) little-endian."""
    c = codes.astype(np.uint32).reshape(codes.shape[:-1] + (8, 4))
    w = c[..., 0] | (c[..., 1] << 6) | (c[..., 2] << 12) | (c[..., 3] << 18)
    out = np.stack([w & 0xFF, (w >> 8) & 0xFF, (w >> 16) & 0xFF], axis=-1).astype(np.uint8)
    return out.reshape(codes.shape[:-1] + (24,))


def gen_packed(qtype, layout, n_elements, rng):
    """Packed bytes (uint8 array) of a tensor of n_elements weights (whole blocks)."""
    be = _BLOCK_ELEMS[qtype]
    nb = (n_elements + be - 1) // be
    bb = _BLOCK_BYTES[layout][qtype]
    out = np.zeros((nb, bb), dtype=np.uint8)
    if qtype == Q4_0:
        d = _f16_scales(rng, nb, 0.02)
        q = rng.integers(0, 16, size=(nb, 32), dtype=np.uint8)
        if layout == RF:   # f32 scale; byte i = q[2i] | q[2i+1] << 4
            out[:, 0:4] = d.astype(np.float32).view(np.uint8).reshape(nb, 4)
            out[:, 4:20] = q[:, 0::2] | (q[:, 1::2] << 4)
        else:              # f16 d; byte j = q[j] | q[j+16] << 4
            out[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
            out[:, 2:18] = q[:, :16] | (q[:, 16:] << 4)
    elif qtype == Q8_0:
        d = _f16_scales(rng, nb, 0.01)
        q = rng.integers(-127, 128, size=(nb, 32), dtype=np.int16)
        if layout == RF:   # f32 scale; unsigned byte = code + 128
            out[:, 0:4] = d.astype(np.float32).view(np.uint8).reshape(nb, 4)
            out[:, 4:36] = (q + 128).astype(np.uint8)
        else:
            out[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
            out[:, 2:34] = q.astype(np.int8).view(np.uint8)
    elif qtype == Q4_K:
        if layout == RF:   # 8 f16 scales @0, 8 int8 mins @16, 16 code bytes per 28-byte stripe @32
            sc = _f16_scales(rng, (nb, 8), 0.02)
            out[:, 0:16] = sc.view(np.uint8).reshape(nb, 16)
            out[:, 16:24] = rng.integers(0, 256, size=(nb, 8), dtype=np.uint8)
            codes = rng.integers(0, 256, size=(nb, 8, 16), dtype=np.uint8)
            for j in range(8):
                out[:, 32 + 28 * j: 32 + 28 * j + 16] = codes[:, j]
        else:              # f16 d, f16 dmin, 12 scale bytes, 128 nibble bytes
            out[:, 0:2] = _f16_scales(rng, nb, 0.02).view(np.uint8).reshape(nb, 2)
            out[:, 2:4] = _f16_scales(rng, nb, 0.02).view(np.uint8).reshape(nb, 2)
            out[:, 4:144] = rng.integers(0, 256, size=(nb, 140), dtype=np.uint8)
    elif qtype == Q6_K:
        if layout == RF:   # 16 f16 scales, 192 code bytes, 32 zero pad bytes
            out[:, 0:32] = _f16_scales(rng, (nb, 16), 0.02).view(np.uint8).reshape(nb, 32)
            out[:, 32:224] = rng.integers(0, 256, size=(nb, 192), dtype=np.uint8)
        else:              # ql 128, qh 64, 16 int8 scales, f16 d
            out[:, 0:208] = rng.integers(0, 256, size=(nb, 208), dtype=np.uint8)
            out[:, 208:210] = _f16_scales(rng, nb, 0.02).view(np.uint8).reshape(nb, 2)
    elif qtype == MXFP4:
        e = rng.integers(-8, 1, size=nb, dtype=np.int16)
        out[:, 0] = (e.astype(np.int8).view(np.uint8) if layout == RF else (e + 127).astype(np.uint8))
        out[:, 1:17] = rng.integers(0, 256, size=(nb, 16), dtype=np.uint8)
    elif qtype in (MXFP6_E2M3, MXFP6_E3M2):
        e = rng.integers(-8, 1, size=nb, dtype=np.int16)
        out[:, 0] = (e.astype(np.int8).view(np.uint8) if layout == RF else (e + 127).astype(np.uint8))
        out[:, 1:25] = rng.integers(0, 256, size=(nb, 24), dtype=np.uint8)
    elif qtype in (Q2_K, Q3_K, Q5_K):
        if layout == RF:   # 16 f16 scales @0, then mins / high bits / packed codes: every remaining byte is data
            out[:, 0:32] = _f16_scales(rng, (nb, 16), 0.02).view(np.uint8).reshape(nb, 32)
            if qtype == Q2_K:   # 16 f16 mins @32
                out[:, 32:64] = _f16_scales(rng, (nb, 16), 0.02).view(np.uint8).reshape(nb, 32)
                out[:, 64:256] = rng.integers(0, 256, size=(nb, 192), dtype=np.uint8)
            else:
                out[:, 32:256] = rng.integers(0, 256, size=(nb, 224), dtype=np.uint8)
        elif qtype == Q2_K:   # scales 16, qs 64, f16 d, f16 dmin
            out[:, 0:80] = rng.integers(0, 256, size=(nb, 80), dtype=np.uint8)
            out[:, 80:82] = _f16_scales(rng, nb, 0.02).view(np.uint8).reshape(nb, 2)
            out[:, 82:84] = _f16_scales(rng, nb, 0.02).view(np.uint8).reshape(nb, 2)
        elif qtype == Q3_K:   # hmask 32, qs 64, scales 12, f16 d
            out[:, 0:108] = rng.integers(0, 256, size=(nb, 108), dtype=np.uint8)
            out[:, 108:110] = _f16_scales(rng, nb, 0.02).view(np.uint8).reshape(nb, 2)
        else:                 # Q5_K: f16 d, f16 dmin, scales 12, qh 32, qs 128
            out[:, 0:2] = _f16_scales(rng, nb, 0.02).view(np.uint8).reshape(nb, 2)
            out[:, 2:4] = _f16_scales(rng, nb, 0.02).view(np.uint8).reshape(nb, 2)
            out[:, 4:176] = rng.integers(0, 256, size=(nb, 172), dtype=np.uint8)
    else:
        raise ValueError(f"unknown qtype {qtype}")
    return out.reshape(-1)


def gen_activations(m, k, rng):
    return rng.standard_normal((m, k), dtype=np.float32)


# ---- the five benchmark configurations (shapes only; contents via gen_packed) ----

def qwen2_0p5b_step():
    """Matmul list of one Qwen2-0.5B-shaped Q4_K_M decode step: (name, qtype, N, K)."""
    ops = []
    for layer in range(24):
        ops += [(f"blk.{layer}.attn_q", Q4_K, 896, 896), (f"blk.{layer}.attn_k", Q4_K, 128, 896),
                (f"blk.{layer}.attn_v", Q4_K, 128, 896), (f"blk.{layer}.attn_output", Q4_K, 896, 896),
                (f"blk.{layer}.ffn_gate", Q4_K, 4864, 896), (f"blk.{layer}.ffn_up", Q4_K, 4864, 896),
                (f"blk.{layer}.ffn_down", Q6_K, 896, 4864)]
    ops.append(("output", Q6_K, 151936, 896))
    return ops


CONFIG_SEEDS = {1: 1001, 2: 1002, 3: 1003, 4: 1004, 5: 1005}
LLAMA7B_SHAPES = [(11008, 4096), (4096, 11008), (4096, 4096)]
LLAMA70B_FFN_SHAPES = [(28672, 8192), (8192, 28672)]
