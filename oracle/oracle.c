/*
 * CPU oracle -- TEST INFRASTRUCTURE ONLY (see oracle.h). Restates, loop for loop,
 * the reference's CPU dequantisation and matmul. File:line citations are paths
 * inside the ROCmForge source tree.
 */
#include "oracle.h"
#include <math.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------ scalars */

float orc_f16_to_f32(uint16_t h) {
    /* half::f16::from_bits(h).to_f32(): exact widening, subnormals, inf, NaN kept. */
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do { e++; man <<= 1; } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

float orc_pow2i(int b) {
    /* f32::powi lowers to compiler-rt __powisf2: square-and-multiply on |b| then a
     * reciprocal for negative b. 2^-127 comes out as the exact subnormal; b = -128
     * overflows the intermediate to +inf and returns 1/inf = 0. */
    float a = 2.0f;
    const int recip = b < 0;
    float r = 1.0f;
    while (1) {
        if (b & 1) r *= a;
        b /= 2;
        if (b == 0) break;
        a *= a;
    }
    return recip ? 1.0f / r : r;
}

static inline float clampf(float v, float lo, float hi) {
    /* f32::clamp: NaN stays NaN. */
    if (v < lo) return lo;
    if (v > hi) return hi;
    return v;
}

/* ---------------------------------------------------------------- RF layout */

void rf_dequant_q4_0(const uint8_t* data, size_t nbytes, size_t n, float* out) {
    /* src/kernels/quant/q4_0.rs:266-310. 20-byte blocks: f32 scale + 16 bytes;
     * element 2i is the low nibble of byte i, element 2i+1 the high nibble. */
    size_t n_blocks = (n + 31) / 32;
    memset(out, 0, n * sizeof(float));
    for (size_t b = 0; b < n_blocks; b++) {
        size_t off = b * 20;
        if (off + 4 > nbytes) break;
        float scale;
        memcpy(&scale, data + off, 4);
        size_t ds = off + 4, base = b * 32;
        for (size_t i = 0; i < 16; i++) {
            if (ds + i >= nbytes) break;
            uint8_t p = data[ds + i];
            int lo = (int)(p & 0x0F) - 8;
            if (base + i * 2 < n) out[base + i * 2] = scale * (float)lo;
            int hi = (int)((p >> 4) & 0x0F) - 8;
            if (base + i * 2 + 1 < n) out[base + i * 2 + 1] = scale * (float)hi;
        }
    }
}

void rf_dequant_q8_0(const uint8_t* data, size_t nbytes, size_t n, float* out) {
    /* src/kernels/quant/q8_0.rs:23-71. 36-byte blocks: f32 scale + 32 bytes read as
     * unsigned, value = (q - 128) * scale. */
    size_t blocks = (n + 31) / 32;
    memset(out, 0, n * sizeof(float));
    for (size_t b = 0; b < blocks; b++) {
        size_t bs = b * 36;
        if (bs + 4 > nbytes) continue;
        float scale;
        memcpy(&scale, data + bs, 4);
        size_t qs = bs + 4;
        size_t qe = qs + 32 < nbytes ? qs + 32 : nbytes;
        for (size_t i = 0; qs + i < qe; i++) {
            size_t e = b * 32 + i;
            if (e < n) out[e] = ((float)data[qs + i] - 128.0f) * scale;
        }
    }
}

void rf_dequant_q8_0_i8(const uint8_t* data, size_t nbytes, size_t n, float* out) {
    /* Variant in src/kernels/matmul/quantized/q8_0.rs:18-54: bytes are int8 and the
     * value is scale * q (no 128 offset). Not the canonical oracle. */
    size_t blocks = (n + 31) / 32;
    memset(out, 0, n * sizeof(float));
    for (size_t b = 0; b < blocks; b++) {
        size_t bs = b * 36;
        if (bs + 4 > nbytes) break;
        float scale;
        memcpy(&scale, data + bs, 4);
        for (size_t i = 0; i < 32; i++) {
            size_t e = b * 32 + i;
            if (bs + 4 + i >= nbytes) break;
            if (e < n) out[e] = scale * (float)(int8_t)data[bs + 4 + i];
        }
    }
}

void rf_dequant_q4_k(const uint8_t* data, size_t nbytes, size_t n, float* out) {
    /* src/kernels/quant/q4_k.rs:201-273. 256-byte super-blocks: 8 f16 scales @0,
     * 8 int8 mins @16, quants @32 with a 28-byte stride per sub-block of which the
     * first 16 bytes carry the 32 nibbles. value = min + q * scale. */
    size_t nsb = (n + 255) / 256;
    memset(out, 0, n * sizeof(float));
    for (size_t sb = 0; sb < nsb; sb++) {
        size_t off = sb * 256;
        if (off + 256 > nbytes) break;
        size_t scales = off, mins = off + 16, quants = off + 32;
        for (size_t j = 0; j < 8; j++) {
            size_t start = sb * 256 + j * 32;
            if (start >= n) break;
            size_t so = scales + j * 2;
            float scale = 1.0f;
            if (so + 2 <= nbytes) scale = orc_f16_to_f32((uint16_t)(data[so] | (data[so + 1] << 8)));
            float mn = 0.0f;
            if (mins + j < nbytes) mn = (float)(int8_t)data[mins + j];
            for (size_t i = 0; i < 32; i++) {
                size_t e = start + i;
                if (e >= n) break;
                size_t bit_pos = i * 4, byte_idx = bit_pos / 8, bit_off = bit_pos % 8;
                size_t qo = quants + j * 28 + byte_idx;
                if (qo + 1 < nbytes) {
                    uint16_t comb = (uint16_t)((data[qo + 1] << 8) | data[qo]);
                    uint8_t q = (uint8_t)((comb >> bit_off) & 0x0F);
                    out[e] = mn + (float)q * scale;
                }
            }
        }
    }
}

void rf_dequant_q6_k(const uint8_t* data, size_t nbytes, size_t n, float* out) {
    /* src/kernels/quant/q6_k.rs:201-266. 256-byte blocks: 16 f16 scales @0, 192 bytes
     * of little-endian 6-bit codes @32, 32 bytes padding. Codes >= 32 mean code-64. */
    size_t nb = (n + 255) / 256;
    memset(out, 0, n * sizeof(float));
    for (size_t b = 0; b < nb; b++) {
        size_t bs = b * 256;
        if (bs + 256 > nbytes) break;
        size_t quants = bs + 32;
        for (size_t i = 0; i < 256; i++) {
            size_t e = b * 256 + i;
            if (e >= n) break;
            size_t so = bs + (i / 16) * 2;
            float scale = 1.0f;
            if (so + 2 <= nbytes) scale = orc_f16_to_f32((uint16_t)(data[so] | (data[so + 1] << 8)));
            size_t bit_off = (i * 6) % 8, byte_idx = (i * 6) / 8;
            if (quants + byte_idx + 1 < nbytes) {
                uint16_t comb = (uint16_t)((data[quants + byte_idx + 1] << 8) | data[quants + byte_idx]);
                uint8_t q = (uint8_t)((comb >> bit_off) & 0x3F);
                float sv = q >= 32 ? (float)((int)(int8_t)q - 64) : (float)q;
                out[e] = sv * scale;
            }
        }
    }
}

float rf_decode_e2m1(uint8_t bits) {
    /* src/loader/mxfp.rs:234-244: 0 -> 0; else sign * (1 + mant) * 2^(exp-1). */
    if (bits == 0) return 0.0f;
    float sign = (bits & 0x08) ? -1.0f : 1.0f;
    int exp = (int)((bits >> 1) & 0x03) - 1;
    float mant = (float)(bits & 0x01);
    return sign * (1.0f + mant) * orc_pow2i(exp);
}

float rf_decode_e2m3(uint8_t bits) {
    /* src/loader/mxfp.rs:283-293: 0 -> 0; else sign * (1 + mant/8) * 2^(exp-1). */
    if (bits == 0) return 0.0f;
    float sign = (bits & 0x20) ? -1.0f : 1.0f;
    int exp = (int)((bits >> 3) & 0x03) - 1;
    float mant = (float)(bits & 0x07) / 8.0f;
    return sign * (1.0f + mant) * orc_pow2i(exp);
}

void rf_dequant_mxfp4(const uint8_t* data, size_t nbytes, size_t n, float* out) {
    /* src/loader/dequant.rs:41-82. 17-byte blocks: int8 exponent then 16 bytes; the
     * HIGH nibble of byte j is element 2j, the low nibble element 2j+1; clamp to +-8. */
    size_t blocks = (n + 31) / 32;
    memset(out, 0, n * sizeof(float));
    for (size_t b = 0; b < blocks; b++) {
        size_t bs = b * 17;
        if (bs + 1 > nbytes) break;
        float scale = orc_pow2i((int)(int8_t)data[bs]);
        size_t ds = bs + 1;
        size_t de = ds + 16 < nbytes ? ds + 16 : nbytes;
        for (size_t bo = 0; ds + bo < de; bo++) {
            uint8_t p = data[ds + bo];
            for (int j = 0; j < 2; j++) {
                size_t e = b * 32 + bo * 2 + (size_t)j;
                if (e < n) {
                    uint8_t code = j == 0 ? (p >> 4) & 0x0F : p & 0x0F;
                    float v = scale * rf_decode_e2m1(code);
                    out[e] = clampf(v, -8.0f, 8.0f);
                }
            }
        }
    }
}

void rf_dequant_mxfp6(const uint8_t* data, size_t nbytes, size_t n, float* out) {
    /* src/loader/dequant.rs:85-132. 25-byte blocks: int8 exponent then 24 bytes.
     * bits = (le16(bytes at 6i/8) >> (10 - 6i%8)) & 63; element 31 of a block is
     * never written (byte_idx + 1 < 24 fails) and stays 0.0; clamp to +-7.5.
     * Both MXFP6 tensor types take this E2M3 path (dequant.rs:693). */
    size_t blocks = (n + 31) / 32;
    memset(out, 0, n * sizeof(float));
    for (size_t b = 0; b < blocks; b++) {
        size_t bs = b * 25;
        if (bs + 1 > nbytes) break;
        float scale = orc_pow2i((int)(int8_t)data[bs]);
        size_t ds = bs + 1;
        size_t de = ds + 24 < nbytes ? ds + 24 : nbytes;
        size_t plen = de - ds;
        const uint8_t* pk = data + ds;
        for (size_t i = 0; i < 32; i++) {
            size_t e = b * 32 + i;
            if (e >= n) break;
            size_t bit_off = (i * 6) % 8, byte_idx = (i * 6) / 8;
            if (byte_idx + 1 < plen) {
                uint16_t comb = (uint16_t)((pk[byte_idx + 1] << 8) | pk[byte_idx]);
                uint8_t bits = (uint8_t)((comb >> (10 - bit_off)) & 0x3F);
                float v = scale * rf_decode_e2m3(bits);
                out[e] = clampf(v, -7.5f, 7.5f);
            }
        }
    }
}

/* MxfpBlock encode / pack helpers (the reference's round-trip tests use them). */

uint8_t rf_encode_e2m1(float value) {
    /* src/loader/mxfp.rs:200-231 */
    if (value == 0.0f) return 0;
    uint8_t sign = value < 0.0f ? 0x8 : 0x0;
    float a = fabsf(value);
    float c = fminf(fmaxf(a, 0.5f), 8.0f);
    uint8_t best = 0;
    float best_err = 3.40282347e+38f;
    for (int e = 0; e < 4; e++)
        for (int m = 0; m < 2; m++) {
            float dec = (1.0f + (float)m) * orc_pow2i(e - 1);
            float err = fabsf(c - dec);
            if (err < best_err) { best_err = err; best = (uint8_t)((e << 1) | m); }
        }
    return sign | best;
}

uint8_t rf_encode_e2m3(float value) {
    /* src/loader/mxfp.rs:249-280 */
    if (value == 0.0f) return 0;
    uint8_t sign = value < 0.0f ? 0x20 : 0x00;
    float a = fabsf(value);
    float c = fminf(fmaxf(a, 0.5f), 7.5f);
    uint8_t best = 0;
    float best_err = 3.40282347e+38f;
    for (int e = 0; e < 4; e++)
        for (int m = 0; m < 8; m++) {
            float dec = (1.0f + (float)m / 8.0f) * orc_pow2i(e - 1);
            float err = fabsf(c - dec);
            if (err < best_err) { best_err = err; best = (uint8_t)((e << 3) | m); }
        }
    return sign | best;
}

int8_t rf_e8m0_from_f32(float v) {
    /* src/loader/mxfp.rs:29-43 */
    if (v == 0.0f || isnan(v)) return 0;
    if (isinf(v)) return 127;
    float l = log2f(fabsf(v));
    if (l < -127.0f) l = -127.0f;
    if (l > 127.0f) l = 127.0f;
    return (int8_t)roundf(l);
}

void rf_pack_6bit(const uint8_t* vals, size_t count, uint8_t* packed) {
    /* src/loader/mxfp.rs:297-320 */
    size_t nb = (count * 6 + 7) / 8;
    memset(packed, 0, nb);
    for (size_t i = 0; i < count; i++) {
        size_t bit_pos = i * 6, byte_idx = bit_pos / 8, bit_off = bit_pos % 8;
        uint8_t v = vals[i] & 0x3F;
        if (bit_off <= 2) {
            packed[byte_idx] |= (uint8_t)(v << bit_off);
        } else {
            size_t first = 8 - bit_off;
            packed[byte_idx] |= (uint8_t)(v << bit_off);
            packed[byte_idx + 1] |= (uint8_t)(v >> first);
        }
    }
}

void rf_unpack_6bit(const uint8_t* packed, size_t nbytes, size_t count, uint8_t* vals) {
    /* src/loader/mxfp.rs:324-353 */
    memset(vals, 0, count);
    for (size_t i = 0; i < count; i++) {
        size_t bit_pos = i * 6, byte_idx = bit_pos / 8, bit_off = bit_pos % 8;
        if (byte_idx < nbytes) {
            if (bit_off <= 2) {
                vals[i] = (packed[byte_idx] >> bit_off) & 0x3F;
            } else {
                size_t first = 8 - bit_off, second = 6 - first;
                uint8_t p1 = (uint8_t)((packed[byte_idx] >> bit_off) & ((1u << first) - 1));
                uint8_t p2 = byte_idx + 1 < nbytes ? (uint8_t)(packed[byte_idx + 1] & ((1u << second) - 1)) : 0;
                vals[i] = (uint8_t)(p1 | (p2 << first));
            }
        }
    }
}

void rf_mxfpblock_pack_mxfp4(const float* v, int8_t* exp_out, uint8_t* el) {
    /* src/loader/mxfp.rs:77-117 */
    float mx = 0.0f;
    for (int i = 0; i < 32; i++) mx = fmaxf(mx, fabsf(v[i]));
    int8_t e = mx == 0.0f ? 0 : rf_e8m0_from_f32(mx);
    float s = orc_pow2i(e);
    memset(el, 0, 16);
    for (int i = 0; i < 32; i++) {
        float nrm = s > 0.0f ? v[i] / s : v[i];
        uint8_t enc = rf_encode_e2m1(nrm);
        if (i % 2 == 0) el[i / 2] |= (uint8_t)(enc << 4);
        else el[i / 2] |= enc & 0x0F;
    }
    *exp_out = e;
}

void rf_mxfpblock_unpack_mxfp4(int8_t e, const uint8_t* el, float* out) {
    /* src/loader/mxfp.rs:120-139 */
    float s = orc_pow2i(e);
    for (int i = 0; i < 32; i++) {
        uint8_t nib = i % 2 == 0 ? (el[i / 2] >> 4) & 0x0F : el[i / 2] & 0x0F;
        out[i] = clampf(s * rf_decode_e2m1(nib), -8.0f, 8.0f);
    }
}

void rf_mxfpblock_pack_mxfp6(const float* v, int8_t* exp_out, uint8_t* el) {
    /* src/loader/mxfp.rs:142-174 */
    float mx = 0.0f;
    for (int i = 0; i < 32; i++) mx = fmaxf(mx, fabsf(v[i]));
    int8_t e = mx == 0.0f ? 0 : rf_e8m0_from_f32(mx);
    float s = orc_pow2i(e);
    uint8_t codes[32];
    for (int i = 0; i < 32; i++) {
        float nrm = s > 0.0f ? v[i] / s : v[i];
        codes[i] = rf_encode_e2m3(nrm);
    }
    rf_pack_6bit(codes, 32, el);
    *exp_out = e;
}

void rf_mxfpblock_unpack_mxfp6(int8_t e, const uint8_t* el, float* out) {
    /* src/loader/mxfp.rs:177-190 (little-endian >> bit_off order; NOT what
     * dequant_mxfp6 uses). */
    uint8_t codes[32];
    rf_unpack_6bit(el, 24, 32, codes);
    float s = orc_pow2i(e);
    for (int i = 0; i < 32; i++) out[i] = clampf(s * rf_decode_e2m3(codes[i]), -7.5f, 7.5f);
}

/* -------------------------------------------------------------- GGUF layout */
/* The llama.cpp / GGUF block formats, restated from their public description.
 * Blocks are complete: n is rounded down to whole blocks of input, a trailing
 * partial block is decoded as far as n. */

static inline uint16_t le16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

void gguf_dequant_q4_0(const uint8_t* data, size_t nbytes, size_t n, float* out) {
    /* 18 bytes: f16 d, 16 bytes; element j = low nibble of byte j, element j+16 =
     * high nibble of byte j; value = d * (q - 8). */
    memset(out, 0, n * sizeof(float));
    size_t nb = (n + 31) / 32;
    for (size_t b = 0; b < nb; b++) {
        if ((b + 1) * 18 > nbytes) break;
        const uint8_t* p = data + b * 18;
        float d = orc_f16_to_f32(le16(p));
        for (size_t j = 0; j < 16; j++) {
            size_t e0 = b * 32 + j, e1 = e0 + 16;
            if (e0 < n) out[e0] = d * (float)((int)(p[2 + j] & 0x0F) - 8);
            if (e1 < n) out[e1] = d * (float)((int)(p[2 + j] >> 4) - 8);
        }
    }
}

void gguf_dequant_q8_0(const uint8_t* data, size_t nbytes, size_t n, float* out) {
    /* 34 bytes: f16 d, 32 int8; value = q * d. */
    memset(out, 0, n * sizeof(float));
    size_t nb = (n + 31) / 32;
    for (size_t b = 0; b < nb; b++) {
        if ((b + 1) * 34 > nbytes) break;
        const uint8_t* p = data + b * 34;
        float d = orc_f16_to_f32(le16(p));
        for (size_t j = 0; j < 32; j++) {
            size_t e = b * 32 + j;
            if (e < n) out[e] = (float)(int8_t)p[2 + j] * d;
        }
    }
}

static inline void q4k_scale_min(const uint8_t* s, int j, uint8_t* sc, uint8_t* m) {
    /* 12 bytes hold eight 6-bit scales and eight 6-bit mins. */
    if (j < 4) {
        *sc = s[j] & 63;
        *m = s[j + 4] & 63;
    } else {
        *sc = (uint8_t)((s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4));
        *m = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
    }
}

void gguf_dequant_q4_k(const uint8_t* data, size_t nbytes, size_t n, float* out) {
    /* 144 bytes: f16 d, f16 dmin, 12 bytes of 6-bit scales/mins, 128 bytes of
     * nibbles. Each 32 bytes of nibbles cover 64 weights: low nibbles are sub-block
     * 2c, high nibbles sub-block 2c+1. value = (d*sc)*q - (dmin*m). */
    memset(out, 0, n * sizeof(float));
    size_t nb = (n + 255) / 256;
    for (size_t b = 0; b < nb; b++) {
        if ((b + 1) * 144 > nbytes) break;
        const uint8_t* p = data + b * 144;
        float d = orc_f16_to_f32(le16(p));
        float dmin = orc_f16_to_f32(le16(p + 2));
        const uint8_t* sc12 = p + 4;
        const uint8_t* qs = p + 16;
        for (int j = 0; j < 8; j++) {
            uint8_t sc, m;
            q4k_scale_min(sc12, j, &sc, &m);
            float d1 = d * (float)sc;
            float dm = dmin * (float)m;
            for (int l = 0; l < 32; l++) {
                size_t e = b * 256 + (size_t)j * 32 + (size_t)l;
                if (e >= n) break;
                uint8_t byte = qs[(j / 2) * 32 + l];
                uint8_t q = (j & 1) ? (byte >> 4) : (byte & 0x0F);
                out[e] = d1 * (float)q - dm;
            }
        }
    }
}

void gguf_dequant_q6_k(const uint8_t* data, size_t nbytes, size_t n, float* out) {
    /* 210 bytes: ql[128], qh[64], int8 scales[16], f16 d. Per 128 weights: 64 bytes
     * of ql and 32 bytes of qh; weight 32g+l of the half takes its low 4 bits from
     * ql[(g&1)*32+l] (low nibble for g<2, high for g>=2) and bits 4..5 from
     * qh[l] >> 2g. value = (d*scale[e/16]) * (q - 32). */
    memset(out, 0, n * sizeof(float));
    size_t nb = (n + 255) / 256;
    for (size_t b = 0; b < nb; b++) {
        if ((b + 1) * 210 > nbytes) break;
        const uint8_t* p = data + b * 210;
        const uint8_t* ql = p;
        const uint8_t* qh = p + 128;
        const int8_t* sc = (const int8_t*)(p + 192);
        float d = orc_f16_to_f32(le16(p + 208));
        for (int i = 0; i < 256; i++) {
            size_t e = b * 256 + (size_t)i;
            if (e >= n) break;
            int h = i / 128, r = i % 128, g = r / 32, l = r % 32;
            uint8_t lb = ql[h * 64 + (g & 1) * 32 + l];
            uint8_t lo = g < 2 ? (lb & 0x0F) : (lb >> 4);
            uint8_t hi = (qh[h * 32 + l] >> (2 * g)) & 3;
            int q = (int)(int8_t)(lo | (hi << 4)) - 32;
            float ds = d * (float)sc[i / 16];
            out[e] = ds * (float)q;
        }
    }
}

/* ------------------------------------------------------------------ remaining K-quants
 * RF layouts: src/loader/dequant.rs:150-233 (Q5_K), :243-322 (Q3_K), :326-419 (Q2_K). All three use 256-byte
 * blocks of 16 sub-blocks with f16 scales at the block start; a block that is not completely inside the
 * stream is skipped (":158 / :251 / :334 break"), so the per-element bounds tests inside are never taken. */

void rf_dequant_q5_k(const uint8_t* data, size_t nbytes, size_t n, float* out) {
    memset(out, 0, n * sizeof(float));
    size_t nb = (n + 255) / 256;
    for (size_t b = 0; b < nb; b++) {
        size_t bs = b * 256;
        if (bs + 256 > nbytes) break;
        for (int sb = 0; sb < 16; sb++) {
            float scale = orc_f16_to_f32(le16(data + bs + (size_t)sb * 2));
            float mn = (float)(int8_t)data[bs + 32 + (size_t)sb];
            for (int i = 0; i < 16; i++) {
                size_t e = b * 256 + (size_t)sb * 16 + (size_t)i;
                if (e >= n) break;
                int bit = i * 5, byte = bit / 8, off = bit % 8;
                size_t qo = bs + 48 + (size_t)sb * 10 + (size_t)byte;
                unsigned comb = ((unsigned)data[qo + 1] << 8) | (unsigned)data[qo];
                unsigned q = (comb >> off) & 0x1F;
                out[e] = mn + (float)q * scale;
            }
        }
    }
}

void rf_dequant_q3_k(const uint8_t* data, size_t nbytes, size_t n, float* out) {
    memset(out, 0, n * sizeof(float));
    size_t nb = (n + 255) / 256;
    for (size_t b = 0; b < nb; b++) {
        size_t bs = b * 256;
        if (bs + 256 > nbytes) break;
        for (int sb = 0; sb < 16; sb++) {
            float scale = orc_f16_to_f32(le16(data + bs + (size_t)sb * 2));
            unsigned qh = (data[bs + 32 + (size_t)(sb / 4)] >> ((sb % 4) * 2)) & 3u;
            for (int i = 0; i < 16; i++) {
                size_t e = b * 256 + (size_t)sb * 16 + (size_t)i;
                if (e >= n) break;
                int bit = i * 3, byte = bit / 8, off = bit % 8;
                size_t qo = bs + 36 + (size_t)sb * 6 + (size_t)byte;
                unsigned comb = ((unsigned)data[qo + 1] << 8) | (unsigned)data[qo];
                unsigned low = (comb >> off) & 7u;
                unsigned high = i < 8 ? ((qh >> i) & 1u) : 0u;   /* qh has two bits: only i = 0, 1 can see one */
                float quant = (float)(int8_t)(low | (high << 3)) - 4.0f;
                out[e] = quant * scale;
            }
        }
    }
}

void rf_dequant_q2_k(const uint8_t* data, size_t nbytes, size_t n, float* out) {
    memset(out, 0, n * sizeof(float));
    size_t nb = (n + 255) / 256;
    for (size_t b = 0; b < nb; b++) {
        size_t bs = b * 256;
        if (bs + 256 > nbytes) break;
        for (int sb = 0; sb < 16; sb++) {
            float scale = orc_f16_to_f32(le16(data + bs + (size_t)sb * 2));
            float mn = orc_f16_to_f32(le16(data + bs + 32 + (size_t)sb * 2));
            unsigned qh = (data[bs + 64 + (size_t)(sb / 8)] >> (sb % 8)) & 1u;
            for (int i = 0; i < 16; i++) {
                size_t e = b * 256 + (size_t)sb * 16 + (size_t)i;
                if (e >= n) break;
                int bit = i * 2, byte = bit / 8, off = bit % 8;
                size_t qo = bs + 68 + (size_t)sb * 4 + (size_t)byte;
                unsigned comb = ((unsigned)data[qo + 1] << 8) | (unsigned)data[qo];
                unsigned low = (comb >> off) & 3u;
                unsigned high = i < 8 ? ((qh >> i) & 1u) : 0u;   /* qh is one bit: only i = 0 can see it */
                float quant = (float)(int8_t)(low | (high << 2));
                out[e] = mn + quant * scale;
            }
        }
    }
}

/* GGUF layouts (llama.cpp block_q2_K 84 B, block_q3_K 110 B, block_q5_K 176 B). */

void gguf_dequant_q2_k(const uint8_t* data, size_t nbytes, size_t n, float* out) {
    /* scales[16] (low nibble scale, high nibble min), qs[64], f16 d, f16 dmin. Element 128h + 32j + l is
     * (qs[32h + l] >> 2j) & 3; value = (d*sc)*q - (dmin*m) with the scale pair of its group of 16. */
    memset(out, 0, n * sizeof(float));
    size_t nb = (n + 255) / 256;
    for (size_t b = 0; b < nb; b++) {
        if ((b + 1) * 84 > nbytes) break;
        const uint8_t* p = data + b * 84;
        float d = orc_f16_to_f32(le16(p + 80)), dmin = orc_f16_to_f32(le16(p + 82));
        for (int i = 0; i < 256; i++) {
            size_t e = b * 256 + (size_t)i;
            if (e >= n) break;
            int h = i / 128, j = (i % 128) / 32, l = i % 32;
            unsigned q = (p[16 + 32 * h + l] >> (2 * j)) & 3u;
            float dl = d * (float)(p[i / 16] & 0x0F);
            float ml = dmin * (float)(p[i / 16] >> 4);
            out[e] = dl * (float)q - ml;
        }
    }
}

void gguf_dequant_q3_k(const uint8_t* data, size_t nbytes, size_t n, float* out) {
    /* hmask[32], qs[64], scales[12], f16 d. Sixteen 6-bit scales (minus 32): low 4 bits from the nibbles of
     * bytes 0..7, high 2 bits from bytes 8..11. Element 128h + 32j + l has low bits (qs[32h + l] >> 2j) & 3 and
     * subtracts 4 when bit (e / 32) of hmask[l] is CLEAR. */
    memset(out, 0, n * sizeof(float));
    size_t nb = (n + 255) / 256;
    for (size_t b = 0; b < nb; b++) {
        if ((b + 1) * 110 > nbytes) break;
        const uint8_t* p = data + b * 110;
        const uint8_t* hm = p;
        const uint8_t* qs = p + 32;
        const uint8_t* sc = p + 96;
        float d = orc_f16_to_f32(le16(p + 108));
        for (int i = 0; i < 256; i++) {
            size_t e = b * 256 + (size_t)i;
            if (e >= n) break;
            int g = i / 16;
            unsigned lo = g < 8 ? (sc[g] & 0x0Fu) : (unsigned)(sc[g - 8] >> 4);
            unsigned hi = (unsigned)(sc[8 + (g % 4)] >> (2 * (g / 4))) & 3u;
            float dl = d * (float)((int)(int8_t)(lo | (hi << 4)) - 32);
            int h = i / 128, j = (i % 128) / 32, l = i % 32;
            int ql = (int)((qs[32 * h + l] >> (2 * j)) & 3u);
            int bitclear = ((hm[l] >> (i / 32)) & 1u) ^ 1u;
            out[e] = dl * (float)(ql - (bitclear << 2));
        }
    }
}

void gguf_dequant_q5_k(const uint8_t* data, size_t nbytes, size_t n, float* out) {
    /* f16 d, f16 dmin, 12 bytes of 6-bit scales/mins (as Q4_K), qh[32], qs[128]. Element 64c + 32nib + l has
     * low 4 bits (qs[32c + l] >> 4nib) & 15 and bit 4 = bit (e / 32) of qh[l]. */
    memset(out, 0, n * sizeof(float));
    size_t nb = (n + 255) / 256;
    for (size_t b = 0; b < nb; b++) {
        if ((b + 1) * 176 > nbytes) break;
        const uint8_t* p = data + b * 176;
        float d = orc_f16_to_f32(le16(p)), dmin = orc_f16_to_f32(le16(p + 2));
        const uint8_t* qh = p + 16;
        const uint8_t* qs = p + 48;
        for (int j = 0; j < 8; j++) {
            uint8_t sc, m;
            q4k_scale_min(p + 4, j, &sc, &m);
            float d1 = d * (float)sc, dm = dmin * (float)m;
            for (int l = 0; l < 32; l++) {
                size_t e = b * 256 + (size_t)j * 32 + (size_t)l;
                if (e >= n) break;
                unsigned lo = (j & 1) ? (unsigned)(qs[(j / 2) * 32 + l] >> 4) : (qs[(j / 2) * 32 + l] & 0x0Fu);
                unsigned hi = (qh[l] >> j) & 1u;
                out[e] = d1 * (float)(lo | (hi << 4)) - dm;
            }
        }
    }
}

static const int8_t k_e2m1_x2[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

static inline float e8m0_half(uint8_t x) {
    /* 2^(x-127) / 2 as an fp32 bit pattern (denormal for x < 2). */
    uint32_t bits = x < 2 ? (0x00200000u << x) : ((uint32_t)(x - 1) << 23);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

void gguf_dequant_mxfp4(const uint8_t* data, size_t nbytes, size_t n, float* out) {
    /* 17 bytes: biased E8M0 exponent, 16 bytes; element j = low nibble of byte j,
     * element j+16 = high nibble; OCP E2M1 values {0,.5,1,1.5,2,3,4,6} held doubled
     * and multiplied by half the block scale. */
    memset(out, 0, n * sizeof(float));
    size_t nb = (n + 31) / 32;
    for (size_t b = 0; b < nb; b++) {
        if ((b + 1) * 17 > nbytes) break;
        const uint8_t* p = data + b * 17;
        float d = e8m0_half(p[0]);
        for (size_t j = 0; j < 16; j++) {
            size_t e0 = b * 32 + j, e1 = e0 + 16;
            if (e0 < n) out[e0] = d * (float)k_e2m1_x2[p[1 + j] & 0x0F];
            if (e1 < n) out[e1] = d * (float)k_e2m1_x2[p[1 + j] >> 4];
        }
    }
}

static inline float e8m0_scale(uint8_t x) {
    /* OCP MX E8M0: 2^(x-127); 255 is NaN. */
    if (x == 255) return NAN;
    return ldexpf(1.0f, (int)x - 127);
}

static inline float ocp_e2m3(uint8_t c) {
    /* OCP FP6 E2M3: sign, 2 exponent bits (bias 1), 3 mantissa bits, subnormals. */
    float s = (c & 0x20) ? -1.0f : 1.0f;
    int e = (c >> 3) & 3, m = c & 7;
    float v = e == 0 ? (float)m * 0.125f : ldexpf(1.0f + (float)m * 0.125f, e - 1);
    return s * v;
}

static inline float ocp_e3m2(uint8_t c) {
    /* OCP FP6 E3M2: sign, 3 exponent bits (bias 3), 2 mantissa bits, subnormals. */
    float s = (c & 0x20) ? -1.0f : 1.0f;
    int e = (c >> 2) & 7, m = c & 3;
    float v = e == 0 ? ldexpf((float)m * 0.25f, -2) : ldexpf(1.0f + (float)m * 0.25f, e - 3);
    return s * v;
}

static void gguf_dequant_mxfp6(const uint8_t* data, size_t nbytes, size_t n, float* out, int e3m2) {
    /* 25 bytes: biased E8M0 exponent, 24 bytes holding 32 six-bit codes, code i at
     * bits [6i, 6i+6) of the little-endian bit stream. No public implementation of
     * a GGUF MXFP6 block exists; this is the OCP element table under a GGUF-style
     * block header ("parity unpinned"). */
    memset(out, 0, n * sizeof(float));
    size_t nb = (n + 31) / 32;
    for (size_t b = 0; b < nb; b++) {
        if ((b + 1) * 25 > nbytes) break;
        const uint8_t* p = data + b * 25;
        float d = e8m0_scale(p[0]);
        for (size_t i = 0; i < 32; i++) {
            size_t e = b * 32 + i;
            if (e >= n) break;
            size_t bit = i * 6, by = bit / 8, sh = bit % 8;
            uint32_t w = p[1 + by] | (by + 1 < 24 ? (uint32_t)p[2 + by] << 8 : 0u);
            uint8_t c = (uint8_t)((w >> sh) & 0x3F);
            out[e] = d * (e3m2 ? ocp_e3m2(c) : ocp_e2m3(c));
        }
    }
}

void gguf_dequant_mxfp6_e2m3(const uint8_t* data, size_t nbytes, size_t n, float* out) { gguf_dequant_mxfp6(data, nbytes, n, out, 0); }
void gguf_dequant_mxfp6_e3m2(const uint8_t* data, size_t nbytes, size_t n, float* out) { gguf_dequant_mxfp6(data, nbytes, n, out, 1); }

/* ------------------------------------------------------------- dispatcher */

size_t orc_block_elems(int qtype) { return (qtype == 2 || qtype == 3 || qtype >= 7) ? 256 : 32; }

size_t orc_block_bytes(int qtype, int layout) {
    static const size_t rf[10] = {20, 36, 256, 256, 17, 25, 25, 256, 256, 256};
    static const size_t gg[10] = {18, 34, 144, 210, 17, 25, 25, 84, 110, 176};
    if (qtype < 0 || qtype > 9) return 0;
    return layout == 0 ? rf[qtype] : gg[qtype];
}

typedef void (*deq_fn)(const uint8_t*, size_t, size_t, float*);

static deq_fn pick(int qtype, int layout) {
    static const deq_fn rf[10] = {rf_dequant_q4_0, rf_dequant_q8_0, rf_dequant_q4_k, rf_dequant_q6_k,
                                  rf_dequant_mxfp4, rf_dequant_mxfp6, rf_dequant_mxfp6,
                                  rf_dequant_q2_k, rf_dequant_q3_k, rf_dequant_q5_k};
    static const deq_fn gg[10] = {gguf_dequant_q4_0, gguf_dequant_q8_0, gguf_dequant_q4_k, gguf_dequant_q6_k,
                                  gguf_dequant_mxfp4, gguf_dequant_mxfp6_e2m3, gguf_dequant_mxfp6_e3m2,
                                  gguf_dequant_q2_k, gguf_dequant_q3_k, gguf_dequant_q5_k};
    if (qtype < 0 || qtype > 9 || layout < 0 || layout > 1) return 0;
    return layout == 0 ? rf[qtype] : gg[qtype];
}

int orc_dequantize(int qtype, int layout, const uint8_t* data, size_t nbytes, size_t n, float* out) {
    deq_fn f = pick(qtype, layout);
    if (!f) return -1;
    f(data, nbytes, n, out);
    return 0;
}

int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

int orc_dequantize_omp(int qtype, int layout, const uint8_t* data, size_t nbytes, size_t n, float* out, int threads) {
    /* Whole blocks are independent; split the stream into block-aligned chunks. */
    deq_fn f = pick(qtype, layout);
    if (!f) return -1;
    if (threads <= 0) threads = orc_max_threads();
    size_t be = orc_block_elems(qtype), bb = orc_block_bytes(qtype, layout);
    size_t nblk = (n + be - 1) / be;
    size_t per = (nblk + (size_t)threads - 1) / (size_t)threads;
    if (per == 0) per = 1;
    long chunks = (long)((nblk + per - 1) / per);
#pragma omp parallel for num_threads(threads) schedule(static)
    for (long c = 0; c < chunks; c++) {
        size_t b0 = (size_t)c * per;
        size_t b1 = b0 + per < nblk ? b0 + per : nblk;
        size_t e0 = b0 * be, e1 = b1 * be < n ? b1 * be : n;
        size_t off = b0 * bb;
        if (off >= nbytes) { memset(out + e0, 0, (e1 - e0) * sizeof(float)); continue; }
        f(data + off, nbytes - off, e1 - e0, out + e0);
    }
    return threads;
}

/* ------------------------------------------------------------------ matmul */

void orc_matmul_f32(const float* a, const float* b, int m, int n, int k, float* c) {
    /* src/tensor/matmul.rs:219-233 */
    for (int i = 0; i < m; i++)
        for (int j = 0; j < n; j++) {
            float sum = 0.0f;
            for (int l = 0; l < k; l++) sum += a[(size_t)i * k + l] * b[(size_t)l * n + j];
            c[(size_t)i * n + j] = sum;
        }
}

void orc_matmul_f32_nk(const float* a, const float* w, int m, int n, int k, float* c) {
    for (int i = 0; i < m; i++)
        for (int j = 0; j < n; j++) {
            float sum = 0.0f;
            const float* wr = w + (size_t)j * k;
            const float* ar = a + (size_t)i * k;
            for (int l = 0; l < k; l++) sum += ar[l] * wr[l];
            c[(size_t)i * n + j] = sum;
        }
}

void orc_matmul_f64(const float* a, const float* b, int m, int n, int k, double* c) {
    for (int i = 0; i < m; i++)
        for (int j = 0; j < n; j++) {
            double sum = 0.0;
            for (int l = 0; l < k; l++) sum += (double)a[(size_t)i * k + l] * (double)b[(size_t)l * n + j];
            c[(size_t)i * n + j] = sum;
        }
}

void orc_matmul_f64_nk(const float* a, const float* w, int m, int n, int k, double* c) {
    for (int i = 0; i < m; i++)
        for (int j = 0; j < n; j++) {
            double sum = 0.0;
            const float* wr = w + (size_t)j * k;
            const float* ar = a + (size_t)i * k;
            for (int l = 0; l < k; l++) sum += (double)ar[l] * (double)wr[l];
            c[(size_t)i * n + j] = sum;
        }
}

int orc_matmul_f32_nk_omp(const float* a, const float* w, int m, int n, int k, float* c, int threads) {
    if (threads <= 0) threads = orc_max_threads();
#pragma omp parallel for num_threads(threads) schedule(static)
    for (int j = 0; j < n; j++) {
        const float* wr = w + (size_t)j * k;
        for (int i = 0; i < m; i++) {
            float sum = 0.0f;
            const float* ar = a + (size_t)i * k;
            for (int l = 0; l < k; l++) sum += ar[l] * wr[l];
            c[(size_t)i * n + j] = sum;
        }
    }
    return threads;
}

int orc_matmul_f32_omp(const float* a, const float* b, int m, int n, int k, float* c, int threads) {
    if (threads <= 0) threads = orc_max_threads();
#pragma omp parallel for num_threads(threads) schedule(static)
    for (int j = 0; j < n; j++) {
        for (int i = 0; i < m; i++) {
            float sum = 0.0f;
            for (int l = 0; l < k; l++) sum += a[(size_t)i * k + l] * b[(size_t)l * n + j];
            c[(size_t)i * n + j] = sum;
        }
    }
    return threads;
}

/* ---------------------------------------------------------------- fused dequant + RMSNorm
 * kernels/fused_dequant_rmsnorm.hip:87-165. */
int orc_fused_dequant_rmsnorm(int qtype, int layout, const uint8_t* data, size_t nbytes, int seq_len, int hidden,
                              const float* weight, float eps, float* out) {
    size_t n = (size_t)seq_len * (size_t)hidden;
    int rc = orc_dequantize(qtype, layout, data, nbytes, n, out);
    if (rc < 0) return rc;
    for (int r = 0; r < seq_len; r++) {
        float* row = out + (size_t)r * hidden;
        float part[256];
        for (int t = 0; t < 256; t++) {
            float s = 0.0f;
            for (int j = t; j < hidden; j += 256) s = s + row[j] * row[j];
            part[t] = s;
        }
        for (int stride = 128; stride > 0; stride >>= 1)
            for (int t = 0; t < stride; t++) part[t] = part[t] + part[t + stride];
        float mean_sq = part[0] / (float)hidden;
        float rms = 1.0f / sqrtf(mean_sq + eps);
        for (int j = 0; j < hidden; j++) row[j] = row[j] * rms * weight[j];
    }
    return 0;
}

/* kernels/swiglu.hip:37-63 */
void orc_swiglu(const float* gate, const float* up, float* out, size_t n) {
    for (size_t i = 0; i < n; i++) {
        const float u = up[i];
        const float sigmoid_up = 1.0f / (1.0f + expf(-u));
        const float swish_up = u * sigmoid_up;
        out[i] = gate[i] * swish_up;
    }
}

/* src/backend/hip_backend/backend.rs:960-972: y_row = 1.0 * bias + y_row */
void orc_add_row_bias(float* y, const float* bias, size_t rows, size_t cols) {
    for (size_t r = 0; r < rows; r++)
        for (size_t j = 0; j < cols; j++) y[r * cols + j] = 1.0f * bias[j] + y[r * cols + j];
}
