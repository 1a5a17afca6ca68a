// Block formats of the quantized-weight path: device-side storage and exact decoding.
//
// A packed tensor lives on the device as up to four "planes". Formats whose blocks are already
// 16-byte multiples stay as one raw plane; the others are split at upload into a header plane and
// 16/8-byte aligned code planes holding exactly the same bytes (same total size):
//
//   fmt = qtype*2 + layout      planes (bytes per block, in the order they occur in the file block)
//   Q4_0  RF   {4 f32 scale, 16 codes}            Q4_0  GGUF {2 f16 d, 16 codes}
//   Q8_0  RF   {4 f32 scale, 32 codes}            Q8_0  GGUF {2 f16 d, 32 codes}
//   Q4_K  RF   {256 raw}                          Q4_K  GGUF {144 raw}
//   Q6_K  RF   {256 raw}                          Q6_K  GGUF {128 ql, 64 qh, 16 scales, 2 d}
//   MXFP4 RF/GGUF {1 exponent, 16 codes}          MXFP6 RF/GGUF {1 exponent, 24 codes}
//   Q2_K/Q3_K/Q5_K RF {256 raw}                   Q2_K GGUF {16 scales, 64 qs, 4 d+dmin}
//   Q3_K  GGUF {32 hmask, 64 qs, 12 scales, 2 d}  Q5_K GGUF {176 raw}
//
// decode8<F>() returns the fp32 values of 8 consecutive weights exactly as the reference CPU code
// computes them (ROCmForge src/kernels/quant/{q4_0,q8_0,q4_k,q6_k}.rs, src/loader/dequant.rs:41-132)
// or, for the GGUF family, as the llama.cpp block definitions give them. Every rounding step is an
// explicit __f*_rn so the compiler cannot contract or reorder it.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace b200q {

enum : int { Q4_0 = 0, Q8_0 = 1, Q4_K = 2, Q6_K = 3, MXFP4 = 4, MXFP6_E2M3 = 5, MXFP6_E3M2 = 6, Q2_K = 7, Q3_K = 8, Q5_K = 9, NUM_QTYPES = 10 };
enum : int { RF = 0, GGUF = 1 };
constexpr int NUM_FMTS = NUM_QTYPES * 2;
__host__ __device__ constexpr int fmt_of(int qtype, int layout) { return qtype * 2 + layout; }

struct WView {
    const uint8_t* p[4];
};

struct FmtInfo {
    int block_elems;
    int block_bytes;
    int nplanes;
    int plane_bytes[4];
};

__host__ __device__ constexpr FmtInfo fmt_info(int fmt) {
    switch (fmt) {
        case fmt_of(Q4_0, RF): return {32, 20, 2, {4, 16, 0, 0}};
        case fmt_of(Q4_0, GGUF): return {32, 18, 2, {2, 16, 0, 0}};
        case fmt_of(Q8_0, RF): return {32, 36, 2, {4, 32, 0, 0}};
        case fmt_of(Q8_0, GGUF): return {32, 34, 2, {2, 32, 0, 0}};
        case fmt_of(Q4_K, RF): return {256, 256, 1, {256, 0, 0, 0}};
        case fmt_of(Q4_K, GGUF): return {256, 144, 1, {144, 0, 0, 0}};
        case fmt_of(Q6_K, RF): return {256, 256, 1, {256, 0, 0, 0}};
        case fmt_of(Q6_K, GGUF): return {256, 210, 4, {128, 64, 16, 2}};
        case fmt_of(MXFP4, RF):
        case fmt_of(MXFP4, GGUF): return {32, 17, 2, {1, 16, 0, 0}};
        case fmt_of(MXFP6_E2M3, RF):
        case fmt_of(MXFP6_E2M3, GGUF):
        case fmt_of(MXFP6_E3M2, RF):
        case fmt_of(MXFP6_E3M2, GGUF): return {32, 25, 2, {1, 24, 0, 0}};
        case fmt_of(Q2_K, RF):
        case fmt_of(Q3_K, RF):
        case fmt_of(Q5_K, RF): return {256, 256, 1, {256, 0, 0, 0}};
        case fmt_of(Q2_K, GGUF): return {256, 84, 3, {16, 64, 4, 0}};
        case fmt_of(Q3_K, GGUF): return {256, 110, 4, {32, 64, 12, 2}};
        case fmt_of(Q5_K, GGUF): return {256, 176, 1, {176, 0, 0, 0}};
        default: return {0, 0, 0, {0, 0, 0, 0}};
    }
}

#ifdef __CUDACC__

__device__ __forceinline__ float f16bits_to_f32(uint16_t b) { return __half2float(__ushort_as_half(b)); }
__device__ __forceinline__ uint16_t ld16(const uint8_t* p) { return *reinterpret_cast<const uint16_t*>(p); }
__device__ __forceinline__ uint32_t ld32(const uint8_t* p) { return *reinterpret_cast<const uint32_t*>(p); }
__device__ __forceinline__ float ldf32(const uint8_t* p) { return *reinterpret_cast<const float*>(p); }

// 2^e for a signed-byte exponent the way f32::powi(2.0, e) evaluates it (src/loader/mxfp.rs:23-25):
// exact for e in [-127, 127] (2^-127 is the fp32 subnormal), 0.0 for e = -128.
__device__ __forceinline__ float rf_e8m0(uint8_t byte) {
    int e = (int)(int8_t)byte;
    uint32_t bits = e == -128 ? 0u : (e == -127 ? 0x00400000u : (uint32_t)(e + 127) << 23);
    return __uint_as_float(bits);
}
// Biased E8M0 halved (2^(x-127)/2), the scale llama.cpp multiplies doubled E2M1 values with.
__device__ __forceinline__ float gguf_e8m0_half(uint8_t x) {
    uint32_t bits = x < 2 ? (0x00200000u << x) : ((uint32_t)(x - 1) << 23);
    return __uint_as_float(bits);
}
// OCP E8M0: 2^(x-127), 255 = NaN.
__device__ __forceinline__ float ocp_e8m0(uint8_t x) {
    uint32_t bits = x == 255 ? 0x7FC00000u : (x == 0 ? 0x00400000u : (uint32_t)x << 23);
    return __uint_as_float(bits);
}
// MxfpBlock::decode_e2m1 (src/loader/mxfp.rs:234-244): 0 -> 0, else sign*(1+m)*2^(e-1).
__device__ __forceinline__ float rf_e2m1(uint32_t c) {
    if (c == 0) return 0.0f;
    float mag = (float)(1 + (c & 1)) * __uint_as_float((126u + ((c >> 1) & 3)) << 23);
    return (c & 8) ? -mag : mag;
}
// MxfpBlock::decode_e2m3 (src/loader/mxfp.rs:283-293): 0 -> 0, else sign*(1+m/8)*2^(e-1).
__device__ __forceinline__ float rf_e2m3(uint32_t c) {
    if (c == 0) return 0.0f;
    float mag = (float)(8 + (c & 7)) * __uint_as_float((123u + ((c >> 3) & 3)) << 23);
    return (c & 0x20) ? -mag : mag;
}
// OCP E2M1 doubled, as an integer in {0,1,2,3,4,6,8,12} with sign (code 8 gives +0).
__device__ __forceinline__ float ocp_e2m1_x2(uint32_t c) {
    uint32_t a = c & 7;
    int mag = a < 2 ? (int)a : (int)((2 + (a & 1)) << ((a >> 1) - 1));
    return (float)((c & 8) ? -mag : mag);
}
__device__ __forceinline__ float ocp_e2m3(uint32_t c) {
    uint32_t e = (c >> 3) & 3, m = c & 7;
    float mag = e == 0 ? (float)m * 0.125f : (float)(8 + m) * __uint_as_float((123u + e) << 23);
    return (c & 0x20) ? -mag : mag;
}
__device__ __forceinline__ float ocp_e3m2(uint32_t c) {
    uint32_t e = (c >> 2) & 7, m = c & 3;
    float mag = e == 0 ? (float)m * 0.0625f : (float)(4 + m) * __uint_as_float((122u + e) << 23);
    return (c & 0x20) ? -mag : mag;
}
__device__ __forceinline__ float clamp_pm(float v, float lim) { return fminf(fmaxf(v, -lim), lim); }

// Six-bit scale / min j of a GGUF Q4_K block from its 12 packed bytes.
__device__ __forceinline__ void q4k_scale_min(const uint8_t* s, int j, uint32_t& sc, uint32_t& m) {
    if (j < 4) {
        sc = s[j] & 63;
        m = s[j + 4] & 63;
    } else {
        sc = (s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4);
        m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

// fp32 values of weights [32*g + 8*part, +8) of the flat element stream. g is the index of the
// 32-weight group, part is 0..3.
template <int F>
__device__ __forceinline__ void decode8(const WView& v, int64_t g, int part, float (&out)[8]) {
    if constexpr (F == fmt_of(Q4_0, RF)) {
        // element 2i = low nibble of byte i, 2i+1 = high nibble; value = scale * (q - 8)
        float s = ldf32(v.p[0] + g * 4);
        uint32_t w = ld32(v.p[1] + g * 16 + part * 4);
#pragma unroll
        for (int j = 0; j < 8; j++) out[j] = __fmul_rn(s, (float)((int)((w >> (4 * j)) & 15) - 8));
    } else if constexpr (F == fmt_of(Q4_0, GGUF)) {
        // element j = low nibble of byte j, element j+16 = high nibble; value = d * (q - 8)
        float d = f16bits_to_f32(ld16(v.p[0] + g * 2));
        const uint8_t* q = v.p[1] + g * 16 + (part & 1) * 8;
        uint32_t w0 = ld32(q), w1 = ld32(q + 4);
        int sh = (part >> 1) * 4;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            out[j] = __fmul_rn(d, (float)((int)((w0 >> (8 * j + sh)) & 15) - 8));
            out[j + 4] = __fmul_rn(d, (float)((int)((w1 >> (8 * j + sh)) & 15) - 8));
        }
    } else if constexpr (F == fmt_of(Q8_0, RF)) {
        // value = ((float)u8 - 128) * scale
        float s = ldf32(v.p[0] + g * 4);
        const uint8_t* q = v.p[1] + g * 32 + part * 8;
        uint32_t w0 = ld32(q), w1 = ld32(q + 4);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            out[j] = __fmul_rn(__fsub_rn((float)((w0 >> (8 * j)) & 255), 128.0f), s);
            out[j + 4] = __fmul_rn(__fsub_rn((float)((w1 >> (8 * j)) & 255), 128.0f), s);
        }
    } else if constexpr (F == fmt_of(Q8_0, GGUF)) {
        float d = f16bits_to_f32(ld16(v.p[0] + g * 2));
        const uint8_t* q = v.p[1] + g * 32 + part * 8;
        uint32_t w0 = ld32(q), w1 = ld32(q + 4);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            out[j] = __fmul_rn((float)(int8_t)((w0 >> (8 * j)) & 255), d);
            out[j + 4] = __fmul_rn((float)(int8_t)((w1 >> (8 * j)) & 255), d);
        }
    } else if constexpr (F == fmt_of(Q4_K, RF)) {
        // 256-byte super-block: f16 scales @0, int8 mins @16, nibbles @32 + 28*sub; value = min + q*scale
        const uint8_t* b = v.p[0] + (g >> 3) * 256;
        int j = (int)(g & 7);
        float sc = f16bits_to_f32(ld16(b + 2 * j));
        float mn = (float)(int8_t)b[16 + j];
        uint32_t w = ld32(b + 32 + 28 * j + part * 4);
#pragma unroll
        for (int i = 0; i < 8; i++) out[i] = __fadd_rn(mn, __fmul_rn((float)((w >> (4 * i)) & 15), sc));
    } else if constexpr (F == fmt_of(Q4_K, GGUF)) {
        // 144-byte super-block: d, dmin, 12 scale bytes, 128 nibble bytes; value = (d*sc)*q - dmin*m
        const uint8_t* b = v.p[0] + (g >> 3) * 144;
        int j = (int)(g & 7);
        float d = f16bits_to_f32(ld16(b)), dmin = f16bits_to_f32(ld16(b + 2));
        uint32_t sc, m;
        q4k_scale_min(b + 4, j, sc, m);
        float d1 = __fmul_rn(d, (float)sc), dm = __fmul_rn(dmin, (float)m);
        const uint8_t* q = b + 16 + (j >> 1) * 32 + part * 8;
        uint32_t w0 = ld32(q), w1 = ld32(q + 4);
        int sh = (j & 1) * 4;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            out[i] = __fsub_rn(__fmul_rn(d1, (float)((w0 >> (8 * i + sh)) & 15)), dm);
            out[i + 4] = __fsub_rn(__fmul_rn(d1, (float)((w1 >> (8 * i + sh)) & 15)), dm);
        }
    } else if constexpr (F == fmt_of(Q6_K, RF)) {
        // 256-byte block: 16 f16 scales @0, little-endian 6-bit stream @32; codes >= 32 mean code-64
        const uint8_t* b = v.p[0] + (g >> 3) * 256;
        int j = (int)(g & 7);
        float sc = f16bits_to_f32(ld16(b + 2 * (2 * j + (part >> 1))));
        const uint8_t* q = b + 32 + 24 * j + 6 * part;
        uint64_t bits = (uint64_t)ld16(q) | ((uint64_t)ld16(q + 2) << 16) | ((uint64_t)ld16(q + 4) << 32);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            int c = (int)((bits >> (6 * i)) & 63);
            out[i] = __fmul_rn((float)(c >= 32 ? c - 64 : c), sc);
        }
    } else if constexpr (F == fmt_of(Q6_K, GGUF)) {
        // planes ql[128], qh[64], int8 scales[16], f16 d; value = (d*scale) * (q - 32)
        int64_t blk = g >> 3;
        int i0 = (int)(g & 7) * 32 + part * 8;   // first element inside the block
        int h = i0 >> 7, r = i0 & 127, gg = r >> 5, l0 = r & 31;
        const uint8_t* ql = v.p[0] + blk * 128 + h * 64 + (gg & 1) * 32 + l0;
        const uint8_t* qh = v.p[1] + blk * 64 + h * 32 + l0;
        float d = f16bits_to_f32(ld16(v.p[3] + blk * 2));
        float ds = __fmul_rn(d, (float)(int8_t)v.p[2][blk * 16 + (i0 >> 4)]);
        uint32_t l0w = ld32(ql), l1w = ld32(ql + 4), h0w = ld32(qh), h1w = ld32(qh + 4);
        int lsh = (gg >> 1) * 4, hsh = 2 * gg;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            int qa = (int)(((l0w >> (8 * i + lsh)) & 15) | (((h0w >> (8 * i + hsh)) & 3) << 4)) - 32;
            int qb = (int)(((l1w >> (8 * i + lsh)) & 15) | (((h1w >> (8 * i + hsh)) & 3) << 4)) - 32;
            out[i] = __fmul_rn(ds, (float)qa);
            out[i + 4] = __fmul_rn(ds, (float)qb);
        }
    } else if constexpr (F == fmt_of(MXFP4, RF)) {
        // int8 exponent; HIGH nibble of byte j is element 2j; clamp to +-8
        float s = rf_e8m0(v.p[0][g]);
        uint32_t w = ld32(v.p[1] + g * 16 + part * 4);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint32_t byte = (w >> (8 * j)) & 255;
            out[2 * j] = clamp_pm(__fmul_rn(s, rf_e2m1(byte >> 4)), 8.0f);
            out[2 * j + 1] = clamp_pm(__fmul_rn(s, rf_e2m1(byte & 15)), 8.0f);
        }
    } else if constexpr (F == fmt_of(MXFP4, GGUF)) {
        float d = gguf_e8m0_half(v.p[0][g]);
        const uint8_t* q = v.p[1] + g * 16 + (part & 1) * 8;
        uint32_t w0 = ld32(q), w1 = ld32(q + 4);
        int sh = (part >> 1) * 4;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            out[j] = __fmul_rn(d, ocp_e2m1_x2((w0 >> (8 * j + sh)) & 15));
            out[j + 4] = __fmul_rn(d, ocp_e2m1_x2((w1 >> (8 * j + sh)) & 15));
        }
    } else if constexpr (F == fmt_of(MXFP6_E2M3, RF) || F == fmt_of(MXFP6_E3M2, RF)) {
        // bits = (le16 at byte 6i/8) >> (10 - 6i%8); element 31 is never written; clamp to +-7.5.
        // Both MXFP6 tensor types decode as E2M3 (src/loader/dequant.rs:693).
        float s = rf_e8m0(v.p[0][g]);
        const uint8_t* q = v.p[1] + g * 24 + 6 * part;
        uint8_t by[8];
#pragma unroll
        for (int i = 0; i < 6; i++) by[i] = q[i];
        by[6] = part < 3 ? q[6] : 0;
        by[7] = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            int bit = 6 * i, bi = bit >> 3, bo = bit & 7;
            uint32_t comb = ((uint32_t)by[bi + 1] << 8) | by[bi];
            uint32_t c = (comb >> (10 - bo)) & 63;
            float val = clamp_pm(__fmul_rn(s, rf_e2m3(c)), 7.5f);
            out[i] = (part == 3 && i == 7) ? 0.0f : val;
        }
    } else if constexpr (F == fmt_of(MXFP6_E2M3, GGUF) || F == fmt_of(MXFP6_E3M2, GGUF)) {
        float d = ocp_e8m0(v.p[0][g]);
        const uint8_t* q = v.p[1] + g * 24 + 6 * part;
        uint64_t bits = (uint64_t)ld16(q) | ((uint64_t)ld16(q + 2) << 16) | ((uint64_t)ld16(q + 4) << 32);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            uint32_t c = (uint32_t)((bits >> (6 * i)) & 63);
            out[i] = __fmul_rn(d, F == fmt_of(MXFP6_E2M3, GGUF) ? ocp_e2m3(c) : ocp_e3m2(c));
        }
    } else if constexpr (F == fmt_of(Q5_K, RF) || F == fmt_of(Q3_K, RF) || F == fmt_of(Q2_K, RF)) {
        // 256-byte blocks of 16 sub-blocks x 16 weights (src/loader/dequant.rs:150-419): f16 scales @0, then
        //   Q5_K: int8 mins @32, 5-bit codes 10 bytes per sub-block @48;            value = min + q * scale
        //   Q3_K: 2 "high" bits per sub-block @32, 3-bit codes 6 bytes per sub-block @36; value = (q - 4) * scale
        //   Q2_K: f16 mins @32, 1 "high" bit per sub-block @64, 2-bit codes 4 bytes @68;  value = min + q * scale
        // The eight weights of a piece lie in one sub-block (i = 0 or 8 inside it).
        const uint8_t* b = v.p[0] + (g >> 3) * 256;
        const int i0 = (int)(g & 7) * 32 + part * 8, sb = i0 >> 4, i = i0 & 15;
        const float scale = f16bits_to_f32((uint16_t)(b[2 * sb] | (b[2 * sb + 1] << 8)));
        constexpr int BITS = F == fmt_of(Q5_K, RF) ? 5 : F == fmt_of(Q3_K, RF) ? 3 : 2;
        constexpr int QOFF = F == fmt_of(Q5_K, RF) ? 48 : F == fmt_of(Q3_K, RF) ? 36 : 68;
        const uint8_t* q = b + QOFF + sb * (2 * BITS) + (i * BITS) / 8;      // i * BITS is a multiple of 8
        uint64_t bits = 0;
#pragma unroll
        for (int t = 0; t < BITS; t++) bits |= (uint64_t)q[t] << (8 * t);   // 8 codes = BITS bytes
        float mn = 0.0f;
        uint32_t qh = 0;
        if constexpr (F == fmt_of(Q5_K, RF)) mn = (float)(int8_t)b[32 + sb];
        if constexpr (F == fmt_of(Q2_K, RF)) {
            mn = f16bits_to_f32((uint16_t)(b[32 + 2 * sb] | (b[33 + 2 * sb] << 8)));
            qh = (b[64 + (sb >> 3)] >> (sb & 7)) & 1u;
        }
        if constexpr (F == fmt_of(Q3_K, RF)) qh = (b[32 + (sb >> 2)] >> ((sb & 3) * 2)) & 3u;
#pragma unroll
        for (int t = 0; t < 8; t++) {
            const uint32_t low = (uint32_t)(bits >> (BITS * t)) & ((1u << BITS) - 1);
            const int e = i + t;                                              // element inside the sub-block
            if constexpr (F == fmt_of(Q5_K, RF)) {
                out[t] = __fadd_rn(mn, __fmul_rn((float)low, scale));
            } else if constexpr (F == fmt_of(Q3_K, RF)) {
                const uint32_t high = e < 8 ? (qh >> e) & 1u : 0u;
                out[t] = __fmul_rn(__fsub_rn((float)(int)(low | (high << 3)), 4.0f), scale);
            } else {
                const uint32_t high = e < 8 ? (qh >> e) & 1u : 0u;
                out[t] = __fadd_rn(mn, __fmul_rn((float)(int)(low | (high << 2)), scale));
            }
        }
    } else if constexpr (F == fmt_of(Q2_K, GGUF) || F == fmt_of(Q3_K, GGUF)) {
        // element 128h + 32j + l of a block has its low two bits at (qs[32h + l] >> 2j) & 3
        const int64_t blk = g >> 3;
        const int i0 = (int)(g & 7) * 32 + part * 8;
        const int h = i0 >> 7, j = (i0 & 127) >> 5, l0 = i0 & 31;
        const uint8_t* qs = v.p[1] + blk * 64 + 32 * h + l0;
        const uint32_t w0 = ld32(qs), w1 = ld32(qs + 4);
        if constexpr (F == fmt_of(Q2_K, GGUF)) {
            // planes scales[16] (scale | min << 4), qs[64], {f16 d, f16 dmin}; value = (d*sc)*q - dmin*m
            const float d = f16bits_to_f32(ld16(v.p[2] + blk * 4)), dmin = f16bits_to_f32(ld16(v.p[2] + blk * 4 + 2));
            const uint32_t sc = v.p[0][blk * 16 + (i0 >> 4)];
            const float dl = __fmul_rn(d, (float)(sc & 15)), ml = __fmul_rn(dmin, (float)(sc >> 4));
#pragma unroll
            for (int t = 0; t < 4; t++) {
                out[t] = __fsub_rn(__fmul_rn(dl, (float)((w0 >> (8 * t + 2 * j)) & 3)), ml);
                out[t + 4] = __fsub_rn(__fmul_rn(dl, (float)((w1 >> (8 * t + 2 * j)) & 3)), ml);
            }
        } else {
            // planes hmask[32], qs[64], scales[12], f16 d; sixteen 6-bit scales minus 32; a CLEAR hmask bit
            // (bit e/32 of hmask[l]) subtracts 4
            const float d = f16bits_to_f32(ld16(v.p[3] + blk * 2));
            const uint8_t* sc = v.p[2] + blk * 12;
            const int g16 = i0 >> 4;
            const uint32_t lo = g16 < 8 ? (sc[g16] & 15u) : (uint32_t)(sc[g16 - 8] >> 4);
            const uint32_t hi = (uint32_t)(sc[8 + (g16 & 3)] >> (2 * (g16 >> 2))) & 3u;
            const float dl = __fmul_rn(d, (float)((int)(lo | (hi << 4)) - 32));
            const uint8_t* hm = v.p[0] + blk * 32 + l0;
            const uint32_t m0 = ld32(hm), m1 = ld32(hm + 4);
            const int bit = i0 >> 5;
#pragma unroll
            for (int t = 0; t < 4; t++) {
                const int qa = (int)((w0 >> (8 * t + 2 * j)) & 3) - (int)((((m0 >> (8 * t + bit)) & 1) ^ 1) << 2);
                const int qb = (int)((w1 >> (8 * t + 2 * j)) & 3) - (int)((((m1 >> (8 * t + bit)) & 1) ^ 1) << 2);
                out[t] = __fmul_rn(dl, (float)qa);
                out[t + 4] = __fmul_rn(dl, (float)qb);
            }
        }
    } else if constexpr (F == fmt_of(Q5_K, GGUF)) {
        // 176-byte block: d, dmin, 12 scale bytes (as Q4_K), qh[32], qs[128]; element 64c + 32nib + l has low
        // bits (qs[32c + l] >> 4nib) & 15 and bit 4 = bit (e / 32) of qh[l]; value = (d*sc)*q - dmin*m
        const uint8_t* b = v.p[0] + (g >> 3) * 176;
        const int j = (int)(g & 7);
        const float d = f16bits_to_f32(ld16(b)), dmin = f16bits_to_f32(ld16(b + 2));
        uint32_t sc, m;
        q4k_scale_min(b + 4, j, sc, m);
        const float d1 = __fmul_rn(d, (float)sc), dm = __fmul_rn(dmin, (float)m);
        const uint8_t* q = b + 48 + (j >> 1) * 32 + part * 8;
        const uint8_t* qh = b + 16 + part * 8;
        const uint32_t w0 = ld32(q), w1 = ld32(q + 4), h0 = ld32(qh), h1 = ld32(qh + 4);
        const int sh = (j & 1) * 4;
#pragma unroll
        for (int t = 0; t < 4; t++) {
            const uint32_t qa = ((w0 >> (8 * t + sh)) & 15) | (((h0 >> (8 * t + j)) & 1) << 4);
            const uint32_t qb = ((w1 >> (8 * t + sh)) & 15) | (((h1 >> (8 * t + j)) & 1) << 4);
            out[t] = __fsub_rn(__fmul_rn(d1, (float)qa), dm);
            out[t + 4] = __fsub_rn(__fmul_rn(d1, (float)qb), dm);
        }
    }
}

// Offset one past the last byte of the FILE stream (block-interleaved, not the planes) that the
// reference CPU code must have in hand to write element e. Streams shorter than this leave the
// element 0.0 (the bounds checks in q4_0.rs:273-292, q8_0.rs:35-58, q4_k.rs:208, q6_k.rs:208,
// dequant.rs:49-59,93-117).
template <int F>
__device__ __forceinline__ int64_t need_end(int64_t e) {
    constexpr FmtInfo I = fmt_info(F);
    int64_t b = e / I.block_elems;
    int i = (int)(e % I.block_elems);
    if constexpr (F == fmt_of(Q4_0, RF)) return b * 20 + 4 + i / 2 + 1;
    else if constexpr (F == fmt_of(Q8_0, RF)) return b * 36 + 4 + i + 1;
    else if constexpr (F == fmt_of(MXFP4, RF)) return b * 17 + 1 + i / 2 + 1;
    else if constexpr (F == fmt_of(MXFP6_E2M3, RF) || F == fmt_of(MXFP6_E3M2, RF)) return b * 25 + 1 + (6 * i) / 8 + 2;
    else return (b + 1) * I.block_bytes;
}

#endif  // __CUDACC__

}  // namespace b200q
