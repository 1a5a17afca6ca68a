// Integer tensor-core decode kernel: fused dequant + matmul for 1..8 activation rows, HBM-bound.
//
// Replaces the per-row-block scalar kernels of the reference (kernels/q4_k_matmul.hip:216, q6_k_matmul.hip:216:
// one thread block per ACTIVATION row, one 4-bit code per inner iteration) and the serial per-op loop of
// BatchQuantizedMatmul::process_batch (src/ggml/hip_backend/ops/batch_quantized.rs:147-161).
//
// Arithmetic. The integer codes go to the tensor cores AS INTEGERS (mma.sync.m16n8k32, u8 x s8 -> s32): a
// nibble masked in place is a u8 (the high nibble of a byte is 16 q, a Q6_K code kept as 4 q), so extraction is
// one logic operation per FOUR weights. Activations are quantised per scale group of the format (32 weights for
// Q4_K, 16 for Q6_K) to a 15-bit integer round(x * 16256 / max|x|) held as two s8 limbs (value = 128 hi + lo),
// so the integer dot product of a group is exact and the only error is the activation rounding: about 4e-5 of
// the result's magnitude for normally distributed activations, inside the 1e-4 bound of this path. The
// group's factor max|x| / 16256, the block scales (d * sc, exact in fp32) and the offsets (- dmin * m * sum x,
// - 32 * sum x) are applied in fp32 once per group and weight row.
//
// Block-diagonal B operand. Thread (g, t) of a warp streams its OWN group of 32 weights of rows g and g+8.
// The 8 columns of the MMA are 4 threads x {hi limb, lo limb}: column 2t holds the hi limbs of the
// activations that meet thread t's k-slots and zeros elsewhere, column 2t+1 the lo limbs. The accumulator
// fragment thread t receives (columns 2t, 2t+1) is then the dot product of ITS group, so block scales are
// applied by the thread that owns the group: no redundant work across the quad. More activation rows repeat
// the MMAs on the same extracted codes.
//
// Data movement. Weights are read from the tensor's DECODE IMAGE (built at upload): items of 16 rows x 128
// weights laid out in the order the lanes consume them, scales already widened to bytes, consecutive items of
// a row tile and consecutive row tiles contiguous. Every warp owns a contiguous byte range of the image and
// pulls it through a private ring in shared memory with one bulk copy (cp.async.bulk, completion on an
// mbarrier) per chunk of items issued by one lane; the other lanes spend no instruction on addressing. A
// launch covers any number of products (a whole decode step): persistent CTAs own contiguous ranges of row
// tiles balanced by bytes; inside a CTA the items of a product segment are split evenly over the 8 warps, at
// any item boundary, and the (at most one per warp) row tile a warp did not start is handed to the warp that
// did through shared memory, added in warp order.
#include <cuda_fp16.h>
#include <stdio.h>
#include <stdlib.h>
#include <atomic>

#include "gemv_i8.cuh"

namespace b200q {

namespace {

constexpr int F_Q4K = fmt_of(Q4_K, GGUF);
constexpr int F_Q6K = fmt_of(Q6_K, GGUF);
constexpr int F_Q80 = fmt_of(Q8_0, GGUF);
constexpr int F_MX6 = fmt_of(MXFP6_E2M3, GGUF);
constexpr int F_MX4 = fmt_of(MXFP4, GGUF);
constexpr int F_Q40 = fmt_of(Q4_0, GGUF);
constexpr int F_Q5K = fmt_of(Q5_K, GGUF);
constexpr int F_Q3K = fmt_of(Q3_K, GGUF);

// ---- item layouts (bytes inside one item; lane = 4 g + t; rows g and g+8 of the row tile; s = sub-block of 32
// weights inside the item's 128). A "chunk" (g, s) is 16 bytes placed at chunk_pos(g, s) * 16 of its 512-byte area,
// so that both kernels read it without bank conflicts.
// Q4_K:   [0,512)      chunk (g, s): codes of sub-block s of row g: byte b = weight b (low nibble) | weight 16+b (high)
//         [512,1024)   the same for row g+8
//         [1024,1152)  per g 16 bytes: for s = 0..3 {scale(g), min(g), scale(g+8), min(g+8)}, one byte each
//         [1152,1216)  per g: f16 d(g), dmin(g), d(g+8), dmin(g+8) of the super-block the half lies in
// Q6_K:   [0,512) / [512,1024) as above with nibble byte b = low 4 bits of weight b | (weight 16+b >> 2) << 4
//         [1024,1536)  chunk (g, s): two words of 2-bit fields for row g, two for row g+8. Word u, byte z:
//                      bits 4-5 = weight 8u+z >> 4, bits 2-3 = weight 16+8u+z & 3,
//                      bits 6-7 = weight 8u+4+z >> 4, bits 0-1 = weight 16+8u+4+z & 3
//         [1536,1664)  per g 16 bytes: for s = 0..3 the int8 scales of weights 0..15 and 16..31 of sub-block s for row
//                      g, then for row g+8
//         [1664,1696)  per g: f16 d(g), d(g+8)
// Q8_0:   [0,512) / [512,1024)      chunk (g, s): int8 codes 0..15 / 16..31 of sub-block s of row g
//         [1024,1536) / [1536,2048) the same for row g+8
//         [2048,2176)  per lane (g, s): f16 d(g), d(g+8) of the sub-block
// MXFP6 (E2M3 element type, GGUF): the 6-bit codes are widened at upload to the int8 value 8 * e2m3(code) (|.| <= 60),
//         so the item is Q8_0's with a one-byte header: [2048,2112) per lane (g, s): E8M0 exponent of row g, of row g+8.
//         The image is 8.25 bits per weight against the format's 6.25: this kernel trades HBM bytes for not
//         decoding a 6-bit float per weight on the integer pipes.
// MXFP4 (GGUF): [0,512)  chunk (g, s): the 32 E2M1 codes of sub-block s of row g in order, nibble k of word j = weight 8j+k
//         [512,1024)   the same for row g+8
//         [1024,1088)  per lane (g, s): E8M0 exponent of row g, of row g+8
//         A code becomes the magnitude 2 * |e2m1(code)| through one byte-permute table look-up; positive and negative
//         codes go through separate MMAs whose sums are subtracted.
// Q4_0:   codes as Q4_K's (a block's 16 bytes are stored as they are); [1024,1152) per lane (g, s): f16 d(g), d(g+8)
// Q5_K:   Q4_K's item followed by [1216,1472): per lane (g, s) the fifth bits of sub-block s of row g, then of row
//         g+8, one word each: bit 8z+j = weight 4j+z, bit 8z+4+j = weight 16+4j+z (j, z = 0..3)
constexpr int Q40_ITEM = 1152;
constexpr int Q5K_ITEM = 1472;
constexpr int MX4_ITEM = 1088;
constexpr int Q4K_ITEM = 1216;
constexpr int Q6K_ITEM = 1696;
constexpr int Q80_ITEM = 2176;
constexpr int MX6_ITEM = 2112;

constexpr int MAX_DEPTH = 8;
constexpr int ZERO_BYTES = 128;                       // lanes that supply the zero columns of B read these
__host__ __device__ constexpr int bar_bytes(int nw) { return nw * MAX_DEPTH * 8; }   // warps x MAX_DEPTH mbarriers
__host__ __device__ constexpr int red_bytes(int nw) { return nw * 16 * 8 * 4; }      // warps x 16 rows x up to 8 activation rows
__host__ __device__ constexpr int fixed_bytes(int nw) { return bar_bytes(nw) + red_bytes(nw) + ZERO_BYTES; }

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// first MMA of a group: the accumulator input is the constant zero
__device__ __forceinline__ void mma_u8s8_z(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                           uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

__device__ __forceinline__ void mma_s8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_s8s8_z(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                           uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// global -> this CTA's shared memory, completion counted in bytes on the mbarrier (no multicast)
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}

// explicit shared-space loads (the addresses are 32-bit shared-window offsets)
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}

// ---- activation images ------------------------------------------------------------------------------------
// Activations are quantised per scale group of the format (G = 32 values for Q4_K, 16 for Q6_K) to the integer
// q = round(x * 16256 * 128 / max|x|), |q| < 2^21, held as three s8 limbs: q = (l0 * 128 + l1) * 128 + l2 with
// l0 in [-127, 127] and l1, l2 in [-64, 63]. Per group the image keeps the factor max|x| / (16256 * 128) and the
// sum of the group's x (times `sum_mul`).
//
// One-row layout (m = 1, block-diagonal kernel), per block b of 32 values:
//   limbs[(b * 3 + L) * 32 + i]   limb L of value 32 b + i
//   fs: G = 32: float2 {f, s} per block; G = 16: float4 {f, s} of values 0..15, {f, s} of values 16..31
// Many-row layout (m = 2..8, activation rows on the MMA's N side), per item h (128 values) and row n < m:
//   lane (n, t) of a warp owns 96 bytes at ((h * m + n) * 4 + t) * 96: for sub-block s and limb L the 8 bytes at
//   (s * 3 + L) * 8 = values 32 s + 4 t .. + 3 and 32 s + 16 + 4 t .. + 3 (the k-slots of that lane's B fragment)
//   fs: G = 32: float2 {f, s} at [(b * mp) + n]; G = 16: [(b * 2 + group) * mp + n]; mp = m rounded up to even
struct ActImg {
    uint8_t* limbs;
    float* fs;
};

__device__ __forceinline__ void split_limbs(int q, int& l0, int& l1, int& l2) {
    l2 = ((q + 64) & 127) - 64;
    const int q1 = (q - l2) >> 7;
    l1 = ((q1 + 64) & 127) - 64;
    l0 = (q1 - l1) >> 7;
}

// x[m, k] (fp32, global) -> image. 8 consecutive values per thread and step, four steps' loads in flight at a time
// (the activations usually come from HBM: the packed weights have pushed them out of L2); the G / 8 lanes of a
// group agree on the group's maximum and sum by shuffles. MANY selects the many-row layout.
// PERM (many-row layout only): the lane t of the fragment owns values 8t..8t+7 of a sub-block (MXFP4's code order)
// instead of 4t..4t+3 and 16+4t..16+4t+3.
template <int G, bool MANY, int NT, bool PERM = false>
__device__ __forceinline__ void prep_x(const float* __restrict__ x, int64_t ldx, int k, int m, const ActImg& img, float sum_mul) {
    const int units = k >> 3;
    const int nb = k >> 5;
    const int mp = (m + 1) & ~1;
    const int total = units * m;
    if (MANY && (m & 1)) {   // the factors of the padding row read as zero
        const int groups = nb * (G == 32 ? 1 : 2);
        for (int i = threadIdx.x; i < groups; i += NT) *reinterpret_cast<float2*>(img.fs + ((size_t)i * mp + m) * 2) = make_float2(0.f, 0.f);
    }
    constexpr int B = 4;
    for (int u0 = 0; u0 < total; u0 += B * NT) {
        float4 xa[B], xb[B];
#pragma unroll
        for (int j = 0; j < B; j++) {
            const int u = u0 + j * NT + threadIdx.x;
            xa[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            xb[j] = xa[j];
            if (u < total) {
                const int n = u / units, p = u - n * units;
                const float4* xp = reinterpret_cast<const float4*>(x + (int64_t)n * ldx + (int64_t)p * 8);
                xa[j] = __ldg(xp);
                xb[j] = __ldg(xp + 1);
            }
        }
#pragma unroll
        for (int j = 0; j < B; j++) {
            if (u0 + j * NT >= total) break;   // uniform: the whole step is past the end
            const int u = u0 + j * NT + threadIdx.x;
            const bool valid = u < total;
            const int n = valid ? u / units : 0;
            const int p = valid ? u - n * units : 0;
            const float v[8] = {xa[j].x, xa[j].y, xa[j].z, xa[j].w, xb[j].x, xb[j].y, xb[j].z, xb[j].w};
            float mx = 0.0f, sm = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; i++) { mx = fmaxf(mx, fabsf(v[i])); sm += v[i]; }
            mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
            sm += __shfl_xor_sync(0xFFFFFFFFu, sm, 1);
            if (G == 32) {
                mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
                sm += __shfl_xor_sync(0xFFFFFFFFu, sm, 2);
            }
            const float s = mx > 0.0f ? 2080768.0f / mx : 0.0f;   // 16256 * 128
            uint32_t w[3][2] = {{0u, 0u}, {0u, 0u}, {0u, 0u}};
#pragma unroll
            for (int i = 0; i < 8; i++) {
                int l0, l1, l2;
                split_limbs(__float2int_rn(v[i] * s), l0, l1, l2);
                w[0][i >> 2] |= (uint32_t)(l0 & 0xFF) << (8 * (i & 3));
                w[1][i >> 2] |= (uint32_t)(l1 & 0xFF) << (8 * (i & 3));
                w[2][i >> 2] |= (uint32_t)(l2 & 0xFF) << (8 * (i & 3));
            }
            if (valid) {
                const int b = p >> 2, jj = p & 3;
                const float f = mx * (1.0f / 2080768.0f);
                if (!MANY) {
                    uint8_t* dst = img.limbs + (size_t)b * 96 + jj * 8;
#pragma unroll
                    for (int L = 0; L < 3; L++) *reinterpret_cast<uint2*>(dst + L * 32) = make_uint2(w[L][0], w[L][1]);
                    if (G == 32) {
                        if (jj == 0) *reinterpret_cast<float2*>(img.fs + (size_t)b * 2) = make_float2(f, sm * sum_mul);
                    } else {
                        if ((jj & 1) == 0) *reinterpret_cast<float2*>(img.fs + (size_t)b * 4 + (jj >> 1) * 2) = make_float2(f, sm * sum_mul);
                    }
                } else {
                    const int h = b >> 2, sb = b & 3;
                    // values 8 jj .. 8 jj + 3 belong to lane t = (2 jj) & 3, values 8 jj + 4 .. to lane t + 1; jj < 2:
                    // first half of the sub-block (b0 of the fragment), else second half (b1)
                    if (PERM) {
                        uint8_t* dst = img.limbs + ((size_t)(h * m + n) * 4 + jj) * 96 + sb * 24;
#pragma unroll
                        for (int L = 0; L < 3; L++) *reinterpret_cast<uint2*>(dst + L * 8) = make_uint2(w[L][0], w[L][1]);
                    } else {
                        const int t0 = (2 * jj) & 3, half = jj >> 1;
                        uint8_t* dst = img.limbs + ((size_t)(h * m + n) * 4 + t0) * 96 + sb * 24 + half * 4;
#pragma unroll
                        for (int L = 0; L < 3; L++) {
                            *reinterpret_cast<uint32_t*>(dst + L * 8) = w[L][0];
                            *reinterpret_cast<uint32_t*>(dst + 96 + L * 8) = w[L][1];
                        }
                    }
                    if (G == 32) {
                        if (jj == 0) *reinterpret_cast<float2*>(img.fs + ((size_t)b * mp + n) * 2) = make_float2(f, sm * sum_mul);
                    } else {
                        if ((jj & 1) == 0) *reinterpret_cast<float2*>(img.fs + ((size_t)(b * 2 + (jj >> 1)) * mp + n) * 2) = make_float2(f, sm * sum_mul);
                    }
                }
            }
        }
    }
}

// bytes of the image of a product with inner dimension k and m rows (limbs, then factors)
__host__ __device__ inline size_t act_limb_bytes(int k, int m) { return (size_t)(k >> 5) * 96 * m; }
__host__ __device__ inline size_t act_image_bytes(int kind, int k, int m) {
    const int mp = m == 1 ? 1 : (m + 1) & ~1;
    return act_limb_bytes(k, m) + (size_t)(k >> 5) * mp * (kind == DK_Q6K ? 16 : 8) + 16;
}

// chunk (g, s) of a 512-byte code area: 16 bytes of row g (or g + 8), sub-block s. Both access patterns -- one
// lane per chunk (16-byte loads) and four lanes per chunk (4-byte loads, fixed s) -- hit every bank once.
__device__ __forceinline__ int chunk_pos(int g, int s) { return 8 * s + ((g + 2 * s) & 7); }

// Per-lane addressing of the one-row B operand. Lanes g == 2t (limb 0) and g == 2t+1 (limb 1) read the limbs of
// thread t's block for the first pass, lane g == 2t limb 2 for the second; all other lanes read the zero region
// with stride 0, so no load is predicated.
struct LaneB1 {
    uint32_t p1, p2;     // shared addresses for item 0 (first / second pass)
    int s1, s2;          // byte steps per item
    uint32_t f0;         // factors of block t of item 0
    int fh;              // byte step per item
};

template <int G>
__device__ __forceinline__ LaneB1 lane_b1(const ActImg& a, const uint8_t* zero, int lane) {
    const int g = lane >> 2, t = lane & 3;
    const bool a1 = (g >> 1) == t, a2 = g == 2 * t;
    LaneB1 r;
    const uint32_t base = smem_addr(a.limbs) + t * 96;
    r.p1 = a1 ? base + (g & 1) * 32 : smem_addr(zero);
    r.p2 = a2 ? base + 64 : smem_addr(zero);
    r.s1 = a1 ? 384 : 0;
    r.s2 = a2 ? 384 : 0;
    constexpr int FPB = G == 32 ? 8 : 16;
    r.f0 = smem_addr(a.fs) + t * FPB;
    r.fh = 4 * FPB;
    return r;
}

// Many-row kernel: lane (g, t) supplies column g = activation row g of the B fragment.
struct LaneBM {
    uint32_t p;          // shared address of the lane's 96 bytes of item 0, or of the zero region
    int sh;              // byte step per item
    uint32_t f0;         // factors {f, s} of rows 2t, 2t+1 for block 0
    int fb;              // byte step per block (G = 32) or per group (G = 16)
};

__device__ __forceinline__ LaneBM lane_bm(const ActImg& a, const uint8_t* zero, int lane, int m) {
    const int g = lane >> 2, t = lane & 3;
    const int mp = (m + 1) & ~1;
    LaneBM r;
    const bool act = g < m;
    r.p = act ? smem_addr(a.limbs) + (g * 4 + t) * 96 : smem_addr(zero);
    r.sh = act ? m * 384 : 0;
    // rows 2t, 2t+1 past the padded row count read the zero region too (their outputs are never stored)
    const bool fact = 2 * t < mp;
    r.f0 = fact ? smem_addr(a.fs) + 2 * t * 8 : smem_addr(zero);
    r.fb = fact ? mp * 8 : 0;
    return r;
}

__device__ __forceinline__ void mma_k16_u8s8_z(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};\n"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

// ------------------------------------------------------------------------------------------- Q4_K (GGUF)
// One row: acc += d * sc * (factor * sum q x_int) - dmin * m * (sum x) for the lane's sub-block of rows g, g+8.
// Q5: the fifth bit of every code joins at bit 4 of its byte.
template <bool Q5>
__device__ __forceinline__ void item_q4k_one(uint32_t it, const LaneB1& lb, int h, float (&acc)[4], int lane) {
    const int g = lane >> 2, t = lane & 3;
    const int cp = chunk_pos(g, t) * 16;
    const uint4 wa = lds128(it + cp);
    const uint4 wb = lds128(it + 512 + cp);
    const uint32_t hs = lds32(it + 1024 + lane * 4);
    const uint2 dd = lds64(it + 1152 + g * 8);
    const uint4 q0 = lds128(lb.p1 + h * lb.s1), q1 = lds128(lb.p1 + h * lb.s1 + 16);
    const uint4 r0 = lds128(lb.p2 + h * lb.s2), r1 = lds128(lb.p2 + h * lb.s2 + 16);
    const uint2 fSb = lds64(lb.f0 + h * lb.fh);
    const float2 d0 = __half22float2(*reinterpret_cast<const __half2*>(&dd.x));
    const float2 d1 = __half22float2(*reinterpret_cast<const __half2*>(&dd.y));
    constexpr uint32_t ML = 0x0F0F0F0Fu, M4 = 0x10101010u;
    uint32_t a[2][4] = {{wa.x & ML, wa.y & ML, wa.z & ML, wa.w & ML}, {wb.x & ML, wb.y & ML, wb.z & ML, wb.w & ML}};
    uint32_t b[2][4] = {{(wa.x >> 4) & ML, (wa.y >> 4) & ML, (wa.z >> 4) & ML, (wa.w >> 4) & ML},
                        {(wb.x >> 4) & ML, (wb.y >> 4) & ML, (wb.z >> 4) & ML, (wb.w >> 4) & ML}};
    if constexpr (Q5) {
        const uint2 hb = lds64(it + 1216 + lane * 8);
        const uint32_t H[2] = {hb.x, hb.y};
#pragma unroll
        for (int r = 0; r < 2; r++) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                a[r][j] |= (H[r] << (4 - j)) & M4;
                b[r][j] |= (H[r] >> j) & M4;
            }
        }
    }
    int c[4], e[4];   // c: columns (limb 0, limb 1); e: columns (limb 2, zero)
    mma_u8s8_z(c, a[0][0], a[1][0], a[0][1], a[1][1], q0.x, q0.y);
    mma_u8s8_z(e, a[0][0], a[1][0], a[0][1], a[1][1], r0.x, r0.y);
    mma_u8s8(c, a[0][2], a[1][2], a[0][3], a[1][3], q0.z, q0.w);
    mma_u8s8(e, a[0][2], a[1][2], a[0][3], a[1][3], r0.z, r0.w);
    mma_u8s8(c, b[0][0], b[1][0], b[0][1], b[1][1], q1.x, q1.y);
    mma_u8s8(e, b[0][0], b[1][0], b[0][1], b[1][1], r1.x, r1.y);
    mma_u8s8(c, b[0][2], b[1][2], b[0][3], b[1][3], q1.z, q1.w);
    mma_u8s8(e, b[0][2], b[1][2], b[0][3], b[1][3], r1.z, r1.w);
    // Q5_K: 32 five-bit codes times 21-bit activations can leave 32 bits, so its last limb joins in floating point
    const float v0 = Q5 ? fmaf((float)(c[0] * 128 + c[1]), 128.0f, (float)e[0]) : (float)((c[0] * 128 + c[1]) * 128 + e[0]);
    const float v1 = Q5 ? fmaf((float)(c[2] * 128 + c[3]), 128.0f, (float)e[2]) : (float)((c[2] * 128 + c[3]) * 128 + e[2]);
    const float f = __uint_as_float(fSb.x), S = __uint_as_float(fSb.y);
    const float A0 = d0.x * (float)(hs & 0xFFu), B0 = -d0.y * (float)((hs >> 8) & 0xFFu);
    const float A1 = d1.x * (float)((hs >> 16) & 0xFFu), B1 = -d1.y * (float)(hs >> 24);
    acc[0] = fmaf(A0, v0 * f, fmaf(B0, S, acc[0]));
    acc[1] = fmaf(A1, v1 * f, fmaf(B1, S, acc[1]));
}

// Many rows: one MMA per sub-block and limb, the activation rows are the MMA's columns; lane (g, t) ends up with
// rows g, g+8 x activation rows 2t, 2t+1.  acc = {(g, 2t), (g, 2t+1), (g+8, 2t), (g+8, 2t+1)}
template <bool Q5>
__device__ __forceinline__ void item_q4k_many(uint32_t it, const LaneBM& lb, int h, float (&acc)[4], int lane) {
    const int g = lane >> 2, t = lane & 3;
    const uint4 hdr = lds128(it + 1024 + g * 16);
    const uint2 dd = lds64(it + 1152 + g * 8);
    const float2 d0 = __half22float2(*reinterpret_cast<const __half2*>(&dd.x));
    const float2 d1 = __half22float2(*reinterpret_cast<const __half2*>(&dd.y));
    const uint32_t hw[4] = {hdr.x, hdr.y, hdr.z, hdr.w};
    const uint32_t bp = lb.p + h * lb.sh;
    constexpr uint32_t ML = 0x0F0F0F0Fu, M4 = 0x10101010u;
#pragma unroll
    for (int s = 0; s < 4; s++) {
        const int cp = chunk_pos(g, s) * 16 + 4 * t;
        const uint32_t w0 = lds32(it + cp), w1 = lds32(it + 512 + cp);
        const uint2 b0 = lds64(bp + s * 24), b1 = lds64(bp + s * 24 + 8), b2 = lds64(bp + s * 24 + 16);
        const uint4 fSb = lds128(lb.f0 + (4 * h + s) * lb.fb);
        uint32_t a0 = w0 & ML, a1 = w1 & ML, a2 = (w0 >> 4) & ML, a3 = (w1 >> 4) & ML;
        if constexpr (Q5) {
            const uint2 hb = lds64(it + 1216 + (4 * g + s) * 8);
            a0 |= (hb.x << (4 - t)) & M4; a2 |= (hb.x >> t) & M4;
            a1 |= (hb.y << (4 - t)) & M4; a3 |= (hb.y >> t) & M4;
        }
        int c0[4], c1[4], c2[4];
        mma_u8s8_z(c0, a0, a1, a2, a3, b0.x, b0.y);
        mma_u8s8_z(c1, a0, a1, a2, a3, b1.x, b1.y);
        mma_u8s8_z(c2, a0, a1, a2, a3, b2.x, b2.y);
        const float A0 = d0.x * (float)(hw[s] & 0xFFu), B0 = -d0.y * (float)((hw[s] >> 8) & 0xFFu);
        const float A1 = d1.x * (float)((hw[s] >> 16) & 0xFFu), B1 = -d1.y * (float)(hw[s] >> 24);
        const float fa = __uint_as_float(fSb.x), Sa = __uint_as_float(fSb.y), fb = __uint_as_float(fSb.z), Sb = __uint_as_float(fSb.w);
        // 32 five-bit codes times 21-bit activations can leave 32 bits: the last limb joins in floating point
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; j++)
            v[j] = Q5 ? fmaf((float)(c0[j] * 128 + c1[j]), 128.0f, (float)c2[j]) : (float)((c0[j] * 128 + c1[j]) * 128 + c2[j]);
        const float v0 = v[0], v1 = v[1], v2 = v[2], v3 = v[3];
        acc[0] = fmaf(A0, v0 * fa, fmaf(B0, Sa, acc[0]));
        acc[1] = fmaf(A0, v1 * fb, fmaf(B0, Sb, acc[1]));
        acc[2] = fmaf(A1, v2 * fa, fmaf(B1, Sa, acc[2]));
        acc[3] = fmaf(A1, v3 * fb, fmaf(B1, Sb, acc[3]));
    }
}

// ------------------------------------------------------------------------------------------- Q4_0 (GGUF)
// acc += d * (factor * sum q x_int - 8 sum x) per block of 32 (the image stores 8 sum x).
__device__ __forceinline__ void item_q40_one(uint32_t it, const LaneB1& lb, int h, float (&acc)[4], int lane) {
    const int g = lane >> 2, t = lane & 3;
    const int cp = chunk_pos(g, t) * 16;
    const uint4 wa = lds128(it + cp);
    const uint4 wb = lds128(it + 512 + cp);
    const uint32_t dd = lds32(it + 1024 + lane * 4);
    const uint4 q0 = lds128(lb.p1 + h * lb.s1), q1 = lds128(lb.p1 + h * lb.s1 + 16);
    const uint4 r0 = lds128(lb.p2 + h * lb.s2), r1 = lds128(lb.p2 + h * lb.s2 + 16);
    const uint2 fSb = lds64(lb.f0 + h * lb.fh);
    const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&dd));
    constexpr uint32_t ML = 0x0F0F0F0Fu;
    const uint32_t a[2][4] = {{wa.x & ML, wa.y & ML, wa.z & ML, wa.w & ML}, {wb.x & ML, wb.y & ML, wb.z & ML, wb.w & ML}};
    const uint32_t b[2][4] = {{(wa.x >> 4) & ML, (wa.y >> 4) & ML, (wa.z >> 4) & ML, (wa.w >> 4) & ML},
                              {(wb.x >> 4) & ML, (wb.y >> 4) & ML, (wb.z >> 4) & ML, (wb.w >> 4) & ML}};
    int c[4], e[4];
    mma_u8s8_z(c, a[0][0], a[1][0], a[0][1], a[1][1], q0.x, q0.y);
    mma_u8s8_z(e, a[0][0], a[1][0], a[0][1], a[1][1], r0.x, r0.y);
    mma_u8s8(c, a[0][2], a[1][2], a[0][3], a[1][3], q0.z, q0.w);
    mma_u8s8(e, a[0][2], a[1][2], a[0][3], a[1][3], r0.z, r0.w);
    mma_u8s8(c, b[0][0], b[1][0], b[0][1], b[1][1], q1.x, q1.y);
    mma_u8s8(e, b[0][0], b[1][0], b[0][1], b[1][1], r1.x, r1.y);
    mma_u8s8(c, b[0][2], b[1][2], b[0][3], b[1][3], q1.z, q1.w);
    mma_u8s8(e, b[0][2], b[1][2], b[0][3], b[1][3], r1.z, r1.w);
    const int v0 = (c[0] * 128 + c[1]) * 128 + e[0];
    const int v1 = (c[2] * 128 + c[3]) * 128 + e[2];
    const float f = __uint_as_float(fSb.x), S8 = __uint_as_float(fSb.y);
    acc[0] = fmaf(d.x, fmaf((float)v0, f, -S8), acc[0]);
    acc[1] = fmaf(d.y, fmaf((float)v1, f, -S8), acc[1]);
}

__device__ __forceinline__ void item_q40_many(uint32_t it, const LaneBM& lb, int h, float (&acc)[4], int lane) {
    const int g = lane >> 2, t = lane & 3;
    const uint4 hdr = lds128(it + 1024 + g * 16);
    const uint32_t hw[4] = {hdr.x, hdr.y, hdr.z, hdr.w};
    const uint32_t bp = lb.p + h * lb.sh;
    constexpr uint32_t ML = 0x0F0F0F0Fu;
#pragma unroll
    for (int s = 0; s < 4; s++) {
        const int cp = chunk_pos(g, s) * 16 + 4 * t;
        const uint32_t w0 = lds32(it + cp), w1 = lds32(it + 512 + cp);
        const uint2 b0 = lds64(bp + s * 24), b1 = lds64(bp + s * 24 + 8), b2 = lds64(bp + s * 24 + 16);
        const uint4 fSb = lds128(lb.f0 + (4 * h + s) * lb.fb);
        const uint32_t a0 = w0 & ML, a1 = w1 & ML, a2 = (w0 >> 4) & ML, a3 = (w1 >> 4) & ML;
        int c0[4], c1[4], c2[4];
        mma_u8s8_z(c0, a0, a1, a2, a3, b0.x, b0.y);
        mma_u8s8_z(c1, a0, a1, a2, a3, b1.x, b1.y);
        mma_u8s8_z(c2, a0, a1, a2, a3, b2.x, b2.y);
        const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&hw[s]));
        const float fa = __uint_as_float(fSb.x), Sa = __uint_as_float(fSb.y), fb = __uint_as_float(fSb.z), Sb = __uint_as_float(fSb.w);
        acc[0] = fmaf(d.x, fmaf((float)((c0[0] * 128 + c1[0]) * 128 + c2[0]), fa, -Sa), acc[0]);
        acc[1] = fmaf(d.x, fmaf((float)((c0[1] * 128 + c1[1]) * 128 + c2[1]), fb, -Sb), acc[1]);
        acc[2] = fmaf(d.y, fmaf((float)((c0[2] * 128 + c1[2]) * 128 + c2[2]), fa, -Sa), acc[2]);
        acc[3] = fmaf(d.y, fmaf((float)((c0[3] * 128 + c1[3]) * 128 + c2[3]), fb, -Sb), acc[3]);
    }
}

// ------------------------------------------------------------------------------------------- Q6_K (GGUF)
// One row: acc += d * sc * (factor * sum q x_int - 32 sum x) per 16 weights (the image stores 32 sum x).
__device__ __forceinline__ void item_q6k_one(uint32_t it, const LaneB1& lb, int h, float (&acc)[4], int lane) {
    const int g = lane >> 2, t = lane & 3;
    const int cp = chunk_pos(g, t) * 16;
    const uint4 wa = lds128(it + cp);
    const uint4 wb = lds128(it + 512 + cp);
    const uint4 hq = lds128(it + 1024 + cp);
    const uint32_t hs = lds32(it + 1536 + lane * 4);
    const uint32_t dd = lds32(it + 1664 + g * 4);
    const uint4 q0 = lds128(lb.p1 + h * lb.s1), q1 = lds128(lb.p1 + h * lb.s1 + 16);
    const uint4 r0 = lds128(lb.p2 + h * lb.s2), r1 = lds128(lb.p2 + h * lb.s2 + 16);
    const uint4 fSb = lds128(lb.f0 + h * lb.fh);
    const float2 d01 = __half22float2(*reinterpret_cast<const __half2*>(&dd));
    constexpr uint32_t ML = 0x0F0F0F0Fu, MH = 0xF0F0F0F0u, M45 = 0x30303030u, M23 = 0x0C0C0C0Cu;
    uint32_t A[2][4], B[2][4];   // [row][nibble word]; B holds 4 q
    {
        const uint32_t w[2][4] = {{wa.x, wa.y, wa.z, wa.w}, {wb.x, wb.y, wb.z, wb.w}};
        const uint32_t q[2][2] = {{hq.x, hq.y}, {hq.z, hq.w}};
#pragma unroll
        for (int r = 0; r < 2; r++) {
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const uint32_t hh = q[r][u];
                A[r][2 * u] = (w[r][2 * u] & ML) | (hh & M45);
                B[r][2 * u] = (w[r][2 * u] & MH) | (hh & M23);
                A[r][2 * u + 1] = (w[r][2 * u + 1] & ML) | ((hh >> 2) & M45);
                B[r][2 * u + 1] = (w[r][2 * u + 1] & MH) | ((hh << 2) & M23);
            }
        }
    }
    int cl[4], el[4], ch[4], eh[4];
    mma_u8s8_z(cl, A[0][0], A[1][0], A[0][1], A[1][1], q0.x, q0.y);
    mma_u8s8_z(el, A[0][0], A[1][0], A[0][1], A[1][1], r0.x, r0.y);
    mma_u8s8_z(ch, B[0][0], B[1][0], B[0][1], B[1][1], q1.x, q1.y);
    mma_u8s8_z(eh, B[0][0], B[1][0], B[0][1], B[1][1], r1.x, r1.y);
    mma_u8s8(cl, A[0][2], A[1][2], A[0][3], A[1][3], q0.z, q0.w);
    mma_u8s8(el, A[0][2], A[1][2], A[0][3], A[1][3], r0.z, r0.w);
    mma_u8s8(ch, B[0][2], B[1][2], B[0][3], B[1][3], q1.z, q1.w);
    mma_u8s8(eh, B[0][2], B[1][2], B[0][3], B[1][3], r1.z, r1.w);
    // the high group's sums carry the factor 4 of its codes: exact shifts before the limbs are combined
    const float l0 = (float)((cl[0] * 128 + cl[1]) * 128 + el[0]), l1 = (float)((cl[2] * 128 + cl[3]) * 128 + el[2]);
    const float h0 = (float)(((ch[0] >> 2) * 128 + (ch[1] >> 2)) * 128 + (eh[0] >> 2));
    const float h1 = (float)(((ch[2] >> 2) * 128 + (ch[3] >> 2)) * 128 + (eh[2] >> 2));
    const float D00 = d01.x * (float)(int)(int8_t)(hs & 0xFFu), D01 = d01.x * (float)(int)(int8_t)((hs >> 8) & 0xFFu);
    const float D10 = d01.y * (float)(int)(int8_t)((hs >> 16) & 0xFFu), D11 = d01.y * (float)(int)(int8_t)(hs >> 24);
    const float fl = __uint_as_float(fSb.x), Sl = __uint_as_float(fSb.y), fh = __uint_as_float(fSb.z), Sh = __uint_as_float(fSb.w);
    acc[0] = fmaf(D00, fmaf(l0, fl, -Sl), fmaf(D01, fmaf(h0, fh, -Sh), acc[0]));
    acc[1] = fmaf(D10, fmaf(l1, fl, -Sl), fmaf(D11, fmaf(h1, fh, -Sh), acc[1]));
}

// Many rows: per sub-block the low group (k-slots 0..15 of the lane's fragment words) and the high group are
// separate k16 MMAs, one per limb.
__device__ __forceinline__ void item_q6k_many(uint32_t it, const LaneBM& lb, int h, float (&acc)[4], int lane) {
    const int g = lane >> 2, t = lane & 3;
    const uint4 hdr = lds128(it + 1536 + g * 16);
    const uint32_t dd = lds32(it + 1664 + g * 4);
    const float2 d01 = __half22float2(*reinterpret_cast<const __half2*>(&dd));
    const uint32_t hw[4] = {hdr.x, hdr.y, hdr.z, hdr.w};
    const uint32_t bp = lb.p + h * lb.sh;
    const int sh = (t & 1) * 2;   // odd nibble words keep their high bits two positions further out
    constexpr uint32_t ML = 0x0F0F0F0Fu, M45 = 0x30303030u, M2345 = 0x3C3C3C3Cu, M01 = 0x03030303u;
#pragma unroll
    for (int s = 0; s < 4; s++) {
        const int cpos = chunk_pos(g, s) * 16;
        const uint32_t w0 = lds32(it + cpos + 4 * t), w1 = lds32(it + 512 + cpos + 4 * t);
        const uint32_t h0 = lds32(it + 1024 + cpos + 4 * (t >> 1)), h1 = lds32(it + 1024 + cpos + 8 + 4 * (t >> 1));
        const uint2 b0 = lds64(bp + s * 24), b1 = lds64(bp + s * 24 + 8), b2 = lds64(bp + s * 24 + 16);
        const uint4 fL = lds128(lb.f0 + (2 * (4 * h + s)) * lb.fb), fH = lds128(lb.f0 + (2 * (4 * h + s) + 1) * lb.fb);
        const uint32_t aL0 = (w0 & ML) | ((h0 >> sh) & M45), aL1 = (w1 & ML) | ((h1 >> sh) & M45);
        // high group as plain codes: the nibble holds q >> 2, the 2-bit field q & 3
        const uint32_t aH0 = ((w0 >> 2) & M2345) | ((h0 >> (2 - sh)) & M01), aH1 = ((w1 >> 2) & M2345) | ((h1 >> (2 - sh)) & M01);
        int l0[4], l1[4], l2[4], g0[4], g1[4], g2[4];
        mma_k16_u8s8_z(l0, aL0, aL1, b0.x);
        mma_k16_u8s8_z(l1, aL0, aL1, b1.x);
        mma_k16_u8s8_z(l2, aL0, aL1, b2.x);
        mma_k16_u8s8_z(g0, aH0, aH1, b0.y);
        mma_k16_u8s8_z(g1, aH0, aH1, b1.y);
        mma_k16_u8s8_z(g2, aH0, aH1, b2.y);
        const float DL0 = d01.x * (float)(int)(int8_t)(hw[s] & 0xFFu), DH0 = d01.x * (float)(int)(int8_t)((hw[s] >> 8) & 0xFFu);
        const float DL1 = d01.y * (float)(int)(int8_t)((hw[s] >> 16) & 0xFFu), DH1 = d01.y * (float)(int)(int8_t)(hw[s] >> 24);
        const float fLa = __uint_as_float(fL.x), SLa = __uint_as_float(fL.y), fLb = __uint_as_float(fL.z), SLb = __uint_as_float(fL.w);
        const float fHa = __uint_as_float(fH.x), SHa = __uint_as_float(fH.y), fHb = __uint_as_float(fH.z), SHb = __uint_as_float(fH.w);
        float vl[4], vh[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            vl[j] = (float)((l0[j] * 128 + l1[j]) * 128 + l2[j]);
            vh[j] = (float)((g0[j] * 128 + g1[j]) * 128 + g2[j]);
        }
        acc[0] = fmaf(DL0, fmaf(vl[0], fLa, -SLa), fmaf(DH0, fmaf(vh[0], fHa, -SHa), acc[0]));
        acc[1] = fmaf(DL0, fmaf(vl[1], fLb, -SLb), fmaf(DH0, fmaf(vh[1], fHb, -SHb), acc[1]));
        acc[2] = fmaf(DL1, fmaf(vl[2], fLa, -SLa), fmaf(DH1, fmaf(vh[2], fHa, -SHa), acc[2]));
        acc[3] = fmaf(DL1, fmaf(vl[3], fLb, -SLb), fmaf(DH1, fmaf(vh[3], fHb, -SHb), acc[3]));
    }
}

// ---------------------------------------------------------------------------------- Q8_0 and MXFP6 as int8
// Block scale of the lane's sub-block for rows g and g+8.
template <int KIND>
__device__ __forceinline__ void s8_scales_lane(uint32_t it, int lane, float& s0, float& s1) {
    if (KIND == DK_Q80) {
        const uint32_t dd = lds32(it + 2048 + lane * 4);
        const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&dd));
        s0 = d.x; s1 = d.y;
    } else {
        const uint32_t w = lds32(it + 2048 + (lane >> 1) * 4) >> ((lane & 1) * 16);
        s0 = ocp_e8m0((uint8_t)(w & 0xFFu)) * 0.125f;   // codes are 8 * value
        s1 = ocp_e8m0((uint8_t)((w >> 8) & 0xFFu)) * 0.125f;
    }
}

// One row: acc += scale * (factor * sum q x_int) for the lane's block of rows g and g+8.
template <int KIND>
__device__ __forceinline__ void item_s8_one(uint32_t it, const LaneB1& lb, int h, float (&acc)[4], int lane) {
    const int g = lane >> 2, t = lane & 3;
    const int cp = chunk_pos(g, t) * 16;
    const uint4 a0 = lds128(it + cp), a1 = lds128(it + 512 + cp);
    const uint4 b0 = lds128(it + 1024 + cp), b1 = lds128(it + 1536 + cp);
    const uint4 q0 = lds128(lb.p1 + h * lb.s1), q1 = lds128(lb.p1 + h * lb.s1 + 16);
    const uint4 r0 = lds128(lb.p2 + h * lb.s2), r1 = lds128(lb.p2 + h * lb.s2 + 16);
    const uint2 fSb = lds64(lb.f0 + h * lb.fh);
    float s0, s1;
    s8_scales_lane<KIND>(it, lane, s0, s1);
    int c[4], e[4];   // c: columns (limb 0, limb 1); e: columns (limb 2, zero)
    mma_s8s8_z(c, a0.x, b0.x, a0.y, b0.y, q0.x, q0.y);
    mma_s8s8_z(e, a0.x, b0.x, a0.y, b0.y, r0.x, r0.y);
    mma_s8s8(c, a0.z, b0.z, a0.w, b0.w, q0.z, q0.w);
    mma_s8s8(e, a0.z, b0.z, a0.w, b0.w, r0.z, r0.w);
    mma_s8s8(c, a1.x, b1.x, a1.y, b1.y, q1.x, q1.y);
    mma_s8s8(e, a1.x, b1.x, a1.y, b1.y, r1.x, r1.y);
    mma_s8s8(c, a1.z, b1.z, a1.w, b1.w, q1.z, q1.w);
    mma_s8s8(e, a1.z, b1.z, a1.w, b1.w, r1.z, r1.w);
    // 32 codes of up to 7 bits times 21-bit activations leave 32 bits: the last limb joins in floating point
    const float v0 = fmaf((float)(c[0] * 128 + c[1]), 128.0f, (float)e[0]);
    const float v1 = fmaf((float)(c[2] * 128 + c[3]), 128.0f, (float)e[2]);
    const float f = __uint_as_float(fSb.x);
    acc[0] = fmaf(s0, v0 * f, acc[0]);
    acc[1] = fmaf(s1, v1 * f, acc[1]);
}

// Many rows: the lane's fragment words are the code bytes as stored, no extraction at all.
template <int KIND>
__device__ __forceinline__ void item_s8_many(uint32_t it, const LaneBM& lb, int h, float (&acc)[4], int lane) {
    const int g = lane >> 2, t = lane & 3;
    const uint32_t bp = lb.p + h * lb.sh;
#pragma unroll
    for (int s = 0; s < 4; s++) {
        const int cp = chunk_pos(g, s) * 16 + 4 * t;
        const uint32_t a0 = lds32(it + cp), a2 = lds32(it + 512 + cp);
        const uint32_t a1 = lds32(it + 1024 + cp), a3 = lds32(it + 1536 + cp);
        const uint2 b0 = lds64(bp + s * 24), b1 = lds64(bp + s * 24 + 8), b2 = lds64(bp + s * 24 + 16);
        const uint4 fSb = lds128(lb.f0 + (4 * h + s) * lb.fb);
        float s0, s1;
        s8_scales_lane<KIND>(it, 4 * g + s, s0, s1);
        int c0[4], c1[4], c2[4];
        mma_s8s8_z(c0, a0, a1, a2, a3, b0.x, b0.y);
        mma_s8s8_z(c1, a0, a1, a2, a3, b1.x, b1.y);
        mma_s8s8_z(c2, a0, a1, a2, a3, b2.x, b2.y);
        const float fa = __uint_as_float(fSb.x), fb = __uint_as_float(fSb.z);
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; j++) v[j] = fmaf((float)(c0[j] * 128 + c1[j]), 128.0f, (float)c2[j]);
        acc[0] = fmaf(s0, v[0] * fa, acc[0]);
        acc[1] = fmaf(s0, v[1] * fb, acc[1]);
        acc[2] = fmaf(s1, v[2] * fa, acc[2]);
        acc[3] = fmaf(s1, v[3] * fb, acc[3]);
    }
}

// ------------------------------------------------------------------------------------------ MXFP4 (GGUF)
// Eight E2M1 codes (one word) -> two byte words of OFFSET codes u = 12 + 2 * e2m1(code) in 0..24, so that one unsigned
// operand carries the signed weights and the -12 is taken back through the group sums (12 * sum x, as Q4_0 does with
// its 8). A byte permute with the raw nibbles as selector returns the table byte where the sign bit is clear and 0x00
// where it is set (its sign-replicate mode on a table of bytes below 0x80); the same on the sign-flipped word with
// the table of the negative codes; the two are disjoint and OR-ed. Five instructions per eight codes.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {   // bit 3 of a selector nibble: replicate the sign
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ void e2m1x8_offset(uint32_t w, uint32_t& u_lo, uint32_t& u_hi) {
    // 12 + {0,1,2,3,4,6,8,12} and 12 - {0,1,2,3,4,6,8,12}
    const uint32_t wn = w ^ 0x88888888u;
    u_lo = prmt(0x0F0E0D0Cu, 0x18141210u, w) | prmt(0x090A0B0Cu, 0x00040608u, wn);
    u_hi = prmt(0x0F0E0D0Cu, 0x18141210u, w >> 16) | prmt(0x090A0B0Cu, 0x00040608u, wn >> 16);
}

__device__ __forceinline__ void mx4_scales_lane(uint32_t it, int lane, float& s0, float& s1) {
    const uint32_t w = lds32(it + 1024 + (lane >> 1) * 4) >> ((lane & 1) * 16);
    s0 = gguf_e8m0_half((uint8_t)(w & 0xFFu));   // codes are 2 * value
    s1 = gguf_e8m0_half((uint8_t)((w >> 8) & 0xFFu));
}

__device__ __forceinline__ void item_mx4_one(uint32_t it, const LaneB1& lb, int h, float (&acc)[4], int lane) {
    const int g = lane >> 2, t = lane & 3;
    const int cp = chunk_pos(g, t) * 16;
    const uint4 wa = lds128(it + cp), wb = lds128(it + 512 + cp);
    const uint4 q0 = lds128(lb.p1 + h * lb.s1), q1 = lds128(lb.p1 + h * lb.s1 + 16);
    const uint4 r0 = lds128(lb.p2 + h * lb.s2), r1 = lds128(lb.p2 + h * lb.s2 + 16);
    const uint2 fSb = lds64(lb.f0 + h * lb.fh);
    float s0, s1;
    mx4_scales_lane(it, lane, s0, s1);
    const uint32_t w0[4] = {wa.x, wa.y, wa.z, wa.w}, w1[4] = {wb.x, wb.y, wb.z, wb.w};
    const uint32_t bq[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    const uint32_t br[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
    int c[4] = {0, 0, 0, 0}, e[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 4; j++) {
        uint32_t u0, u2, u1, u3;
        e2m1x8_offset(w0[j], u0, u2);
        e2m1x8_offset(w1[j], u1, u3);
        mma_u8s8(c, u0, u1, u2, u3, bq[2 * j], bq[2 * j + 1]);
        mma_u8s8(e, u0, u1, u2, u3, br[2 * j], br[2 * j + 1]);
    }
    const int v0 = (c[0] * 128 + c[1]) * 128 + e[0];
    const int v1 = (c[2] * 128 + c[3]) * 128 + e[2];
    const float f = __uint_as_float(fSb.x), S12 = __uint_as_float(fSb.y);
    acc[0] = fmaf(s0, fmaf((float)v0, f, -S12), acc[0]);
    acc[1] = fmaf(s1, fmaf((float)v1, f, -S12), acc[1]);
}

__device__ __forceinline__ void item_mx4_many(uint32_t it, const LaneBM& lb, int h, float (&acc)[4], int lane) {
    const int g = lane >> 2, t = lane & 3;
    const uint32_t bp = lb.p + h * lb.sh;
#pragma unroll
    for (int s = 0; s < 4; s++) {
        const int cp = chunk_pos(g, s) * 16 + 4 * t;
        const uint32_t w0 = lds32(it + cp), w1 = lds32(it + 512 + cp);
        const uint2 b0 = lds64(bp + s * 24), b1 = lds64(bp + s * 24 + 8), b2 = lds64(bp + s * 24 + 16);
        const uint4 fSb = lds128(lb.f0 + (4 * h + s) * lb.fb);
        float s0, s1;
        mx4_scales_lane(it, 4 * g + s, s0, s1);
        uint32_t u0, u1, u2, u3;
        e2m1x8_offset(w0, u0, u2);
        e2m1x8_offset(w1, u1, u3);
        int c0[4], c1[4], c2[4];
        mma_u8s8_z(c0, u0, u1, u2, u3, b0.x, b0.y);
        mma_u8s8_z(c1, u0, u1, u2, u3, b1.x, b1.y);
        mma_u8s8_z(c2, u0, u1, u2, u3, b2.x, b2.y);
        const float fa = __uint_as_float(fSb.x), Sa = __uint_as_float(fSb.y), fb = __uint_as_float(fSb.z), Sb = __uint_as_float(fSb.w);
        acc[0] = fmaf(s0, fmaf((float)((c0[0] * 128 + c1[0]) * 128 + c2[0]), fa, -Sa), acc[0]);
        acc[1] = fmaf(s0, fmaf((float)((c0[1] * 128 + c1[1]) * 128 + c2[1]), fb, -Sb), acc[1]);
        acc[2] = fmaf(s1, fmaf((float)((c0[2] * 128 + c1[2]) * 128 + c2[2]), fa, -Sa), acc[2]);
        acc[3] = fmaf(s1, fmaf((float)((c0[3] * 128 + c1[3]) * 128 + c2[3]), fb, -Sb), acc[3]);
    }
}

// What a warp streams for one product segment.
struct Stream {
    const uint8_t* src;   // next byte to copy
    int to_issue;         // items not yet requested
    int item_bytes;
};

// Per-warp ring bookkeeping (uniform across the lanes of a warp).
struct Ring {
    uint32_t bar0;        // shared address of the warp's first mbarrier
    uint32_t slot0;       // shared address of the warp's first slot
    int depth, slot_bytes, chunk;
    int pslot, cslot;     // next slot to fill / to consume
    uint32_t parity;      // bit s: parity the next wait on slot s uses
    int inflight;         // chunks requested and not yet consumed
};

__device__ __forceinline__ void ring_issue(Ring& r, Stream& s, int lane) {
    const int cnt = min(r.chunk, s.to_issue);
    const uint32_t bytes = (uint32_t)cnt * (uint32_t)s.item_bytes;
    if (lane == 0) {
        const uint32_t bar = r.bar0 + r.pslot * 8;
        // the slot's previous contents were read through the generic proxy; order those reads before the
        // asynchronous write
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_expect_tx(bar, bytes);
        bulk_g2s(r.slot0 + r.pslot * r.slot_bytes, s.src, bytes, bar);
    }
    s.src += bytes;
    s.to_issue -= cnt;
    r.pslot = r.pslot + 1 == r.depth ? 0 : r.pslot + 1;
    r.inflight++;
}

__device__ __forceinline__ void ring_fill(Ring& r, Stream& s, int lane) {
    while (r.inflight < r.depth && s.to_issue > 0) ring_issue(r, s, lane);
}

// Waits (bounded) for the chunk in the consumer slot; false when the wait gave up.
__device__ __forceinline__ bool ring_wait(const Ring& r, long long budget) {
    const uint32_t bar = r.bar0 + r.cslot * 8;
    const uint32_t par = (r.parity >> r.cslot) & 1u;
    if (mbar_try_wait(bar, par)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; i++)
            if (mbar_try_wait(bar, par)) return true;
        if (clock64() - t0 > budget) return false;
    }
}

__device__ __forceinline__ void ring_release(Ring& r) {
    r.parity ^= 1u << r.cslot;
    r.cslot = r.cslot + 1 == r.depth ? 0 : r.cslot + 1;
    r.inflight--;
}

// The four values a lane accumulates. One-row kernel: acc[0], acc[1] = its share of rows g, g+8 (the quad's four
// shares are added at the end of a row tile). Many-row kernel: complete sums of (g, 2t), (g, 2t+1), (g+8, 2t),
// (g+8, 2t+1).
template <bool MANY>
__device__ __forceinline__ void finish_acc(float (&acc)[4]) {
    if (!MANY) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            float s = acc[i];
            s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
            s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);
            acc[i] = s;
        }
    }
}

template <bool MANY>
__device__ __forceinline__ void store_tile(const DOp& op, int prt, const float (&acc)[4], int m, int lane) {
    const int g = lane >> 2, t = lane & 3;
    if (!MANY) {
        // every lane of a quad holds the sums of rows g and g + 8: lanes t = 0 store the first, lanes t = 1 the second, so
        // ONE instruction writes the tile's 64 contiguous bytes (outputs in host memory travel as one PCIe write, not two)
        if (t > 1) return;
        const int row = prt * 16 + g + 8 * t;
        const float v = t ? acc[1] : acc[0];
        if (row < op.n_rows) {
            op.y[row] = v;
            for (int pp = 0; pp < op.n_extra; pp++) op.y_extra[pp][row] = v;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int row = prt * 16 + g + 8 * (j >> 1), n = 2 * t + (j & 1);
            if (row < op.n_rows && n < m) {
                op.y[(int64_t)n * op.ldy + row] = acc[j];
                for (int pp = 0; pp < op.n_extra; pp++) op.y_extra[pp][(int64_t)n * op.ldy + row] = acc[j];
            }
        }
    }
}

// hand-over slot of a warp: 16 rows x 8 activation rows
template <bool MANY>
__device__ __forceinline__ void slot_write(float* red, int warp, const float (&acc)[4], int lane) {
    const int g = lane >> 2, t = lane & 3;
    float* s = red + warp * 128;
    if (!MANY) {
        if (t == 0) { s[g * 8] = acc[0]; s[(g + 8) * 8] = acc[1]; }
    } else {
        s[g * 8 + 2 * t] = acc[0]; s[g * 8 + 2 * t + 1] = acc[1];
        s[(g + 8) * 8 + 2 * t] = acc[2]; s[(g + 8) * 8 + 2 * t + 1] = acc[3];
    }
}
template <bool MANY>
__device__ __forceinline__ void slot_add(const float* red, int warp, float (&acc)[4], int lane) {
    const int g = lane >> 2, t = lane & 3;
    const float* s = red + warp * 128;
    if (!MANY) {
        acc[0] += s[g * 8]; acc[1] += s[(g + 8) * 8];   // all four lanes of a quad keep the same sums (store_tile relies on it)
    } else {
        acc[0] += s[g * 8 + 2 * t]; acc[1] += s[g * 8 + 2 * t + 1];
        acc[2] += s[(g + 8) * 8 + 2 * t]; acc[3] += s[(g + 8) * 8 + 2 * t + 1];
    }
}

constexpr long long WAIT_BUDGET = 2000000000ll;   // SM clock cycles (about a second)

// One product segment: this warp's items [i0, i1) of the segment that starts at product row tile rtb. When the
// warp's own stream is exhausted the ring goes on with `nx`, the warp's share of the NEXT segment, so the copies
// never pause at a segment boundary. Returns false when a bounded wait expired.
template <int KIND, bool MANY>
__device__ __forceinline__ bool run_segment(const DOp& op, int rtb, int i0, int i1, Ring& ring, Stream& st, Stream& nx, const LaneB1& lb1,
                                            const LaneBM& lbm, int m, float* red, float (&pend)[4], int& pend_rt, int lane, int warp) {
    const int nh = op.nh;
    int prt = rtb + i0 / nh;
    int h = i0 - (i0 / nh) * nh;
    bool mine = h == 0;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    int remaining = i1 - i0;
    pend_rt = -1;
    const int item_bytes = op.item_bytes;
    while (ring.inflight < ring.depth && st.to_issue == 0 && nx.to_issue > 0) ring_issue(ring, nx, lane);
    while (remaining > 0) {
        const int cnt = min(ring.chunk, remaining);
        bool ok = ring_wait(ring, WAIT_BUDGET);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) return false;
        uint32_t it = ring.slot0 + ring.cslot * ring.slot_bytes;
        for (int c = 0; c < cnt; c++, it += item_bytes) {
            if (KIND == DK_Q4K || KIND == DK_Q5K) {
                if (MANY) item_q4k_many<KIND == DK_Q5K>(it, lbm, h, acc, lane); else item_q4k_one<KIND == DK_Q5K>(it, lb1, h, acc, lane);
            } else if (KIND == DK_Q40) {
                if (MANY) item_q40_many(it, lbm, h, acc, lane); else item_q40_one(it, lb1, h, acc, lane);
            } else if (KIND == DK_Q6K) {
                if (MANY) item_q6k_many(it, lbm, h, acc, lane); else item_q6k_one(it, lb1, h, acc, lane);
            } else if (KIND == DK_MX4) {
                if (MANY) item_mx4_many(it, lbm, h, acc, lane); else item_mx4_one(it, lb1, h, acc, lane);
            } else {
                if (MANY) item_s8_many<KIND>(it, lbm, h, acc, lane); else item_s8_one<KIND>(it, lb1, h, acc, lane);
            }
            if (++h == nh) {   // the row tile is complete as far as this warp is concerned
                finish_acc<MANY>(acc);
                if (mine) store_tile<MANY>(op, prt, acc, m, lane);
                else slot_write<MANY>(red, warp, acc, lane);
                h = 0; prt++; mine = true;
                acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
            }
        }
        remaining -= cnt;
        __syncwarp();   // every lane has read the slot before it is refilled
        ring_release(ring);
        if (st.to_issue > 0) ring_issue(ring, st, lane);
        else if (nx.to_issue > 0) ring_issue(ring, nx, lane);
    }
    if (h != 0) {   // the range ends inside a row tile
        finish_acc<MANY>(acc);
        if (mine) {   // this warp started it: it collects the other parts after the CTA has met
            pend_rt = prt;
            pend[0] = acc[0]; pend[1] = acc[1]; pend[2] = acc[2]; pend[3] = acc[3];
        } else {
            slot_write<MANY>(red, warp, acc, lane);
        }
    }
    return true;
}

template <int NW>
__device__ __forceinline__ void warp_range(int items, int warp, int& i0, int& i1) {
    i0 = (int)(((int64_t)items * warp) / NW);
    i1 = (int)(((int64_t)items * (warp + 1)) / NW);
}

// A segment: row tiles [b, e) (launch-wide indices) of the product in `slot` of the descriptor cache.
struct Seg {
    int b, e;     // launch-wide row tiles
    int opi;      // index of the product
    int ub, ue;   // the work unit the segment belongs to
};

// NW warps per CTA; MANY = activation rows on the MMA's N side (m = 2..8), else the one-row block-diagonal form.
template <int NW, bool MANY>
__global__ void __launch_bounds__(NW * 32, NW == 8 ? 2 : 1)
gemv_i8_kernel(const __grid_constant__ DOp single, const DOp* __restrict__ ops, int n_ops, const int2* __restrict__ ranges, int n_units,
               int total_rt, int m, int* status, int* sched, int chunk, int depth, int slot_bytes, const __grid_constant__ PeerSignal sig) {
    // `single` and `sig` are indexed by lane / by peer: as grid constants they are read where the launch put them;
    // as plain parameters every thread would first copy them to its stack (216 bytes x 75776 threads of DRAM writes)
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ DOp s_op[3];    // descriptors of the previous, the current and the next segment's product
    __shared__ int s_next;     // next work unit of the CTA
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* red = reinterpret_cast<float*>(smem + bar_bytes(NW));
    uint8_t* zero = smem + bar_bytes(NW) + red_bytes(NW);
    uint8_t* ring_base = smem + fixed_bytes(NW);
    uint8_t* ximg = ring_base + (size_t)NW * depth * slot_bytes;

    Ring ring;
    ring.bar0 = smem_addr(smem) + warp * MAX_DEPTH * 8;
    ring.slot0 = smem_addr(ring_base + (size_t)warp * depth * slot_bytes);
    ring.depth = depth; ring.slot_bytes = slot_bytes; ring.chunk = chunk;
    ring.pslot = 0; ring.cslot = 0; ring.parity = 0u; ring.inflight = 0;
    if (lane == 0)
        for (int s = 0; s < depth; s++) mbar_init(ring.bar0 + s * 8, 1);
    if (threadIdx.x < ZERO_BYTES / 4) reinterpret_cast<uint32_t*>(zero)[threadIdx.x] = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");

    // Work units are contiguous ranges of row tiles (of one or several products). Unit blockIdx.x is this CTA's
    // first; further units are handed out by an atomic counter. Every fetch happens after griddepcontrol.wait,
    // i.e. after the launch ahead in the stream (which uses the same counter) has completed and reset it.
    auto unit_range = [&](int u, int& b, int& e) {
        if (ranges) {
            const int2 rg = ranges[u];
            b = rg.x; e = rg.y;
        } else {
            b = (int)(((int64_t)u * total_rt) / n_units);
            e = (int)(((int64_t)(u + 1) * total_rt) / n_units);
        }
    };
    auto find_op = [&](int rt) {   // product whose row tiles contain rt
        int lo = 0, hi = n_ops - 1;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (ops[mid].rt0 + ops[mid].nrt <= rt) lo = mid + 1; else hi = mid;
        }
        return lo;
    };
    // a warp copies one 128-byte descriptor into the cache
    static_assert(sizeof(DOp) == 128, "one word per lane");
    auto cache_op = [&](int slot, int opi) {
        const uint32_t* src = n_ops > 1 ? reinterpret_cast<const uint32_t*>(ops + opi) : nullptr;
        reinterpret_cast<uint32_t*>(&s_op[slot])[lane] = src ? __ldg(src + lane) : reinterpret_cast<const uint32_t*>(&single)[lane];
    };

    Seg cur;
    unit_range(blockIdx.x, cur.ub, cur.ue);
    cur.b = cur.ub;
    cur.opi = n_ops > 1 ? find_op(cur.b) : 0;
    if (warp == 0) cache_op(0, cur.opi);
    __syncthreads();
    cur.e = min(cur.ue, s_op[0].rt0 + s_op[0].nrt);
    // Programmatic dependent launch: the next kernel of the stream may start its CTAs as ours retire; like this
    // kernel it touches nothing an earlier kernel writes (activations, outputs) before its griddepcontrol.wait,
    // only the immutable packed weights.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // this warp's share of a segment as a stream of items
    auto stream_of = [&](const DOp& o, const Seg& sg, int& i0, int& i1) {
        warp_range<NW>((sg.e - sg.b) * o.nh, warp, i0, i1);
        Stream st;
        st.src = o.img + ((int64_t)(sg.b - o.rt0) * o.nh + i0) * o.item_bytes;
        st.to_issue = i1 - i0;
        st.item_bytes = o.item_bytes;
        return st;
    };
    int i0, i1;
    Stream st = stream_of(s_op[0], cur, i0, i1);
    ring_fill(ring, st, lane);   // the weights are immutable: start them before anything else

    // only now wait for the kernels ahead in the stream, whose outputs the activations may be
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // thread 0: the unit after the current one (asked for at the start of the current unit); launches whose units
    // all start on a CTA of their own never touch the counter
    const bool dynamic = n_units > (int)gridDim.x;
    int fetched = n_units;
    if (dynamic && threadIdx.x == 0) fetched = (int)gridDim.x + atomicAdd(&sched[0], 1);

    bool alive = true;
    int si = 0;   // descriptor slot of the current segment; the previous one is (si + 2) % 3, the next (si + 1) % 3
    // hand-over of the previous segment, completed after the CTA has met
    float pend[4];
    int pend_rt = -1, prev_b = 0, prev_items = 0, prev_i1 = 0;
    for (;;) {
        const DOp& op = s_op[si];
        const int sp = si == 0 ? 2 : si - 1, sn = si == 2 ? 0 : si + 1;
        const bool last_seg = cur.e >= cur.ue;   // the unit ends with this segment
        if (last_seg && threadIdx.x == 0) s_next = fetched;
        __syncthreads();   // the previous segment is done: its hand-over slots are written, its activations free
        if (alive && pend_rt >= 0) {
            // parts of the pending row tile lie with the following warps, in order, until one reaches its end
            const DOp& po = s_op[sp];
            const int tile_end = (pend_rt - prev_b + 1) * po.nh;
            int pos = prev_i1;
            for (int w2 = warp + 1; w2 < NW && pos < tile_end; w2++) {
                int j0, j1;
                warp_range<NW>(prev_items, w2, j0, j1);
                if (j0 == j1) continue;
                slot_add<MANY>(red, w2, pend, lane);
                pos = j1;
            }
            store_tile<MANY>(po, pend_rt, pend, m, lane);
        }
        // the segment after this one; its descriptor goes into the slot nobody reads any more
        Seg nxt;
        bool have_next = true;
        if (!last_seg) {
            nxt.ub = cur.ub; nxt.ue = cur.ue; nxt.b = cur.e; nxt.opi = cur.opi + 1;   // products are consecutive in row tiles
        } else {
            const int nu = s_next;
            if (nu < n_units) {
                unit_range(nu, nxt.ub, nxt.ue);
                nxt.b = nxt.ub;
                nxt.opi = n_ops > 1 ? find_op(nxt.b) : 0;
                if (threadIdx.x == 0) fetched = (int)gridDim.x + atomicAdd(&sched[0], 1);   // only reached when dynamic
            } else {
                have_next = false;
            }
        }
        if (have_next && warp == NW - 1) cache_op(sn, nxt.opi);
        // activation image of this segment
        ActImg ai;
        ai.limbs = ximg;
        ai.fs = reinterpret_cast<float*>(ximg + act_limb_bytes(op.k, m));
        LaneB1 lb1{};
        LaneBM lbm{};
        if (op.kind == DK_MX4) {
            prep_x<32, MANY, NW * 32, true>(op.x, op.ldx, op.k, m, ai, 12.0f);
            if (MANY) lbm = lane_bm(ai, zero, lane, m); else lb1 = lane_b1<32>(ai, zero, lane);
        } else if (op.kind == DK_Q40) {   // the image keeps 8 sum x
            prep_x<32, MANY, NW * 32>(op.x, op.ldx, op.k, m, ai, 8.0f);
            if (MANY) lbm = lane_bm(ai, zero, lane, m); else lb1 = lane_b1<32>(ai, zero, lane);
        } else if (op.kind != DK_Q6K) {   // scale groups of 32; only Q4_K and Q5_K use the sums
            prep_x<32, MANY, NW * 32>(op.x, op.ldx, op.k, m, ai, 1.0f);
            if (MANY) lbm = lane_bm(ai, zero, lane, m); else lb1 = lane_b1<32>(ai, zero, lane);
        } else {
            prep_x<16, MANY, NW * 32>(op.x, op.ldx, op.k, m, ai, 32.0f);
            if (MANY) lbm = lane_bm(ai, zero, lane, m); else lb1 = lane_b1<16>(ai, zero, lane);
        }
        __syncthreads();   // the image is complete and the next descriptor is cached
        Stream nx{nullptr, 0, 0};
        int n0 = 0, n1 = 0;
        if (have_next) {
            const DOp& no = s_op[sn];
            nxt.e = min(nxt.ue, no.rt0 + no.nrt);
            nx = stream_of(no, nxt, n0, n1);
            if (!alive) nx.to_issue = 0;
        }

        prev_b = cur.b - op.rt0; prev_items = (cur.e - cur.b) * op.nh; prev_i1 = i1;
        pend_rt = -1;
        if (alive) {
            bool ok;
            if (op.kind == DK_Q4K) ok = run_segment<DK_Q4K, MANY>(op, prev_b, i0, i1, ring, st, nx, lb1, lbm, m, red, pend, pend_rt, lane, warp);
            else if (op.kind == DK_Q6K) ok = run_segment<DK_Q6K, MANY>(op, prev_b, i0, i1, ring, st, nx, lb1, lbm, m, red, pend, pend_rt, lane, warp);
            else if (op.kind == DK_Q80) ok = run_segment<DK_Q80, MANY>(op, prev_b, i0, i1, ring, st, nx, lb1, lbm, m, red, pend, pend_rt, lane, warp);
            else if (op.kind == DK_MX4) ok = run_segment<DK_MX4, MANY>(op, prev_b, i0, i1, ring, st, nx, lb1, lbm, m, red, pend, pend_rt, lane, warp);
            else if (op.kind == DK_Q40) ok = run_segment<DK_Q40, MANY>(op, prev_b, i0, i1, ring, st, nx, lb1, lbm, m, red, pend, pend_rt, lane, warp);
            else if (op.kind == DK_Q5K) ok = run_segment<DK_Q5K, MANY>(op, prev_b, i0, i1, ring, st, nx, lb1, lbm, m, red, pend, pend_rt, lane, warp);
            else ok = run_segment<DK_MX6, MANY>(op, prev_b, i0, i1, ring, st, nx, lb1, lbm, m, red, pend, pend_rt, lane, warp);
            if (!ok) {
                alive = false;
                pend_rt = -1;
                if (lane == 0) atomicExch(status, 100 + warp);
            }
        }
        if (!have_next) break;
        cur = nxt; st = nx; i0 = n0; i1 = n1;
        si = sn;
    }
    __syncthreads();   // hand-over slots of the last segment are written
    if (alive && pend_rt >= 0) {
        const DOp& po = s_op[si];
        const int tile_end = (pend_rt - prev_b + 1) * po.nh;
        int pos = prev_i1;
        for (int w2 = warp + 1; w2 < NW && pos < tile_end; w2++) {
            int j0, j1;
            warp_range<NW>(prev_items, w2, j0, j1);
            if (j0 == j1) continue;
            slot_add<MANY>(red, w2, pend, lane);
            pos = j1;
        }
        store_tile<MANY>(po, pend_rt, pend, m, lane);
    }
    // scattered products: when every CTA's stores to the peers are out, the last CTA tells the peers. One system-scope
    // fence per CTA (after the barrier it covers the whole CTA's stores), one more in the last CTA between its
    // observation of the counter and the flag stores, which are then plain system-scope stores issued back to back
    // (a release store per peer would wait for a round trip over NVLink each).
    if (sig.n > 0) {
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence_system();
            if (atomicAdd(&sched[2], 1) == (int)gridDim.x - 1) {
                sched[2] = 0;
                if (sig.status_out) *reinterpret_cast<volatile int*>(sig.status_out) = *reinterpret_cast<volatile int*>(status);
                __threadfence_system();
                for (int p = 0; p < sig.n; p++)
                    if (p != sig.my) asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(sig.flag[p] + sig.my), "r"(sig.epoch) : "memory");
            }
        }
    }
    // the last CTA to run out of units resets the counters for the next launch
    if (dynamic && threadIdx.x == 0 && atomicAdd(&sched[1], 1) == (int)gridDim.x - 1) {
        sched[0] = 0;
        sched[1] = 0;
        __threadfence();
    }
    // a wait that gave up leaves copies in flight: they must land before the CTA's shared memory is released
    if (!alive) {
        while (ring.inflight > 0) {
            ring_wait(ring, WAIT_BUDGET);
            ring_release(ring);
        }
    }
}

// ---------------------------------------------------------------------------------------------- image build
// One thread per (item, lane): gathers the lane's bytes of rows g and g+8 from the stream-layout planes.
__global__ void __launch_bounds__(256) build_image_q4k_kernel(const uint8_t* __restrict__ raw, uint8_t* __restrict__ img, int n_rows, int nh,
                                                               int64_t n_items) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t item = idx >> 5;
    if (item >= n_items) return;
    const int lane = (int)(idx & 31), g = lane >> 2, t = lane & 3;
    const int64_t T = item / nh;
    const int h = (int)(item - T * nh);
    uint8_t* it = img + item * Q4K_ITEM;
    uint32_t hs = 0;
    uint32_t dd[2] = {0u, 0u};
    for (int i = 0; i < 2; i++) {
        const int64_t row = T * 16 + g + 8 * i;
        uint4 out = make_uint4(0u, 0u, 0u, 0u);
        if (row < n_rows) {
            const int64_t hsi = row * nh + h;
            const uint8_t* blk = raw + (hsi >> 1) * 144;
            const int j = 4 * (int)(hsi & 1) + t;   // sub-block of the super-block
            const uint8_t* qs = blk + 16 + 32 * (j >> 1);
            uint8_t o[16];
            for (int b = 0; b < 16; b++)
                o[b] = (j & 1) ? (uint8_t)((qs[b] >> 4) | (qs[16 + b] & 0xF0)) : (uint8_t)((qs[b] & 0x0F) | ((qs[16 + b] & 0x0F) << 4));
            out = *reinterpret_cast<uint4*>(o);
            uint32_t sc, mn;
            q4k_scale_min(blk + 4, j, sc, mn);
            hs |= (sc | (mn << 8)) << (16 * i);
            dd[i] = ld32(blk);
        }
        *reinterpret_cast<uint4*>(it + 512 * i + chunk_pos(g, t) * 16) = out;
    }
    *reinterpret_cast<uint32_t*>(it + 1024 + lane * 4) = hs;
    if (t == 0) *reinterpret_cast<uint2*>(it + 1152 + g * 8) = make_uint2(dd[0], dd[1]);
}

// Q3K = true: a GGUF Q3_K tensor re-encoded, exactly, in Q6_K's item form. value = d (sc6 - 32) (q3 - 4) with q3 - 4 in
// -4..3 is d * sc * (q6 - 32) with the int8 scale sc = sc6 - 32 and q6 = q3 + 28: the decode kernel then runs its Q6_K
// code on the image (which holds 6.6 bit per weight where the file has 3.4).
template <bool Q3K>
__global__ void __launch_bounds__(256) build_image_q6k_kernel(WView v, uint8_t* __restrict__ img, int n_rows, int nh, int64_t n_items) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t item = idx >> 5;
    if (item >= n_items) return;
    const int lane = (int)(idx & 31), g = lane >> 2, t = lane & 3;
    const int64_t T = item / nh;
    const int h = (int)(item - T * nh);
    uint8_t* it = img + item * Q6K_ITEM;
    uint32_t hs = 0, dd = 0;
    uint32_t hq[4] = {0u, 0u, 0u, 0u};
    for (int i = 0; i < 2; i++) {
        const int64_t row = T * 16 + g + 8 * i;
        uint4 out = make_uint4(0u, 0u, 0u, 0u);
        if (row < n_rows) {
            const int64_t hsi = row * nh + h;
            const int64_t blk = hsi >> 1;
            const int sec = (int)(hsi & 1);
            uint8_t q[32];   // the lane's 32 codes: weights 32 t + e of the half
            uint32_t sc2 = 0;  // the two int8 scales of those weights (16 each)
            if (Q3K) {
                // planes hmask[32], qs[64], scales[12], d: element 128 sec + 32 t + e has its low two bits at
                // (qs[32 sec + e] >> 2 t) & 3 and its third bit at bit 4 sec + t of hmask[e]
                const uint8_t* hm = v.p[0] + blk * 32;
                const uint8_t* qs = v.p[1] + blk * 64 + sec * 32;
                for (int e = 0; e < 32; e++)
                    q[e] = (uint8_t)(((qs[e] >> (2 * t)) & 3u) + (((hm[e] >> (4 * sec + t)) & 1u) << 2) + 28u);
                const uint8_t* sc = v.p[2] + blk * 12;
                for (int u = 0; u < 2; u++) {
                    const int g16 = 8 * sec + 2 * t + u;
                    const uint32_t lo = g16 < 8 ? (sc[g16] & 15u) : (uint32_t)(sc[g16 - 8] >> 4);
                    const uint32_t hi = (uint32_t)(sc[8 + (g16 & 3)] >> (2 * (g16 >> 2))) & 3u;
                    sc2 |= (uint32_t)(uint8_t)(int8_t)((int)(lo | (hi << 4)) - 32) << (8 * u);
                }
            } else {
                const uint8_t* ql = v.p[0] + blk * 128 + sec * 64 + 32 * (t & 1);
                const uint8_t* qh = v.p[1] + blk * 64 + sec * 32;
                for (int e = 0; e < 32; e++) {
                    const uint32_t lo4 = (t < 2) ? (ql[e] & 0x0Fu) : (uint32_t)(ql[e] >> 4);
                    const uint32_t hi2 = (qh[e] >> (2 * t)) & 3u;
                    q[e] = (uint8_t)(lo4 | (hi2 << 4));
                }
                const uint8_t* sc = v.p[2] + blk * 16 + sec * 8 + 2 * t;
                sc2 = (uint32_t)sc[0] | ((uint32_t)sc[1] << 8);
            }
            uint8_t o[16];
            for (int b = 0; b < 16; b++) o[b] = (uint8_t)((q[b] & 0x0F) | ((q[16 + b] >> 2) << 4));
            out = *reinterpret_cast<uint4*>(o);
            for (int u = 0; u < 2; u++) {
                uint32_t word = 0;
                for (int z = 0; z < 4; z++) {
                    const uint32_t byte = ((uint32_t)(q[8 * u + z] >> 4) << 4) | ((uint32_t)(q[16 + 8 * u + z] & 3) << 2) |
                                          ((uint32_t)(q[8 * u + 4 + z] >> 4) << 6) | (uint32_t)(q[16 + 8 * u + 4 + z] & 3);
                    word |= byte << (8 * z);
                }
                hq[2 * i + u] = word;
            }
            hs |= sc2 << (16 * i);
            dd |= (uint32_t)ld16(v.p[3] + blk * 2) << (16 * i);
        }
        *reinterpret_cast<uint4*>(it + 512 * i + chunk_pos(g, t) * 16) = out;
    }
    *reinterpret_cast<uint4*>(it + 1024 + chunk_pos(g, t) * 16) = make_uint4(hq[0], hq[1], hq[2], hq[3]);
    *reinterpret_cast<uint32_t*>(it + 1536 + lane * 4) = hs;
    if (t == 0) *reinterpret_cast<uint32_t*>(it + 1664 + g * 4) = dd;
}

// Q8_0 (codes as stored) and MXFP6 E2M3 (codes widened to 8 * value): one thread per (item, lane).
// e3m2 (MXFP6 only): the bytes are not int8 codes but the E3M2 code s|eee|mm spread to s00eeemm, which is the high byte of
// the f16 holding value * 2^-12 (the tensor-memory prefill kernel's form; the integer decode kernel cannot use it).
template <int KIND>
__global__ void __launch_bounds__(256) build_image_s8_kernel(WView v, uint8_t* __restrict__ img, int n_rows, int nh, int64_t n_items,
                                                              int e3m2 = 0) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t item = idx >> 5;
    if (item >= n_items) return;
    const int lane = (int)(idx & 31), g = lane >> 2, t = lane & 3;
    const int64_t T = item / nh;
    const int h = (int)(item - T * nh);
    uint8_t* it = img + item * (KIND == DK_Q80 ? Q80_ITEM : MX6_ITEM);
    uint16_t sc[2] = {0, 0};
    for (int i = 0; i < 2; i++) {
        const int64_t row = T * 16 + g + 8 * i;
        uint8_t o[32];
        for (int b = 0; b < 32; b++) o[b] = 0;
        if (row < n_rows) {
            const int64_t blk = (row * nh + h) * 4 + t;   // 32-weight block in the flat stream
            if (KIND == DK_Q80) {
                const uint8_t* q = v.p[1] + blk * 32;
                for (int b = 0; b < 32; b++) o[b] = q[b];
                sc[i] = ld16(v.p[0] + blk * 2);
            } else {
                const uint8_t* q = v.p[1] + blk * 24;
                for (int b = 0; b < 32; b++) {
                    const int bit = 6 * b;
                    const uint32_t comb = (uint32_t)q[bit >> 3] | ((bit >> 3) + 1 < 24 ? (uint32_t)q[(bit >> 3) + 1] << 8 : 0u);
                    const uint32_t code = (comb >> (bit & 7)) & 63u;
                    o[b] = e3m2 ? (uint8_t)(((code & 0x20u) << 2) | (code & 0x1Fu)) : (uint8_t)(int8_t)__float2int_rn(ocp_e2m3(code) * 8.0f);
                }
                sc[i] = v.p[0][blk];
            }
        }
        const int cp = chunk_pos(g, t) * 16;
        *reinterpret_cast<uint4*>(it + 1024 * i + cp) = *reinterpret_cast<uint4*>(o);
        *reinterpret_cast<uint4*>(it + 1024 * i + 512 + cp) = *reinterpret_cast<uint4*>(o + 16);
    }
    if (KIND == DK_Q80) *reinterpret_cast<uint32_t*>(it + 2048 + lane * 4) = (uint32_t)sc[0] | ((uint32_t)sc[1] << 16);
    else *reinterpret_cast<uint16_t*>(it + 2048 + lane * 2) = (uint16_t)((sc[0] & 0xFF) | ((sc[1] & 0xFF) << 8));
}

__global__ void __launch_bounds__(256) build_image_mx4_kernel(WView v, uint8_t* __restrict__ img, int n_rows, int nh, int64_t n_items) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t item = idx >> 5;
    if (item >= n_items) return;
    const int lane = (int)(idx & 31), g = lane >> 2, t = lane & 3;
    const int64_t T = item / nh;
    const int h = (int)(item - T * nh);
    uint8_t* it = img + item * MX4_ITEM;
    uint32_t sc = 0;
    for (int i = 0; i < 2; i++) {
        const int64_t row = T * 16 + g + 8 * i;
        uint32_t o[4] = {0u, 0u, 0u, 0u};
        if (row < n_rows) {
            const int64_t blk = (row * nh + h) * 4 + t;
            const uint8_t* q = v.p[1] + blk * 16;   // byte i: element i (low nibble), element i + 16 (high nibble)
            for (int e = 0; e < 32; e++) {
                const uint32_t code = e < 16 ? (q[e] & 0x0Fu) : (uint32_t)(q[e - 16] >> 4);
                o[e >> 3] |= code << (4 * (e & 7));
            }
            sc |= (uint32_t)v.p[0][blk] << (8 * i);
        }
        *reinterpret_cast<uint4*>(it + 512 * i + chunk_pos(g, t) * 16) = make_uint4(o[0], o[1], o[2], o[3]);
    }
    *reinterpret_cast<uint16_t*>(it + 1024 + lane * 2) = (uint16_t)sc;
}

// Q4_0: the block's 16 code bytes as they are, f16 d per block.
__global__ void __launch_bounds__(256) build_image_q40_kernel(WView v, uint8_t* __restrict__ img, int n_rows, int nh, int64_t n_items) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t item = idx >> 5;
    if (item >= n_items) return;
    const int lane = (int)(idx & 31), g = lane >> 2, t = lane & 3;
    const int64_t T = item / nh;
    const int h = (int)(item - T * nh);
    uint8_t* it = img + item * Q40_ITEM;
    uint32_t dd = 0;
    for (int i = 0; i < 2; i++) {
        const int64_t row = T * 16 + g + 8 * i;
        uint4 out = make_uint4(0u, 0u, 0u, 0u);
        if (row < n_rows) {
            const int64_t blk = (row * nh + h) * 4 + t;
            const uint8_t* q = v.p[1] + blk * 16;
            uint8_t o[16];
            for (int b = 0; b < 16; b++) o[b] = q[b];
            out = *reinterpret_cast<uint4*>(o);
            dd |= (uint32_t)ld16(v.p[0] + blk * 2) << (16 * i);
        }
        *reinterpret_cast<uint4*>(it + 512 * i + chunk_pos(g, t) * 16) = out;
    }
    *reinterpret_cast<uint32_t*>(it + 1024 + lane * 4) = dd;
}

// Q5_K: Q4_K's item plus the fifth bits.
__global__ void __launch_bounds__(256) build_image_q5k_kernel(const uint8_t* __restrict__ raw, uint8_t* __restrict__ img, int n_rows, int nh,
                                                               int64_t n_items) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t item = idx >> 5;
    if (item >= n_items) return;
    const int lane = (int)(idx & 31), g = lane >> 2, t = lane & 3;
    const int64_t T = item / nh;
    const int h = (int)(item - T * nh);
    uint8_t* it = img + item * Q5K_ITEM;
    uint32_t hs = 0;
    uint32_t dd[2] = {0u, 0u}, hb[2] = {0u, 0u};
    for (int i = 0; i < 2; i++) {
        const int64_t row = T * 16 + g + 8 * i;
        uint4 out = make_uint4(0u, 0u, 0u, 0u);
        if (row < n_rows) {
            const int64_t hsi = row * nh + h;
            const uint8_t* blk = raw + (hsi >> 1) * 176;   // d, dmin, scales[12], qh[32], qs[128]
            const int j = 4 * (int)(hsi & 1) + t;           // sub-block of the super-block
            const uint8_t* qh = blk + 16;
            const uint8_t* qs = blk + 48 + 32 * (j >> 1);
            uint8_t o[16];
            for (int b = 0; b < 16; b++)
                o[b] = (j & 1) ? (uint8_t)((qs[b] >> 4) | (qs[16 + b] & 0xF0)) : (uint8_t)((qs[b] & 0x0F) | ((qs[16 + b] & 0x0F) << 4));
            out = *reinterpret_cast<uint4*>(o);
            uint32_t H = 0;
            for (int e = 0; e < 32; e++) {   // weight e of the sub-block: fifth bit = bit j of qh[e]
                const uint32_t bit = (qh[e] >> j) & 1u;
                const int z = e & 3, jj = (e & 15) >> 2;
                H |= bit << (8 * z + (e < 16 ? jj : 4 + jj));
            }
            hb[i] = H;
            uint32_t sc, mn;
            q4k_scale_min(blk + 4, j, sc, mn);
            hs |= (sc | (mn << 8)) << (16 * i);
            dd[i] = ld32(blk);
        }
        *reinterpret_cast<uint4*>(it + 512 * i + chunk_pos(g, t) * 16) = out;
    }
    *reinterpret_cast<uint32_t*>(it + 1024 + lane * 4) = hs;
    if (t == 0) *reinterpret_cast<uint2*>(it + 1152 + g * 8) = make_uint2(dd[0], dd[1]);
    *reinterpret_cast<uint2*>(it + 1216 + lane * 8) = make_uint2(hb[0], hb[1]);
}

}  // namespace

int decode_kind_of(int fmt) {
    if (fmt == F_Q4K) return DK_Q4K;
    if (fmt == F_Q6K) return DK_Q6K;
    if (fmt == F_Q80) return DK_Q80;
    if (fmt == F_MX6) return DK_MX6;
    if (fmt == F_MX4) return DK_MX4;
    if (fmt == F_Q40) return DK_Q40;
    if (fmt == F_Q5K) return DK_Q5K;
    if (fmt == F_Q3K) return DK_Q6K;   // re-encoded in Q6_K's item form when the image is built
    return DK_NONE;
}

int decode_item_bytes(int kind) {
    return kind == DK_Q4K ? Q4K_ITEM : kind == DK_Q6K ? Q6K_ITEM : kind == DK_Q80 ? Q80_ITEM : kind == DK_MX6 ? MX6_ITEM : kind == DK_MX4 ? MX4_ITEM : kind == DK_Q40 ? Q40_ITEM : kind == DK_Q5K ? Q5K_ITEM : 0;
}

bool decode_image_wanted(int fmt, int orient, int64_t n_rows, int64_t k) {
    if (decode_kind_of(fmt) == DK_NONE || orient != B200Q_ORIENT_NK) return false;
    if (k % 128 || k > (1 << 24) || n_rows > 0x7FFFFFF0ll) return false;
    const int64_t items = ((n_rows + 15) / 16) * (k / 128);
    return items < (1ll << 31) / 8;   // item counts of a CTA's segment stay inside 32-bit arithmetic
}

size_t decode_image_bytes(int fmt, int64_t n_rows, int64_t k) {
    const int kind = decode_kind_of(fmt);
    if (kind == DK_NONE) return 0;
    return (size_t)((n_rows + 15) / 16) * (size_t)(k / 128) * decode_item_bytes(kind) + 256;
}

int build_decode_image(b200q_ctx* ctx, const b200q_weight* w, DImage* out, uint8_t* place) {
    *out = DImage{};
    const int kind = decode_kind_of(w->fmt);
    if (kind == DK_NONE) return B200Q_OK;
    DImage d;
    d.kind = kind;
    d.item_bytes = decode_item_bytes(kind);
    d.nh = (int)(w->k / 128);
    d.nrt = (int)((w->n_local + 15) / 16);
    const int64_t n_items = (int64_t)d.nrt * d.nh;
    d.bytes = (size_t)n_items * d.item_bytes;
    void* p = place;
    if (!place) B200Q_CUDA(cudaMalloc(&p, d.bytes + 256), B200Q_ERR_ALLOC);
    d.base = static_cast<uint8_t*>(p);
    const int64_t threads = n_items * 32;
    const int64_t grid = (threads + 255) / 256;
    if (grid > 0x7FFFFFFF) {
        if (!place) cudaFree(p);
        return fail(B200Q_ERR_INVALID, "upload: tensor too large for one image-build launch");
    }
    if (kind == DK_Q4K) build_image_q4k_kernel<<<(unsigned)grid, 256, 0, ctx->stream>>>(w->view.p[0], d.base, (int)w->n_local, d.nh, n_items);
    else if (kind == DK_Q6K && w->fmt == F_Q3K) build_image_q6k_kernel<true><<<(unsigned)grid, 256, 0, ctx->stream>>>(w->view, d.base, (int)w->n_local, d.nh, n_items);
    else if (kind == DK_Q6K) build_image_q6k_kernel<false><<<(unsigned)grid, 256, 0, ctx->stream>>>(w->view, d.base, (int)w->n_local, d.nh, n_items);
    else if (kind == DK_Q80) build_image_s8_kernel<DK_Q80><<<(unsigned)grid, 256, 0, ctx->stream>>>(w->view, d.base, (int)w->n_local, d.nh, n_items);
    else if (kind == DK_Q40) build_image_q40_kernel<<<(unsigned)grid, 256, 0, ctx->stream>>>(w->view, d.base, (int)w->n_local, d.nh, n_items);
    else if (kind == DK_Q5K) build_image_q5k_kernel<<<(unsigned)grid, 256, 0, ctx->stream>>>(w->view.p[0], d.base, (int)w->n_local, d.nh, n_items);
    else if (kind == DK_MX4) build_image_mx4_kernel<<<(unsigned)grid, 256, 0, ctx->stream>>>(w->view, d.base, (int)w->n_local, d.nh, n_items);
    else build_image_s8_kernel<DK_MX6><<<(unsigned)grid, 256, 0, ctx->stream>>>(w->view, d.base, (int)w->n_local, d.nh, n_items);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess && !place) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        if (!place) cudaFree(p);
        return cuda_fail(B200Q_ERR_LAUNCH, e, "upload: decode image");
    }
    *out = d;
    return B200Q_OK;
}

// GGUF MXFP6 E3M2: an image in MXFP6 E2M3's item form for the tensor-memory prefill kernel only (own allocation).
int build_e3m2_prefill_image(b200q_ctx* ctx, const b200q_weight* w, DImage* out) {
    *out = DImage{};
    if (w->fmt != fmt_of(MXFP6_E3M2, GGUF) || w->orient != B200Q_ORIENT_NK || (w->k % 128) != 0)
        return fail(B200Q_ERR_INVALID, "prefill image: needs a GGUF MXFP6 E3M2 NK tensor with k %% 128 == 0");
    DImage d;
    d.kind = DK_MX6;
    d.item_bytes = MX6_ITEM;
    d.nh = (int)(w->k / 128);
    d.nrt = (int)((w->n_local + 15) / 16);
    const int64_t n_items = (int64_t)d.nrt * d.nh;
    d.bytes = (size_t)n_items * d.item_bytes;
    const int64_t grid = (n_items * 32 + 255) / 256;
    if (grid > 0x7FFFFFFF) return fail(B200Q_ERR_INVALID, "prefill image: tensor too large for one image-build launch");
    void* p = nullptr;
    B200Q_CUDA(cudaMalloc(&p, d.bytes + 256), B200Q_ERR_ALLOC);
    d.base = static_cast<uint8_t*>(p);
    build_image_s8_kernel<DK_MX6><<<(unsigned)grid, 256, 0, ctx->stream>>>(w->view, d.base, (int)w->n_local, d.nh, n_items, 1);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        cudaFree(p);
        return cuda_fail(B200Q_ERR_LAUNCH, e, "prefill image");
    }
    *out = d;
    return B200Q_OK;
}

size_t gemv_i8_image_smem(int kind, int k, int m) { return act_image_bytes(kind, k, m); }

bool gemv_i8_plan(int max_item_bytes, int kmax, int kind_mask, int m, DecodeLaunch* out) {
    size_t image = 0;
    for (int kd = 0; kd < DK_COUNT; kd++)
        if (kind_mask & (1 << kd)) image = max(image, act_image_bytes(kd, kmax, m));
    // one activation row: 8 warps per CTA, two CTAs per SM; more rows: 16 warps, one CTA per SM (one image per SM)
    const int nw = m == 1 ? 8 : 16;
    // tuning knob (like the reference's ROCFORGE_TILE_* variables, src/ggml/hip_backend/tuning.rs:237-275):
    // B200Q_DECODE_RING="items per copy,slots per warp"
    int chunk = 4, depth = 2;
    if (const char* e = getenv("B200Q_DECODE_RING")) {
        int c = 0, d = 0;
        if (sscanf(e, "%d,%d", &c, &d) == 2 && c >= 1 && c <= 8 && d >= 2 && d <= MAX_DEPTH) { chunk = c; depth = d; }
    }
    const size_t cap = nw == 8 ? 112 * 1024 : 225 * 1024, cap1 = 225 * 1024;
    const size_t fixed = fixed_bytes(nw);
    for (int pass = 0; pass < 2; pass++) {
        // first pass: the preferred occupancy; second pass (8-warp form only): one CTA per SM
        const size_t limit = pass == 0 ? cap : cap1;
        int c = chunk, d = depth;
        for (;;) {
            const int slot = ((c * max_item_bytes + 127) / 128) * 128;
            const size_t total = fixed + (size_t)nw * d * slot + image;
            if (total <= limit) {
                out->chunk_items = c; out->depth = d; out->slot_bytes = slot; out->smem_bytes = total;
                out->ctas_per_sm = (nw == 8 && total <= 112 * 1024) ? 2 : 1;
                out->nw = nw; out->many = m > 1;
                return true;
            }
            if (d > 2) d--;
            else if (c > 1) c--;
            else break;
        }
    }
    return false;
}

void gemv_i8_make_units(const std::vector<double>& tile_cost, const std::vector<int>& tile_op, int n_ctas, std::vector<int2>* units) {
    // Contiguous ranges of (nearly) equal cost. A range that starts a new product pays for the barrier, the
    // activation image and the hand-over of a segment: `seg_cost` bytes' worth of time.
    // tuning knobs: B200Q_DECODE_UNITS="static share in percent,tail units per CTA,segment cost in KiB": the first
    // n_ctas units split that share of the work evenly, the rest is cut into smaller units handed out dynamically
    double share = 100.0, seg_cost = 96.0 * 1024;
    int tail = 0;
    if (const char* e = getenv("B200Q_DECODE_UNITS")) {
        double a = 0, c = 0;
        int t = 0;
        if (sscanf(e, "%lf,%d,%lf", &a, &t, &c) == 3 && a >= 10 && a <= 100 && t >= 0 && t <= 16 && c >= 0) { share = a; tail = t; seg_cost = c * 1024; }
    }
    const int total = (int)tile_cost.size();
    std::vector<double> cost(total);
    double sum = 0;
    for (int t = 0; t < total; t++) {
        cost[t] = tile_cost[t] + ((t == 0 || tile_op[t] != tile_op[t - 1]) ? seg_cost : 0.0);
        sum += cost[t];
    }
    units->clear();
    if (tail == 0) share = 100.0;
    const double first_part = sum * share / 100.0;
    double acc = 0;
    int t = 0;
    for (int c = 0; c < n_ctas && t < total; c++) {
        int2 u;
        u.x = t;
        const double limit = first_part * (c + 1) / n_ctas;
        const bool last = share >= 100.0 && c == n_ctas - 1;
        // a range that does not start a product pays for its segment all the same
        double own = (tile_op[t] == (t ? tile_op[t - 1] : -1)) ? seg_cost : 0.0;
        while (t < total && (last || acc + own + cost[t] * 0.5 <= limit || t == u.x)) acc += cost[t++];
        u.y = t;
        units->push_back(u);
    }
    if (t < total) {
        const int n_tail = n_ctas * tail;
        const double rest = sum - acc;
        double acc2 = 0;
        for (int c = 0; c < n_tail && t < total; c++) {
            int2 u;
            u.x = t;
            const double limit = rest * (c + 1) / n_tail;
            while (t < total && (c == n_tail - 1 || acc2 + cost[t] * 0.5 <= limit || t == u.x)) acc2 += cost[t++];
            u.y = t;
            units->push_back(u);
        }
    }
}

bool gemv_i8_supported(const b200q_weight* w, int m) {
    if (!w->dimg.base || m < 1 || m > 8) return false;
    DecodeLaunch L;
    return gemv_i8_plan(w->dimg.item_bytes, (int)w->k, 1 << w->dimg.kind, m, &L);
}

int launch_gemv_i8(b200q_ctx* ctx, const DOp* h_single, const DOp* d_ops, int n_ops, const int2* d_ranges, int n_units, int n_ctas,
                   int total_rt, int m, const DecodeLaunch& L, const PeerSignal* sig_in) {
    if (total_rt <= 0) return B200Q_OK;
    if (n_units > total_rt) n_units = total_rt;
    if (n_ctas > n_units) n_ctas = n_units;
    static std::atomic<bool> configured[64][2] = {};
    const int ki = L.many ? 1 : 0;
    const void* kernels[2] = {(const void*)gemv_i8_kernel<8, false>, (const void*)gemv_i8_kernel<16, true>};
    if (!configured[ctx->device & 63][ki]) {
        B200Q_CUDA(cudaFuncSetAttribute(kernels[ki], cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024), B200Q_ERR_LAUNCH);
        configured[ctx->device & 63][ki] = true;
    }
    DOp single{};
    if (h_single) single = *h_single;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)n_ctas);
    cfg.blockDim = dim3(L.nw * 32);
    cfg.dynamicSmemBytes = L.smem_bytes;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // overlap with the tail of the kernel ahead
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int* status = ctx->d_status;
    int* sched = ctx->d_status + 2;   // {next unit, CTAs done, CTAs done storing to peers}: zero between launches
    PeerSignal sig{};
    if (sig_in) sig = *sig_in;
    int chunk = L.chunk_items, depth = L.depth, slot = L.slot_bytes;
    void* args[] = {&single, &d_ops, &n_ops, &d_ranges, &n_units, &total_rt, &m, &status, &sched, &chunk, &depth, &slot, &sig};
    B200Q_CUDA(cudaLaunchKernelExC(&cfg, kernels[ki], args), B200Q_ERR_LAUNCH);
    B200Q_CUDA(cudaGetLastError(), B200Q_ERR_LAUNCH);
    ctx->tc_pending = true;   // the next synchronise reads the status word
    return B200Q_OK;
}

}  // namespace b200q
