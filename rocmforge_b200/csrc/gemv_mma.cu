// Grouped decode kernel: fused dequant + matmul for 1..8 activation rows, HBM-bound.
//
// Replaces the per-row-block scalar kernels of the reference (kernels/q4_k_matmul.hip:216,
// q6_k_matmul.hip:216: one thread block per ACTIVATION row, one 4-bit code per inner iteration) and the
// serial per-op loop of BatchQuantizedMatmul::process_batch (src/ggml/hip_backend/ops/batch_quantized.rs:147-161).
//
// Why tensor cores for a GEMV. A B200 SM has to consume ~40 4.5-bit weights per clock to keep up with HBM
// but issues at most 4 warp instructions per clock, so the budget is ~2.5 thread instructions per weight:
// converting every code to fp32 and multiplying it on the CUDA cores does not fit. Here the raw integer
// codes go to the tensor cores as f16 SUBNORMALS: a 4- or 6-bit code q masked into the low bits of an f16
// lane is exactly q * 2^-24 (q * 2^-20 for a nibble left in bits 4..7). Extraction is one AND per pair of
// weights; everything else is per 16-weight run.
//
// Block-diagonal B operand. In mma.sync.m16n8k16 thread t of a quad supplies k-slots {2t,2t+1,2t+8,2t+9}
// of the 16 weight rows. Each thread streams its OWN 16-weight runs (16 contiguous bytes of one row), so
// the 16 k-slots of one MMA belong to four different runs with four different block scales. The 8 columns
// of B are therefore used as 4 threads x {hi, lo}: column 2t holds the f16 "hi" part of the activations for
// the k-slots of thread t and zeros elsewhere, column 2t+1 the "lo" part. The accumulator fragment that
// thread t receives (columns 2t, 2t+1) is then exactly the dot product of ITS run with hi and lo, and the
// block scale (d * sc, exact in fp32), the 2^24 and the "- dmin * m" / "- 32" offsets (one FMA with the
// pre-computed sum of the run's activations) are applied once per run by the thread that owns it.
// Activations are x = s * (hi + lo) with s a power of two per 16-weight run, so products carry 22 mantissa
// bits and accumulate in fp32: results stay within 1e-4 of the fp32 oracle. More activation rows repeat
// the MMAs (the extracted codes are reused), so cost grows slowly with m.
//
// Work decomposition. A CTA tile is (8 >> kw_log2) tiles of 16 weight rows x the whole k, the 8 warps of
// the CTA arranged as row-tiles x k-parts; partial sums meet in shared memory. A launch covers any number
// of products (a whole decode step): CTAs are persistent and own a contiguous range of CTA tiles balanced
// by bytes, so each CTA prepares the activations of only the products it touches.
#include <cuda_fp16.h>

#include "gemv_mma.cuh"

namespace b200q {

namespace {

constexpr int F_Q4K = fmt_of(Q4_K, GGUF);
constexpr int F_Q6K = fmt_of(Q6_K, GGUF);
constexpr int RED_FLOATS = 8 * 16 * 8;   // 8 warps x 16 rows x up to 8 activation rows

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// First MMA of a run: the accumulator input is the constant zero (no register initialisation needed).
__device__ __forceinline__ void mma16816_z(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                           uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

__device__ __forceinline__ uint4 ldg128(const uint8_t* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
// Pulls the line into L2 ahead of use; costs no register and may point past the end of a row (never past
// the tensor's allocation: callers clamp to `lim`).
__device__ __forceinline__ void prefetch_l2(const uint8_t* p, const uint8_t* lim) {
    if (p < lim) asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}
__device__ __forceinline__ uint32_t ldg16(const uint8_t* p) { return __ldg(reinterpret_cast<const uint16_t*>(p)); }
__device__ __forceinline__ uint32_t ldg8(const uint8_t* p) { return __ldg(p); }

// Shared-memory image of one product's activations, per 16-weight run R and activation row n:
//   img[(R*m + n)*4 + {0,1}] : f16 hi parts of the 16 activations, in MMA order (4 per MMA)
//   img[(R*m + n)*4 + {2,3}] : f16 lo parts
//   ss[R*m + n]              : {power-of-two scale of the run, sum of its fp32 activations}
struct XImg {
    uint4* img;
    float2* ss;
};

// The first 32 bytes of the activation area stay zero: lanes that supply the zero columns of B read them.
constexpr int XZERO_BYTES = 32;

__device__ __forceinline__ XImg ximg_carve(uint8_t* base, int k, int m) {
    XImg s;
    s.img = reinterpret_cast<uint4*>(base + XZERO_BYTES);
    s.ss = reinterpret_cast<float2*>(base + XZERO_BYTES + (size_t)(k >> 4) * m * 64);
    return s;
}

// Per-lane view of the B operand: lanes g == 2t (hi) and g == 2t+1 (lo) read the image of their run, every
// other lane reads the zero region (stride 0), so the loads need no predicate.
struct BLane {
    const uint4* base;
    int mult;   // 4 uint4 per (run, activation row) for data lanes, 0 for zero lanes
};

__device__ __forceinline__ BLane blane_make(const XImg& xs, uint8_t* xbase, int g, int t) {
    BLane b;
    bool active = (g >> 1) == t;
    b.base = active ? xs.img + (g & 1) * 2 : reinterpret_cast<const uint4*>(xbase);
    b.mult = active ? 4 : 0;
    return b;
}

__device__ __forceinline__ void load_b(const BLane& bl, int run_row, uint4& b01, uint4& b23) {
    const uint4* p = bl.base + run_row * bl.mult;
    b01 = p[0];
    b23 = p[1];
}

// x[m, k] (fp32, global) -> image. PERM: MMA j of a run takes elements (4j, 4j+2 | 4j+1, 4j+3), the pairs
// the nibble masks produce from bytes (0,2) and (1,3); otherwise natural order.
template <bool PERM>
__device__ __forceinline__ void prep_x(const float* __restrict__ x, int64_t ldx, int k, int m, const XImg& s) {
    const int total = (k >> 4) * m;
    for (int q = threadIdx.x; q < total; q += blockDim.x) {
        int R = q / m, n = q - R * m;
        const float4* xp = reinterpret_cast<const float4*>(x + (int64_t)n * ldx + (int64_t)R * 16);
        float v[16];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float4 f = __ldg(xp + i);
            v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
        }
        float mx = 0.0f, sum = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; i++) { mx = fmaxf(mx, fabsf(v[i])); sum += v[i]; }
        int e = (int)((__float_as_uint(mx) >> 23) & 255u);
        e = mx == 0.0f ? 127 : min(max(e, 1), 253);
        float sdown = __uint_as_float((uint32_t)(254 - e) << 23);   // 2^(127-e): the run lands in (-2, 2)
        float sup = __uint_as_float((uint32_t)e << 23);
        __align__(16) __half h[16];
        __align__(16) __half l[16];
#pragma unroll
        for (int i = 0; i < 16; i++) {
            int src = PERM ? ((i & ~3) | ((i & 1) << 1) | ((i & 2) >> 1)) : i;   // 0,2,1,3 inside each group of 4
            float xs = v[src] * sdown;
            h[i] = __float2half_rn(xs);
            l[i] = __float2half_rn(xs - __half2float(h[i]));
        }
        uint4* dst = s.img + (size_t)q * 4;
        dst[0] = reinterpret_cast<uint4*>(h)[0];
        dst[1] = reinterpret_cast<uint4*>(h)[1];
        dst[2] = reinterpret_cast<uint4*>(l)[0];
        dst[3] = reinterpret_cast<uint4*>(l)[1];
        s.ss[q] = make_float2(sup, sum);
    }
}

// ------------------------------------------------------------------------------------------- Q4_K (GGUF)
// A byte placed in an f16 lane is the subnormal byte * 2^-24: integer -> float without the integer pipe.
__device__ __forceinline__ float2 bytes_as_f16x2(uint32_t bits) {
    __half2 h;
    *reinterpret_cast<uint32_t*>(&h) = bits;
    return __half22float2(h);
}

// The block scales one thread needs from one super-block header of one weight row, multiplied out:
// per 128-weight half, d*sc*2^24 (low-nibble sub-block), d*sc*2^20 (high-nibble sub-block) and dmin*m of both.
struct Q4KHalfScales {
    float dA, dB, nA, nB;
};

// sel picks the chunk of each half the thread owns: sub-blocks 2tp, 2tp+1 (half 0) and 4+2tp, 5+2tp (half 1).
__device__ __forceinline__ void q4k_decode_hdr(uint4 h, uint32_t sel, Q4KHalfScales& h0, Q4KHalfScales& h1) {
    float d = __half2float(__ushort_as_half((unsigned short)(h.x & 0xFFFFu)));
    float dmin = __half2float(__ushort_as_half((unsigned short)(h.x >> 16)));
    uint32_t sc_lo = h.y & 0x3F3F3F3Fu, m_lo = h.z & 0x3F3F3F3Fu;
    uint32_t sc_hi = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
    uint32_t m_hi = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
    // bytes {A of half 0, B of half 0, A of half 1, B of half 1}
    uint32_t sc4 = __byte_perm(sc_lo, sc_hi, sel), m4 = __byte_perm(m_lo, m_hi, sel);
    float2 s01 = bytes_as_f16x2(__byte_perm(sc4, 0, 0x4140)), s23 = bytes_as_f16x2(__byte_perm(sc4, 0, 0x4342));
    float2 m01 = bytes_as_f16x2(__byte_perm(m4, 0, 0x4140)), m23 = bytes_as_f16x2(__byte_perm(m4, 0, 0x4342));
    const float T24 = 16777216.0f;
    float d48 = d * T24 * T24, d44 = d * T24 * 1048576.0f, dm24 = dmin * T24;
    h0.dA = d48 * s01.x; h0.dB = d44 * s01.y; h0.nA = dm24 * m01.x; h0.nB = dm24 * m01.y;
    h1.dA = d48 * s23.x; h1.dB = d44 * s23.y; h1.nA = dm24 * m23.x; h1.nB = dm24 * m23.y;
}

// One 16-row tile x halves [hb, he) (a half = 128 weights of a row). Thread (g, t) owns, in every half and
// for rows g and g+8, bytes [16*(t&1), +16) of chunk (t>>1): 16 weights of a low-nibble sub-block and 16 of
// the high-nibble sub-block. acc[i][n]: partial sum of row g+8i, activation row n, over this thread's runs.
template <int MT>
__device__ __forceinline__ void tile_q4k(const GOp& op, int m, int rtile, int hb, int he, const XImg& xs,
                                         const BLane& bl, float (&acc)[2][MT]) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3, tp = t >> 1;
    if (hb >= he) return;
    const uint8_t* base = op.v.p[0];
    const uint8_t* plim = base + ((((int64_t)op.n_rows * op.k) >> 8) * 144);   // end of the packed tensor
    const int qoff = 16 + tp * 32 + (t & 1) * 16;   // this thread's 16 bytes inside the first chunk pair
    const uint32_t sel = tp ? 0x7632u : 0x5410u;
    // Two look-ahead slots per row; slot s always holds halves of one parity, so its pointer advances by one
    // whole super-block (144 bytes) per use and whether it sees FIRST halves of super-blocks never changes.
    const uint8_t* ps[2][2];      // [slot][row]
    bool first_half[2][2];
    const uint8_t* hp[2];         // header of the super-block whose first half comes next
    uint4 hraw[2];                // ... prefetched
    Q4KHalfScales sc[2][2];       // [slot][row] scales of the half the slot processes next
    uint4 wn[2][2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        int64_t r = min((int64_t)rtile * 16 + g + 8 * i, (int64_t)op.n_rows - 1);
        int64_t hs = ((r * op.k) >> 7) + hb;   // stream index of the first half
        const uint8_t* sb = base + (hs >> 1) * 144;
        const bool par = (hs & 1) != 0;
        ps[0][i] = sb + (par ? 64 : 0) + qoff;
        ps[1][i] = sb + (par ? 144 : 64) + qoff;
        first_half[0][i] = !par;
        first_half[1][i] = par;
        hraw[i] = make_uint4(0, 0, 0, 0);
        if (par) {   // the row starts in the second half of a super-block: its header is needed at once
            Q4KHalfScales unused;
            q4k_decode_hdr(ldg128(sb), sel, unused, sc[0][i]);
            hp[i] = sb + 144;
            if (hb + 1 < he) hraw[i] = ldg128(hp[i]);
        } else {
            hp[i] = sb;
            hraw[i] = ldg128(hp[i]);
        }
        wn[0][i] = ldg128(ps[0][i]);
        wn[1][i] = make_uint4(0, 0, 0, 0);
        if (hb + 1 < he) wn[1][i] = ldg128(ps[1][i]);
    }
    for (int h0 = hb; h0 < he; h0 += 2) {
#pragma unroll
        for (int j2 = 0; j2 < 2; j2++) {
            const int h = h0 + j2;
            if (h < he) {
                uint4 w[2] = {wn[j2][0], wn[j2][1]};
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    if (first_half[j2][i]) {
                        q4k_decode_hdr(hraw[i], sel, sc[j2][i], sc[j2 ^ 1][i]);
                        hp[i] += 144;
                        if (h + 2 < he) hraw[i] = ldg128(hp[i]);
                    }
                    if (h + 2 < he) {
                        ps[j2][i] += 144;
                        wn[j2][i] = ldg128(ps[j2][i]);
                        prefetch_l2(ps[j2][i] + 6 * 144, plim);
                    }
                }
                const uint32_t ML = 0x000F000Fu, MH = 0x00F000F0u;
                const uint32_t w0[4] = {w[0].x, w[0].y, w[0].z, w[0].w};
                const uint32_t w1[4] = {w[1].x, w[1].y, w[1].z, w[1].w};
                uint32_t s0[4], s1[4];
#pragma unroll
                for (int j = 0; j < 4; j++) { s0[j] = w0[j] >> 8; s1[j] = w1[j] >> 8; }
                const int RA = 8 * h + 4 * tp + (t & 1);   // run of the low-nibble weights; high nibbles: RA + 2
#pragma unroll
                for (int n = 0; n < MT; n++) {
                    if (n < m) {
                        uint4 b01, b23;
                        float cA[4], cB[4];
                        load_b(bl, RA * m + n, b01, b23);
                        mma16816_z(cA, w0[0] & ML, w1[0] & ML, s0[0] & ML, s1[0] & ML, b01.x, b01.y);
                        mma16816(cA, w0[1] & ML, w1[1] & ML, s0[1] & ML, s1[1] & ML, b01.z, b01.w);
                        mma16816(cA, w0[2] & ML, w1[2] & ML, s0[2] & ML, s1[2] & ML, b23.x, b23.y);
                        mma16816(cA, w0[3] & ML, w1[3] & ML, s0[3] & ML, s1[3] & ML, b23.z, b23.w);
                        load_b(bl, (RA + 2) * m + n, b01, b23);
                        mma16816_z(cB, w0[0] & MH, w1[0] & MH, s0[0] & MH, s1[0] & MH, b01.x, b01.y);
                        mma16816(cB, w0[1] & MH, w1[1] & MH, s0[1] & MH, s1[1] & MH, b01.z, b01.w);
                        mma16816(cB, w0[2] & MH, w1[2] & MH, s0[2] & MH, s1[2] & MH, b23.x, b23.y);
                        mma16816(cB, w0[3] & MH, w1[3] & MH, s0[3] & MH, s1[3] & MH, b23.z, b23.w);
                        float2 sa = xs.ss[RA * m + n], sb = xs.ss[(RA + 2) * m + n];
#pragma unroll
                        for (int i = 0; i < 2; i++) {
                            float va = cA[2 * i] + cA[2 * i + 1], vb = cB[2 * i] + cB[2 * i + 1];   // hi + lo columns
                            const Q4KHalfScales& q = sc[j2][i];
                            acc[i][n] += va * (q.dA * sa.x) - q.nA * sa.y + vb * (q.dB * sb.x) - q.nB * sb.y;
                        }
                    }
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------------- Q6_K (GGUF)
// Thread (g, t) owns, in every 128-weight half and for rows g and g+8, 16 bytes of ql (32-run a = t>>1 in
// its low nibbles, 32-run a+2 in its high nibbles; 16-weight half lh = t&1 of each) and the matching 16
// bytes of qh: two runs of 16 weights with one int8 scale each. All four planes are linear in the stream
// index of the half, so every pointer advances by a constant per half.
struct Q6KW {
    uint4 ql, qh;
    uint32_t s_lo, s_hi;   // int8 scales of the two runs
    uint32_t d;            // f16 bits
};

struct Q6KPtr {
    const uint8_t *ql, *qh, *sc, *d0;   // d0: d plane; indexed with the block number
    int hs;                             // stream index of the half the pointers address
};

__device__ __forceinline__ Q6KW q6k_load(const Q6KPtr& p) {
    Q6KW w;
    w.ql = ldg128(p.ql);
    w.qh = ldg128(p.qh);
    w.s_lo = ldg8(p.sc);
    w.s_hi = ldg8(p.sc + 4);
    w.d = ldg16(p.d0 + (p.hs >> 1) * 2);
    return w;
}

__device__ __forceinline__ void q6k_advance(Q6KPtr& p) {
    p.ql += 64; p.qh += 32; p.sc += 8; p.hs += 1;
}

template <int MT>
__device__ __forceinline__ void tile_q6k(const GOp& op, int m, int rtile, int hb, int he, const XImg& xs,
                                         const BLane& bl, float (&acc)[2][MT]) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3, a = t >> 1, lh = t & 1;
    if (hb >= he) return;
    Q6KPtr pp[2];
    Q6KW wn[2];   // one half of look-ahead
#pragma unroll
    for (int i = 0; i < 2; i++) {
        int64_t r = min((int64_t)rtile * 16 + g + 8 * i, (int64_t)op.n_rows - 1);
        int64_t hs = ((r * op.k) >> 7) + hb;
        pp[i].ql = op.v.p[0] + hs * 64 + a * 32 + lh * 16;
        pp[i].qh = op.v.p[1] + hs * 32 + lh * 16;
        pp[i].sc = op.v.p[2] + hs * 8 + 2 * a + lh;
        pp[i].d0 = op.v.p[3];
        pp[i].hs = (int)hs;
        wn[i] = q6k_load(pp[i]);
    }
    const int shl = 4 - 2 * a, shr = 2 * a;
    for (int h = hb; h < he; h++) {
        Q6KW w[2] = {wn[0], wn[1]};
        if (h + 1 < he) {
#pragma unroll
            for (int i = 0; i < 2; i++) { q6k_advance(pp[i]); wn[i] = q6k_load(pp[i]); }
        }
        uint32_t aL[2][4][2], aH[2][4][2];   // [row][word][pair] f16x2 codes * 2^-24
        float dL[2], dH[2];
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const uint32_t ql[4] = {w[i].ql.x, w[i].ql.y, w[i].ql.z, w[i].ql.w};
            const uint32_t qh[4] = {w[i].qh.x, w[i].qh.y, w[i].qh.z, w[i].qh.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                uint32_t cl = (ql[j] & 0x0F0F0F0Fu) | ((qh[j] << shl) & 0x30303030u);          // 32-run a
                uint32_t ch = ((ql[j] >> 4) & 0x0F0F0F0Fu) | ((qh[j] >> shr) & 0x30303030u);   // 32-run a+2
                aL[i][j][0] = __byte_perm(cl, 0, 0x4140); aL[i][j][1] = __byte_perm(cl, 0, 0x4342);
                aH[i][j][0] = __byte_perm(ch, 0, 0x4140); aH[i][j][1] = __byte_perm(ch, 0, 0x4342);
            }
            float d24 = __half2float(__ushort_as_half((unsigned short)w[i].d)) * 16777216.0f;
            dL[i] = d24 * (float)(int)(int8_t)w[i].s_lo;   // d * scale * 2^24
            dH[i] = d24 * (float)(int)(int8_t)w[i].s_hi;
        }
        const int RL = 8 * h + 2 * a + lh;   // run of the low-nibble codes; high nibbles: RL + 4
#pragma unroll
        for (int n = 0; n < MT; n++) {
            if (n < m) {
                uint4 b01, b23;
                float cL[4], cH[4];
                load_b(bl, RL * m + n, b01, b23);
                mma16816_z(cL, aL[0][0][0], aL[1][0][0], aL[0][0][1], aL[1][0][1], b01.x, b01.y);
                mma16816(cL, aL[0][1][0], aL[1][1][0], aL[0][1][1], aL[1][1][1], b01.z, b01.w);
                mma16816(cL, aL[0][2][0], aL[1][2][0], aL[0][2][1], aL[1][2][1], b23.x, b23.y);
                mma16816(cL, aL[0][3][0], aL[1][3][0], aL[0][3][1], aL[1][3][1], b23.z, b23.w);
                load_b(bl, (RL + 4) * m + n, b01, b23);
                mma16816_z(cH, aH[0][0][0], aH[1][0][0], aH[0][0][1], aH[1][0][1], b01.x, b01.y);
                mma16816(cH, aH[0][1][0], aH[1][1][0], aH[0][1][1], aH[1][1][1], b01.z, b01.w);
                mma16816(cH, aH[0][2][0], aH[1][2][0], aH[0][2][1], aH[1][2][1], b23.x, b23.y);
                mma16816(cH, aH[0][3][0], aH[1][3][0], aH[0][3][1], aH[1][3][1], b23.z, b23.w);
                float2 sl = xs.ss[RL * m + n], sh = xs.ss[(RL + 4) * m + n];
                const float k32 = 32.0f / 16777216.0f;
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    float vl = cL[2 * i] + cL[2 * i + 1], vh = cH[2 * i] + cH[2 * i + 1];
                    // d * sc * (sum q x - 32 sum x)
                    acc[i][n] += dL[i] * (vl * sl.x - k32 * sl.y) + dH[i] * (vh * sh.x - k32 * sh.y);
                }
            }
        }
    }
}

// --------------------------------------------------------------------------------------------- kernel
template <int MT>
__global__ void __launch_bounds__(256, 2)
gemv_mma_kernel(GOp single, const GOp* __restrict__ ops, int n_ops, const int2* __restrict__ ranges, int total_tiles, int m) {
    extern __shared__ __align__(16) uint8_t smem[];
    float* red = reinterpret_cast<float*>(smem);
    uint8_t* xbase = smem + RED_FLOATS * sizeof(float);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int tb, te;
    if (ranges) {
        int2 rg = ranges[blockIdx.x];
        tb = rg.x; te = rg.y;
    } else {
        tb = (int)(((int64_t)blockIdx.x * total_tiles) / gridDim.x);
        te = (int)(((int64_t)(blockIdx.x + 1) * total_tiles) / gridDim.x);
    }
    int opi = 0, cur = -1;
    if (n_ops > 1) {   // first product whose tile range reaches tb
        int lo = 0, hi = n_ops - 1;
        while (lo < hi) {
            int mid = (lo + hi) >> 1;
            if (ops[mid].tile0 + ops[mid].ntiles <= tb) lo = mid + 1; else hi = mid;
        }
        opi = lo;
    }
    GOp op = single;
    XImg xs{};
    BLane bl{};
    if (threadIdx.x < XZERO_BYTES / 4) reinterpret_cast<uint32_t*>(xbase)[threadIdx.x] = 0u;   // published by the first barrier
    for (int tile = tb; tile < te; tile++) {
        if (n_ops > 1) {
            while (opi < n_ops - 1 && tile >= ops[opi].tile0 + ops[opi].ntiles) opi++;
        }
        if (opi != cur) {
            if (n_ops > 1) op = ops[opi];
            __syncthreads();   // everyone is done with the previous product's activations
            xs = ximg_carve(xbase, op.k, m);
            bl = blane_make(xs, xbase, lane >> 2, lane & 3);
            if (op.fmt == F_Q4K) prep_x<true>(op.x, op.ldx, op.k, m, xs);
            else prep_x<false>(op.x, op.ldx, op.k, m, xs);
            __syncthreads();
            cur = opi;
        }
        const int kw = 1 << op.kw_log2;
        const int rtile = (tile - op.tile0) * (8 >> op.kw_log2) + (warp >> op.kw_log2);
        const int kpart = warp & (kw - 1);
        float acc[2][MT];
#pragma unroll
        for (int n = 0; n < MT; n++) { acc[0][n] = 0.f; acc[1][n] = 0.f; }
        const bool live = (int64_t)rtile * 16 < op.n_rows;
        if (live) {
            int nh = op.k >> 7, per = (nh + kw - 1) >> op.kw_log2;
            int hb = kpart * per, he = min(nh, (kpart + 1) * per);
            if (op.fmt == F_Q4K) tile_q4k<MT>(op, m, rtile, hb, he, xs, bl, acc);
            else tile_q6k<MT>(op, m, rtile, hb, he, xs, bl, acc);
        }
        // the four threads of a quad hold partial sums of the same two rows
#pragma unroll
        for (int n = 0; n < MT; n++) {
#pragma unroll
            for (int i = 0; i < 2; i++) {
                float s = acc[i][n];
                s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
                s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);
                acc[i][n] = s;
            }
        }
        const int g = lane >> 2, t = lane & 3;
        if (kw > 1) {
            if (t == 0) {
#pragma unroll
                for (int n = 0; n < MT; n++) {
                    red[(warp * 16 + g) * MT + n] = acc[0][n];
                    red[(warp * 16 + g + 8) * MT + n] = acc[1][n];
                }
            }
            __syncthreads();
            if (kpart == 0 && live) {
                for (int o = lane; o < 16 * MT; o += 32) {
                    int r = o / MT, n = o - r * MT;
                    float s = 0.f;
                    for (int j = 0; j < kw; j++) s += red[((warp + j) * 16 + r) * MT + n];
                    int64_t row = (int64_t)rtile * 16 + r;
                    if (row < op.n_rows && n < m) op.y[(int64_t)n * op.ldy + row] = s;
                }
            }
            __syncthreads();   // the reduction buffer is free again
        } else if (live && t == 0) {
#pragma unroll
            for (int n = 0; n < MT; n++) {
                if (n < m) {
#pragma unroll
                    for (int i = 0; i < 2; i++) {
                        int64_t row = (int64_t)rtile * 16 + g + 8 * i;
                        if (row < op.n_rows) op.y[(int64_t)n * op.ldy + row] = acc[i][n];
                    }
                }
            }
        }
    }
}

}  // namespace

size_t gemv_mma_smem_bytes(int fmt, int k, int m) {
    (void)fmt;
    return RED_FLOATS * sizeof(float) + XZERO_BYTES + (size_t)(k >> 4) * m * (64 + sizeof(float2)) + 16;
}

bool gemv_mma_supported(const b200q_weight* w, int m) {
    if (w->orient != B200Q_ORIENT_NK || m < 1 || m > 8) return false;
    if (w->n_local > 0x7FFFFFF0ll || w->k > (1 << 24) || w->n_elements >= (1ll << 37)) return false;
    if (w->fmt != F_Q4K && w->fmt != F_Q6K) return false;
    if (w->k % 128) return false;
    return gemv_mma_smem_bytes(w->fmt, (int)w->k, m) <= 200 * 1024;
}

void gemv_mma_plan(GOp* op, bool few_tiles) {
    // Fewest k-parts (most work per warp, no cross-warp reduction) that still give the launch enough CTA
    // tiles; a warp never gets less than two 128-weight halves when k allows it.
    const int units = op->k / 128;
    const int row_tiles = (op->n_rows + 15) / 16;
    const int want_tiles = few_tiles ? 4 * 148 : 1;
    int kw_log2 = 0;
    while (kw_log2 < 3 && (row_tiles * (1 << kw_log2) + 7) / 8 < want_tiles && units / (2 << kw_log2) >= 2) kw_log2++;
    // very long rows: keep a CTA tile under ~160 KB of packed weights so tiles stay balanceable
    FmtInfo I = fmt_info(op->fmt);
    const double row_bytes = (double)op->k * I.block_bytes / I.block_elems;
    while (kw_log2 < 3 && (8 >> kw_log2) * 16 * row_bytes > 160.0 * 1024 && units / (2 << kw_log2) >= 2) kw_log2++;
    while (kw_log2 > 0 && (1 << kw_log2) > units) kw_log2--;
    op->kw_log2 = kw_log2;
    const int rt = 8 >> kw_log2;
    op->ntiles = (row_tiles + rt - 1) / rt;
}

int launch_gemv_mma(b200q_ctx* ctx, const GOp* h_single, const GOp* d_ops, int n_ops, const int2* d_ranges, int n_ctas,
                    int total_tiles, int m, size_t smem_bytes) {
    if (total_tiles <= 0) return B200Q_OK;
    static bool configured[64][4] = {};
    const int mi = m <= 1 ? 0 : m <= 2 ? 1 : m <= 4 ? 2 : 3;
    const int smem_cap = 200 * 1024 + 8192;
    if (!configured[ctx->device & 63][mi]) {
        cudaError_t e = cudaSuccess;
        switch (mi) {
            case 0: e = cudaFuncSetAttribute(gemv_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_cap); break;
            case 1: e = cudaFuncSetAttribute(gemv_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_cap); break;
            case 2: e = cudaFuncSetAttribute(gemv_mma_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_cap); break;
            default: e = cudaFuncSetAttribute(gemv_mma_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_cap); break;
        }
        B200Q_CUDA(e, B200Q_ERR_LAUNCH);
        configured[ctx->device & 63][mi] = true;
    }
    GOp single{};
    if (h_single) single = *h_single;
    switch (mi) {
        case 0: gemv_mma_kernel<1><<<n_ctas, 256, smem_bytes, ctx->stream>>>(single, d_ops, n_ops, d_ranges, total_tiles, m); break;
        case 1: gemv_mma_kernel<2><<<n_ctas, 256, smem_bytes, ctx->stream>>>(single, d_ops, n_ops, d_ranges, total_tiles, m); break;
        case 2: gemv_mma_kernel<4><<<n_ctas, 256, smem_bytes, ctx->stream>>>(single, d_ops, n_ops, d_ranges, total_tiles, m); break;
        default: gemv_mma_kernel<8><<<n_ctas, 256, smem_bytes, ctx->stream>>>(single, d_ops, n_ops, d_ranges, total_tiles, m); break;
    }
    B200Q_CUDA(cudaGetLastError(), B200Q_ERR_LAUNCH);
    return B200Q_OK;
}

}  // namespace b200q
