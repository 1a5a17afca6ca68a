// Grouped decode kernel: fused dequant + matmul for 1..8 activation rows, HBM-bound.
//
// Replaces the per-row-block scalar kernels of the reference (kernels/q4_k_matmul.hip:216,
// q6_k_matmul.hip:216: one thread block per ACTIVATION row, one 4-bit code per inner iteration) and the
// serial per-op loop of BatchQuantizedMatmul::process_batch (src/ggml/hip_backend/ops/batch_quantized.rs:147-161).
//
// Design. Streaming 4.5-bit weights at HBM speed leaves ~1 integer instruction per weight, which rules out
// converting every code to fp32 on the CUDA cores. Instead the raw integer codes are fed to the tensor
// cores as f16 SUBNORMALS: a 4- or 6-bit code q masked into the low bits of an f16 lane is the number
// q * 2^-24 (q * 2^-20 for a nibble left in bits 4..7), exactly. One mma.sync.m16n8k16 then multiplies 16
// weight rows x 16 codes with up to 8 activation rows; the block scale (d * sc, an exact fp32 product) and
// the 2^24 are applied to the fp32 accumulator afterwards, once per 16/32-weight scale group, and the
// "- dmin * m" / "- 32" offsets become one FMA with the pre-computed sum of the activations of that group.
// Activations are split into f16 hi + lo parts (x = s * (hi + lo), s a per-group power of two), so the
// products carry 22 mantissa bits and accumulate in fp32: the result stays within 1e-4 of the fp32 oracle.
//
// Work decomposition. A CTA tile is (8 >> kw_log2) tiles of 16 weight rows x the whole k, the 8 warps of
// the CTA being arranged as row-tiles x k-parts; partial sums of the k-parts meet in shared memory. A
// launch covers any number of products (a whole decode step): CTAs are persistent and own a contiguous
// range of CTA tiles balanced by bytes, so each CTA prepares the activations of only the products it
// touches. Weight loads are software-pipelined 4 chunks deep in registers.
#include <cuda_fp16.h>

#include "gemv_mma.cuh"

namespace b200q {

namespace {

constexpr int F_Q4K = fmt_of(Q4_K, GGUF);
constexpr int F_Q6K = fmt_of(Q6_K, GGUF);

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg128(const uint8_t* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ uint2 ldg64(const uint8_t* p) { return __ldg(reinterpret_cast<const uint2*>(p)); }
__device__ __forceinline__ uint32_t ldg32(const uint8_t* p) { return __ldg(reinterpret_cast<const uint32_t*>(p)); }
__device__ __forceinline__ uint32_t ldg16(const uint8_t* p) { return __ldg(reinterpret_cast<const uint16_t*>(p)); }

// Shared-memory image of one product's activations.
//   hi / lo : per x-group (4*EPT weights), activation row n and quad lane t: EPT f16 values, in the order
//             the MMA B fragments want them
//   ss      : per x-group and row: {2^e scale of the group, sum of the fp32 activations of the group}
struct XSmem {
    uint8_t* hi;
    uint8_t* lo;
    float2* ss;
};

template <int EPT>
__device__ __forceinline__ XSmem xsmem_carve(uint8_t* base, int k, int m) {
    int nxg = k / (4 * EPT);
    size_t frag = (size_t)nxg * m * 4 * EPT * 2;
    XSmem s;
    s.hi = base;
    s.lo = base + frag;
    s.ss = reinterpret_cast<float2*>(base + 2 * frag);
    return s;
}

// Converts x[m, k] (fp32, global) into the hi/lo fragment image. One quad of threads per (x-group, row).
template <int EPT, bool PERM>
__device__ __forceinline__ void prep_x(const float* __restrict__ x, int64_t ldx, int k, int m, const XSmem& s) {
    const int nq = (k / (4 * EPT)) * m;
    const int t = threadIdx.x & 3;
    for (int base = 0; base < nq; base += (int)(blockDim.x >> 2)) {
        int q = base + (int)(threadIdx.x >> 2);
        bool valid = q < nq;
        int qq = valid ? q : 0;
        int G = qq / m, n = qq - G * m;
        const float* xp = x + (int64_t)n * ldx + (int64_t)G * 4 * EPT + t * EPT;
        float v[EPT];
#pragma unroll
        for (int i = 0; i < EPT; i += 4) {
            float4 f = __ldg(reinterpret_cast<const float4*>(xp + i));
            v[i] = f.x; v[i + 1] = f.y; v[i + 2] = f.z; v[i + 3] = f.w;
        }
        float mx = 0.0f, sum = 0.0f;
#pragma unroll
        for (int i = 0; i < EPT; i++) { mx = fmaxf(mx, fabsf(v[i])); sum += v[i]; }
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
        // power-of-two normalisation of the group so the f16 split never overflows or underflows badly
        int e = (int)((__float_as_uint(mx) >> 23) & 255u);
        e = mx == 0.0f ? 127 : min(max(e, 1), 253);
        float sdown = __uint_as_float((uint32_t)(254 - e) << 23);
        float sup = __uint_as_float((uint32_t)e << 23);
        __align__(16) __half h[EPT], l[EPT];
#pragma unroll
        for (int i = 0; i < EPT; i++) {
            float xs = v[i] * sdown;
            h[i] = __float2half_rn(xs);
            l[i] = __float2half_rn(xs - __half2float(h[i]));
        }
        if (valid) {
            size_t idx = ((size_t)qq * 4 + t);
            if constexpr (EPT == 8) {
                // order e0,e2,e1,e3,e4,e6,e5,e7: the pairs the nibble masks (bytes 0/2, bytes 1/3) produce
                constexpr int P[8] = {0, 2, 1, 3, 4, 6, 5, 7};
                __align__(16) __half hp[8], lp[8];
#pragma unroll
                for (int i = 0; i < 8; i++) { hp[i] = h[PERM ? P[i] : i]; lp[i] = l[PERM ? P[i] : i]; }
                reinterpret_cast<uint4*>(s.hi)[idx] = *reinterpret_cast<uint4*>(hp);
                reinterpret_cast<uint4*>(s.lo)[idx] = *reinterpret_cast<uint4*>(lp);
            } else {
                reinterpret_cast<uint2*>(s.hi)[idx] = *reinterpret_cast<uint2*>(h);
                reinterpret_cast<uint2*>(s.lo)[idx] = *reinterpret_cast<uint2*>(l);
            }
            if (t == 0) s.ss[qq] = make_float2(sup, sum);
        }
    }
}

// ------------------------------------------------------------------------------------------- Q4_K (GGUF)
// Decoded super-block header of one weight row: d * 2^20, dmin and the eight 6-bit scales / mins as bytes.
struct Q4KHdr {
    float d20, dmin;
    uint32_t sc_lo, sc_hi, m_lo, m_hi;
};

__device__ __forceinline__ Q4KHdr q4k_decode_hdr(uint4 h) {
    Q4KHdr r;
    r.d20 = __half2float(__ushort_as_half((unsigned short)(h.x & 0xFFFFu))) * 1048576.0f;
    r.dmin = __half2float(__ushort_as_half((unsigned short)(h.x >> 16)));
    r.sc_lo = h.y & 0x3F3F3F3Fu;
    r.m_lo = h.z & 0x3F3F3F3Fu;
    r.sc_hi = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
    r.m_hi = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
    return r;
}

// One 16-row tile x chunk range [cb, ce) of 64-weight chunks. acc: rows (g, g+8) x activation rows (2t, 2t+1).
__device__ __forceinline__ void tile_q4k(const GOp& op, int m, int rtile, int cb, int ce, const XSmem& xs, float (&acc)[4]) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const uint8_t* base = op.v.p[0];
    int64_t r[2];
    r[0] = min((int64_t)rtile * 16 + g, (int64_t)op.n_rows - 1);
    r[1] = min((int64_t)rtile * 16 + g + 8, (int64_t)op.n_rows - 1);
    int64_t ci[2] = {(r[0] * op.k) >> 6, (r[1] * op.k) >> 6};   // index of the row's first chunk in the stream
    Q4KHdr cur[2];
    uint4 nxt[2];
    uint2 wb[4][2];
    if (cb >= ce) return;
#pragma unroll
    for (int i = 0; i < 2; i++) {
        cur[i] = q4k_decode_hdr(ldg128(base + ((ci[i] + cb) >> 2) * 144));
        nxt[i] = make_uint4(0, 0, 0, 0);
    }
    auto load_w = [&](int c, int i) -> uint2 {
        int64_t s = ci[i] + c;
        return ldg64(base + (s >> 2) * 144 + 16 + (int)(s & 3) * 32 + t * 8);
    };
#pragma unroll
    for (int j = 0; j < 4; j++)
        if (cb + j < ce) { wb[j][0] = load_w(cb + j, 0); wb[j][1] = load_w(cb + j, 1); }

    const uint4* xhi = reinterpret_cast<const uint4*>(xs.hi);
    const uint4* xlo = reinterpret_cast<const uint4*>(xs.lo);
    const bool have_b = g < m;
    const int tok0 = 2 * t, tok1 = 2 * t + 1;

    for (int c0 = cb; c0 < ce; c0 += 4) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int c = c0 + j;
            if (c < ce) {
                uint2 w[2] = {wb[j][0], wb[j][1]};
                if (c + 4 < ce) { wb[j][0] = load_w(c + 4, 0); wb[j][1] = load_w(c + 4, 1); }
                int cc[2];
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    int64_t s = ci[i] + c;
                    cc[i] = (int)(s & 3);
                    if (cc[i] == 0 && c != cb) cur[i] = q4k_decode_hdr(nxt[i]);
                    if (cc[i] == 0 || c == cb) {
                        // prefetch the header of the following super-block if this warp will reach it
                        int64_t nsb = (s >> 2) + 1;
                        if (nsb * 4 - ci[i] < ce) nxt[i] = ldg128(base + nsb * 144);
                    }
                }
                // B fragments of the two 32-weight groups of this chunk
                uint4 bhA = make_uint4(0, 0, 0, 0), blA = bhA, bhB = bhA, blB = bhA;
                if (have_b) {
                    size_t ia = ((size_t)(2 * c) * m + g) * 4 + t, ib = ((size_t)(2 * c + 1) * m + g) * 4 + t;
                    bhA = xhi[ia]; blA = xlo[ia]; bhB = xhi[ib]; blB = xlo[ib];
                }
                float cA[4] = {0.f, 0.f, 0.f, 0.f}, cB[4] = {0.f, 0.f, 0.f, 0.f};
                {
                    // low nibbles -> sub-block 2cc (codes * 2^-24), high nibbles -> sub-block 2cc+1 (codes * 2^-20)
                    uint32_t x0 = w[0].x, x1 = w[1].x, y0 = w[0].y, y1 = w[1].y;
                    uint32_t x0s = x0 >> 8, x1s = x1 >> 8, y0s = y0 >> 8, y1s = y1 >> 8;
                    const uint32_t ML = 0x000F000Fu, MH = 0x00F000F0u;
                    mma16816(cA, x0 & ML, x1 & ML, x0s & ML, x1s & ML, bhA.x, bhA.y);
                    mma16816(cA, y0 & ML, y1 & ML, y0s & ML, y1s & ML, bhA.z, bhA.w);
                    mma16816(cA, x0 & ML, x1 & ML, x0s & ML, x1s & ML, blA.x, blA.y);
                    mma16816(cA, y0 & ML, y1 & ML, y0s & ML, y1s & ML, blA.z, blA.w);
                    mma16816(cB, x0 & MH, x1 & MH, x0s & MH, x1s & MH, bhB.x, bhB.y);
                    mma16816(cB, y0 & MH, y1 & MH, y0s & MH, y1s & MH, bhB.z, bhB.w);
                    mma16816(cB, x0 & MH, x1 & MH, x0s & MH, x1s & MH, blB.x, blB.y);
                    mma16816(cB, y0 & MH, y1 & MH, y0s & MH, y1s & MH, blB.z, blB.w);
                }
                // scales of the activations (2^e, sum) for the activation rows this thread accumulates
                float2 sA0 = make_float2(0.f, 0.f), sA1 = sA0, sB0 = sA0, sB1 = sA0;
                if (tok0 < m) { sA0 = xs.ss[(size_t)(2 * c) * m + tok0]; sB0 = xs.ss[(size_t)(2 * c + 1) * m + tok0]; }
                if (tok1 < m) { sA1 = xs.ss[(size_t)(2 * c) * m + tok1]; sB1 = xs.ss[(size_t)(2 * c + 1) * m + tok1]; }
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    uint32_t scw = cc[i] < 2 ? cur[i].sc_lo : cur[i].sc_hi;
                    uint32_t mw = cc[i] < 2 ? cur[i].m_lo : cur[i].m_hi;
                    int sh = (cc[i] & 1) * 16;
                    float scA = (float)((scw >> sh) & 0xFFu), scB = (float)((scw >> (sh + 8)) & 0xFFu);
                    float mA = (float)((mw >> sh) & 0xFFu), mB = (float)((mw >> (sh + 8)) & 0xFFu);
                    float dA = cur[i].d20 * 16.0f * scA;   // d * sc * 2^24
                    float dB = cur[i].d20 * scB;           // d * sc * 2^20
                    float nA = cur[i].dmin * mA, nB = cur[i].dmin * mB;
                    acc[2 * i] += cA[2 * i] * (dA * sA0.x) - nA * sA0.y + cB[2 * i] * (dB * sB0.x) - nB * sB0.y;
                    acc[2 * i + 1] += cA[2 * i + 1] * (dA * sA1.x) - nA * sA1.y + cB[2 * i + 1] * (dB * sB1.x) - nB * sB1.y;
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------------- Q6_K (GGUF)
struct Q6KUnit {      // the bytes one thread needs of one 128-weight half of one row
    uint32_t ql[4];   // [a*2 + lh]: ql word at a*32 + lh*16 + 4t
    uint32_t qh[2];   // [lh]
    uint2 sc;         // 8 int8 scales of the half
    uint32_t d;       // f16 bits
};

__device__ __forceinline__ Q6KUnit q6k_load(const WView& v, int64_t unit, int t) {
    int64_t blk = unit >> 1;
    int half = (int)(unit & 1);
    const uint8_t* ql = v.p[0] + blk * 128 + half * 64 + 4 * t;
    const uint8_t* qh = v.p[1] + blk * 64 + half * 32 + 4 * t;
    Q6KUnit u;
    u.ql[0] = ldg32(ql); u.ql[1] = ldg32(ql + 16); u.ql[2] = ldg32(ql + 32); u.ql[3] = ldg32(ql + 48);
    u.qh[0] = ldg32(qh); u.qh[1] = ldg32(qh + 16);
    u.sc = ldg64(v.p[2] + blk * 16 + half * 8);
    u.d = ldg16(v.p[3] + blk * 2);
    return u;
}

__device__ __forceinline__ void tile_q6k(const GOp& op, int m, int rtile, int ub, int ue, const XSmem& xs, float (&acc)[4]) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    int64_t r[2];
    r[0] = min((int64_t)rtile * 16 + g, (int64_t)op.n_rows - 1);
    r[1] = min((int64_t)rtile * 16 + g + 8, (int64_t)op.n_rows - 1);
    int64_t ui[2] = {(r[0] * op.k) >> 7, (r[1] * op.k) >> 7};
    if (ub >= ue) return;
    Q6KUnit nb[2][2];
#pragma unroll
    for (int j = 0; j < 2; j++)
        if (ub + j < ue) { nb[j][0] = q6k_load(op.v, ui[0] + ub + j, t); nb[j][1] = q6k_load(op.v, ui[1] + ub + j, t); }
    const uint2* xhi = reinterpret_cast<const uint2*>(xs.hi);
    const uint2* xlo = reinterpret_cast<const uint2*>(xs.lo);
    const bool have_b = g < m;
    const int tok0 = 2 * t, tok1 = 2 * t + 1;
    for (int u0 = ub; u0 < ue; u0 += 2) {
#pragma unroll
        for (int j = 0; j < 2; j++) {
            int u = u0 + j;
            if (u < ue) {
                Q6KUnit w[2] = {nb[j][0], nb[j][1]};
                if (u + 2 < ue) { nb[j][0] = q6k_load(op.v, ui[0] + u + 2, t); nb[j][1] = q6k_load(op.v, ui[1] + u + 2, t); }
                float d24[2];
#pragma unroll
                for (int i = 0; i < 2; i++)
                    d24[i] = __half2float(__ushort_as_half((unsigned short)w[i].d)) * 16777216.0f;
#pragma unroll
                for (int gg = 0; gg < 4; gg++) {
#pragma unroll
                    for (int lh = 0; lh < 2; lh++) {
                        const int s = 2 * gg + lh;                 // scale group inside the half
                        uint32_t c4[2];
#pragma unroll
                        for (int i = 0; i < 2; i++) {
                            uint32_t qlw = w[i].ql[(gg & 1) * 2 + lh], qhw = w[i].qh[lh];
                            uint32_t lo4 = gg < 2 ? (qlw & 0x0F0F0F0Fu) : ((qlw >> 4) & 0x0F0F0F0Fu);
                            uint32_t hs = gg == 0 ? (qhw << 4) : gg == 1 ? (qhw << 2) : gg == 2 ? qhw : (qhw >> 2);
                            c4[i] = lo4 | (hs & 0x30303030u);      // four 6-bit codes, one per byte
                        }
                        // bytes -> f16 lanes (code * 2^-24): (b0,b1) and (b2,b3)
                        uint32_t a0 = __byte_perm(c4[0], 0, 0x4140), a2 = __byte_perm(c4[0], 0, 0x4342);
                        uint32_t a1 = __byte_perm(c4[1], 0, 0x4140), a3 = __byte_perm(c4[1], 0, 0x4342);
                        size_t xg = (size_t)u * 8 + s;
                        uint2 bh = make_uint2(0, 0), bl = bh;
                        if (have_b) { size_t ix = (xg * m + g) * 4 + t; bh = xhi[ix]; bl = xlo[ix]; }
                        float c[4] = {0.f, 0.f, 0.f, 0.f};
                        mma16816(c, a0, a1, a2, a3, bh.x, bh.y);
                        mma16816(c, a0, a1, a2, a3, bl.x, bl.y);
                        float2 s0 = make_float2(0.f, 0.f), s1 = s0;
                        if (tok0 < m) s0 = xs.ss[xg * m + tok0];
                        if (tok1 < m) s1 = xs.ss[xg * m + tok1];
#pragma unroll
                        for (int i = 0; i < 2; i++) {
                            uint32_t scw = s < 4 ? w[i].sc.x : w[i].sc.y;
                            float sc = (float)(int)(int8_t)((scw >> (8 * (s & 3))) & 0xFFu);
                            float ds = d24[i] * sc;                     // d * scale * 2^24
                            float off = ds * (32.0f / 16777216.0f);     // 32 * d * scale
                            acc[2 * i] += c[2 * i] * (ds * s0.x) - off * s0.y;
                            acc[2 * i + 1] += c[2 * i + 1] * (ds * s1.x) - off * s1.y;
                        }
                    }
                }
            }
        }
    }
}

// --------------------------------------------------------------------------------------------- kernel
__global__ void __launch_bounds__(256, 2)
gemv_mma_kernel(GOp single, const GOp* __restrict__ ops, int n_ops, const int2* __restrict__ ranges, int total_tiles, int m) {
    extern __shared__ __align__(16) uint8_t smem[];
    float* red = reinterpret_cast<float*>(smem);          // 8 warps x 32 lanes x 4 partial sums
    uint8_t* xbase = smem + 8 * 32 * 4 * sizeof(float);
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
    XSmem xs{};
    for (int tile = tb; tile < te; tile++) {
        if (n_ops > 1) {
            while (opi < n_ops - 1 && tile >= ops[opi].tile0 + ops[opi].ntiles) opi++;
        }
        if (opi != cur) {
            if (n_ops > 1) op = ops[opi];
            __syncthreads();   // everyone is done with the previous product's activations
            if (op.fmt == F_Q4K) {
                xs = xsmem_carve<8>(xbase, op.k, m);
                prep_x<8, true>(op.x, op.ldx, op.k, m, xs);
            } else {
                xs = xsmem_carve<4>(xbase, op.k, m);
                prep_x<4, false>(op.x, op.ldx, op.k, m, xs);
            }
            __syncthreads();
            cur = opi;
        }
        const int kw = 1 << op.kw_log2;
        const int rtile = (tile - op.tile0) * (8 >> op.kw_log2) + (warp >> op.kw_log2);
        const int kpart = warp & (kw - 1);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        const bool live = (int64_t)rtile * 16 < op.n_rows;
        if (live) {
            if (op.fmt == F_Q4K) {
                int n = op.k >> 6, per = (n + kw - 1) >> op.kw_log2;
                tile_q4k(op, m, rtile, kpart * per, min(n, (kpart + 1) * per), xs, acc);
            } else {
                int n = op.k >> 7, per = (n + kw - 1) >> op.kw_log2;
                tile_q6k(op, m, rtile, kpart * per, min(n, (kpart + 1) * per), xs, acc);
            }
        }
        if (kw > 1) {
            if (kpart != 0) {
                float4* dst = reinterpret_cast<float4*>(red) + warp * 32 + lane;
                *dst = make_float4(acc[0], acc[1], acc[2], acc[3]);
            }
            __syncthreads();
            if (kpart == 0) {
                for (int j = 1; j < kw; j++) {
                    float4 p = reinterpret_cast<const float4*>(red)[(warp + j) * 32 + lane];
                    acc[0] += p.x; acc[1] += p.y; acc[2] += p.z; acc[3] += p.w;
                }
            }
        }
        if (kpart == 0 && live) {
            const int g = lane >> 2, t = lane & 3;
#pragma unroll
            for (int i = 0; i < 2; i++) {
                int64_t row = (int64_t)rtile * 16 + g + 8 * i;
                if (row < op.n_rows) {
                    if (2 * t < m) op.y[(int64_t)(2 * t) * op.ldy + row] = acc[2 * i];
                    if (2 * t + 1 < m) op.y[(int64_t)(2 * t + 1) * op.ldy + row] = acc[2 * i + 1];
                }
            }
        }
        if (kw > 1) __syncthreads();   // the reduction buffer is free again
    }
}

}  // namespace

bool gemv_mma_supported(const b200q_weight* w, int m) {
    if (w->orient != B200Q_ORIENT_NK || m < 1 || m > 8) return false;
    if (w->n_local > 0x7FFFFFF0ll || w->k > (1 << 24)) return false;
    if (w->fmt == F_Q4K) { if (w->k % 64) return false; }
    else if (w->fmt == F_Q6K) { if (w->k % 128) return false; }
    else return false;
    return gemv_mma_smem_bytes(w->fmt, (int)w->k, m) <= 200 * 1024;
}

size_t gemv_mma_smem_bytes(int fmt, int k, int m) {
    int ept = fmt == F_Q4K ? 8 : 4;
    size_t nxg = (size_t)k / (4 * ept);
    return 8 * 32 * 4 * sizeof(float) + 2 * nxg * m * 4 * ept * 2 + nxg * m * sizeof(float2) + 16;
}

void gemv_mma_plan(GOp* op, bool few_tiles) {
    FmtInfo I = fmt_info(op->fmt);
    double row_bytes = (double)op->k * I.block_bytes / I.block_elems;
    int units = op->fmt == F_Q4K ? op->k / 64 : op->k / 128;
    // aim at ~48 KB of packed weights per CTA tile, at least one k-unit per warp
    int rt = 8;
    while (rt > 1 && rt * 16 * row_bytes > 48.0 * 1024) rt >>= 1;
    int row_tiles = (op->n_rows + 15) / 16;
    if (few_tiles) {
        while (rt > 1 && (row_tiles + rt - 1) / rt < 2 * 148) rt >>= 1;
    }
    while (rt < 8 && (8 / rt) > units) rt <<= 1;
    int kw_log2 = 0;
    while ((8 >> kw_log2) > rt) kw_log2++;
    op->kw_log2 = kw_log2;
    op->ntiles = (row_tiles + rt - 1) / rt;
}

int launch_gemv_mma(b200q_ctx* ctx, const GOp* h_single, const GOp* d_ops, int n_ops, const int2* d_ranges, int n_ctas,
                    int total_tiles, int m, size_t smem_bytes) {
    if (total_tiles <= 0) return B200Q_OK;
    static size_t configured[64] = {0};
    if (smem_bytes > configured[ctx->device & 63]) {
        B200Q_CUDA(cudaFuncSetAttribute(gemv_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(200 * 1024 + 8192)),
                   B200Q_ERR_LAUNCH);
        configured[ctx->device & 63] = 200 * 1024 + 8192;
    }
    GOp single{};
    if (h_single) single = *h_single;
    gemv_mma_kernel<<<n_ctas, 256, smem_bytes, ctx->stream>>>(single, d_ops, n_ops, d_ranges, total_tiles, m);
    B200Q_CUDA(cudaGetLastError(), B200Q_ERR_LAUNCH);
    return B200Q_OK;
}

}  // namespace b200q
