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
// by bytes, so each CTA prepares the activations of only the products it touches. Weights reach the warps
// through per-warp cp.async rings in shared memory (see "weight streaming" below).
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

// ------------------------------------------------------------------------------------ weight streaming
// Every warp streams its weights through a private ring in shared memory filled with cp.async (16 bytes
// per thread and copy), `ring_d` items deep. An item is one 128-weight half of the warp's 16 rows; the
// producer cursor runs ring_d items ahead of the consumer over a FLAT stream of (tile, half) items, so the
// prefetch crosses tile boundaries and no load latency is exposed when a warp starts a new tile. No
// registers are held for look-ahead. Slot layout (per warp): [row g / g+8][piece 0/1][lane] x 16 B of codes,
// then [row][quad] x 16 B of block header written by the quad's first lane.
constexpr int RING_DATA_BYTES = 2 * 2 * 32 * 16;
constexpr int RING_HDR_BYTES = 2 * 8 * 16;
constexpr int RING_SLOT_BYTES = RING_DATA_BYTES + RING_HDR_BYTES;   // 2304

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_wait_keep(int keep) {   // wait until at most `keep` groups are pending
    if (keep >= 3) asm volatile("cp.async.wait_group 3;" ::: "memory");
    else asm volatile("cp.async.wait_group 1;" ::: "memory");
}

// ---- Q4_K: thread (g, t) owns, in every half and for rows g and g+8, bytes [16*(t&1), +16) of chunk (t>>1):
// 16 weights of a low-nibble sub-block and 16 of the high-nibble sub-block.
struct Q4KCursor {
    const uint8_t* p;   // this thread's 16 bytes of the half the cursor is on
    bool second;        // the half is the second half of its super-block
};

__device__ __forceinline__ Q4KCursor q4k_cursor(const GOp& op, int64_t row, int h, int qoff) {
    int64_t hs = ((row * op.k) >> 7) + h;
    Q4KCursor c;
    c.second = (hs & 1) != 0;
    c.p = op.v.p[0] + (hs >> 1) * 144 + (c.second ? 64 : 0) + qoff;
    return c;
}
// copies the cursor's half (and the super-block header, by the quad's first lane, when the consumer will
// need it: first half of a super-block or first item of a tile) into ring slot `slot`, row index i
__device__ __forceinline__ void q4k_issue(Q4KCursor& c, uint32_t slot, int i, int lane, bool tile_start) {
    cp_async16(slot + (i * 2) * 512 + lane * 16, c.p);
    if ((lane & 3) == 0 && (tile_start || !c.second))
        cp_async16(slot + RING_DATA_BYTES + (i * 8 + (lane >> 2)) * 16, c.p - 16 - (c.second ? 64 : 0));
    c.p += c.second ? 80 : 64;
    c.second = !c.second;
}

// ---- Q6_K: thread (g, t) owns 16 bytes of ql (32-run a = t>>1 in the low nibbles, a+2 in the high nibbles,
// 16-weight half lh = t&1 of each) and the matching 16 bytes of qh; header = 8 int8 scales + the f16 d pair.
struct Q6KCursor {
    const uint8_t *ql, *qh, *sc;
    int hs;
};

__device__ __forceinline__ Q6KCursor q6k_cursor(const GOp& op, int64_t row, int h, int t) {
    int64_t hs = ((row * op.k) >> 7) + h;
    Q6KCursor c;
    c.ql = op.v.p[0] + hs * 64 + (t >> 1) * 32 + (t & 1) * 16;
    c.qh = op.v.p[1] + hs * 32 + (t & 1) * 16;
    c.sc = op.v.p[2] + hs * 8;
    c.hs = (int)hs;
    return c;
}
__device__ __forceinline__ void q6k_issue(Q6KCursor& c, const uint8_t* dplane, uint32_t slot, int i, int lane) {
    cp_async16(slot + (i * 2) * 512 + lane * 16, c.ql);
    cp_async16(slot + (i * 2 + 1) * 512 + lane * 16, c.qh);
    if ((lane & 3) == 0) {
        uint32_t h = slot + RING_DATA_BYTES + (i * 8 + (lane >> 2)) * 16;
        cp_async8(h, c.sc);
        cp_async4(h + 8, dplane + ((c.hs >> 2) << 2));   // the 4 aligned bytes holding d of this block pair
    }
    c.ql += 64; c.qh += 32; c.sc += 8; c.hs += 1;
}

// ---------------------------------------------------------------------------------------------- kernel
template <int MT>
__global__ void __launch_bounds__(256, 2)
gemv_mma_kernel(GOp single, const GOp* __restrict__ ops, int n_ops, const int2* __restrict__ ranges, int total_tiles, int m,
                int ring_d) {
    extern __shared__ __align__(16) uint8_t smem[];
    float* red = reinterpret_cast<float*>(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3, tp = t >> 1;
    uint8_t* ring_gen = smem + RED_FLOATS * sizeof(float) + warp * ring_d * RING_SLOT_BYTES;
    const uint32_t ring = smem_addr(ring_gen);
    uint8_t* xbase = smem + RED_FLOATS * sizeof(float) + 8 * ring_d * RING_SLOT_BYTES;
    int tb, te;
    if (ranges) {
        int2 rg = ranges[blockIdx.x];
        tb = rg.x; te = rg.y;
    } else {
        tb = (int)(((int64_t)blockIdx.x * total_tiles) / gridDim.x);
        te = (int)(((int64_t)(blockIdx.x + 1) * total_tiles) / gridDim.x);
    }
    int opi = 0;
    if (n_ops > 1) {   // first product whose tile range reaches tb
        int lo = 0, hi = n_ops - 1;
        while (lo < hi) {
            int mid = (lo + hi) >> 1;
            if (ops[mid].tile0 + ops[mid].ntiles <= tb) lo = mid + 1; else hi = mid;
        }
        opi = lo;
    }
    if (threadIdx.x < XZERO_BYTES / 4) reinterpret_cast<uint32_t*>(xbase)[threadIdx.x] = 0u;   // published by the first barrier
    const int qoff = 16 + tp * 32 + (t & 1) * 16;        // Q4_K: this thread's 16 bytes inside the first chunk pair
    const uint32_t sel = tp ? 0x7632u : 0x5410u;         // Q4_K: which scale bytes of a header belong to this thread
    const int a6 = t >> 1, lh6 = t & 1, shl6 = 4 - 2 * a6, shr6 = 2 * a6;   // Q6_K
    const int keep = ring_d - 1;

    for (int seg_b = tb; seg_b < te;) {
        // ---- one product: tiles [seg_b, seg_e) of this CTA belong to it
        GOp op = single;
        if (n_ops > 1) {
            while (opi < n_ops - 1 && seg_b >= ops[opi].tile0 + ops[opi].ntiles) opi++;
            op = ops[opi];
        }
        const int seg_e = min(te, op.tile0 + op.ntiles);
        __syncthreads();   // everyone is done with the previous product's activations
        XImg xs = ximg_carve(xbase, op.k, m);
        BLane bl = blane_make(xs, xbase, g, t);
        const bool q4 = op.fmt == F_Q4K;
        if (q4) prep_x<true>(op.x, op.ldx, op.k, m, xs);
        else prep_x<false>(op.x, op.ldx, op.k, m, xs);
        __syncthreads();

        const int kw = 1 << op.kw_log2, rt = 8 >> op.kw_log2;
        const int kpart = warp & (kw - 1);
        const int nh = op.k >> 7, per = (nh + kw - 1) >> op.kw_log2;
        const int hb = kpart * per, he = min(nh, (kpart + 1) * per);
        const bool has_items = hb < he;
        auto row_of = [&](int tile, int i) -> int64_t {
            return min(((int64_t)(tile - op.tile0) * rt + (warp >> op.kw_log2)) * 16 + g + 8 * i, (int64_t)op.n_rows - 1);
        };

        // ---- producer cursor over the flat (tile, half) stream
        int pt = seg_b, ph = hb, pslot = 0;
        Q4KCursor c4[2] = {};
        Q6KCursor c6[2] = {};
        auto cursor_init = [&]() {
            if (q4) { c4[0] = q4k_cursor(op, row_of(pt, 0), ph, qoff); c4[1] = q4k_cursor(op, row_of(pt, 1), ph, qoff); }
            else { c6[0] = q6k_cursor(op, row_of(pt, 0), ph, t); c6[1] = q6k_cursor(op, row_of(pt, 1), ph, t); }
        };
        auto issue_next = [&]() {
            if (has_items && pt < seg_e) {
                const uint32_t slot = ring + pslot * RING_SLOT_BYTES;
                if (q4) { q4k_issue(c4[0], slot, 0, lane, ph == hb); q4k_issue(c4[1], slot, 1, lane, ph == hb); }
                else { q6k_issue(c6[0], op.v.p[3], slot, 0, lane); q6k_issue(c6[1], op.v.p[3], slot, 1, lane); }
                if (++ph == he) {
                    ph = hb;
                    if (++pt < seg_e) cursor_init();
                }
            }
            cp_commit();
            pslot = pslot + 1 == ring_d ? 0 : pslot + 1;
        };
        if (has_items && pt < seg_e) cursor_init();
        for (int d = 0; d < ring_d; d++) issue_next();
        int cslot = 0;

        for (int tile = seg_b; tile < seg_e; tile++) {
            const int rtile = (tile - op.tile0) * rt + (warp >> op.kw_log2);
            const bool live = (int64_t)rtile * 16 < op.n_rows;
            float acc[2][MT];
#pragma unroll
            for (int n = 0; n < MT; n++) { acc[0][n] = 0.f; acc[1][n] = 0.f; }
            // stream index of the current half of each row (its parity = position inside the super-block)
            int hs_c[2];
#pragma unroll
            for (int i = 0; i < 2; i++) hs_c[i] = (int)(((row_of(tile, i) * op.k) >> 7) + hb);
            Q4KHalfScales cur[2], nxt[2];
            for (int h = hb; h < he; h++) {
                cp_wait_keep(keep);
                __syncwarp();   // the quad leader's header copy is visible to its quad
                const uint8_t* slot = ring_gen + cslot * RING_SLOT_BYTES;
                const uint4* sd = reinterpret_cast<const uint4*>(slot);
                const uint4* sh = reinterpret_cast<const uint4*>(slot + RING_DATA_BYTES);
                if (q4) {
                    const uint4 wa = sd[lane], wb = sd[64 + lane];
#pragma unroll
                    for (int i = 0; i < 2; i++) {
                        const bool second = (hs_c[i] & 1) != 0;
                        if (h == hb || !second) {
                            Q4KHalfScales h0, h1;
                            q4k_decode_hdr(sh[i * 8 + g], sel, h0, h1);
                            cur[i] = second ? h1 : h0;
                            nxt[i] = h1;
                        } else {
                            cur[i] = nxt[i];
                        }
                    }
                    const uint32_t ML = 0x000F000Fu, MH = 0x00F000F0u;
                    const uint32_t w0[4] = {wa.x, wa.y, wa.z, wa.w};
                    const uint32_t w1[4] = {wb.x, wb.y, wb.z, wb.w};
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
                            const float2 sa = xs.ss[RA * m + n], sb = xs.ss[(RA + 2) * m + n];
#pragma unroll
                            for (int i = 0; i < 2; i++) {
                                const float va = cA[2 * i] + cA[2 * i + 1], vb = cB[2 * i] + cB[2 * i + 1];   // hi + lo columns
                                acc[i][n] += va * (cur[i].dA * sa.x) - cur[i].nA * sa.y + vb * (cur[i].dB * sb.x) - cur[i].nB * sb.y;
                            }
                        }
                    }
                } else {
                    uint32_t aL[2][4][2], aH[2][4][2];   // [row][word][pair] f16x2 codes * 2^-24
                    float dL[2], dH[2];
#pragma unroll
                    for (int i = 0; i < 2; i++) {
                        const uint4 qlv = sd[(i * 2) * 32 + lane], qhv = sd[(i * 2 + 1) * 32 + lane];
                        const uint4 hd = sh[i * 8 + g];   // x,y: eight int8 scales of the half; z: f16 d of two blocks
                        const uint32_t ql[4] = {qlv.x, qlv.y, qlv.z, qlv.w};
                        const uint32_t qh[4] = {qhv.x, qhv.y, qhv.z, qhv.w};
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            uint32_t cl = (ql[j] & 0x0F0F0F0Fu) | ((qh[j] << shl6) & 0x30303030u);          // 32-run a
                            uint32_t ch = ((ql[j] >> 4) & 0x0F0F0F0Fu) | ((qh[j] >> shr6) & 0x30303030u);   // 32-run a+2
                            aL[i][j][0] = __byte_perm(cl, 0, 0x4140); aL[i][j][1] = __byte_perm(cl, 0, 0x4342);
                            aH[i][j][0] = __byte_perm(ch, 0, 0x4140); aH[i][j][1] = __byte_perm(ch, 0, 0x4342);
                        }
                        // block = hs >> 1 picks the f16 d inside the copied pair
                        const uint32_t dbits = (hs_c[i] & 2) ? (hd.z >> 16) : (hd.z & 0xFFFFu);
                        const float d24 = __half2float(__ushort_as_half((unsigned short)dbits)) * 16777216.0f;
                        const uint32_t scw = a6 ? hd.x >> 16 : hd.x;     // scales 2a+lh (low run) ...
                        const uint32_t scw2 = a6 ? hd.y >> 16 : hd.y;    // ... and 2a+4+lh (high run)
                        dL[i] = d24 * (float)(int)(int8_t)((scw >> (8 * lh6)) & 0xFFu);
                        dH[i] = d24 * (float)(int)(int8_t)((scw2 >> (8 * lh6)) & 0xFFu);
                    }
                    const int RL = 8 * h + 2 * a6 + lh6;   // run of the low-nibble codes; high nibbles: RL + 4
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
                            const float2 sl = xs.ss[RL * m + n], sh2 = xs.ss[(RL + 4) * m + n];
                            const float k32 = 32.0f / 16777216.0f;
#pragma unroll
                            for (int i = 0; i < 2; i++) {
                                const float vl = cL[2 * i] + cL[2 * i + 1], vh = cH[2 * i] + cH[2 * i + 1];
                                // d * sc * (sum q x - 32 sum x)
                                acc[i][n] += dL[i] * (vl * sl.x - k32 * sl.y) + dH[i] * (vh * sh2.x - k32 * sh2.y);
                            }
                        }
                    }
                }
                hs_c[0]++; hs_c[1]++;
                __syncwarp();   // every lane has read the slot before it is refilled
                issue_next();
                cslot = cslot + 1 == ring_d ? 0 : cslot + 1;
            }
            // the four threads of a quad hold partial sums of the same two rows
#pragma unroll
            for (int n = 0; n < MT; n++) {
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    float sacc = acc[i][n];
                    sacc += __shfl_xor_sync(0xFFFFFFFFu, sacc, 1);
                    sacc += __shfl_xor_sync(0xFFFFFFFFu, sacc, 2);
                    acc[i][n] = sacc;
                }
            }
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
                        float sacc = 0.f;
                        for (int j = 0; j < kw; j++) sacc += red[((warp + j) * 16 + r) * MT + n];
                        int64_t row = (int64_t)rtile * 16 + r;
                        if (row < op.n_rows && n < m) op.y[(int64_t)n * op.ldy + row] = sacc;
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
        // drain: nothing of this product's ring may still be in flight when the next product reuses it
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        seg_b = seg_e;
    }
}

}  // namespace

// Ring depth: 4 items when that still lets two CTAs share an SM (or when nothing smaller helps), else 2.
int gemv_mma_ring_depth(int k, int m) {
    size_t image = XZERO_BYTES + (size_t)(k >> 4) * m * (64 + sizeof(float2)) + 16 + RED_FLOATS * sizeof(float);
    if (image + 8 * 4 * RING_SLOT_BYTES <= 110 * 1024) return 4;
    if (image + 8 * 2 * RING_SLOT_BYTES <= 110 * 1024) return 2;
    return image + 8 * 4 * RING_SLOT_BYTES <= 220 * 1024 ? 4 : 2;
}

size_t gemv_mma_smem_bytes(int fmt, int k, int m) {
    (void)fmt;
    return RED_FLOATS * sizeof(float) + 8 * (size_t)gemv_mma_ring_depth(k, m) * RING_SLOT_BYTES + XZERO_BYTES +
           (size_t)(k >> 4) * m * (64 + sizeof(float2)) + 16;
}

bool gemv_mma_supported(const b200q_weight* w, int m) {
    if (w->orient != B200Q_ORIENT_NK || m < 1 || m > 8) return false;
    if (w->n_local > 0x7FFFFFF0ll || w->k > (1 << 24) || w->n_elements >= (1ll << 37)) return false;
    if (w->fmt != F_Q4K && w->fmt != F_Q6K) return false;
    if (w->k % 128) return false;
    return gemv_mma_smem_bytes(w->fmt, (int)w->k, m) <= 220 * 1024;
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

size_t gemv_mma_smem_for(int ring_d, int kmax, int m) {
    return RED_FLOATS * sizeof(float) + 8 * (size_t)ring_d * RING_SLOT_BYTES + XZERO_BYTES +
           (size_t)(kmax >> 4) * m * (64 + sizeof(float2)) + 16;
}

int launch_gemv_mma(b200q_ctx* ctx, const GOp* h_single, const GOp* d_ops, int n_ops, const int2* d_ranges, int n_ctas,
                    int total_tiles, int m, size_t smem_bytes, int ring_d) {
    if (total_tiles <= 0) return B200Q_OK;
    static bool configured[64][4] = {};
    const int mi = m <= 1 ? 0 : m <= 2 ? 1 : m <= 4 ? 2 : 3;
    const int smem_cap = 226 * 1024;
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
        case 0: gemv_mma_kernel<1><<<n_ctas, 256, smem_bytes, ctx->stream>>>(single, d_ops, n_ops, d_ranges, total_tiles, m, ring_d); break;
        case 1: gemv_mma_kernel<2><<<n_ctas, 256, smem_bytes, ctx->stream>>>(single, d_ops, n_ops, d_ranges, total_tiles, m, ring_d); break;
        case 2: gemv_mma_kernel<4><<<n_ctas, 256, smem_bytes, ctx->stream>>>(single, d_ops, n_ops, d_ranges, total_tiles, m, ring_d); break;
        default: gemv_mma_kernel<8><<<n_ctas, 256, smem_bytes, ctx->stream>>>(single, d_ops, n_ops, d_ranges, total_tiles, m, ring_d); break;
    }
    B200Q_CUDA(cudaGetLastError(), B200Q_ERR_LAUNCH);
    return B200Q_OK;
}

}  // namespace b200q
