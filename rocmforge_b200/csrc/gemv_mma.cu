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
constexpr int F_MX4 = fmt_of(MXFP4, GGUF);
constexpr int F_Q40 = fmt_of(Q4_0, GGUF);
constexpr int F_Q80 = fmt_of(Q8_0, GGUF);
constexpr int F_Q5K = fmt_of(Q5_K, GGUF);
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

// Shared-memory image of one product's activations. Activation row n is first scaled by a power of two so that
// its largest magnitude lies in [256, 512); per 16-weight run R and activation row n:
//   img[(R*m + n)*4 + {0,1}] : f16 hi parts of the 16 scaled activations, in MMA order (4 per MMA)
//   img[(R*m + n)*4 + {2,3}] : f16 lo parts (scaled value minus hi)
//   sum[R*m + n]             : sum of the run's activations times `sum_mul`, in the units of the accumulators
//   fin[n]                   : factor that takes an accumulator back to real units (2^24 / the row's scale)
// Runs that Q4_K multiplies with high nibbles (left in bits 4..7, i.e. 16 q) are stored divided by 16.
struct XImg {
    uint4* img;
    float* sum;
    float* fin;
};

// The first 32 bytes of the activation area stay zero: lanes that supply the zero columns of B read them.
constexpr int XZERO_BYTES = 32;

__device__ __forceinline__ XImg ximg_carve(uint8_t* base, int k, int m) {
    XImg s;
    s.img = reinterpret_cast<uint4*>(base + XZERO_BYTES);
    s.sum = reinterpret_cast<float*>(base + XZERO_BYTES + (size_t)(k >> 4) * m * 64);
    s.fin = s.sum + (size_t)(k >> 4) * m;
    return s;
}

// x[m, k] (fp32, global) -> image. MODE 1 (Q4_K) and 2 (MXFP4): MMA j of a run takes elements
// (4j, 4j+2 | 4j+1, 4j+3), the pairs the nibble masks produce from bytes (0,2) and (1,3); MODE 1 also stores
// the runs that meet high nibbles divided by 16. MODE 0 (Q6_K): natural order.
// `red` is scratch for the row maxima (8 warps x up to 8 rows); the caller synchronises before and after.
template <int MODE>
__device__ __forceinline__ void prep_x(const float* __restrict__ x, int64_t ldx, int k, int m, const XImg& s, float* red,
                                       float sum_mul) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int n = 0; n < m; n++) {
        const float4* xr = reinterpret_cast<const float4*>(x + (int64_t)n * ldx);
        float mx = 0.0f;
        for (int i = threadIdx.x; i < (k >> 2); i += 256) {
            const float4 f = __ldg(xr + i);
            mx = fmaxf(fmaxf(mx, fmaxf(fabsf(f.x), fabsf(f.y))), fmaxf(fabsf(f.z), fabsf(f.w)));
        }
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        if (lane == 0) red[warp * 8 + n] = mx;
    }
    __syncthreads();
    const int total = (k >> 4) * m;
    for (int q = threadIdx.x; q < total; q += 256) {
        const int R = q / m, n = q - R * m;
        float mx = red[n];
#pragma unroll
        for (int w = 1; w < 8; w++) mx = fmaxf(mx, red[w * 8 + n]);
        int e = (int)((__float_as_uint(mx) >> 23) & 255u);
        e = mx == 0.0f ? 127 : min(max(e, 9), 238);
        const float sdown = __uint_as_float((uint32_t)(262 - e) << 23);   // 2^(135-e): the row's maximum lands in [256, 512)
        const float run_mul = (MODE == 1 && (R & 2)) ? sdown * 0.0625f : sdown;
        const float4* xp = reinterpret_cast<const float4*>(x + (int64_t)n * ldx + (int64_t)R * 16);
        float v[16];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float4 f = __ldg(xp + i);
            v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
        }
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; i++) sum += v[i];
        __align__(16) __half h[16];
        __align__(16) __half l[16];
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const int src = MODE != 0 ? ((i & ~3) | ((i & 1) << 1) | ((i & 2) >> 1)) : i;   // 0,2,1,3 inside each group of 4
            const float xs = v[src] * run_mul;
            h[i] = __float2half_rn(xs);
            l[i] = __float2half_rn(xs - __half2float(h[i]));
        }
        uint4* dst = s.img + (size_t)q * 4;
        dst[0] = reinterpret_cast<uint4*>(h)[0];
        dst[1] = reinterpret_cast<uint4*>(h)[1];
        dst[2] = reinterpret_cast<uint4*>(l)[0];
        dst[3] = reinterpret_cast<uint4*>(l)[1];
        s.sum[q] = sum * (sdown * (1.0f / 16777216.0f)) * sum_mul;
        if (R == 0) s.fin[n] = __uint_as_float((uint32_t)(e + 16) << 23);   // 2^24 / sdown = 2^(e-111)
    }
}

// ------------------------------------------------------------------------------------ weight streaming
// Every warp streams its weights through a private ring in shared memory filled with cp.async (16 bytes
// per thread and copy), `ring_d` items deep. An item is one 128-weight half of the warp's 16 rows together
// with the block headers it needs; the producer cursor runs ring_d items ahead of the consumer over a FLAT
// stream of (tile, half) items, so the prefetch crosses tile boundaries and no load latency is exposed when
// a warp starts a new tile. No registers are held for look-ahead. Slot layout (per warp):
// [row g / g+8][piece 0/1][lane] x 16 B of codes, then [row][quad] x 16 B of block header written by the
// quad's first lane. Rows g and g+8 of a thread are a whole number of super-blocks apart, so one cursor plus
// a constant byte distance serves both.
// Q6_K slots hold two pieces (ql, qh) per row, Q4_K slots one, so a warp's ring (ring_d units of
// RING_UNIT_BYTES) is ring_d items deep for Q6_K and 2 * ring_d items deep for Q4_K: about 9 KB of weights
// in flight per warp either way, which is what hides the HBM latency.
constexpr int RING_HDR_BYTES = 2 * 8 * 16;
constexpr int Q6K_DATA_BYTES = 2 * 2 * 32 * 16, Q6K_SLOT_BYTES = Q6K_DATA_BYTES + RING_HDR_BYTES;   // 2304
constexpr int Q4K_DATA_BYTES = 2 * 32 * 16, Q4K_SLOT_BYTES = Q4K_DATA_BYTES + RING_HDR_BYTES;       // 1280
constexpr int RING_UNIT_BYTES = 2 * Q4K_SLOT_BYTES;                                                // 2560 >= 2304
constexpr int MX4_DATA_BYTES = 2 * 32 * 16, MX4_SLOT_BYTES = MX4_DATA_BYTES + 2 * 8 * 4;           // 1088
constexpr int Q40_SLOT_BYTES = MX4_DATA_BYTES + 2 * 8 * 8;                                          // 1152: four f16 scales per row
constexpr int Q80_DATA_BYTES = 2 * 2 * 32 * 16, Q80_SLOT_BYTES = Q80_DATA_BYTES + 2 * 8 * 8;        // 2176: 32 code bytes per block

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
    if (keep >= 7) asm volatile("cp.async.wait_group 7;" ::: "memory");
    else if (keep >= 3) asm volatile("cp.async.wait_group 3;" ::: "memory");
    else asm volatile("cp.async.wait_group 1;" ::: "memory");
}

// What a warp knows about the product segment it is working on.
struct Seg {
    int seg_b, seg_e;     // CTA tiles of this product owned by the CTA
    int hb, he;           // 128-weight halves of every row owned by this warp (its k-part)
    int rt_shift;         // log2 of the row tiles per CTA tile
    int wrow;             // this warp's row tile inside a CTA tile
    int tile0;            // first CTA tile of the product
    int n_rows, nh;       // rows of the tensor, halves per row
};

__device__ __forceinline__ int seg_row_base(const Seg& sg, int tile) { return (((tile - sg.tile0) << sg.rt_shift) + sg.wrow) * 16; }

// ---- Q4_K cursor: thread (g, t) owns, in every half and for rows g and g+8, bytes [16*(t&1), +16) of chunk
// (t>>1): 16 weights of a low-nibble sub-block and 16 of the high-nibble sub-block.
struct Q4KCursor {
    const uint8_t* p;   // this thread's 16 bytes of the half the cursor is on (row g)
    int64_t d1;         // byte distance to the same piece of row g+8 (0 when that row is past the end)
    int sec;            // 1 when the half is the second half of its super-block
};

// Q5 = GGUF Q5_K: the same block with 32 bytes of fifth bits (qh) between the 16 header bytes and the nibbles.
template <bool Q5>
__device__ __forceinline__ void q4k_seek(Q4KCursor& c, const uint8_t* base, const Seg& sg, int tile, int g, int qo) {
    constexpr int BB = Q5 ? 176 : 144, NO = Q5 ? 48 : 16;   // block bytes, offset of the nibbles
    const int rb = seg_row_base(sg, tile) + g;
    const int64_t r0 = min((int64_t)rb, (int64_t)sg.n_rows - 1);
    const int64_t hs = r0 * sg.nh + sg.hb;
    c.sec = (int)(hs & 1);
    c.p = base + (hs >> 1) * BB + NO + c.sec * 64 + qo;
    c.d1 = (rb + 8 <= sg.n_rows - 1) ? (int64_t)sg.nh * (4 * BB) : 0;
}
// Copies the cursor's half of both rows (and, by the quad's first lane, the two super-block headers) into
// the ring slot and steps to the next half.
template <bool Q5>
__device__ __forceinline__ void q4k_issue(Q4KCursor& c, uint32_t slot, int lane) {
    constexpr int BB = Q5 ? 176 : 144, NO = Q5 ? 48 : 16, DATA = Q5 ? 2 * Q4K_DATA_BYTES : Q4K_DATA_BYTES;
    cp_async16(slot + lane * 16, c.p);
    cp_async16(slot + 512 + lane * 16, c.p + c.d1);
    const int t = lane & 3;
    const uint8_t* blk = c.p - NO - c.sec * 64 - ((t >> 1) * 32 + (t & 1) * 16);   // start of the super-block
    if constexpr (Q5) {   // the 16 fifth-bit bytes that go with this thread's 16 nibble bytes
        cp_async16(slot + 1024 + lane * 16, blk + 16 + (t & 1) * 16);
        cp_async16(slot + 1536 + lane * 16, blk + 16 + (t & 1) * 16 + c.d1);
    }
    if (t == 0) {
        cp_async16(slot + DATA + (lane >> 2) * 16, blk);
        cp_async16(slot + DATA + 128 + (lane >> 2) * 16, blk + c.d1);
    }
    c.p += 64 + c.sec * (BB - 128);
    c.sec ^= 1;
}

// ---- Q6_K cursor: thread (g, t) owns 16 bytes of ql (32-run a = t>>1 in the low nibbles, a+2 in the high
// nibbles, 16-weight half lh = t&1 of each) and the matching 16 bytes of qh; header = 8 int8 scales + the
// aligned 4 bytes that hold the f16 d of the block.
struct Q6KCursor {
    const uint8_t *ql, *qh, *sc;
    int64_t hs;          // index of the half in the tensor's flat stream (row g)
    int64_t dh;          // halves between row g and row g+8 (0 when that row is past the end)
};

__device__ __forceinline__ void q6k_seek(Q6KCursor& c, const GOp& op, const Seg& sg, int tile, int g, int t) {
    const int rb = seg_row_base(sg, tile) + g;
    const int64_t r0 = min((int64_t)rb, (int64_t)sg.n_rows - 1);
    c.hs = r0 * sg.nh + sg.hb;
    c.ql = op.v.p[0] + c.hs * 64 + (t >> 1) * 32 + (t & 1) * 16;
    c.qh = op.v.p[1] + c.hs * 32 + (t & 1) * 16;
    c.sc = op.v.p[2] + c.hs * 8;
    c.dh = (rb + 8 <= sg.n_rows - 1) ? (int64_t)sg.nh * 8 : 0;
}
__device__ __forceinline__ void q6k_issue(Q6KCursor& c, const uint8_t* dplane, uint32_t slot, int lane) {
    cp_async16(slot + lane * 16, c.ql);
    cp_async16(slot + 512 + lane * 16, c.qh);
    cp_async16(slot + 1024 + lane * 16, c.ql + c.dh * 64);
    cp_async16(slot + 1536 + lane * 16, c.qh + c.dh * 32);
    if ((lane & 3) == 0) {
        const uint32_t h = slot + Q6K_DATA_BYTES + (lane >> 2) * 16;
        const uint8_t* dp = dplane + (c.hs & ~(int64_t)3);
        cp_async8(h, c.sc);
        cp_async4(h + 8, dp);
        cp_async8(h + 128, c.sc + c.dh * 8);
        cp_async4(h + 136, dp + c.dh);
    }
    c.ql += 64; c.qh += 32; c.sc += 8; c.hs += 1;
}

// Reduction of the k-parts of a tile through shared memory, or the direct store when a warp owns whole rows.
template <int MT>
__device__ __forceinline__ void finish_tile(float (&acc)[2][MT], const GOp& op, const Seg& sg, const XImg& xs, int tile, int m,
                                            int kw, float* red, int warp, int lane) {
    const int g = lane >> 2, t = lane & 3;
    const int row_base = seg_row_base(sg, tile);
    const bool live = row_base < sg.n_rows;
#pragma unroll
    for (int n = 0; n < MT; n++) {
#pragma unroll
        for (int i = 0; i < 2; i++) {   // the four threads of a quad hold partial sums of the same two rows
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
        if ((warp & (kw - 1)) == 0 && live) {
            for (int o = lane; o < 16 * MT; o += 32) {
                const int r = o / MT, n = o - r * MT;
                float sacc = 0.f;
                for (int j = 0; j < kw; j++) sacc += red[((warp + j) * 16 + r) * MT + n];
                const int row = row_base + r;
                if (row < sg.n_rows && n < m) {
                    const float val = sacc * xs.fin[n];
                    op.y[(int64_t)n * op.ldy + row] = val;
                    for (int pp = 0; pp < op.n_extra; pp++) op.y_extra[pp][(int64_t)n * op.ldy + row] = val;
                }
            }
        }
        __syncthreads();   // the reduction buffer is free again
    } else if (live && t == 0) {
#pragma unroll
        for (int n = 0; n < MT; n++) {
            if (n < m) {
                const float f = xs.fin[n];
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const int row = row_base + g + 8 * i;
                    if (row < sg.n_rows) {
                        const float val = acc[i][n] * f;
                        op.y[(int64_t)n * op.ldy + row] = val;
                        for (int pp = 0; pp < op.n_extra; pp++) op.y_extra[pp][(int64_t)n * op.ldy + row] = val;
                    }
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------------- Q4_K (GGUF)
// One product segment, Q4_K. Per item and row: the two 6-bit scales and minima of the thread's chunk are cut
// out of the 12 packed bytes (different bit positions in the first and second half of a super-block), the 64
// codes become 16 A registers (one AND per pair of weights), 8 MMAs per activation row, and the block
// scales are folded into the accumulator: acc += d * (scA * vA + scB * vB) - dmin * (mA * sumA + mB * sumB).
template <int MT, bool Q5, class Late>
__device__ __forceinline__ void run_q4k(const GOp& op, const Seg& sg, const XImg& xs, const uint8_t* xzero, uint8_t* ring_gen,
                                        int ring_d, int m, int kw, float* red, Late&& late) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3, tp = t >> 1;
    constexpr int SLOT_BYTES = Q5 ? Q6K_SLOT_BYTES : Q4K_SLOT_BYTES;   // Q5_K: two more 512-byte pieces (the fifth bits)
    constexpr int DATA_BYTES = Q5 ? 2 * Q4K_DATA_BYTES : Q4K_DATA_BYTES;
    const int depth = Q5 ? ring_d : 2 * ring_d;
    const uint32_t ring = smem_addr(ring_gen), ring_end = ring + depth * SLOT_BYTES;
    const int keep = depth - 1;
    const int qo = tp * 32 + (t & 1) * 16;
    const int sh16 = tp * 16;
    const bool has_items = sg.hb < sg.he;
    // B operand: lanes g == 2t (hi) and g == 2t+1 (lo) read the image of their run, all other lanes the zero
    // region (stride 0), so the loads need no predicate
    const bool active = (g >> 1) == t;
    const uint4* bbase = active ? xs.img + (g & 1) * 2 + (4 * tp + (t & 1)) * m * 4 : reinterpret_cast<const uint4*>(xzero);
    const int bstep = active ? 8 * m * 4 : 0;       // uint4 per half
    const int bhigh = active ? 2 * m * 4 : 0;       // from the low-nibble run to the high-nibble run
    const int bn = active ? 4 : 0;                  // per activation row
    const float* sbase = xs.sum + (4 * tp + (t & 1)) * m;

    // ---- producer
    Q4KCursor cur{};
    int pt = sg.seg_b, ph = sg.hb;
    uint32_t pslot = ring;
    if (has_items && pt < sg.seg_e) q4k_seek<Q5>(cur, op.v.p[0], sg, pt, g, qo);
    auto issue_next = [&]() {
        if (has_items && pt < sg.seg_e) {
            q4k_issue<Q5>(cur, pslot, lane);
            if (++ph == sg.he) {
                ph = sg.hb;
                if (++pt < sg.seg_e) q4k_seek<Q5>(cur, op.v.p[0], sg, pt, g, qo);
            }
        }
        cp_commit();
        pslot += SLOT_BYTES;
        if (pslot == ring_end) pslot = ring;
    };
    for (int d = 0; d < depth; d++) issue_next();
    late();   // the first product of a CTA builds its activation image only now: the weights are already on their way
    const uint8_t* cslot = ring_gen;
    const uint8_t* cend = ring_gen + depth * SLOT_BYTES;

    for (int tile = sg.seg_b; tile < sg.seg_e; tile++) {
        float acc[2][MT];
#pragma unroll
        for (int n = 0; n < MT; n++) { acc[0][n] = 0.f; acc[1][n] = 0.f; }
        const int64_t r0 = min((int64_t)seg_row_base(sg, tile) + g, (int64_t)sg.n_rows - 1);
        int csec = (int)((r0 * sg.nh + sg.hb) & 1);
        const uint4* bp = bbase + sg.hb * bstep;
        const float* sp = sbase + sg.hb * 8 * m;
        for (int h = sg.hb; h < sg.he; h++) {
            cp_wait_keep(keep);
            __syncwarp();   // the quad leader's header copies are visible to its quad
            const uint4* sd = reinterpret_cast<const uint4*>(cslot);
            const uint4* sh = reinterpret_cast<const uint4*>(cslot + DATA_BYTES);
            const uint4 wa = sd[lane], wb = sd[32 + lane];
            const uint4 hd[2] = {sh[g], sh[8 + g]};
            const uint32_t MA = csec ? 0x0F0Fu : 0x3F3Fu, MB = csec ? 0x3030u : 0u;
            float dd[2], dmn[2], scA[2], scB[2], mnA[2], mnB[2];
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const float2 df = __half22float2(*reinterpret_cast<const __half2*>(&hd[i].x));
                dd[i] = df.x; dmn[i] = -df.y;
                const uint32_t y1 = hd[i].y >> sh16, z1 = hd[i].z >> sh16, w1 = hd[i].w >> sh16;
                const uint32_t scp = ((csec ? w1 : y1) & MA) | ((y1 >> 2) & MB);
                const uint32_t mp = ((csec ? (w1 >> 4) : z1) & MA) | ((z1 >> 2) & MB);
                scA[i] = (float)(scp & 0xFFu); scB[i] = (float)(scp >> 8);
                mnA[i] = (float)(mp & 0xFFu); mnB[i] = (float)(mp >> 8);
            }
            const uint32_t ML = 0x000F000Fu, MH = 0x00F000F0u;
            const uint32_t w0[4] = {wa.x, wa.y, wa.z, wa.w};
            const uint32_t w1[4] = {wb.x, wb.y, wb.z, wb.w};
            uint32_t s0[4], s1[4];
#pragma unroll
            for (int j = 0; j < 4; j++) { s0[j] = w0[j] >> 8; s1[j] = w1[j] >> 8; }
            // Q5_K: bit (4 sec + 2 tp) of a qh byte is the fifth bit of its low-nibble weight, the next bit that of
            // its high-nibble weight; it joins the code at bit 4 (bit 8 where the nibble stays in bits 4..7). The
            // operands are completed once per item: [row g bytes 0,2 | row g+8 bytes 0,2 | row g bytes 1,3 | row g+8 bytes 1,3]
            uint32_t qL[4][4], qH[4][4];
            if constexpr (Q5) {
                const uint4 qa = sd[64 + lane], qb = sd[96 + lane];
                const uint32_t q0[4] = {qa.x, qa.y, qa.z, qa.w};
                const uint32_t q1[4] = {qb.x, qb.y, qb.z, qb.w};
                const int jl = 4 * csec + 2 * tp;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const uint32_t a0 = q0[j] >> jl, a1 = q1[j] >> jl;
                    qL[0][j] = (w0[j] & ML) | ((a0 & 0x00010001u) << 4);
                    qL[1][j] = (w1[j] & ML) | ((a1 & 0x00010001u) << 4);
                    qL[2][j] = (s0[j] & ML) | (((a0 >> 8) & 0x00010001u) << 4);
                    qL[3][j] = (s1[j] & ML) | (((a1 >> 8) & 0x00010001u) << 4);
                    qH[0][j] = (w0[j] & MH) | (((a0 >> 1) & 0x00010001u) << 8);
                    qH[1][j] = (w1[j] & MH) | (((a1 >> 1) & 0x00010001u) << 8);
                    qH[2][j] = (s0[j] & MH) | (((a0 >> 9) & 0x00010001u) << 8);
                    qH[3][j] = (s1[j] & MH) | (((a1 >> 9) & 0x00010001u) << 8);
                }
            }
            auto AL = [&](int which, int j) -> uint32_t {
                if constexpr (Q5) return qL[which][j];
                else return (which == 0 ? w0[j] : which == 1 ? w1[j] : which == 2 ? s0[j] : s1[j]) & ML;
            };
            auto AH = [&](int which, int j) -> uint32_t {
                if constexpr (Q5) return qH[which][j];
                else return (which == 0 ? w0[j] : which == 1 ? w1[j] : which == 2 ? s0[j] : s1[j]) & MH;
            };
#pragma unroll
            for (int n = 0; n < MT; n++) {
                if (n < m) {
                    float cA[4], cB[4];
                    const uint4* bq = bp + n * bn;
                    uint4 b01 = bq[0], b23 = bq[1];
                    mma16816_z(cA, AL(0, 0), AL(1, 0), AL(2, 0), AL(3, 0), b01.x, b01.y);
                    mma16816(cA, AL(0, 1), AL(1, 1), AL(2, 1), AL(3, 1), b01.z, b01.w);
                    mma16816(cA, AL(0, 2), AL(1, 2), AL(2, 2), AL(3, 2), b23.x, b23.y);
                    mma16816(cA, AL(0, 3), AL(1, 3), AL(2, 3), AL(3, 3), b23.z, b23.w);
                    b01 = bq[bhigh]; b23 = bq[bhigh + 1];
                    mma16816_z(cB, AH(0, 0), AH(1, 0), AH(2, 0), AH(3, 0), b01.x, b01.y);
                    mma16816(cB, AH(0, 1), AH(1, 1), AH(2, 1), AH(3, 1), b01.z, b01.w);
                    mma16816(cB, AH(0, 2), AH(1, 2), AH(2, 2), AH(3, 2), b23.x, b23.y);
                    mma16816(cB, AH(0, 3), AH(1, 3), AH(2, 3), AH(3, 3), b23.z, b23.w);
                    const float sa = sp[n], sb = sp[2 * m + n];
#pragma unroll
                    for (int i = 0; i < 2; i++) {
                        const float va = cA[2 * i] + cA[2 * i + 1], vb = cB[2 * i] + cB[2 * i + 1];   // hi + lo columns
                        const float u = fmaf(scB[i], vb, scA[i] * va);
                        const float mn = fmaf(mnB[i], sb, mnA[i] * sa);
                        acc[i][n] = fmaf(dmn[i], mn, fmaf(dd[i], u, acc[i][n]));
                    }
                }
            }
            csec ^= 1;
            bp += bstep;
            sp += 8 * m;
            __syncwarp();   // every lane has read the slot before it is refilled
            issue_next();
            cslot += SLOT_BYTES;
            if (cslot == cend) cslot = ring_gen;
        }
        finish_tile<MT>(acc, op, sg, xs, tile, m, kw, red, warp, lane);
    }
    // drain: nothing of this product's ring may still be in flight when the next product reuses it
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// ------------------------------------------------------------------------------------------- Q6_K (GGUF)
// One product segment, Q6_K: acc += d * sc * (sum q x - 32 sum x) per 16-weight run (the activation image
// stores 32 sum x).
template <int MT, class Late>
__device__ __forceinline__ void run_q6k(const GOp& op, const Seg& sg, const XImg& xs, const uint8_t* xzero, uint8_t* ring_gen,
                                        int ring_d, int m, int kw, float* red, Late&& late) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const uint32_t ring = smem_addr(ring_gen), ring_end = ring + ring_d * Q6K_SLOT_BYTES;
    const int keep = ring_d - 1;
    const int a6 = t >> 1, lh6 = t & 1, shl6 = 4 - 2 * a6, shr6 = 2 * a6;
    const int scsh = 16 * a6 + 8 * lh6;   // bit position of scale 2a+lh inside its word of four
    const bool has_items = sg.hb < sg.he;
    const bool active = (g >> 1) == t;
    const uint4* bbase = active ? xs.img + (g & 1) * 2 + (2 * a6 + lh6) * m * 4 : reinterpret_cast<const uint4*>(xzero);
    const int bstep = active ? 8 * m * 4 : 0;
    const int bhigh = active ? 4 * m * 4 : 0;
    const int bn = active ? 4 : 0;
    const float* sbase = xs.sum + (2 * a6 + lh6) * m;

    Q6KCursor cur{};
    int pt = sg.seg_b, ph = sg.hb;
    uint32_t pslot = ring;
    if (has_items && pt < sg.seg_e) q6k_seek(cur, op, sg, pt, g, t);
    auto issue_next = [&]() {
        if (has_items && pt < sg.seg_e) {
            q6k_issue(cur, op.v.p[3], pslot, lane);
            if (++ph == sg.he) {
                ph = sg.hb;
                if (++pt < sg.seg_e) q6k_seek(cur, op, sg, pt, g, t);
            }
        }
        cp_commit();
        pslot += Q6K_SLOT_BYTES;
        if (pslot == ring_end) pslot = ring;
    };
    for (int d = 0; d < ring_d; d++) issue_next();
    late();   // the first product of a CTA builds its activation image only now: the weights are already on their way
    const uint8_t* cslot = ring_gen;
    const uint8_t* cend = ring_gen + ring_d * Q6K_SLOT_BYTES;

    for (int tile = sg.seg_b; tile < sg.seg_e; tile++) {
        float acc[2][MT];
#pragma unroll
        for (int n = 0; n < MT; n++) { acc[0][n] = 0.f; acc[1][n] = 0.f; }
        const int64_t r0 = min((int64_t)seg_row_base(sg, tile) + g, (int64_t)sg.n_rows - 1);
        int chs = (int)((r0 * sg.nh + sg.hb) & 3);   // bit 1: which f16 of the copied d pair
        const uint4* bp = bbase + sg.hb * bstep;
        const float* sp = sbase + sg.hb * 8 * m;
        for (int h = sg.hb; h < sg.he; h++) {
            cp_wait_keep(keep);
            __syncwarp();
            const uint4* sd = reinterpret_cast<const uint4*>(cslot);
            const uint4* sh = reinterpret_cast<const uint4*>(cslot + Q6K_DATA_BYTES);
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
                    const uint32_t cl = (ql[j] & 0x0F0F0F0Fu) | ((qh[j] << shl6) & 0x30303030u);          // 32-run a
                    const uint32_t ch = ((ql[j] >> 4) & 0x0F0F0F0Fu) | ((qh[j] >> shr6) & 0x30303030u);   // 32-run a+2
                    aL[i][j][0] = __byte_perm(cl, 0, 0x4140); aL[i][j][1] = __byte_perm(cl, 0, 0x4342);
                    aH[i][j][0] = __byte_perm(ch, 0, 0x4140); aH[i][j][1] = __byte_perm(ch, 0, 0x4342);
                }
                const uint32_t dbits = (chs & 2) ? (hd.z >> 16) : (hd.z & 0xFFFFu);
                const float d = __half2float(__ushort_as_half((unsigned short)dbits));
                dL[i] = d * (float)(int)(int8_t)((hd.x >> scsh) & 0xFFu);    // scale 2a+lh (low run)
                dH[i] = d * (float)(int)(int8_t)((hd.y >> scsh) & 0xFFu);    // scale 2a+4+lh (high run)
            }
#pragma unroll
            for (int n = 0; n < MT; n++) {
                if (n < m) {
                    float cL[4], cH[4];
                    const uint4* bq = bp + n * bn;
                    uint4 b01 = bq[0], b23 = bq[1];
                    mma16816_z(cL, aL[0][0][0], aL[1][0][0], aL[0][0][1], aL[1][0][1], b01.x, b01.y);
                    mma16816(cL, aL[0][1][0], aL[1][1][0], aL[0][1][1], aL[1][1][1], b01.z, b01.w);
                    mma16816(cL, aL[0][2][0], aL[1][2][0], aL[0][2][1], aL[1][2][1], b23.x, b23.y);
                    mma16816(cL, aL[0][3][0], aL[1][3][0], aL[0][3][1], aL[1][3][1], b23.z, b23.w);
                    b01 = bq[bhigh]; b23 = bq[bhigh + 1];
                    mma16816_z(cH, aH[0][0][0], aH[1][0][0], aH[0][0][1], aH[1][0][1], b01.x, b01.y);
                    mma16816(cH, aH[0][1][0], aH[1][1][0], aH[0][1][1], aH[1][1][1], b01.z, b01.w);
                    mma16816(cH, aH[0][2][0], aH[1][2][0], aH[0][2][1], aH[1][2][1], b23.x, b23.y);
                    mma16816(cH, aH[0][3][0], aH[1][3][0], aH[0][3][1], aH[1][3][1], b23.z, b23.w);
                    const float s32l = sp[n], s32h = sp[4 * m + n];
#pragma unroll
                    for (int i = 0; i < 2; i++) {
                        const float vl = cL[2 * i] + cL[2 * i + 1] - s32l, vh = cH[2 * i] + cH[2 * i + 1] - s32h;
                        acc[i][n] = fmaf(dH[i], vh, fmaf(dL[i], vl, acc[i][n]));
                    }
                }
            }
            chs++;
            bp += bstep;
            sp += 8 * m;
            __syncwarp();
            issue_next();
            cslot += Q6K_SLOT_BYTES;
            if (cslot == cend) cslot = ring_gen;
        }
        finish_tile<MT>(acc, op, sg, xs, tile, m, kw, red, warp, lane);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// ------------------------------------------------------------------------------------------ MXFP4 (GGUF)
// Blocks of 32: one E8M0 exponent byte (plane 0) and 16 code bytes (plane 1), byte i = element i in the low
// nibble and element i+16 in the high nibble. An E2M1 code s|ee|m is itself a tiny float: placed at bits
// 15|11..9 of an f16 lane it is exactly value * 2^-14 (ee = 0 lands in the f16 subnormals, as E2M1 demands),
// so codes go to the tensor cores after two ANDs and two shift-adds per pair, and the block scale
// 2^(e-127) * 2^14 is applied once per 32 weights. Thread (g, t) owns block t of the half for rows g, g+8:
// its low nibbles are 16-weight run 2t, its high nibbles run 2t+1.
struct MX4Cursor {
    const uint8_t *q, *e;   // this thread's 16 code bytes; the four exponents of the half (row g)
    int64_t dq, de;         // byte distances to row g+8 (0 when that row is past the end)
};

// KIND 1 = GGUF Q4_0 on the same path: the same 16 code bytes per block (byte i = elements i and i+16), and an
// f16 scale d per block (2 bytes) where MXFP4 (KIND 0) has its exponent byte. KIND 2 = GGUF Q8_0: f16 d and 32
// int8 codes per block, two 16-byte pieces per thread and row (elements 0..15 = run 2t, 16..31 = run 2t+1).
template <int KIND>
__device__ __forceinline__ void mx4_seek(MX4Cursor& c, const GOp& op, const Seg& sg, int tile, int g, int t) {
    constexpr int SB = KIND ? 8 : 4;          // scale bytes of one row's half (four blocks)
    constexpr int CB = KIND == 2 ? 32 : 16;   // code bytes of one block
    const int rb = seg_row_base(sg, tile) + g;
    const int64_t r0 = min((int64_t)rb, (int64_t)sg.n_rows - 1);
    const int64_t hs = r0 * sg.nh + sg.hb;
    c.q = op.v.p[1] + hs * (4 * CB) + t * CB;
    c.e = op.v.p[0] + hs * SB;
    const bool two = rb + 8 <= sg.n_rows - 1;
    c.dq = two ? (int64_t)sg.nh * 8 * (4 * CB) : 0;
    c.de = two ? (int64_t)sg.nh * 8 * SB : 0;
}
template <int KIND>
__device__ __forceinline__ void mx4_issue(MX4Cursor& c, uint32_t slot, int lane) {
    constexpr int DATA = KIND == 2 ? Q80_DATA_BYTES : MX4_DATA_BYTES;
    if constexpr (KIND == 2) {   // [row g | g+8][piece 0 | 1][lane]
        cp_async16(slot + lane * 16, c.q);
        cp_async16(slot + 512 + lane * 16, c.q + 16);
        cp_async16(slot + 1024 + lane * 16, c.q + c.dq);
        cp_async16(slot + 1536 + lane * 16, c.q + c.dq + 16);
    } else {
        cp_async16(slot + lane * 16, c.q);
        cp_async16(slot + 512 + lane * 16, c.q + c.dq);
    }
    if ((lane & 3) == 0) {
        if constexpr (KIND != 0) {
            cp_async8(slot + DATA + (lane >> 2) * 8, c.e);
            cp_async8(slot + DATA + 64 + (lane >> 2) * 8, c.e + c.de);
        } else {
            cp_async4(slot + DATA + (lane >> 2) * 4, c.e);
            cp_async4(slot + DATA + 32 + (lane >> 2) * 4, c.e + c.de);
        }
    }
    c.q += KIND == 2 ? 128 : 64; c.e += KIND ? 8 : 4;
}

// two E2M1 codes (bits 0..3 and 16..19 of v) -> f16x2 holding value * 2^-14
__device__ __forceinline__ uint32_t e2m1x2_to_f16x2(uint32_t v) {
    return (v & 0x00070007u) * 512u + (v & 0x00080008u) * 4096u;
}

template <int MT, int KIND, class Late>
__device__ __forceinline__ void run_mx4(const GOp& op, const Seg& sg, const XImg& xs, const uint8_t* xzero, uint8_t* ring_gen,
                                        int ring_d, int m, int kw, float* red, Late&& late) {
    constexpr bool Q40 = KIND == 1, Q80 = KIND == 2;
    constexpr int SLOT_BYTES = Q80 ? Q80_SLOT_BYTES : Q40 ? Q40_SLOT_BYTES : MX4_SLOT_BYTES;
    constexpr int DATA_BYTES = Q80 ? Q80_DATA_BYTES : MX4_DATA_BYTES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    // slots the warp's ring holds: 8 or 4 of the small slots, ring_d (4 or 2) of the 2176-byte Q8_0 slots
    const int depth = Q80 ? ring_d : (min(8, ring_d * RING_UNIT_BYTES / SLOT_BYTES) >= 8 ? 8 : 4);
    const uint32_t ring = smem_addr(ring_gen), ring_end = ring + depth * SLOT_BYTES;
    const int keep = depth - 1;
    const bool has_items = sg.hb < sg.he;
    const bool active = (g >> 1) == t;
    const uint4* bbase = active ? xs.img + (g & 1) * 2 + (2 * t) * m * 4 : reinterpret_cast<const uint4*>(xzero);
    const int bstep = active ? 8 * m * 4 : 0;
    const int bhigh = active ? m * 4 : 0;
    const int bn = active ? 4 : 0;

    MX4Cursor cur{};
    int pt = sg.seg_b, ph = sg.hb;
    uint32_t pslot = ring;
    if (has_items && pt < sg.seg_e) mx4_seek<KIND>(cur, op, sg, pt, g, t);
    auto issue_next = [&]() {
        if (has_items && pt < sg.seg_e) {
            mx4_issue<KIND>(cur, pslot, lane);
            if (++ph == sg.he) {
                ph = sg.hb;
                if (++pt < sg.seg_e) mx4_seek<KIND>(cur, op, sg, pt, g, t);
            }
        }
        cp_commit();
        pslot += SLOT_BYTES;
        if (pslot == ring_end) pslot = ring;
    };
    for (int d = 0; d < depth; d++) issue_next();
    late();   // the first product of a CTA builds its activation image only now: the weights are already on their way
    const uint8_t* cslot = ring_gen;
    const uint8_t* cend = ring_gen + depth * SLOT_BYTES;

    for (int tile = sg.seg_b; tile < sg.seg_e; tile++) {
        float acc[2][MT];
#pragma unroll
        for (int n = 0; n < MT; n++) { acc[0][n] = 0.f; acc[1][n] = 0.f; }
        const uint4* bp = bbase + sg.hb * bstep;
        const float* sp = xs.sum + ((size_t)sg.hb * 8 + 2 * t) * m;   // Q4_0: 8 * sum(x) of the block's two 16-weight runs
        for (int h = sg.hb; h < sg.he; h++) {
            cp_wait_keep(keep);
            __syncwarp();
            const uint4* sd = reinterpret_cast<const uint4*>(cslot);
            const uint4 wa = sd[lane], wb = sd[(Q80 ? 64 : 32) + lane];
            float S[2];
            const uint32_t w0[4] = {wa.x, wa.y, wa.z, wa.w};
            const uint32_t w1[4] = {wb.x, wb.y, wb.z, wb.w};
            uint32_t aL[2][4][2], aH[2][4][2];   // [row][word][bytes (0,2) | (1,3)]
            if constexpr (Q80) {
                const uint16_t* sdh = reinterpret_cast<const uint16_t*>(cslot + DATA_BYTES);
#pragma unroll
                for (int i = 0; i < 2; i++) S[i] = __half2float(__ushort_as_half(sdh[(i * 8 + g) * 4 + t]));   // d of block t
                const uint4 wc = sd[32 + lane], wd = sd[96 + lane];   // second pieces: elements 16..31 of the block
                const uint32_t h0[4] = {wc.x, wc.y, wc.z, wc.w};
                const uint32_t h1[4] = {wd.x, wd.y, wd.z, wd.w};
                // int8 code ^ 0x80 = q + 128 in 0..255: in the low byte of an f16 lane that is (q + 128) * 2^-24
                const uint32_t MB = 0x00FF00FFu, SX = 0x80808080u;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    aL[0][j][0] = (w0[j] ^ SX) & MB;   aL[0][j][1] = ((w0[j] ^ SX) >> 8) & MB;
                    aH[0][j][0] = (h0[j] ^ SX) & MB;   aH[0][j][1] = ((h0[j] ^ SX) >> 8) & MB;
                    aL[1][j][0] = (w1[j] ^ SX) & MB;   aL[1][j][1] = ((w1[j] ^ SX) >> 8) & MB;
                    aH[1][j][0] = (h1[j] ^ SX) & MB;   aH[1][j][1] = ((h1[j] ^ SX) >> 8) & MB;
                }
            } else if constexpr (Q40) {
                const uint16_t* sdh = reinterpret_cast<const uint16_t*>(cslot + DATA_BYTES);
#pragma unroll
                for (int i = 0; i < 2; i++) S[i] = __half2float(__ushort_as_half(sdh[(i * 8 + g) * 4 + t]));   // d of block t
                const uint32_t ML = 0x000F000Fu;   // an integer code in the low bits of an f16 lane is code * 2^-24
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    aL[0][j][0] = w0[j] & ML;          aL[0][j][1] = (w0[j] >> 8) & ML;
                    aH[0][j][0] = (w0[j] >> 4) & ML;   aH[0][j][1] = (w0[j] >> 12) & ML;
                    aL[1][j][0] = w1[j] & ML;          aL[1][j][1] = (w1[j] >> 8) & ML;
                    aH[1][j][0] = (w1[j] >> 4) & ML;   aH[1][j][1] = (w1[j] >> 12) & ML;
                }
            } else {
                const uint32_t* se = reinterpret_cast<const uint32_t*>(cslot + DATA_BYTES);
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const uint32_t eb = (se[i * 8 + g] >> (8 * t)) & 0xFFu;
                    // 2^(e-127) * 2^14, over the 2^24 every product's final factor carries for the integer-coded formats
                    S[i] = gguf_e8m0_half((uint8_t)eb) * (1.0f / 512.0f);
                }
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    aL[0][j][0] = e2m1x2_to_f16x2(w0[j]);       aL[0][j][1] = e2m1x2_to_f16x2(w0[j] >> 8);
                    aH[0][j][0] = e2m1x2_to_f16x2(w0[j] >> 4);  aH[0][j][1] = e2m1x2_to_f16x2(w0[j] >> 12);
                    aL[1][j][0] = e2m1x2_to_f16x2(w1[j]);       aL[1][j][1] = e2m1x2_to_f16x2(w1[j] >> 8);
                    aH[1][j][0] = e2m1x2_to_f16x2(w1[j] >> 4);  aH[1][j][1] = e2m1x2_to_f16x2(w1[j] >> 12);
                }
            }
#pragma unroll
            for (int n = 0; n < MT; n++) {
                if (n < m) {
                    float cL[4], cH[4];
                    const uint4* bq = bp + n * bn;
                    uint4 b01 = bq[0], b23 = bq[1];
                    mma16816_z(cL, aL[0][0][0], aL[1][0][0], aL[0][0][1], aL[1][0][1], b01.x, b01.y);
                    mma16816(cL, aL[0][1][0], aL[1][1][0], aL[0][1][1], aL[1][1][1], b01.z, b01.w);
                    mma16816(cL, aL[0][2][0], aL[1][2][0], aL[0][2][1], aL[1][2][1], b23.x, b23.y);
                    mma16816(cL, aL[0][3][0], aL[1][3][0], aL[0][3][1], aL[1][3][1], b23.z, b23.w);
                    b01 = bq[bhigh]; b23 = bq[bhigh + 1];
                    mma16816_z(cH, aH[0][0][0], aH[1][0][0], aH[0][0][1], aH[1][0][1], b01.x, b01.y);
                    mma16816(cH, aH[0][1][0], aH[1][1][0], aH[0][1][1], aH[1][1][1], b01.z, b01.w);
                    mma16816(cH, aH[0][2][0], aH[1][2][0], aH[0][2][1], aH[1][2][1], b23.x, b23.y);
                    mma16816(cH, aH[0][3][0], aH[1][3][0], aH[0][3][1], aH[1][3][1], b23.z, b23.w);
                    // Q4_0: d * (sum q x - 8 sum x) over the block; Q8_0: d * (sum (q + 128) x - 128 sum x)
                    const float off = KIND ? sp[n] + sp[m + n] : 0.0f;
#pragma unroll
                    for (int i = 0; i < 2; i++)
                        acc[i][n] = fmaf(S[i], (cL[2 * i] + cL[2 * i + 1]) + (cH[2 * i] + cH[2 * i + 1]) - off, acc[i][n]);
                }
            }
            bp += bstep;
            sp += 8 * m;
            __syncwarp();
            issue_next();
            cslot += SLOT_BYTES;
            if (cslot == cend) cslot = ring_gen;
        }
        finish_tile<MT>(acc, op, sg, xs, tile, m, kw, red, warp, lane);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------- kernel
// Q40K: the instantiation that also carries the GGUF Q4_0 path. Launches without a Q4_0 product use the other
// one, whose code (and register allocation) is exactly that of the three-format kernel.
template <int MT, bool Q40K>
__global__ void __launch_bounds__(256, 2)
gemv_mma_kernel(GOp single, const GOp* __restrict__ ops, int n_ops, const int2* __restrict__ ranges, int total_tiles, int m,
                int ring_d) {
    extern __shared__ __align__(16) uint8_t smem[];
    float* red = reinterpret_cast<float*>(smem);
    const int warp = threadIdx.x >> 5;
    uint8_t* ring_gen = smem + RED_FLOATS * sizeof(float) + warp * ring_d * RING_UNIT_BYTES;
    uint8_t* xbase = smem + RED_FLOATS * sizeof(float) + 8 * ring_d * RING_UNIT_BYTES;
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
    // Programmatic dependent launch: the next kernel of the stream may start its CTAs as ours retire; like this
    // kernel it touches nothing an earlier kernel writes (activations, outputs) before its griddepcontrol.wait,
    // only the immutable packed weights.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    bool first = true;

    for (int seg_b = tb; seg_b < te;) {
        // ---- one product: tiles [seg_b, seg_e) of this CTA belong to it
        GOp op = single;
        if (n_ops > 1) {
            while (opi < n_ops - 1 && seg_b >= ops[opi].tile0 + ops[opi].ntiles) opi++;
            op = ops[opi];
        }
        const int seg_e = min(te, op.tile0 + op.ntiles);
        __syncthreads();   // everyone is done with the previous product's activations and the reduction scratch
        XImg xs = ximg_carve(xbase, op.k, m);
        const bool q5 = Q40K && op.fmt == F_Q5K;
        const bool q4 = op.fmt == F_Q4K || q5;
        auto prep = [&]() {
            if (q4) prep_x<1>(op.x, op.ldx, op.k, m, xs, red, 1.0f);
            else if (op.fmt == F_Q6K) prep_x<0>(op.x, op.ldx, op.k, m, xs, red, 32.0f);
            else prep_x<2>(op.x, op.ldx, op.k, m, xs, red, !Q40K ? 1.0f : op.fmt == F_Q40 ? 8.0f : op.fmt == F_Q80 ? 128.0f : 1.0f);
            __syncthreads();
        };
        // The CTA's first product starts streaming its weights BEFORE it waits for the kernels ahead of it in the
        // stream (whose outputs its activations may be) and builds the activation image; later products find the
        // dependency resolved and prepare first.
        const bool late_prep = first;
        first = false;
        if (!late_prep) prep();
        auto late = [&]() {
            if (late_prep) {
                asm volatile("griddepcontrol.wait;" ::: "memory");
                prep();
            }
        };

        const int kw = 1 << op.kw_log2;
        const int kpart = warp & (kw - 1);
        const int nh = op.k >> 7, per = (nh + kw - 1) >> op.kw_log2;
        Seg sg;
        sg.seg_b = seg_b; sg.seg_e = seg_e;
        sg.hb = kpart * per; sg.he = min(nh, (kpart + 1) * per);
        sg.rt_shift = 3 - op.kw_log2;
        sg.wrow = warp >> op.kw_log2;
        sg.tile0 = op.tile0;
        sg.n_rows = op.n_rows; sg.nh = nh;
        if (q5) run_q4k<MT, Q40K>(op, sg, xs, xbase, ring_gen, ring_d, m, kw, red, late);
        else if (q4) run_q4k<MT, false>(op, sg, xs, xbase, ring_gen, ring_d, m, kw, red, late);
        else if (op.fmt == F_Q6K) run_q6k<MT>(op, sg, xs, xbase, ring_gen, ring_d, m, kw, red, late);
        else if (Q40K && op.fmt == F_Q40) run_mx4<MT, Q40K ? 1 : 0>(op, sg, xs, xbase, ring_gen, ring_d, m, kw, red, late);
        else if (Q40K && op.fmt == F_Q80) run_mx4<MT, Q40K ? 2 : 0>(op, sg, xs, xbase, ring_gen, ring_d, m, kw, red, late);
        else run_mx4<MT, 0>(op, sg, xs, xbase, ring_gen, ring_d, m, kw, red, late);
        seg_b = seg_e;
    }
}

}  // namespace

// Ring depth in units of RING_UNIT_BYTES per warp: 4 when that still lets two CTAs share an SM (or when
// nothing smaller helps), else 2. (Three CTAs per SM with a shallower ring measured slower.)
int gemv_mma_ring_depth(int k, int m) {
    size_t image = XZERO_BYTES + (size_t)(k >> 4) * m * (64 + sizeof(float2)) + 16 + RED_FLOATS * sizeof(float);
    if (image + 8 * 4 * RING_UNIT_BYTES <= 110 * 1024) return 4;
    if (image + 8 * 2 * RING_UNIT_BYTES <= 110 * 1024) return 2;
    return image + 8 * 4 * RING_UNIT_BYTES <= 220 * 1024 ? 4 : 2;
}

size_t gemv_mma_smem_bytes(int fmt, int k, int m) {
    (void)fmt;
    return RED_FLOATS * sizeof(float) + 8 * (size_t)gemv_mma_ring_depth(k, m) * RING_UNIT_BYTES + XZERO_BYTES +
           (size_t)(k >> 4) * m * (64 + sizeof(float2)) + 16;
}

bool gemv_mma_is_q4_0(int fmt) { return fmt == F_Q40 || fmt == F_Q80 || fmt == F_Q5K; }

bool gemv_mma_supported(const b200q_weight* w, int m) {
    if (w->orient != B200Q_ORIENT_NK || m < 1 || m > 8) return false;
    if (w->n_local > 0x7FFFFFF0ll || w->k > (1 << 24) || w->n_elements >= (1ll << 37)) return false;
    if (w->fmt != F_Q4K && w->fmt != F_Q6K && w->fmt != F_MX4 && w->fmt != F_Q40 && w->fmt != F_Q80 && w->fmt != F_Q5K) return false;
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
    return RED_FLOATS * sizeof(float) + 8 * (size_t)ring_d * RING_UNIT_BYTES + XZERO_BYTES +
           (size_t)(kmax >> 4) * m * (64 + sizeof(float2)) + 16;
}

int launch_gemv_mma(b200q_ctx* ctx, const GOp* h_single, const GOp* d_ops, int n_ops, const int2* d_ranges, int n_ctas,
                    int total_tiles, int m, size_t smem_bytes, int ring_d, bool has_q4_0) {
    if (total_tiles <= 0) return B200Q_OK;
    static bool configured[64][4][2] = {};
    const int mi = m <= 1 ? 0 : m <= 2 ? 1 : m <= 4 ? 2 : 3;
    const int qi = has_q4_0 ? 1 : 0;
    const int smem_cap = 226 * 1024;
    const void* kernels[4][2] = {
        {(const void*)gemv_mma_kernel<1, false>, (const void*)gemv_mma_kernel<1, true>},
        {(const void*)gemv_mma_kernel<2, false>, (const void*)gemv_mma_kernel<2, true>},
        {(const void*)gemv_mma_kernel<4, false>, (const void*)gemv_mma_kernel<4, true>},
        {(const void*)gemv_mma_kernel<8, false>, (const void*)gemv_mma_kernel<8, true>}};
    if (!configured[ctx->device & 63][mi][qi]) {
        B200Q_CUDA(cudaFuncSetAttribute(kernels[mi][qi], cudaFuncAttributeMaxDynamicSharedMemorySize, smem_cap), B200Q_ERR_LAUNCH);
        configured[ctx->device & 63][mi][qi] = true;
    }
    GOp single{};
    if (h_single) single = *h_single;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)n_ctas);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // overlap with the tail of the kernel ahead
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    void* args[] = {&single, &d_ops, &n_ops, &d_ranges, &total_tiles, &m, &ring_d};
    cudaError_t le = cudaLaunchKernelExC(&cfg, kernels[mi][qi], args);
    B200Q_CUDA(le, B200Q_ERR_LAUNCH);
    B200Q_CUDA(cudaGetLastError(), B200Q_ERR_LAUNCH);
    return B200Q_OK;
}

}  // namespace b200q
