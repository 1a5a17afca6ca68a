// Prefill kernels: fused dequant + GEMM on the 5th-generation tensor cores (tcgen05, accumulators in TMEM).
//
// Replaces what the reference does for m > 1 today: dequantise the whole tensor to fp32 and call an fp32
// library GEMM with host-side transposes (src/kernels/matmul/quantized/q8_0.rs:69-106,
// src/tensor/matmul.rs:153-214). Here packed weights are expanded tile by tile to f16 next to the tensor
// cores and never touch HBM as fp32.
//
//   y[m, n] = x[m, k] * W[n, k]^T   computed as   D[128 weight rows, BN activation rows] += A * B^T
//
//   A (UMMA M side) : 128 weight rows x 64 k per stage, f16. Three producers, one per kernel below:
//                     gemm_tc_kernel<F>        every format: decode8 (exact fp32 values) + one rounding to f16,
//                                              K-major tile with 128-byte swizzle in SHARED memory
//                     gemm_q4k_tmem_kernel     GGUF Q4_K: raw super-blocks by TMA, converted into TENSOR memory
//                                              (tcgen05.st), TS-form MMA; one CTA per tile
//                     gemm_tmem_sk_kernel<QF>  GGUF Q4_K / Q5_K / Q6_K / MXFP4 / Q4_0 / Q8_0: the same in tensor memory, persistent
//                                              CTAs with a stream-K split over all tiles
//                     (f16, not bf16: an 11-bit mantissa keeps the result inside the 2e-3 tolerance, bf16
//                     weights do not)
//   B (UMMA N side) : BN <= 256 activation rows x 64 k, f16, loaded by TMA (cp.async.bulk.tensor, no
//                     multicast) with 128-byte swizzle. Activations (fp32 or bf16 from the caller) are first
//                     copied to f16 with one power-of-two scale per row, so neither large nor small rows
//                     leave the f16 range; the scale is multiplied back in the epilogue
//   D               : fp32 in tensor memory, 128 lanes x BN columns; read back with tcgen05.ld by eight
//                     warps (two per lane quarter). The persistent kernel scales each warp's 32 x 32 block into
//                     a private shared-memory buffer and writes it with one TMA store per warp (and per rank
//                     of a scattered product); the other kernels store from registers, coalesced along n
//
// Warp roles (384 threads): warp 0 = TMA producer + TMEM allocator, warp 1 = MMA issuer (one elected
// thread), warp 2 = raw-weight loader (tensor-memory kernels), warp 3 = partial-sum publisher and prefetcher
// (persistent kernel), 8 producer / converter warps that are also the epilogue warps. The persistent kernel
// is launched with programmatic stream serialisation: weight copies and conversion start while the
// activation conversion kernel ahead of it still runs (griddepcontrol.wait before the first activation copy). Rings of stages are handed over with mbarriers: full (producer arrivals + TMA
// transaction bytes), empty (tcgen05.commit).
// Every wait is bounded by a clock budget; on expiry the kernel raises a status word, all roles leave
// their loops, outstanding copies are waited for (again bounded), TMEM is freed and the kernel returns.
#include <algorithm>
#include <atomic>
#include <mutex>

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "gemv_i8.cuh"

namespace b200q {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int STAGES = 4;   // power of two: stage = kb & 3, phase = (kb >> 2) & 1
constexpr int NTHREADS = 384;
constexpr int A_STAGE_BYTES = BM * BK * 2;   // 16 KB
constexpr long long WAIT_BUDGET = 1ll << 31; // clock cycles (~1 s) before a wait gives up

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
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
// Waits for the phase with the given parity. The fast path is a bare try_wait loop; every 4096 failed tries
// it looks at the clock and at the CTA's abort flag, gives up after WAIT_BUDGET cycles (or when another role
// already gave up), raises the abort flag and the launch's status word and returns false.
__device__ __forceinline__ bool mbar_wait_for(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                              long long budget) {
    long long t0 = 0;
    for (uint32_t spin = 1;; spin++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 4095u) == 0) {
            if (*abort_flag != 0) return false;
            long long now = clock64();
            if (t0 == 0) t0 = now;
            if (now - t0 > budget) {
                *abort_flag = 1;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
    return mbar_wait_for(bar, parity, abort_flag, status, code, WAIT_BUDGET);
}


__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int cx, int cy, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(cx), "r"(cy)
        : "memory");
}

// Untiled bulk copy global -> shared (both addresses 16-byte aligned, size a multiple of 16), completion on an mbarrier.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// Tiled store shared -> global (clipped at the tensor's edges), tracked by the thread's bulk-copy groups.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int cx, int cy) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(src), "r"(cx), "r"(cy)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// MMA issue: D[tmem] (+)= A[smem desc] * B[smem desc]^T. Descriptors are passed as {lo word computed per
// stage, constant hi word}; the first MMA of a tile overwrites the accumulator, the others accumulate.
__device__ __forceinline__ void umma_f16_acc(uint32_t tmem_d, uint32_t alo, uint32_t ahi, uint32_t blo, uint32_t bhi, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .b64 da, db;\n\t.reg .pred p;\n\t"
        "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
        "setp.eq.b32 p, 1, 1;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
        ::"r"(tmem_d), "r"(alo), "r"(ahi), "r"(blo), "r"(bhi), "r"(idesc)
        : "memory");
}
__device__ __forceinline__ void umma_f16_first(uint32_t tmem_d, uint32_t alo, uint32_t ahi, uint32_t blo, uint32_t bhi, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .b64 da, db;\n\t.reg .pred p;\n\t"
        "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
        "setp.eq.b32 p, 1, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
        ::"r"(tmem_d), "r"(alo), "r"(ahi), "r"(blo), "r"(bhi), "r"(idesc)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// A operand read from tensor memory (lanes = rows, two f16 per 32-bit column), B from a shared-memory descriptor.
__device__ __forceinline__ void umma_ts_f16_acc(uint32_t tmem_d, uint32_t tmem_a, uint32_t blo, uint32_t bhi, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .b64 db;\n\t.reg .pred p;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "setp.eq.b32 p, 1, 1;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "r"(blo), "r"(bhi), "r"(idesc)
        : "memory");
}
__device__ __forceinline__ void umma_ts_f16_first(uint32_t tmem_d, uint32_t tmem_a, uint32_t blo, uint32_t bhi, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .b64 db;\n\t.reg .pred p;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "setp.eq.b32 p, 1, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "r"(blo), "r"(bhi), "r"(idesc)
        : "memory");
}

// Each thread of the warp writes 16 consecutive 32-bit columns of its own TMEM lane.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
          "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// K-major operand tile with 128-byte swizzle: rows at a 128-byte pitch, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFFu);   // start address
    d |= (uint64_t)1 << 16;                        // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                        // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Specialised A-tile producer for GGUF Q4_K: two threads expand the 64 weights of one row of the k-block
// (one 32-byte chunk: low nibbles = sub-block 2c, high nibbles = sub-block 2c+1) to f16, 16 bytes each.
//   (w & 0x000F000F) | 0x64006400  is the f16 pair (1024 + q_byte0, 1024 + q_byte2); minus 1024 gives q exactly;
//   one HFMA2 forms q * (d*sc) - dmin*m with a single rounding. High nibbles stay in bits 4..7 (1024 + 16 q)
//   and use (d*sc)/16. Weights come out in the order 0,2,1,3 inside each group of four; the f16 copy of the
//   activations is stored in the same order, so no byte shuffles are needed.
struct Q4KRaw {
    uint4 hdr, q;
    int c;   // chunk of the super-block (0..3)
};

__device__ __forceinline__ Q4KRaw q4k_load_raw(const uint8_t* __restrict__ base, int64_t chunk_index, int half) {
    const uint8_t* sb = base + (chunk_index >> 2) * 144;
    Q4KRaw r;
    r.c = (int)(chunk_index & 3);
    r.hdr = __ldg(reinterpret_cast<const uint4*>(sb));
    r.q = __ldg(reinterpret_cast<const uint4*>(sb + 16 + r.c * 32 + half * 16));
    return r;
}

// half: which 16 bytes of the chunk (weights 16*half .. 16*half+15 of both sub-blocks); r: row inside the tile.
__device__ __forceinline__ void q4k_convert(const Q4KRaw& raw, int half, int r, uint8_t* tile) {
    const uint4 hdr = raw.hdr;
    const int c = raw.c;
    const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xFFFFu)));
    const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
    uint32_t scA, scB, mA, mB;
    {
        const uint32_t sc_lo = hdr.y & 0x3F3F3F3Fu, m_lo = hdr.z & 0x3F3F3F3Fu;
        const uint32_t sc_hi = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
        const uint32_t m_hi = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
        const uint32_t scw = c < 2 ? sc_lo : sc_hi, mw = c < 2 ? m_lo : m_hi;
        const int sh = (c & 1) * 16;
        scA = (scw >> sh) & 0xFFu; scB = (scw >> (sh + 8)) & 0xFFu;
        mA = (mw >> sh) & 0xFFu; mB = (mw >> (sh + 8)) & 0xFFu;
    }
    const __half2 dsA = __float2half2_rn(d * (float)scA), dsB = __float2half2_rn(d * (float)scB * 0.0625f);
    const __half2 ndA = __float2half2_rn(-dmin * (float)mA), ndB = __float2half2_rn(-dmin * (float)mB);
    const __half2 k1024 = __float2half2_rn(1024.0f);
    const uint32_t MAGIC = 0x64006400u, ML = 0x000F000Fu, MH = 0x00F000F0u;
    const uint32_t w[4] = {raw.q.x, raw.q.y, raw.q.z, raw.q.w};
    uint32_t lo[8], hi[8];   // f16x2 weights of sub-block A (k 0..31 of the block) and B (k 32..63)
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const uint32_t v = w[j], vs = v >> 8;
        uint32_t t0 = (v & ML) | MAGIC, t1 = (vs & ML) | MAGIC, t2 = (v & MH) | MAGIC, t3 = (vs & MH) | MAGIC;
        __half2 a0 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&t0), k1024), dsA, ndA);
        __half2 a1 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&t1), k1024), dsA, ndA);
        __half2 b0 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&t2), k1024), dsB, ndB);
        __half2 b1 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&t3), k1024), dsB, ndB);
        lo[2 * j] = *reinterpret_cast<uint32_t*>(&a0); lo[2 * j + 1] = *reinterpret_cast<uint32_t*>(&a1);
        hi[2 * j] = *reinterpret_cast<uint32_t*>(&b0); hi[2 * j + 1] = *reinterpret_cast<uint32_t*>(&b1);
    }
    uint8_t* rowp = tile + r * 128;
#pragma unroll
    for (int cc = 0; cc < 2; cc++) {   // 16-byte chunks 2*half+cc (sub-block A) and 4+2*half+cc (sub-block B)
        const int ca = 2 * half + cc;
        *reinterpret_cast<uint4*>(rowp + ((ca ^ (r & 7)) << 4)) = make_uint4(lo[4 * cc], lo[4 * cc + 1], lo[4 * cc + 2], lo[4 * cc + 3]);
        *reinterpret_cast<uint4*>(rowp + (((ca + 4) ^ (r & 7)) << 4)) = make_uint4(hi[4 * cc], hi[4 * cc + 1], hi[4 * cc + 2], hi[4 * cc + 3]);
    }
}

struct GemmArgs {
    WView v;
    const float* xscale;   // per activation row: the power of two its f16 copy was divided by
    float* y;
    int64_t ldy;
    int n_rows, k, m, bn, tmem_cols;
    int a_col0;            // first TMEM column of the weight-operand slots (kernel with the A operand in TMEM)
    int* status;
    int n_extra;           // further copies of y to write: the same slice inside other GPUs' full outputs
    float* y_extra[7];     // (peer-mapped pointers; stores over NVLink only, plain or TMA, never loads)
    int staged_epilogue;   // persistent kernel: finished tiles leave through shared memory and tiled TMA stores
    int y_bf16;            // staged epilogue only: y (and its copies on other GPUs) are bf16, rounded once from fp32
};

// Warp roles (384 threads = 12 warps; a warp may only read the TMEM lane quarter warp_id % 4):
//   warp 0          TMA producer for the activation tiles, TMEM allocator
//   warp 1          MMA issuer (one thread). Warps 5 and 9 share its scheduler and therefore stay asleep on a
//                   hardware barrier during the main loop: the issuer's instruction stream is the critical path
//   warps 2,3,4,6,7,8,10,11   weight-tile producers (two threads per weight row)
//   epilogue        warps 4,5,6,7 (lane quarters 0,1,2,3) take the even 32-column groups, warps 8,9,10,11 the odd
__device__ __forceinline__ bool is_producer_warp(int warp) { return warp >= 2 && warp != 5 && warp != 9; }
// dense index 0..7 of a producer warp
__device__ __forceinline__ int producer_index(int warp) { return warp - 2 - (warp > 5) - (warp > 9); }

template <int F>
__global__ void __launch_bounds__(NTHREADS, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, GemmArgs a) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte aligned by an OFFSET on the shared array (a round trip through an integer would hide the
    // address space from the compiler and turn every access below into a generic one)
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int b_stage_bytes = a.bn * BK * 2;
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sB + STAGES * b_stage_bytes);
    uint64_t* full_a = bars;
    uint64_t* full_b = bars + STAGES;
    uint64_t* empty = bars + 2 * STAGES;
    uint64_t* accum = bars + 3 * STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * STAGES + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row0 = blockIdx.x * BM;
    const int tok0 = blockIdx.y * a.bn;
    const int nkb = a.k / BK;

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(smem_u32(&full_a[s]), 9);   // 8 producer warps + the TMA thread's expect_tx arrival
            mbar_init(smem_u32(&full_b[s]), 1);   // unused (kept so the barrier block keeps its layout)
            mbar_init(smem_u32(&empty[s]), 1);
        }
        mbar_init(smem_u32(accum), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)a.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer (activations)
        if (lane == 0) {
            int issued = 0;
            for (int kb = 0; kb < nkb; kb++) {
                const int s = kb & (STAGES - 1);
                const uint32_t ph = (kb >> 2) & 1;
                if (!mbar_wait(smem_u32(&empty[s]), ph ^ 1, abort_flag, a.status, 1)) break;
                mbar_arrive_expect_tx(smem_u32(&full_a[s]), (uint32_t)b_stage_bytes);
                tma_load_2d(smem_u32(sB + s * b_stage_bytes), &tmap_x, kb * BK, tok0, smem_u32(&full_a[s]));
                issued = kb + 1;
            }
            // do not leave copies in flight behind: the last STAGES tiles issued must have landed
            for (int kb = max(0, issued - STAGES); kb < issued; kb++) {
                const int s = kb & (STAGES - 1);
                const uint32_t ph = (kb >> 2) & 1;
                long long t0 = clock64();
                while (!mbar_try_wait(smem_u32(&full_a[s]), ph)) {
                    if (clock64() - t0 > WAIT_BUDGET) { atomicCAS(a.status, 0, 5); break; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            // D fp32, A and B f16. The two operand formats of kind::f16 must be equal: f16 weights with bf16
            // activations raise an illegal-instruction fault on sm_100a.
            const uint32_t idesc = (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(a.bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            const uint64_t adesc0 = umma_desc_sw128(smem_u32(sA));
            const uint64_t bdesc0 = umma_desc_sw128(smem_u32(sB));
            const uint32_t ahi = (uint32_t)(adesc0 >> 32), bhi = (uint32_t)(bdesc0 >> 32);
            const uint32_t alo0 = (uint32_t)adesc0, blo0 = (uint32_t)bdesc0;
            const uint32_t a_step = (uint32_t)(A_STAGE_BYTES >> 4), b_step = (uint32_t)(b_stage_bytes >> 4);
            const uint32_t fu0 = smem_u32(full_a), em0 = smem_u32(empty);
            for (int kb = 0; kb < nkb; kb++) {
                const uint32_t s = (uint32_t)kb & (STAGES - 1);
                const uint32_t ph = ((uint32_t)kb >> 2) & 1;
                if (!mbar_wait(fu0 + s * 8, ph, abort_flag, a.status, 2)) break;
                tc_fence_after();
                const uint32_t al = alo0 + s * a_step, bl = blo0 + s * b_step;
                // 16 f16 = 32 bytes further along k inside the swizzle atom: +2 in the encoded address
                if (kb == 0) umma_f16_first(tmem_base, al, ahi, bl, bhi, idesc);
                else umma_f16_acc(tmem_base, al, ahi, bl, bhi, idesc);
                umma_f16_acc(tmem_base, al + 2, ahi, bl + 2, bhi, idesc);
                umma_f16_acc(tmem_base, al + 4, ahi, bl + 4, bhi, idesc);
                umma_f16_acc(tmem_base, al + 6, ahi, bl + 6, bhi, idesc);
                umma_commit(em0 + s * 8);
            }
            umma_commit(smem_u32(accum));   // arrives once every MMA issued so far has completed
        }
    } else if (is_producer_warp(warp)) {
        // ---------------------------------------------------------------- weight-tile producers
        const int dt = producer_index(warp) * 32 + lane;   // 0..255
        constexpr bool FAST = F == fmt_of(Q4_K, GGUF);
        Q4KRaw pre{};
        const int64_t frow = min((int64_t)row0 + (dt >> 1), (int64_t)a.n_rows - 1);
        const int64_t fchunk0 = (frow * a.k) >> 6;
        if (FAST && nkb > 0) pre = q4k_load_raw(a.v.p[0], fchunk0, dt & 1);
        for (int kb = 0; kb < nkb && ok; kb++) {
            const int s = kb & (STAGES - 1);
            const uint32_t ph = (kb >> 2) & 1;
            Q4KRaw cur = pre;
            if (FAST && kb + 1 < nkb) pre = q4k_load_raw(a.v.p[0], fchunk0 + kb + 1, dt & 1);   // next block's bytes fly while this one converts
            // one lane polls, the warp follows: keeps the shared-memory pipe free for the MMA issuer
            if (lane == 0) ok = mbar_wait(smem_u32(&empty[s]), ph ^ 1, abort_flag, a.status, 4);
            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
            if (!ok) break;
            uint8_t* tile = sA + s * A_STAGE_BYTES;
            if constexpr (FAST) {
                q4k_convert(cur, dt & 1, dt >> 1, tile);
            } else {
#pragma unroll 2
                for (int it = 0; it < (BM * BK / 8) / 256; it++) {
                    const int idx = it * 256 + dt;
                    const int r = idx >> 3, c = idx & 7;
                    const int64_t row = min((int64_t)row0 + r, (int64_t)a.n_rows - 1);
                    const int64_t piece = (row * a.k + (int64_t)kb * BK + c * 8) >> 3;
                    float w[8];
                    decode8<F>(a.v, piece >> 2, (int)(piece & 3), w);
                    __half2 p0 = __floats2half2_rn(w[0], w[1]), p1 = __floats2half2_rn(w[2], w[3]);
                    __half2 p2 = __floats2half2_rn(w[4], w[5]), p3 = __floats2half2_rn(w[6], w[7]);
                    uint4 pk;
                    pk.x = *reinterpret_cast<uint32_t*>(&p0); pk.y = *reinterpret_cast<uint32_t*>(&p1);
                    pk.z = *reinterpret_cast<uint32_t*>(&p2); pk.w = *reinterpret_cast<uint32_t*>(&p3);
                    *reinterpret_cast<uint4*>(tile + r * 128 + ((c ^ (r & 7)) << 4)) = pk;
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> tensor-core reads
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&full_a[s]));
        }
    }
    // ---------------------------------------------------------------- epilogue: warps 4..11
    if (warp >= 4) {
        // warp 4 waits for the accumulator, everyone else sleeps on hardware barrier 1 until it is released
        if (warp == 4) {
            if (lane == 0 && ok) ok = mbar_wait(smem_u32(accum), 0, abort_flag, a.status, 6);
            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
            if (!ok) *abort_flag = 1;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (*abort_flag == 0) {
            tc_fence_after();
            const int q = warp & 3;                       // the lane quarter this warp may read
            const int row = row0 + q * 32 + lane;
            for (int c0 = (warp >= 8 ? 32 : 0); c0 < a.bn; c0 += 64) {
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
                if (row < a.n_rows) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int tok = tok0 + c0 + j;
                        if (tok < a.m) {
                                const float val = __uint_as_float(v[j]) * __ldg(a.xscale + tok);
                                a.y[(int64_t)tok * a.ldy + row] = val;
                                for (int pp = 0; pp < a.n_extra; pp++) a.y_extra[pp][(int64_t)tok * a.ldy + row] = val;
                            }
                    }
                }
            }
        }
    }
    // ---------------------------------------------------------------- teardown (every path ends here)
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)a.tmem_cols) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------
// GGUF Q4_K with the weight operand in tensor memory.
//
// With both operands in shared memory the kernel above is bound by the SM's shared-memory data pipe: per 64-k
// block it carries the TMA writes and tensor-core reads of the activation tile (32 KB each), the producers'
// scattered global loads, their 16 KB of f16 stores and the tensor-core reads of those. Here the weights never
// exist as f16 in shared memory:
//   * warp 2 copies the raw super-blocks (144 bytes per row per 256 k) with one tiled TMA copy per 128 rows
//     into a 3-deep ring: 18 KB per 256 k instead of 64 KB of f16 (one copy per row was tried first and was
//     bound by the copy engine's request rate);
//   * warps 4..11 (thread = weight row; warps 4-7 take the low nibbles = first 32 k of each 64-k chunk, warps
//     8-11 the high nibbles = last 32 k) expand 32 weights to 16 packed f16x2 registers and write them with
//     tcgen05.st into the TMEM slot of the stage (32 columns per stage: lane = row, column c = k 2c, 2c+1);
//   * the MMA takes A from TMEM ([taddr] operand) and B from the swizzled shared-memory tile as before.
// TMEM columns: [0, bn) accumulator, [a_col0, a_col0 + 32 * STAGES) weight slots.
constexpr int RAW_STAGES = 3;
constexpr int RAW_ROW_BYTES = 144;
constexpr int RAW_STAGE_BYTES = BM * RAW_ROW_BYTES;   // 18,432
constexpr int A_SLOT_COLS = BK / 2;                   // 32

__global__ void __launch_bounds__(NTHREADS, 1) gemm_q4k_tmem_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, GemmArgs a) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte aligned by an OFFSET on the shared array (a round trip through an integer would hide the
    // address space from the compiler and turn every access below into a generic one)
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int b_stage_bytes = a.bn * BK * 2;
    uint8_t* sB = smem;
    uint8_t* sRaw = sB + STAGES * b_stage_bytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sRaw + RAW_STAGES * RAW_STAGE_BYTES);
    uint64_t* full = bars;                            // 8 converter warps + the TMA thread's expect_tx arrival
    uint64_t* empty = bars + STAGES;                  // tcgen05.commit
    uint64_t* raw_full = bars + 2 * STAGES;           // bulk-copy bytes
    uint64_t* raw_empty = raw_full + RAW_STAGES;      // 8 converter warps
    uint64_t* accum = raw_empty + RAW_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row0 = blockIdx.x * BM;
    const int tok0 = blockIdx.y * a.bn;
    const int nkb = a.k / BK;
    const int nsb = a.k >> 8;

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(smem_u32(&full[s]), 9);
            mbar_init(smem_u32(&empty[s]), 1);
        }
        for (int s = 0; s < RAW_STAGES; s++) {
            mbar_init(smem_u32(&raw_full[s]), 1);
            mbar_init(smem_u32(&raw_empty[s]), 8);
        }
        mbar_init(smem_u32(accum), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)a.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer (activations)
        if (lane == 0) {
            int issued = 0;
            for (int kb = 0; kb < nkb; kb++) {
                const int s = kb & (STAGES - 1);
                const uint32_t ph = (kb >> 2) & 1;
                if (!mbar_wait(smem_u32(&empty[s]), ph ^ 1, abort_flag, a.status, 1)) break;
                mbar_arrive_expect_tx(smem_u32(&full[s]), (uint32_t)b_stage_bytes);
                tma_load_2d(smem_u32(sB + s * b_stage_bytes), &tmap_x, kb * BK, tok0, smem_u32(&full[s]));
                issued = kb + 1;
            }
            for (int kb = max(0, issued - STAGES); kb < issued; kb++) {   // nothing stays in flight behind us
                const int s = kb & (STAGES - 1);
                const uint32_t ph = (kb >> 2) & 1;
                long long t0 = clock64();
                while (!mbar_try_wait(smem_u32(&full[s]), ph)) {
                    if (clock64() - t0 > WAIT_BUDGET) { atomicCAS(a.status, 0, 5); break; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(a.bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            const uint64_t bdesc0 = umma_desc_sw128(smem_u32(sB));
            const uint32_t bhi = (uint32_t)(bdesc0 >> 32), blo0 = (uint32_t)bdesc0;
            const uint32_t b_step = (uint32_t)(b_stage_bytes >> 4);
            const uint32_t fu0 = smem_u32(full), em0 = smem_u32(empty);
            const uint32_t at0 = tmem_base + (uint32_t)a.a_col0;
            for (int kb = 0; kb < nkb; kb++) {
                const uint32_t s = (uint32_t)kb & (STAGES - 1);
                const uint32_t ph = ((uint32_t)kb >> 2) & 1;
                if (!mbar_wait(fu0 + s * 8, ph, abort_flag, a.status, 2)) break;
                tc_fence_after();
                const uint32_t at = at0 + s * A_SLOT_COLS, bl = blo0 + s * b_step;
                // 16 k further: 8 TMEM columns on the A side, 32 bytes (+2 encoded) inside the swizzle atom on the B side
                if (kb == 0) umma_ts_f16_first(tmem_base, at, bl, bhi, idesc);
                else umma_ts_f16_acc(tmem_base, at, bl, bhi, idesc);
                umma_ts_f16_acc(tmem_base, at + 8, bl + 2, bhi, idesc);
                umma_ts_f16_acc(tmem_base, at + 16, bl + 4, bhi, idesc);
                umma_ts_f16_acc(tmem_base, at + 24, bl + 6, bhi, idesc);
                umma_commit(em0 + s * 8);
            }
            umma_commit(smem_u32(accum));
        }
    } else if (warp == 2) {
        // ---------------------------------------------------------------- raw super-block loader
        // The packed tensor is a 2-D byte array [n_rows, k / 256 * 144]; one tiled copy brings the 144-byte
        // super-block of each of the 128 rows (rows past the end of the tensor read as zeros = zero weights).
        if (lane == 0) {
            int issued = 0;
            for (int sb = 0; sb < nsb; sb++) {
                const int rs = sb % RAW_STAGES;
                const uint32_t ph = (uint32_t)(sb / RAW_STAGES) & 1;
                if (!mbar_wait(smem_u32(&raw_empty[rs]), ph ^ 1, abort_flag, a.status, 7)) break;
                mbar_arrive_expect_tx(smem_u32(&raw_full[rs]), (uint32_t)RAW_STAGE_BYTES);
                tma_load_2d(smem_u32(sRaw + rs * RAW_STAGE_BYTES), &tmap_w, sb * RAW_ROW_BYTES, row0, smem_u32(&raw_full[rs]));
                issued = sb + 1;
            }
            for (int sb = max(0, issued - RAW_STAGES); sb < issued; sb++) {   // every copy issued has landed
                const int rs = sb % RAW_STAGES;
                const uint32_t ph = (uint32_t)(sb / RAW_STAGES) & 1;
                long long t0 = clock64();
                while (!mbar_try_wait(smem_u32(&raw_full[rs]), ph)) {
                    if (clock64() - t0 > WAIT_BUDGET) { atomicCAS(a.status, 0, 9); break; }
                }
            }
        }
    } else if (warp >= 4) {
        // ---------------------------------------------------------------- converters: raw bytes -> f16 in TMEM
        const int q = warp & 3;                 // TMEM lane quarter this warp may touch
        const int nib = (warp - 4) >> 2;        // 0: low nibbles (k 0..31 of a chunk), 1: high nibbles (k 32..63)
        const int r = q * 32 + lane;
        const uint32_t slot0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)a.a_col0 + (uint32_t)nib * 16;
        const uint32_t mask = nib ? 0x00F000F0u : 0x000F000Fu;
        const float nibscale = nib ? 0.0625f : 1.0f;
        const __half2 k1024 = __float2half2_rn(1024.0f);
        for (int sb = 0; sb < nsb && ok; sb++) {
            const int rs = sb % RAW_STAGES;
            const uint32_t rph = (uint32_t)(sb / RAW_STAGES) & 1;
            if (lane == 0) ok = mbar_wait(smem_u32(&raw_full[rs]), rph, abort_flag, a.status, 8);
            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
            if (!ok) break;
            const uint8_t* rowp = sRaw + rs * RAW_STAGE_BYTES + r * RAW_ROW_BYTES;
            const uint4 hdr = *reinterpret_cast<const uint4*>(rowp);
            const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xFFFFu)));
            const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
            const uint32_t sc_lo = hdr.y & 0x3F3F3F3Fu, m_lo = hdr.z & 0x3F3F3F3Fu;
            const uint32_t sc_hi = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
            const uint32_t m_hi = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const int kb = sb * 4 + c;
                const int s = kb & (STAGES - 1);
                const uint32_t ph = (uint32_t)(kb >> 2) & 1;
                // sub-block 2c + nib of the super-block: byte (2 (c & 1) + nib) of the low or high scale word
                const int sh = ((c & 1) * 2 + nib) * 8;
                const uint32_t sc = ((c < 2 ? sc_lo : sc_hi) >> sh) & 0xFFu, mn = ((c < 2 ? m_lo : m_hi) >> sh) & 0xFFu;
                const __half2 ds = __float2half2_rn(d * (float)sc * nibscale);
                const __half2 nd = __float2half2_rn(-dmin * (float)mn);
                const uint4 qa = *reinterpret_cast<const uint4*>(rowp + 16 + c * 32);
                const uint4 qb = *reinterpret_cast<const uint4*>(rowp + 32 + c * 32);
                const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
                uint32_t v[16];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    uint32_t t0 = (w[j] & mask) | 0x64006400u, t1 = ((w[j] >> 8) & mask) | 0x64006400u;
                    __half2 h0 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&t0), k1024), ds, nd);
                    __half2 h1 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&t1), k1024), ds, nd);
                    v[2 * j] = *reinterpret_cast<uint32_t*>(&h0);
                    v[2 * j + 1] = *reinterpret_cast<uint32_t*>(&h1);
                }
                if (lane == 0) ok = mbar_wait(smem_u32(&empty[s]), ph ^ 1, abort_flag, a.status, 4);
                ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
                if (!ok) break;
                tc_fence_after();
                tmem_st16(slot0 + (uint32_t)s * A_SLOT_COLS, v);
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&full[s]));
            }
            if (!ok) break;
            __syncwarp();   // every lane has read its bytes of this raw stage
            if (lane == 0) mbar_arrive(smem_u32(&raw_empty[rs]));
        }
        // ------------------------------------------------------------ epilogue (same warps)
        if (warp == 4) {
            if (lane == 0 && ok) ok = mbar_wait(smem_u32(accum), 0, abort_flag, a.status, 6);
            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
            if (!ok) *abort_flag = 1;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (*abort_flag == 0) {
            tc_fence_after();
            const int row = row0 + q * 32 + lane;
            for (int c0 = (warp >= 8 ? 32 : 0); c0 < a.bn; c0 += 64) {
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
                if (row < a.n_rows) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int tok = tok0 + c0 + j;
                        if (tok < a.m) {
                                const float val = __uint_as_float(v[j]) * __ldg(a.xscale + tok);
                                a.y[(int64_t)tok * a.ldy + row] = val;
                                for (int pp = 0; pp < a.n_extra; pp++) a.y_extra[pp][(int64_t)tok * a.ldy + row] = val;
                            }
                    }
                }
            }
        }
    }
    // ---------------------------------------------------------------- teardown (every path ends here)
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)a.tmem_cols) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------
// Persistent form of the kernel above: one CTA per SM, work split evenly in units of one super-block step
// (128 weight rows x bn activation rows x 256 k) over ALL tiles, so 172 tiles on 148 SMs cost 1.16 tile
// times instead of 2. A CTA's range is a run of consecutive (tile, super-block) units: it may begin in the
// middle of a tile and end in the middle of another.
//   * A segment that does not start at k = 0 is a partial sum: it is written raw (fp32, unscaled) to the
//     CTA's workspace slot and published with a flag that carries the launch number.
//   * The CTA whose segment starts at k = 0 owns the tile: after its own part it adds the partial sums of
//     the following CTAs, in CTA order (deterministic), scales and stores. Those CTAs computed their parts
//     first thing in their ranges, the owner computes its part last, so the owner normally finds the flags
//     already set; the wait is bounded like every other wait.
// Only the first segment of a CTA can be a partial one, hence one workspace slot per CTA.
struct SkArgs {
    GemmArgs a;
    int tiles_x;         // tiles along the weight rows; tile t = (t % tiles_x, t / tiles_x)
    int nsb;             // super-blocks (256 k) per tile
    int total_units;     // tiles * nsb
    float* ws;           // [gridDim.x][bn][128] partial accumulators
    int* flags;          // [gridDim.x]
    int epoch;
    // MXFP6 (QF 6): the tensor's decode image (items of 16 rows x 128 k, 2048 code bytes + 64 exponent bytes each)
    const uint8_t* img;
    int img_nh;          // items per row tile
    int img_nrt;         // row tiles of 16 rows
    int img_e3m2;        // the image's bytes are E3M2 codes spread to s00eeemm (high bytes of f16 value * 2^-12), not int8 codes
};

constexpr int SK_SLOT_FLOATS = BM * 256;

__device__ __forceinline__ int sk_unit_begin(int cta, int total, int ctas) { return (int)(((int64_t)cta * total) / ctas); }

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// QF selects the weight format: 0 = GGUF Q4_K (raw rows of 144-byte super-blocks), 1 = GGUF MXFP4 (raw rows of
// 8 x 16 code bytes per 256 k from the code plane; the 8 exponent bytes come by a plain load). MXFP4 codes
// become f16 by bit placement (E2M1 s|ee|m at bits 15|11..9 is value * 2^-14) and one HMUL2 with the block
// scale 2^(e-127) * 2^14, which has to lie in the f16 range (block exponents 2^-28 .. 2^1).
// Output tensor maps of the other GPUs' buffers for a scattered product (peer-mapped memory; TMA STORES only)
struct PeerMaps {
    CUtensorMap m[7];
};

template <int QF>
__global__ void __launch_bounds__(NTHREADS, 1)
gemm_tmem_sk_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                    const __grid_constant__ CUtensorMap tmap_w2, const __grid_constant__ CUtensorMap tmap_w3,
                    const __grid_constant__ CUtensorMap tmap_y, const __grid_constant__ CUtensorMap tmap_ws,
                    const __grid_constant__ PeerMaps peers, SkArgs k) {
    // bytes of one weight row per 256-k step in the raw ring; Q6_K keeps its three planes one after the other
    // inside a stage: [128 rows x 128 B ql][128 rows x 64 B qh][128 rows x 16 B scales]
    // QF 3 = GGUF Q4_0: MXFP4's code rows; QF 4 = GGUF Q8_0: 256 code bytes per row and step, two 128-byte boxes
    // QF 5 = GGUF Q5_K: Q4_K's block with 32 bytes of fifth bits (qh) between the scales and the nibbles
    // QF 6 = GGUF MXFP6 E2M3 from the decode image: codes widened to int8 (8 x value) at upload, 256 bytes per row and step,
    //        fetched as the 2048 code bytes of 16 items (8 row tiles x 2 k-halves) by untiled bulk copies
    constexpr int RAW_ROW_BYTES = QF == 0 ? 144 : QF == 5 ? 176 : (QF == 1 || QF == 3) ? 128 : (QF == 4 || QF == 6) ? 256 : 208;
    constexpr int RAW_STAGE_BYTES = BM * RAW_ROW_BYTES;
    constexpr int RS = (QF == 2 || QF == 4 || QF == 5 || QF == 6) ? 2 : RAW_STAGES;   // raw ring depth; Q6_K's 26 KB stages leave room for two beside the staging tile
    const GemmArgs& a = k.a;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte aligned by an OFFSET on the shared array (a round trip through an integer would hide the
    // address space from the compiler and turn every access below into a generic one)
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int b_stage_bytes = a.bn * BK * 2;
    uint8_t* sB = smem;
    uint8_t* sRaw = sB + STAGES * b_stage_bytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sRaw + RS * RAW_STAGE_BYTES);
    uint64_t* full = bars;
    uint64_t* empty = bars + STAGES;
    uint64_t* raw_full = bars + 2 * STAGES;
    uint64_t* raw_empty = raw_full + RS;
    uint64_t* accum = raw_empty + RS;    // MMAs of a segment complete -> epilogue
    uint64_t* dfree = accum + 1;                 // epilogue has read the accumulator -> next segment's MMAs
    uint64_t* pfull = dfree + 1;                 // [4] rounds of a partial tile prefetched into the idle activation stages
    uint64_t* pgo = pfull + 4;                   // MMAs of the CTA's last segment complete -> the stages are idle
    uint64_t* gfree = pgo + 1;                   // [2] staging tile of an epilogue group may be overwritten (its stores have read it)
    uint64_t* gready = gfree + 2;                // [2] the four warps of a group have written their blocks
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gready + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* stored = const_cast<int*>(abort_flag) + 1;   // epilogue warps whose partial-sum stores are fenced
    // staging tiles of the epilogue: per group of four warps 32 activation rows x 128 weight rows of fp32 (one TMA store box)
    float* stg = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(stored + 1) + ((128u - (smem_u32(stored + 1) & 127u)) & 127u));

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x, nctas = gridDim.x;
    const int u0 = sk_unit_begin(cta, k.total_units, nctas), u1 = sk_unit_begin(cta + 1, k.total_units, nctas);

    if (tid == 0) {
        for (int s = 0; s < STAGES / 2; s++) {   // one pair of barriers per PAIR of stages
            mbar_init(smem_u32(&full[s]), 9);    // 8 converter warps + the TMA thread's expect_tx arrival
            mbar_init(smem_u32(&empty[s]), 1);   // tcgen05.commit
        }
        for (int s = 0; s < RS; s++) {
            mbar_init(smem_u32(&raw_full[s]), 1);
            mbar_init(smem_u32(&raw_empty[s]), 8);
        }
        mbar_init(smem_u32(accum), 1);
        mbar_init(smem_u32(dfree), 8);
        for (int s = 0; s < 4; s++) mbar_init(smem_u32(&pfull[s]), 1);
        mbar_init(smem_u32(pgo), 1);
        for (int s = 0; s < 2; s++) {
            mbar_init(smem_u32(&gfree[s]), 1);
            mbar_init(smem_u32(&gready[s]), 4);
        }
        *abort_flag = 0;
        *stored = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)a.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // a kernel behind this one may start its CTAs as ours retire

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer (activations)
        if (lane == 0) {
            // programmatic dependent launch: the f16 activations come from the kernel ahead of this one; the raw
            // weight copies and their conversion into tensor memory (warps 2, 4..11) do not wait for it
            asm volatile("griddepcontrol.wait;" ::: "memory");
            int it = 0;
            for (int u = u0; u < u1 && ok;) {
                const int tile = u / k.nsb, sb0 = u - tile * k.nsb, sb1 = min(k.nsb, sb0 + (u1 - u));
                const int tok0 = (tile / k.tiles_x) * a.bn;
                for (int kb = 4 * sb0; kb < 4 * sb1; kb += 2, it += 2) {
                    const int s = it & (STAGES - 1);                    // first stage of the pair
                    const uint32_t ph = (it >> 2) & 1;
                    const uint32_t fb = smem_u32(&full[s >> 1]);
                    {
                    if (!mbar_wait(smem_u32(&empty[s >> 1]), ph ^ 1, abort_flag, a.status, 1)) { ok = false; break; }
 }
                    mbar_arrive_expect_tx(fb, 2u * (uint32_t)b_stage_bytes);
                    tma_load_2d(smem_u32(sB + s * b_stage_bytes), &tmap_x, kb * BK, tok0, fb);
                    tma_load_2d(smem_u32(sB + (s + 1) * b_stage_bytes), &tmap_x, (kb + 1) * BK, tok0, fb);
                }
                u += sb1 - sb0;
            }
            for (int j = max(0, it - STAGES); j < it; j += 2) {   // nothing stays in flight behind us
                const int s = j & (STAGES - 1);
                const uint32_t ph = (j >> 2) & 1;
                long long t0 = clock64();
                while (!mbar_try_wait(smem_u32(&full[s >> 1]), ph)) {
                    if (clock64() - t0 > WAIT_BUDGET) { atomicCAS(a.status, 0, 5); break; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(a.bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            const uint64_t bdesc0 = umma_desc_sw128(smem_u32(sB));
            const uint32_t bhi = (uint32_t)(bdesc0 >> 32), blo0 = (uint32_t)bdesc0;
            const uint32_t b_step = (uint32_t)(b_stage_bytes >> 4);
            const uint32_t fu0 = smem_u32(full), em0 = smem_u32(empty);
            const uint32_t at0 = tmem_base + (uint32_t)a.a_col0;
            int it = 0, seg = 0;
            for (int u = u0; u < u1 && ok; seg++) {
                const int tile = u / k.nsb, sb0 = u - tile * k.nsb, sb1 = min(k.nsb, sb0 + (u1 - u));
                // the previous segment's accumulator must have been read out
                if (!mbar_wait(smem_u32(dfree), (uint32_t)(seg & 1) ^ 1, abort_flag, a.status, 10)) break;
                tc_fence_after();
                for (int kb = 4 * sb0; kb < 4 * sb1; kb += 2, it += 2) {
                    const uint32_t s = (uint32_t)it & (STAGES - 1);     // first stage of the pair
                    const uint32_t ph = ((uint32_t)it >> 2) & 1;
                    {
                    if (!mbar_wait(fu0 + (s >> 1) * 8, ph, abort_flag, a.status, 2)) { ok = false; break; }
 }
                    tc_fence_after();
                    const uint32_t at = at0 + s * A_SLOT_COLS, bl = blo0 + s * b_step;
                    // 16 k further: 8 TMEM columns on the A side, 32 bytes (+2 encoded) inside the swizzle atom on the B
                    // side; the second stage of the pair is one A slot / one B stage further on
                    if (kb == 4 * sb0) umma_ts_f16_first(tmem_base, at, bl, bhi, idesc);
                    else umma_ts_f16_acc(tmem_base, at, bl, bhi, idesc);
                    umma_ts_f16_acc(tmem_base, at + 8, bl + 2, bhi, idesc);
                    umma_ts_f16_acc(tmem_base, at + 16, bl + 4, bhi, idesc);
                    umma_ts_f16_acc(tmem_base, at + 24, bl + 6, bhi, idesc);
                    const uint32_t at2 = at + A_SLOT_COLS, bl2 = bl + b_step;
                    umma_ts_f16_acc(tmem_base, at2, bl2, bhi, idesc);
                    umma_ts_f16_acc(tmem_base, at2 + 8, bl2 + 2, bhi, idesc);
                    umma_ts_f16_acc(tmem_base, at2 + 16, bl2 + 4, bhi, idesc);
                    umma_ts_f16_acc(tmem_base, at2 + 24, bl2 + 6, bhi, idesc);
                    umma_commit(em0 + (s >> 1) * 8);
                }
                if (!ok) break;
                umma_commit(smem_u32(accum));
                if (u + (sb1 - sb0) == u1) umma_commit(smem_u32(pgo));
                u += sb1 - sb0;
            }
        }
    } else if (warp == 2) {
        // ---------------------------------------------------------------- raw super-block loader
        if (lane == 0) {
            int rit = 0;
            for (int u = u0; u < u1 && ok;) {
                const int tile = u / k.nsb, sb0 = u - tile * k.nsb, sb1 = min(k.nsb, sb0 + (u1 - u));
                const int row0 = (tile % k.tiles_x) * BM;
                for (int sb = sb0; sb < sb1; sb++, rit++) {
                    const int rs = rit % RS;
                    const uint32_t ph = (uint32_t)(rit / RS) & 1;
                    if (!mbar_wait(smem_u32(&raw_empty[rs]), ph ^ 1, abort_flag, a.status, 7)) { ok = false; break; }
                    if constexpr (QF == 6) {
                        // row tiles past the tensor's last one are not copied (their rows are never stored)
                        const int T0 = row0 >> 4, nT = min(8, k.img_nrt - T0);
                        const uint32_t st = smem_u32(sRaw + rs * RAW_STAGE_BYTES), bar = smem_u32(&raw_full[rs]);
                        mbar_arrive_expect_tx(bar, (uint32_t)nT * 4096u);
                        for (int j = 0; j < nT; j++) {
                            const uint8_t* src = k.img + ((int64_t)(T0 + j) * k.img_nh + 2 * sb) * 2112;
                            bulk_load(st + (uint32_t)j * 4096u, src, 2048u, bar);
                            bulk_load(st + (uint32_t)j * 4096u + 2048u, src + 2112, 2048u, bar);
                        }
                        continue;
                    }
                    mbar_arrive_expect_tx(smem_u32(&raw_full[rs]), (uint32_t)RAW_STAGE_BYTES);
                    if constexpr (QF == 2) {
                        const uint32_t st = smem_u32(sRaw + rs * RAW_STAGE_BYTES), bar = smem_u32(&raw_full[rs]);
                        tma_load_2d(st, &tmap_w, sb * 128, row0, bar);
                        tma_load_2d(st + BM * 128, &tmap_w2, sb * 64, row0, bar);
                        tma_load_2d(st + BM * 192, &tmap_w3, sb * 16, row0, bar);
                    } else if constexpr (QF == 4) {
                        const uint32_t st = smem_u32(sRaw + rs * RAW_STAGE_BYTES), bar = smem_u32(&raw_full[rs]);
                        tma_load_2d(st, &tmap_w, sb * 256, row0, bar);                 // blocks 0..3 of the step
                        tma_load_2d(st + BM * 128, &tmap_w, sb * 256 + 128, row0, bar);   // blocks 4..7
                    } else {
                        tma_load_2d(smem_u32(sRaw + rs * RAW_STAGE_BYTES), &tmap_w, sb * RAW_ROW_BYTES, row0, smem_u32(&raw_full[rs]));
                    }
                }
                u += sb1 - sb0;
            }
            for (int j = max(0, rit - RS); j < rit; j++) {
                const int rs = j % RS;
                const uint32_t ph = (uint32_t)(j / RS) & 1;
                long long t0 = clock64();
                while (!mbar_try_wait(smem_u32(&raw_full[rs]), ph)) {
                    if (clock64() - t0 > WAIT_BUDGET) { atomicCAS(a.status, 0, 9); break; }
                }
            }
        }
    } else if (warp == 3) {
        // ---------------------------------------------------------------- publisher, then partial-tile prefetcher
        // A range that ends inside a tile makes this CTA the tile's owner, and that segment is its last one, so
        // the activation stages are idle once its MMAs are complete. This thread waits, beside the main loop,
        // for the next CTA's partial tile (its flag), then for those MMAs, and lets the copy engine bring the
        // partial tile into the stages, 64 activation rows per copy: the owner's adds read shared memory.
        if (lane == 0 && u1 > u0 && u0 % k.nsb != 0) {
            // publisher: this CTA's first segment starts inside a tile, so it leaves partial sums in the workspace;
            // once the eight epilogue warps have fenced their stores the flag tells the tile's owner
            long long t0 = clock64();
            bool all = true;
            while (*reinterpret_cast<volatile int*>(stored) < 8) {
                if (*abort_flag != 0 || clock64() - t0 > WAIT_BUDGET) { all = false; atomicCAS(a.status, 0, 12); break; }
                __nanosleep(100);
            }
            if (all) {
                __threadfence();
                st_release_gpu(k.flags + cta, k.epoch);
            }
        }
        if (lane == 0 && a.staged_epilogue && (a.bn & 63) == 0 && u1 > u0 && cta + 1 < nctas) {
            const int tl = (u1 - 1) / k.nsb;
            const int s0 = max(u0, tl * k.nsb) - tl * k.nsb, s1 = u1 - tl * k.nsb;
            if (s0 == 0 && s1 < k.nsb) {
                long long t0 = clock64();
                while (ld_acquire_gpu(k.flags + cta + 1) != k.epoch) {
                    if (*abort_flag != 0 || clock64() - t0 > WAIT_BUDGET) {
                        *abort_flag = 1;
                        atomicCAS(a.status, 0, 11);
                        ok = false;
                        break;
                    }
                    __nanosleep(200);
                }
                asm volatile("fence.proxy.async;" ::: "memory");   // the flag was acquired by a plain load; the copy engine reads next
                if (ok && mbar_wait(smem_u32(pgo), 0, abort_flag, a.status, 15)) {
                    for (int rnd = 0; rnd < a.bn; rnd += 64) {
                        const uint32_t pb = smem_u32(&pfull[rnd >> 6]);
                        mbar_arrive_expect_tx(pb, 64u * BM * 4u);
                        tma_load_2d(smem_u32(sB + (rnd >> 6) * (64 * BM * 4)), &tmap_ws, 0, (cta + 1) * 256 + rnd, pb);
                    }
                    // nothing stays in flight behind this thread
                    for (int rnd = 0; rnd < a.bn; rnd += 64)
                        if (!mbar_wait(smem_u32(&pfull[rnd >> 6]), 0, abort_flag, a.status, 14)) break;
                }
            }
        }
    } else if (warp >= 4) {
        // ---------------------------------------------------------------- converters, then epilogue, per segment
        const int q = warp & 3;
        const int nib = (warp - 4) >> 2;
        const int r = q * 32 + lane;
        const uint32_t slot0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)a.a_col0 + (uint32_t)nib * 16;
        const uint32_t mask = nib ? 0x00F000F0u : 0x000F000Fu;
        const float nibscale = nib ? 0.0625f : 1.0f;
        const __half2 k1024 = __float2half2_rn(1024.0f);
        int it = 0, rit = 0, seg = 0;
        // Partial sums are written with plain stores; the fence that completes them costs a round trip to L2,
        // so it waits until the next segment's first super-block is converted (the stores have landed by
        // then), and the publisher (warp 3) releases the flag once all eight warps have fenced.
        int ep_round = 0;   // rounds of the staged epilogue so far (phase of the group's hand-over barriers)
        bool fence_due = false;
        auto fence_and_count = [&]() {
            __threadfence();
            __syncwarp();
            if (lane == 0) atomicAdd(stored, 1);
            fence_due = false;
        };
        for (int u = u0; u < u1 && ok; seg++) {
            const int tile = u / k.nsb, sb0 = u - tile * k.nsb, sb1 = min(k.nsb, sb0 + (u1 - u));
            const int row0 = (tile % k.tiles_x) * BM, tok0 = (tile / k.tiles_x) * a.bn;
            for (int sb = sb0; sb < sb1 && ok; sb++, rit++) {
                const int rs = rit % RS;
                const uint32_t rph = (uint32_t)(rit / RS) & 1;
                if (lane == 0) ok = mbar_wait(smem_u32(&raw_full[rs]), rph, abort_flag, a.status, 8);
                ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
                if (!ok) break;
                if constexpr (QF == 0 || QF == 5) {
                const uint8_t* rowp = sRaw + rs * RAW_STAGE_BYTES + r * RAW_ROW_BYTES;
                const uint4 hdr = *reinterpret_cast<const uint4*>(rowp);
                // Q5_K: the fifth bit of weight l of sub-block j is bit j of qh[l]; it lands on bit 4 of the code
                // (bit 8 where the high nibble stays in place and the scale carries 1/16)
                uint32_t qhw[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
                if constexpr (QF == 5) {
                    const uint4 ha = *reinterpret_cast<const uint4*>(rowp + 16), hb = *reinterpret_cast<const uint4*>(rowp + 32);
                    qhw[0] = ha.x; qhw[1] = ha.y; qhw[2] = ha.z; qhw[3] = ha.w;
                    qhw[4] = hb.x; qhw[5] = hb.y; qhw[6] = hb.z; qhw[7] = hb.w;
                }
                constexpr int QS0 = QF == 5 ? 48 : 16;   // first nibble byte of the block
                const int hs = nib ? 8 : 4;
                const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xFFFFu)));
                const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
                const uint32_t sc_lo = hdr.y & 0x3F3F3F3Fu, m_lo = hdr.z & 0x3F3F3F3Fu;
                const uint32_t sc_hi = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
                const uint32_t m_hi = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
#pragma unroll
                for (int c = 0; c < 4; c++, it++) {
                    const int s = it & (STAGES - 1);
                    const uint32_t ph = (uint32_t)(it >> 2) & 1;
                    const int sh = ((c & 1) * 2 + nib) * 8;
                    const uint32_t sc = ((c < 2 ? sc_lo : sc_hi) >> sh) & 0xFFu, mn = ((c < 2 ? m_lo : m_hi) >> sh) & 0xFFu;
                    const __half2 ds = __float2half2_rn(d * (float)sc * nibscale);
                    const __half2 nd = __float2half2_rn(-dmin * (float)mn);
                    const uint4 qa = *reinterpret_cast<const uint4*>(rowp + QS0 + c * 32);
                    const uint4 qb = *reinterpret_cast<const uint4*>(rowp + QS0 + 16 + c * 32);
                    const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
                    uint32_t v[16];
                    const int jb = 2 * c + nib;   // sub-block of this thread's 32 weights
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        uint32_t t0 = (w[j] & mask) | 0x64006400u, t1 = ((w[j] >> 8) & mask) | 0x64006400u;
                        if constexpr (QF == 5) {
                            t0 |= ((qhw[j] >> jb) & 0x00010001u) << hs;
                            t1 |= ((qhw[j] >> (jb + 8)) & 0x00010001u) << hs;
                        }
                        __half2 h0 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&t0), k1024), ds, nd);
                        __half2 h1 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&t1), k1024), ds, nd);
                        v[2 * j] = *reinterpret_cast<uint32_t*>(&h0);
                        v[2 * j + 1] = *reinterpret_cast<uint32_t*>(&h1);
                    }
                    // stages are handed over in pairs (128 k): one wait before the first store, one arrival after the second
                    if ((c & 1) == 0) {
                        if (lane == 0) ok = mbar_wait(smem_u32(&empty[s >> 1]), ph ^ 1, abort_flag, a.status, 4);
                        ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
                        if (!ok) break;
                        tc_fence_after();
                    }
                    tmem_st16(slot0 + (uint32_t)s * A_SLOT_COLS, v);
                    if (c & 1) {
                        tmem_st_wait();
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&full[s >> 1]));
                    }
                }
                } else if constexpr (QF == 2) {
                    // GGUF Q6_K: per 128-weight half, ql[64] low/high nibbles and qh[32] two-bit fields; k-block c
                    // of the 256-k step = half c >> 1, nibble c & 1; this thread takes weights 32 nib .. 32 nib + 31.
                    const uint8_t* stage = sRaw + rs * RAW_STAGE_BYTES;
                    const uint8_t* qlr = stage + r * 128;
                    const uint8_t* qhr = stage + BM * 128 + r * 64;
                    const uint4 scv = *reinterpret_cast<const uint4*>(stage + BM * 192 + r * 16);
                    const uint32_t scw[4] = {scv.x, scv.y, scv.z, scv.w};
                    const int64_t grow = min((int64_t)row0 + r, (int64_t)a.n_rows - 1);
                    const float d = __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short*>(a.v.p[3]) + grow * k.nsb + sb)));
                    const __half2 k1056 = __float2half2_rn(1056.0f);
#pragma unroll
                    for (int c = 0; c < 4; c++, it++) {
                        const int s = it & (STAGES - 1);
                        const uint32_t ph = (uint32_t)(it >> 2) & 1;
                        const int half = c >> 1, hn = c & 1;
                        // int8 scales 4c + 2 nib and + 1 (16 weights each): bytes 2 nib, 2 nib + 1 of scale word c
                        const int sc0 = (int)(int8_t)((scw[c] >> (16 * nib)) & 0xFFu), sc1 = (int)(int8_t)((scw[c] >> (16 * nib + 8)) & 0xFFu);
                        const __half2 ds0 = __float2half2_rn(d * (float)sc0), ds1 = __float2half2_rn(d * (float)sc1);
                        // 128-byte and 64-byte rows are stored swizzled by the copy (bank conflicts otherwise)
                        const int lc = 4 * half + 2 * nib, hc = 2 * half;
                        const uint4 la = *reinterpret_cast<const uint4*>(qlr + ((lc ^ (r & 7)) << 4));
                        const uint4 lb = *reinterpret_cast<const uint4*>(qlr + (((lc + 1) ^ (r & 7)) << 4));
                        const uint4 ha = *reinterpret_cast<const uint4*>(qhr + ((hc ^ ((r >> 1) & 3)) << 4));
                        const uint4 hb = *reinterpret_cast<const uint4*>(qhr + (((hc + 1) ^ ((r >> 1) & 3)) << 4));
                        const uint32_t lw[8] = {la.x, la.y, la.z, la.w, lb.x, lb.y, lb.z, lb.w};
                        const uint32_t hw[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
                        const int lsh = 4 * hn, hsh = 4 * hn + 2 * nib;
                        uint32_t v[16];
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const uint32_t code4 = ((lw[j] >> lsh) & 0x0F0F0F0Fu) | (((hw[j] >> hsh) & 0x03030303u) << 4);
                            uint32_t t0 = __byte_perm(code4, 0x64646464u, 0x5140), t1 = __byte_perm(code4, 0x64646464u, 0x7362);
                            const __half2 dsj = j < 4 ? ds0 : ds1;
                            __half2 h0 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&t0), k1056), dsj);   // (q - 32) exactly, then one rounding
                            __half2 h1 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&t1), k1056), dsj);
                            v[2 * j] = *reinterpret_cast<uint32_t*>(&h0);
                            v[2 * j + 1] = *reinterpret_cast<uint32_t*>(&h1);
                        }
                        // stages are handed over in pairs (128 k): one wait before the first store, one arrival after the second
                        if ((c & 1) == 0) {
                            if (lane == 0) ok = mbar_wait(smem_u32(&empty[s >> 1]), ph ^ 1, abort_flag, a.status, 4);
                            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
                            if (!ok) break;
                            tc_fence_after();
                        }
                        tmem_st16(slot0 + (uint32_t)s * A_SLOT_COLS, v);
                        if (c & 1) {
                            tmem_st_wait();
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(smem_u32(&full[s >> 1]));
                        }
                    }
                } else if constexpr (QF == 6) {
                    // MXFP6 E2M3 from the decode image: int8 codes = 8 x value (exact). A stage holds, per row tile j of
                    // 16 rows and k-half hh, 2048 bytes: [rows g | rows g + 8] x [first | second 16 codes of a block],
                    // 16-byte chunk (g, t) of block t at 8 t + ((g + 2 t) & 7). This thread takes block 2c + nib of
                    // k-block c; byte ^ 0x80 widened by one PRMT per pair to 1152 + q, minus 1152, times 2^(e-127) / 8:
                    // exact in f16 for block exponents 106..140. Natural weight order.
                    const uint8_t* stage = sRaw + rs * RAW_STAGE_BYTES + (r >> 4) * 4096 + ((r >> 3) & 1) * 1024;
                    const int g8 = r & 7;
                    const int64_t grow = min((int64_t)row0 + r, (int64_t)a.n_rows - 1);
                    const uint2 ex = __ldg(reinterpret_cast<const uint2*>(a.v.p[0] + grow * (a.k >> 5) + sb * 8));
                    const __half2 k1152 = __float2half2_rn(1152.0f);
#pragma unroll
                    for (int c = 0; c < 4; c++, it++) {
                        const int s = it & (STAGES - 1);
                        const uint32_t ph = (uint32_t)(it >> 2) & 1;
                        const int blk = 2 * c + nib, t4 = blk & 3;
                        const uint32_t eb = ((blk < 4 ? ex.x : ex.y) >> (8 * t4)) & 0xFFu;
                        // 2^(eb - 130) built from bits: eb <= 116 lands in the f16 subnormals, still exact down to 2^-24
                        // (E3M2: 2^(eb - 115), exact for block exponents 107..130)
                        const __half2 S = __float2half2_rn(__uint_as_float(k.img_e3m2 ? (eb + 12u) << 23 : eb >= 4u ? (eb - 3u) << 23 : 0u));
                        const uint8_t* cp = stage + (blk >> 2) * 2048 + ((8 * t4 + ((g8 + 2 * t4) & 7)) << 4);
                        const uint4 qa = *reinterpret_cast<const uint4*>(cp);
                        const uint4 qb = *reinterpret_cast<const uint4*>(cp + 512);
                        const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
                        uint32_t v[16];
                        if (k.img_e3m2) {
                            // a byte s00eeemm in the high half of an f16 is the E3M2 value * 2^-12, subnormals included
#pragma unroll
                            for (int j = 0; j < 8; j++) {
                                uint32_t t0 = __byte_perm(w[j], 0u, 0x1404), t1 = __byte_perm(w[j], 0u, 0x3424);
                                __half2 h0 = __hmul2(*reinterpret_cast<__half2*>(&t0), S);
                                __half2 h1 = __hmul2(*reinterpret_cast<__half2*>(&t1), S);
                                v[2 * j] = *reinterpret_cast<uint32_t*>(&h0);
                                v[2 * j + 1] = *reinterpret_cast<uint32_t*>(&h1);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 8; j++) {
                                const uint32_t u4 = w[j] ^ 0x80808080u;
                                uint32_t t0 = __byte_perm(u4, 0x64646464u, 0x5140), t1 = __byte_perm(u4, 0x64646464u, 0x7362);
                                __half2 h0 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&t0), k1152), S);
                                __half2 h1 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&t1), k1152), S);
                                v[2 * j] = *reinterpret_cast<uint32_t*>(&h0);
                                v[2 * j + 1] = *reinterpret_cast<uint32_t*>(&h1);
                            }
                        }
                        if ((c & 1) == 0) {
                            if (lane == 0) ok = mbar_wait(smem_u32(&empty[s >> 1]), ph ^ 1, abort_flag, a.status, 4);
                            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
                            if (!ok) break;
                            tc_fence_after();
                        }
                        tmem_st16(slot0 + (uint32_t)s * A_SLOT_COLS, v);
                        if (c & 1) {
                            tmem_st_wait();
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(smem_u32(&full[s >> 1]));
                        }
                    }
                } else if constexpr (QF == 4) {
                    // GGUF Q8_0: block = f16 d + 32 int8 codes. The step's 256 code bytes of a row arrive as two
                    // swizzled 128-byte rows (blocks 0..3 and 4..7); this thread takes block 2c + nib of k-block c:
                    // byte ^ 0x80 = q + 128, widened with one PRMT per pair to 1024 + 128 + q, minus 1152 = q exactly,
                    // one rounding in the multiply by d. Natural weight order (activations are not permuted).
                    const uint8_t* stage = sRaw + rs * RAW_STAGE_BYTES;
                    const int64_t grow = min((int64_t)row0 + r, (int64_t)a.n_rows - 1);
                    const uint4 dv = __ldg(reinterpret_cast<const uint4*>(a.v.p[0] + (grow * (a.k >> 5) + sb * 8) * 2));
                    const __half2 k1152 = __float2half2_rn(1152.0f);
#pragma unroll
                    for (int c = 0; c < 4; c++, it++) {
                        const int s = it & (STAGES - 1);
                        const uint32_t ph = (uint32_t)(it >> 2) & 1;
                        const int blk = 2 * c + nib;
                        const uint32_t dw = blk < 2 ? dv.x : blk < 4 ? dv.y : blk < 6 ? dv.z : dv.w;
                        const __half2 S = __half2half2(__ushort_as_half((unsigned short)((blk & 1) ? (dw >> 16) : (dw & 0xFFFFu))));
                        const uint8_t* rowp = stage + (blk >> 2) * (BM * 128) + r * 128;
                        const int ch = (blk & 3) * 2;
                        const uint4 qa = *reinterpret_cast<const uint4*>(rowp + ((ch ^ (r & 7)) << 4));
                        const uint4 qb = *reinterpret_cast<const uint4*>(rowp + (((ch + 1) ^ (r & 7)) << 4));
                        const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
                        uint32_t v[16];
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const uint32_t u4 = w[j] ^ 0x80808080u;
                            uint32_t t0 = __byte_perm(u4, 0x64646464u, 0x5140), t1 = __byte_perm(u4, 0x64646464u, 0x7362);
                            __half2 h0 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&t0), k1152), S);
                            __half2 h1 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&t1), k1152), S);
                            v[2 * j] = *reinterpret_cast<uint32_t*>(&h0);
                            v[2 * j + 1] = *reinterpret_cast<uint32_t*>(&h1);
                        }
                        if ((c & 1) == 0) {
                            if (lane == 0) ok = mbar_wait(smem_u32(&empty[s >> 1]), ph ^ 1, abort_flag, a.status, 4);
                            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
                            if (!ok) break;
                            tc_fence_after();
                        }
                        tmem_st16(slot0 + (uint32_t)s * A_SLOT_COLS, v);
                        if (c & 1) {
                            tmem_st_wait();
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(smem_u32(&full[s >> 1]));
                        }
                    }
                } else {
                const uint8_t* rowp = sRaw + rs * RAW_STAGE_BYTES + r * RAW_ROW_BYTES;
                const int64_t grow = min((int64_t)row0 + r, (int64_t)a.n_rows - 1);
                // block scales of the 256-k step: eight exponent bytes (MXFP4) or eight f16 d (Q4_0)
                uint4 ex = make_uint4(0u, 0u, 0u, 0u);
                if constexpr (QF == 3) ex = __ldg(reinterpret_cast<const uint4*>(a.v.p[0] + (grow * (a.k >> 5) + sb * 8) * 2));
                else {
                    const uint2 e2 = __ldg(reinterpret_cast<const uint2*>(a.v.p[0] + grow * (a.k >> 5) + sb * 8));
                    ex.x = e2.x; ex.y = e2.y;
                }
                const __half2 k1032 = __float2half2_rn(1032.0f);
#pragma unroll
                for (int c = 0; c < 4; c++, it++) {
                    const int s = it & (STAGES - 1);
                    const uint32_t ph = (uint32_t)(it >> 2) & 1;
                    const int blk = 2 * c + nib;                      // block of 32 inside the 256-k step
                    __half2 S;
                    if constexpr (QF == 3) {
                        const uint32_t dw = blk < 2 ? ex.x : blk < 4 ? ex.y : blk < 6 ? ex.z : ex.w;
                        S = __half2half2(__ushort_as_half((unsigned short)((blk & 1) ? (dw >> 16) : (dw & 0xFFFFu))));
                    } else {
                        const uint32_t eb = ((blk < 4 ? ex.x : ex.y) >> (8 * (blk & 3))) & 0xFFu;
                        S = __float2half2_rn(gguf_e8m0_half((uint8_t)eb) * 32768.0f);
                    }
                    // rows are 128 bytes: the copy swizzles the 16-byte chunks with the row number so that the
                    // 32 rows of a warp do not all hit the same banks
                    const uint4 q = *reinterpret_cast<const uint4*>(rowp + ((blk ^ (r & 7)) << 4));
                    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
                    uint32_t v[16];
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        // low nibbles: elements 4j..4j+3 of the block (as 0,2 | 1,3), high nibbles: 16 further on
                        const uint32_t x0 = w[j], x1 = w[j] >> 8, x2 = w[j] >> 4, x3 = w[j] >> 12;
                        uint32_t t0, t1, t2, t3;
                        __half2 h0, h1, h2, h3;
                        if constexpr (QF == 3) {
                            // Q4_0: (1024 + q) - 1032 = q - 8 exactly, then one rounding in the multiply by d
                            t0 = (x0 & 0x000F000Fu) | 0x64006400u; t1 = (x1 & 0x000F000Fu) | 0x64006400u;
                            t2 = (x2 & 0x000F000Fu) | 0x64006400u; t3 = (x3 & 0x000F000Fu) | 0x64006400u;
                            h0 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&t0), k1032), S);
                            h1 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&t1), k1032), S);
                            h2 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&t2), k1032), S);
                            h3 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&t3), k1032), S);
                        } else {
                            t0 = (x0 & 0x00070007u) * 512u + (x0 & 0x00080008u) * 4096u;
                            t1 = (x1 & 0x00070007u) * 512u + (x1 & 0x00080008u) * 4096u;
                            t2 = (x2 & 0x00070007u) * 512u + (x2 & 0x00080008u) * 4096u;
                            t3 = (x3 & 0x00070007u) * 512u + (x3 & 0x00080008u) * 4096u;
                            h0 = __hmul2(*reinterpret_cast<__half2*>(&t0), S); h1 = __hmul2(*reinterpret_cast<__half2*>(&t1), S);
                            h2 = __hmul2(*reinterpret_cast<__half2*>(&t2), S); h3 = __hmul2(*reinterpret_cast<__half2*>(&t3), S);
                        }
                        v[2 * j] = *reinterpret_cast<uint32_t*>(&h0); v[2 * j + 1] = *reinterpret_cast<uint32_t*>(&h1);
                        v[8 + 2 * j] = *reinterpret_cast<uint32_t*>(&h2); v[8 + 2 * j + 1] = *reinterpret_cast<uint32_t*>(&h3);
                    }
                    // stages are handed over in pairs (128 k): one wait before the first store, one arrival after the second
                    if ((c & 1) == 0) {
                        if (lane == 0) ok = mbar_wait(smem_u32(&empty[s >> 1]), ph ^ 1, abort_flag, a.status, 4);
                        ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
                        if (!ok) break;
                        tc_fence_after();
                    }
                    tmem_st16(slot0 + (uint32_t)s * A_SLOT_COLS, v);
                    if (c & 1) {
                        tmem_st_wait();
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&full[s >> 1]));
                    }
                }
                }
                if (!ok) break;
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&raw_empty[rs]));
                if (fence_due) fence_and_count();
            }
            if (!ok) break;
            // ------------------------------------------------------------ epilogue of this segment
            if (seg == 0) asm volatile("griddepcontrol.wait;" ::: "memory");   // the row scales come from the kernel ahead
            if (lane == 0) ok = mbar_wait(smem_u32(accum), (uint32_t)(seg & 1), abort_flag, a.status, 6);
            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
            if (!ok) break;
            tc_fence_after();
            const bool head = sb0 == 0, whole = head && sb1 == k.nsb;
            const int row = row0 + r;
            // partial sums this (owning) CTA has to add: the CTAs after it, until the tile's k range is covered
            int p_end = cta + 1;
            bool pf = false;   // the first partial tile arrives in shared memory (prefetcher warp)
            if (head && !whole) {
                const int tile_end = (tile + 1) * k.nsb;
                while (p_end < nctas && sk_unit_begin(p_end, k.total_units, nctas) < tile_end) p_end++;
                pf = a.staged_epilogue && (a.bn & 63) == 0 && p_end > cta + 1 && u + (sb1 - sb0) == u1;
                for (int p = cta + 1 + (pf ? 1 : 0); p < p_end && ok; p++) {
                    if (lane == 0) {
                        long long t0 = clock64();
                        while (ld_acquire_gpu(k.flags + p) != k.epoch) {
                            if (*abort_flag != 0 || clock64() - t0 > WAIT_BUDGET) {
                                *abort_flag = 1;
                                atomicCAS(a.status, 0, 11);
                                ok = false;
                                break;
                            }
                        }
                    }
                    ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
                }
            }
            float* myslot = k.ws + (size_t)cta * SK_SLOT_FLOATS;
            if (head && a.staged_epilogue) {
                // Finished tile -> shared memory -> TMA stores. Every warp owns a 32 x 32 block of the round
                // (its 32 weight rows x 32 activation rows), stages it in a private 4 KB buffer and stores it
                // with its own copy (clipped at the edges of y), so the eight warps never wait for one another
                // and no thread waits for global memory; the copies drain while the next segment's main loop runs.
                // Scattered product (one store per GPU): the four warps that share a 32-row half of the round (warps 4..7:
                // activation rows 0..31, warps 8..11: 32..63) write their 32 x 32 blocks side by side into ONE tile of [32 activation rows][128 weight
                // rows], and the group's first warp stores it with one copy whose rows are 512 contiguous bytes (256
                // in bf16): the copy engine spends its time per row, so four times fewer rows per byte. The hand-over
                // inside a group goes through two mbarriers with bounded waits.
                // A product stored to one output keeps a private 4 KB buffer and a store of its own per warp (no
                // hand-over at all; measured faster there).
                const int half_off = warp >= 8 ? 32 : 0;
                const int grp = warp >= 8 ? 1 : 0;
                const bool coop = a.n_extra > 0;
                float* wstg = coop ? stg + grp * 4096 : stg + (warp - 4) * 1024;
                const int wpitch = coop ? 128 : 32;            // elements per activation row of the staging tile
                const int wcol = coop ? q * 32 + lane : lane;
                const bool leader = (warp & 3) == 0;
                const uint32_t gfree_b = smem_u32(&gfree[grp]), gready_b = smem_u32(&gready[grp]);
                const int last_rnd = ((a.bn + 63) >> 6) * 64 - 64;
                bool freed = false;
                for (int rnd = 0; rnd < a.bn && ok; rnd += 64) {
                    const int c0 = rnd + half_off;
                    uint32_t v[32];
                    tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)min(c0, 480), v);
                    if (rnd == last_rnd) {
                        // every TMEM read of this warp is complete: the accumulator may be overwritten
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(dfree));
                        freed = true;
                    }
                    if (pf) {
                        if (lane == 0) ok = mbar_wait(smem_u32(&pfull[rnd >> 6]), 0, abort_flag, a.status, 14);
                        ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
                        if (!ok) break;
                        const float* sp = reinterpret_cast<const float*>(sB + (rnd >> 6) * (64 * BM * 4)) + half_off * BM + r;
#pragma unroll
                        for (int j = 0; j < 32; j++) v[j] = __float_as_uint(__uint_as_float(v[j]) + sp[j * BM]);
                    }
                    for (int p = cta + 1 + (pf ? 1 : 0); p < p_end; p++) {
                        const float* ps = k.ws + (size_t)p * SK_SLOT_FLOATS + c0 * BM + r;
                        if (c0 < a.bn) {
#pragma unroll
                            for (int j = 0; j < 32; j++) v[j] = __float_as_uint(__uint_as_float(v[j]) + __ldcg(ps + j * BM));
                        }
                    }
                    // the group's previous store must have finished READING the tile before it is overwritten
                    if (lane == 0) {
                        if (!coop) {
                            bulk_wait_read0();
                        } else {
                            if (leader) {
                                bulk_wait_read0();
                                mbar_arrive(gfree_b);
                            }
                            ok = mbar_wait(gfree_b, (uint32_t)(ep_round & 1), abort_flag, a.status, 16);
                        }
                    }
                    ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
                    if (!ok) break;
                    // row scales of the block's 32 activation rows: 128-byte aligned, read four at a time (the
                    // scale array is padded, and rows past m are clipped by the store)
                    const float4* sc4 = reinterpret_cast<const float4*>(a.xscale + tok0 + c0);
                    if (a.y_bf16) {
                        // bf16 outputs: the block is staged as [32 activation rows][32 weight rows] of 2 bytes
                        __nv_bfloat16* w16 = reinterpret_cast<__nv_bfloat16*>(wstg) + wcol;
#pragma unroll
                        for (int j4 = 0; j4 < 8; j4++) {
                            const float4 sc = __ldg(sc4 + j4);
                            w16[(4 * j4 + 0) * wpitch] = __float2bfloat16_rn(__uint_as_float(v[4 * j4 + 0]) * sc.x);
                            w16[(4 * j4 + 1) * wpitch] = __float2bfloat16_rn(__uint_as_float(v[4 * j4 + 1]) * sc.y);
                            w16[(4 * j4 + 2) * wpitch] = __float2bfloat16_rn(__uint_as_float(v[4 * j4 + 2]) * sc.z);
                            w16[(4 * j4 + 3) * wpitch] = __float2bfloat16_rn(__uint_as_float(v[4 * j4 + 3]) * sc.w);
                        }
                    } else {
                        float* w32 = wstg + wcol;
#pragma unroll
                        for (int j4 = 0; j4 < 8; j4++) {
                            const float4 sc = __ldg(sc4 + j4);
                            w32[(4 * j4 + 0) * wpitch] = __uint_as_float(v[4 * j4 + 0]) * sc.x;
                            w32[(4 * j4 + 1) * wpitch] = __uint_as_float(v[4 * j4 + 1]) * sc.y;
                            w32[(4 * j4 + 2) * wpitch] = __uint_as_float(v[4 * j4 + 2]) * sc.z;
                            w32[(4 * j4 + 3) * wpitch] = __uint_as_float(v[4 * j4 + 3]) * sc.w;
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        if (!coop) {
                            if (c0 < a.bn) {
                                tma_store_2d(&tmap_y, smem_u32(wstg), row0 + q * 32, tok0 + c0);
                                bulk_commit();
                            }
                        } else {
                            mbar_arrive(gready_b);
                            if (leader) {
                                ok = mbar_wait(gready_b, (uint32_t)(ep_round & 1), abort_flag, a.status, 17);
                                if (ok && c0 < a.bn) {
                                    tma_store_2d(&tmap_y, smem_u32(wstg), row0, tok0 + c0);
                                    // the same tile into the other GPUs' outputs, over NVLink
                                    for (int pp = 0; pp < a.n_extra; pp++) tma_store_2d(&peers.m[pp], smem_u32(wstg), row0, tok0 + c0);
                                    bulk_commit();
                                }
                            }
                        }
                    }
                    ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
                    ep_round++;
                }
                if (!freed) {   // a wait gave up before the last read: the MMA thread leaves through the abort flag
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(dfree));
                }
            } else
            for (int c0 = (warp >= 8 ? 32 : 0); c0 < a.bn; c0 += 64) {
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
                if (!ok) continue;
                if (!head) {
#pragma unroll
                    for (int j = 0; j < 32; j++) __stcg(myslot + (c0 + j) * BM + r, __uint_as_float(v[j]));
                } else {
                    for (int p = cta + 1; p < p_end; p++) {
                        const float* ps = k.ws + (size_t)p * SK_SLOT_FLOATS + c0 * BM + r;
#pragma unroll
                        for (int j = 0; j < 32; j++) v[j] = __float_as_uint(__uint_as_float(v[j]) + __ldcg(ps + j * BM));
                    }
                    if (row < a.n_rows) {
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            const int tok = tok0 + c0 + j;
                            if (tok < a.m) {
                                const float val = __uint_as_float(v[j]) * __ldg(a.xscale + tok);
                                a.y[(int64_t)tok * a.ldy + row] = val;
                                for (int pp = 0; pp < a.n_extra; pp++) a.y_extra[pp][(int64_t)tok * a.ldy + row] = val;
                            }
                        }
                    }
                }
            }
            if (!(head && a.staged_epilogue)) {
                // every TMEM read of this warp is complete: the accumulator may be overwritten
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(dfree));
            }
            if (!head) fence_due = true;   // partial sums written: fence and count later (see above)
            u += sb1 - sb0;
        }
        if (fence_due) fence_and_count();
        if (lane == 0) bulk_wait0();   // the tile stores of this thread are complete before shared memory goes away
    }
    // ---------------------------------------------------------------- teardown (every path ends here)
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)a.tmem_cols) : "memory");
    }
}

// Activation rows -> f16 with a power-of-two scale per row (max |x| of the row lands in [1, 2)).
// perm: inside every aligned group of four k positions the order becomes 0,2,1,3 -- the order in which the
// nibble masks of the Q4_K tile producers emit weights (bytes 0 and 2, then bytes 1 and 3).
// One CTA per row; VEC = 4 reads 16 bytes (fp32) or 8 bytes (bf16) per thread and needs k % 4 == 0 with
// aligned rows, VEC = 1 is the general path. The second pass re-reads the row from L1/L2.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xFFFF0000u), __uint_as_float(u.y << 16),
                       __uint_as_float(u.y & 0xFFFF0000u));
}

// With `up` set (fp32 rows of the same shape and pitch) the row converted is x * swish(up), swish(u) = u * 1 / (1 + expf(-u)),
// in the operation order of the stand-alone SwiGLU kernel (kernels/swiglu.hip:55-62): the activation of an MLP
// block's down projection is formed here, in the pass that reads it anyway.
__device__ __forceinline__ float4 swiglu4(float4 g, float4 u) {
    float4 o;
    o.x = g.x * (u.x * (1.0f / (1.0f + expf(-u.x))));
    o.y = g.y * (u.y * (1.0f / (1.0f + expf(-u.y))));
    o.z = g.z * (u.z * (1.0f / (1.0f + expf(-u.z))));
    o.w = g.w * (u.w * (1.0f / (1.0f + expf(-u.w))));
    return o;
}

template <typename T, int VEC>
__global__ void __launch_bounds__(256) x_to_f16_kernel(const T* __restrict__ x, int64_t ldx, __half* __restrict__ out,
                                                       float* __restrict__ scale, int k, int perm, const float* __restrict__ up) {
    // the prefill kernel behind this one may start: it streams and converts weights, and waits for this
    // kernel's completion (griddepcontrol.wait) before it touches the f16 activations or their scales
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // this kernel itself is launched with programmatic stream serialisation: its CTAs may be resident while the
    // kernel ahead of it still runs (it may produce x, or still read the f16 copy this kernel overwrites), so
    // nothing is read or written before that kernel has completed
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int row = blockIdx.x;
    const T* xr = x + (int64_t)row * ldx;
    const float* ur = up ? up + (int64_t)row * ldx : nullptr;
    float mx = 0.0f;
    if constexpr (VEC == 4) {
        for (int i = threadIdx.x * 4; i < k; i += 1024) {
            float4 v = load4(xr + i);
            if (ur) v = swiglu4(v, load4(ur + i));
            mx = fmaxf(fmaxf(mx, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
        }
    } else {
        for (int i = threadIdx.x; i < k; i += 256) {
            float v = (float)xr[i];
            if (ur) { const float u = ur[i]; v = v * (u * (1.0f / (1.0f + expf(-u)))); }
            mx = fmaxf(mx, fabsf(v));
        }
    }
    __shared__ float red[8];
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = red[0];
    for (int i = 1; i < 8; i++) mx = fmaxf(mx, red[i]);
    int e = (int)((__float_as_uint(mx) >> 23) & 255u);
    e = (mx == 0.0f || !(mx <= 3.0e38f)) ? 127 : min(max(e, 1), 253);
    const float sdown = __uint_as_float((uint32_t)(254 - e) << 23);
    __half* orow = out + (int64_t)row * k;
    if constexpr (VEC == 4) {
        for (int i = threadIdx.x * 4; i < k; i += 1024) {
            float4 v = load4(xr + i);
            if (ur) v = swiglu4(v, load4(ur + i));
            const __half2 a = perm ? __floats2half2_rn(v.x * sdown, v.z * sdown) : __floats2half2_rn(v.x * sdown, v.y * sdown);
            const __half2 b = perm ? __floats2half2_rn(v.y * sdown, v.w * sdown) : __floats2half2_rn(v.z * sdown, v.w * sdown);
            uint2 pk;
            pk.x = *reinterpret_cast<const uint32_t*>(&a);
            pk.y = *reinterpret_cast<const uint32_t*>(&b);
            *reinterpret_cast<uint2*>(orow + i) = pk;
        }
    } else {
        for (int i = threadIdx.x; i < k; i += 256) {
            const int src = perm ? ((i & ~3) | ((i & 1) << 1) | ((i & 2) >> 1)) : i;
            float v = (float)xr[src];
            if (ur) { const float u = ur[src]; v = v * (u * (1.0f / (1.0f + expf(-u)))); }
            orow[i] = __float2half_rn(v * sdown);
        }
    }
    if (threadIdx.x == 0) scale[row] = __uint_as_float((uint32_t)e << 23);
}

// The same conversion for short rows of up to 1024 * NC elements (k % 4 == 0, aligned rows): every thread keeps its NC
// groups of four values in registers between the row maximum and the conversion, so the row is read once and all of a
// thread's loads are in flight together. Same arithmetic, element for element, as the two-pass kernel above.
template <typename T, int NC>
__global__ void __launch_bounds__(256) x_to_f16_regs_kernel(const T* __restrict__ x, int64_t ldx, __half* __restrict__ out,
                                                            float* __restrict__ scale, int k, int perm, const float* __restrict__ up) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");   // see x_to_f16_kernel
    const int row = blockIdx.x;
    const T* xr = x + (int64_t)row * ldx;
    float4 v[NC];
#pragma unroll
    for (int j = 0; j < NC; j++) {
        const int i = (threadIdx.x + j * 256) * 4;
        v[j] = i < k ? load4(xr + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    if (up) {
        const float* ur = up + (int64_t)row * ldx;
        float4 u[NC];
#pragma unroll
        for (int j = 0; j < NC; j++) {
            const int i = (threadIdx.x + j * 256) * 4;
            u[j] = i < k ? load4(ur + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
#pragma unroll
        for (int j = 0; j < NC; j++) v[j] = swiglu4(v[j], u[j]);
    }
    float mx = 0.0f;
#pragma unroll
    for (int j = 0; j < NC; j++) mx = fmaxf(fmaxf(mx, fmaxf(fabsf(v[j].x), fabsf(v[j].y))), fmaxf(fabsf(v[j].z), fabsf(v[j].w)));
    __shared__ float red[8];
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = red[0];
    for (int i = 1; i < 8; i++) mx = fmaxf(mx, red[i]);
    int e = (int)((__float_as_uint(mx) >> 23) & 255u);
    e = (mx == 0.0f || !(mx <= 3.0e38f)) ? 127 : min(max(e, 1), 253);
    const float sdown = __uint_as_float((uint32_t)(254 - e) << 23);
    __half* orow = out + (int64_t)row * k;
#pragma unroll
    for (int j = 0; j < NC; j++) {
        const int i = (threadIdx.x + j * 256) * 4;
        if (i < k) {
            const float4 w = v[j];
            const __half2 a = perm ? __floats2half2_rn(w.x * sdown, w.z * sdown) : __floats2half2_rn(w.x * sdown, w.y * sdown);
            const __half2 b = perm ? __floats2half2_rn(w.y * sdown, w.w * sdown) : __floats2half2_rn(w.z * sdown, w.w * sdown);
            uint2 pk;
            pk.x = *reinterpret_cast<const uint32_t*>(&a);
            pk.y = *reinterpret_cast<const uint32_t*>(&b);
            *reinterpret_cast<uint2*>(orow + i) = pk;
        }
    }
    if (threadIdx.x == 0) scale[row] = __uint_as_float((uint32_t)e << 23);
}

// Longer rows (up to 47 KB of fp32, k % 4 == 0, aligned rows): the values wait in shared memory instead, written and
// read back by the same thread, so several rows per SM stay in flight at a small register count.
template <typename T>
__global__ void __launch_bounds__(256) x_to_f16_smem_kernel(const T* __restrict__ x, int64_t ldx, __half* __restrict__ out,
                                                            float* __restrict__ scale, int k, int perm, const float* __restrict__ up) {
    extern __shared__ float4 srow[];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");   // see x_to_f16_kernel
    const int row = blockIdx.x;
    const T* xr = x + (int64_t)row * ldx;
    const float* ur = up ? up + (int64_t)row * ldx : nullptr;
    const int k4 = k >> 2;
    float mx = 0.0f;
    for (int i0 = threadIdx.x; i0 < k4; i0 += 1024) {
        float4 v[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const int i = i0 + q * 256;
            v[q] = i < k4 ? load4(xr + 4 * i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
        if (ur) {
            float4 u[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const int i = i0 + q * 256;
                u[q] = i < k4 ? load4(ur + 4 * i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (int q = 0; q < 4; q++) v[q] = swiglu4(v[q], u[q]);
        }
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const int i = i0 + q * 256;
            if (i < k4) srow[i] = v[q];
            mx = fmaxf(fmaxf(mx, fmaxf(fabsf(v[q].x), fabsf(v[q].y))), fmaxf(fabsf(v[q].z), fabsf(v[q].w)));
        }
    }
    __shared__ float red[8];
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = red[0];
    for (int i = 1; i < 8; i++) mx = fmaxf(mx, red[i]);
    int e = (int)((__float_as_uint(mx) >> 23) & 255u);
    e = (mx == 0.0f || !(mx <= 3.0e38f)) ? 127 : min(max(e, 1), 253);
    const float sdown = __uint_as_float((uint32_t)(254 - e) << 23);
    __half* orow = out + (int64_t)row * k;
    for (int i = threadIdx.x; i < k4; i += 256) {
        const float4 w = srow[i];
        const __half2 a = perm ? __floats2half2_rn(w.x * sdown, w.z * sdown) : __floats2half2_rn(w.x * sdown, w.y * sdown);
        const __half2 b = perm ? __floats2half2_rn(w.y * sdown, w.w * sdown) : __floats2half2_rn(w.z * sdown, w.w * sdown);
        uint2 pk;
        pk.x = *reinterpret_cast<const uint32_t*>(&a);
        pk.y = *reinterpret_cast<const uint32_t*>(&b);
        *reinterpret_cast<uint2*>(orow + 4 * i) = pk;
    }
    if (threadIdx.x == 0) scale[row] = __uint_as_float((uint32_t)e << 23);
}

template <typename T>
int launch_x_to_f16(b200q_ctx* ctx, const T* x, int64_t ldx, __half* out, float* scale, int m, int k, int perm, const float* up = nullptr) {
    const bool vec = (k % 4) == 0 && (ldx % 4) == 0 && (reinterpret_cast<uintptr_t>(x) % 16) == 0 && (reinterpret_cast<uintptr_t>(up) % 16) == 0;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)m);
    cfg.blockDim = dim3(256);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (vec && k <= 4096) B200Q_CUDA(cudaLaunchKernelEx(&cfg, x_to_f16_regs_kernel<T, 4>, x, ldx, out, scale, k, perm, up), B200Q_ERR_LAUNCH);
    else if (vec && k <= 12032) {   // the row and the eight partial maxima within the 48 KB a launch may ask for unconfigured
        cfg.dynamicSmemBytes = (size_t)k * sizeof(float);
        B200Q_CUDA(cudaLaunchKernelEx(&cfg, x_to_f16_smem_kernel<T>, x, ldx, out, scale, k, perm, up), B200Q_ERR_LAUNCH);
    }
    else if (vec) B200Q_CUDA(cudaLaunchKernelEx(&cfg, x_to_f16_kernel<T, 4>, x, ldx, out, scale, k, perm, up), B200Q_ERR_LAUNCH);
    else B200Q_CUDA(cudaLaunchKernelEx(&cfg, x_to_f16_kernel<T, 1>, x, ldx, out, scale, k, perm, up), B200Q_ERR_LAUNCH);
    return B200Q_OK;
}

// Exercises the give-up path of the bounded waits without touching the tensor cores: one thread waits on a
// barrier nobody will ever arrive on, with a caller-chosen budget, raises the launch's status word exactly
// as the GEMM kernels do, and returns. The host then sees B200Q_ERR_TIMEOUT from b200q_synchronize.
__global__ void bounded_wait_selftest_kernel(int* status, long long budget) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mbar_wait_for(smem_u32(&bar), 0, &abort_flag, status, 99, budget);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

template <typename K>
// The flags are atomics: contexts of one device may be driven from different threads (setting the attribute twice is harmless).
int configure_once(b200q_ctx* ctx, K kernel, std::atomic<bool>* configured) {
    if (!configured[ctx->device & 63]) {
        B200Q_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024), B200Q_ERR_LAUNCH);
        configured[ctx->device & 63] = true;
    }
    return B200Q_OK;
}

template <int F>
int launch_fmt(b200q_ctx* ctx, const CUtensorMap& map, const GemmArgs& a, dim3 grid, size_t smem) {
    static std::atomic<bool> configured[64] = {};
    int rc = configure_once(ctx, gemm_tc_kernel<F>, configured);
    if (rc != B200Q_OK) return rc;
    gemm_tc_kernel<F><<<grid, NTHREADS, smem, ctx->stream>>>(map, a);
    B200Q_CUDA(cudaGetLastError(), B200Q_ERR_LAUNCH);
    return B200Q_OK;
}

// The product itself, once the f16 copy of the activations (row-major [m, k]) and their row scales exist.
// Workspace of the persistent kernel: `ctas` partial tiles, then `ctas` flag words (zeroed when allocated).
int ensure_sk_workspace(b200q_ctx* ctx, int ctas) {
    if (ctx->sk_ws && ctx->sk_ctas >= ctas) return B200Q_OK;
    if (ctx->sk_ws) {
        B200Q_CUDA(cudaStreamSynchronize(ctx->stream), B200Q_ERR_DEVICE);
        cudaFree(ctx->sk_ws);
        ctx->sk_ws = nullptr;
        ctx->sk_ctas = 0;
    }
    const size_t slots = (size_t)ctas * SK_SLOT_FLOATS * sizeof(float);
    B200Q_CUDA(cudaMalloc(&ctx->sk_ws, slots + (size_t)ctas * sizeof(int)), B200Q_ERR_ALLOC);
    B200Q_CUDA(cudaMemsetAsync(static_cast<uint8_t*>(ctx->sk_ws) + slots, 0, (size_t)ctas * sizeof(int), ctx->stream), B200Q_ERR_DEVICE);
    ctx->sk_ctas = ctas;
    ctx->sk_epoch = 0;
    return B200Q_OK;
}

// MXFP4, Q4_0 and Q8_0 (GGUF) take the tensor-memory kernel when their 256-k steps are whole and the unit count fits an int.
bool mx4_tmem_path(const b200q_weight* w, int m) {
    // GGUF Q4_0 shares the path: the same 16 code bytes per block, an f16 d per block where MXFP4 has an exponent byte
    if ((w->fmt != fmt_of(MXFP4, GGUF) && w->fmt != fmt_of(Q4_0, GGUF) && w->fmt != fmt_of(Q8_0, GGUF)) || (w->k % 256) != 0) return false;
    if (!w->f16_scales_ok) return false;   // a block scale outside the f16 converters' range: shared-memory-operand kernel
    const int bn = m >= 256 ? 256 : ((m + 15) / 16) * 16;
    const int64_t tiles = ((w->n_local + BM - 1) / BM) * (int64_t)((m + bn - 1) / bn);
    return tiles * (w->k / 256) < (1ll << 30);
}

// GGUF MXFP6 E2M3 takes the tensor-memory kernel through its decode image (int8 codes), when the tensor has one; E3M2
// through an image of the same form that only this kernel reads (built by the tensor's first prefill product).
bool mx6_tmem_path(const b200q_weight* w, int m) {
    const bool e3m2 = w->fmt == fmt_of(MXFP6_E3M2, GGUF);
    if ((w->fmt != fmt_of(MXFP6_E2M3, GGUF) && !e3m2) || (w->k % 256) != 0 || !w->f16_scales_ok) return false;
    if (!e3m2 && (!w->dimg.base || w->dimg.kind != DK_MX6)) return false;
    if (e3m2 && ((w->n_local + 15) / 16) * (w->k / 128) / 8 > 0x7FFFFFFFll) return false;   // one image-build launch
    const int bn = m >= 256 ? 256 : ((m + 15) / 16) * 16;
    const int64_t tiles = ((w->n_local + BM - 1) / BM) * (int64_t)((m + bn - 1) / bn);
    return tiles * (w->k / 256) < (1ll << 30);
}

// GGUF Q5_K takes the tensor-memory kernel under the same conditions (persistent kernel only).
bool q5k_tmem_path(const b200q_weight* w, int m) {
    if (w->fmt != fmt_of(Q5_K, GGUF) || (w->k % 256) != 0 || !w->f16_scales_ok) return false;
    const int bn = m >= 256 ? 256 : ((m + 15) / 16) * 16;
    const int64_t tiles = ((w->n_local + BM - 1) / BM) * (int64_t)((m + bn - 1) / bn);
    return tiles * (w->k / 256) < (1ll << 30);
}

// Launch of the persistent prefill kernel with programmatic stream serialisation: its CTAs may start while the
// kernel ahead of it in the stream (the activation conversion) is still running.
template <class K>
cudaError_t launch_sk(b200q_ctx* ctx, K kernel, int ctas, size_t smem, const CUtensorMap& m0, const CUtensorMap& m1,
                      const CUtensorMap& m2, const CUtensorMap& m3, const CUtensorMap& m4, const CUtensorMap& m5,
                      const PeerMaps& peers, const SkArgs& k) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, m0, m1, m2, m3, m4, m5, peers, k);
}

// GGUF Q3_K planes -> GGUF Q6_K planes holding the same weights exactly: d (sc6 - 32) (q3 - 4) is d * sc * (q6 - 32) with the
// int8 scale sc = sc6 - 32 and q6 = q3 + 28 in 28..35. One thread per (block, half of 128, position e of 32): its four
// weights 32 t + e of the half share one byte of each Q6_K code plane.
__global__ void __launch_bounds__(256) q3k_to_q6k_planes_kernel(WView q3, WView q6, int64_t n_blocks) {
    const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
    const int64_t blk = idx >> 6;
    if (blk >= n_blocks) return;
    const int sec = (int)(idx >> 5) & 1, e = (int)idx & 31;
    const uint32_t hm = q3.p[0][blk * 32 + e];
    const uint32_t qs = q3.p[1][blk * 64 + sec * 32 + e];
    uint32_t q[4];
#pragma unroll
    for (int t = 0; t < 4; t++) q[t] = ((qs >> (2 * t)) & 3u) + (((hm >> (4 * sec + t)) & 1u) << 2) + 28u;
    const_cast<uint8_t*>(q6.p[0])[blk * 128 + sec * 64 + e] = (uint8_t)((q[0] & 15u) | ((q[2] & 15u) << 4));
    const_cast<uint8_t*>(q6.p[0])[blk * 128 + sec * 64 + 32 + e] = (uint8_t)((q[1] & 15u) | ((q[3] & 15u) << 4));
    const_cast<uint8_t*>(q6.p[1])[blk * 64 + sec * 32 + e] = (uint8_t)((q[0] >> 4) | ((q[1] >> 4) << 2) | ((q[2] >> 4) << 4) | ((q[3] >> 4) << 6));
    if (e < 8) {
        const uint8_t* sc = q3.p[2] + blk * 12;
        const int g16 = 8 * sec + e;
        const uint32_t lo = g16 < 8 ? (sc[g16] & 15u) : (uint32_t)(sc[g16 - 8] >> 4);
        const uint32_t hi = (uint32_t)(sc[8 + (g16 & 3)] >> (2 * (g16 >> 2))) & 3u;
        const_cast<uint8_t*>(q6.p[2])[blk * 16 + g16] = (uint8_t)(int8_t)((int)(lo | (hi << 4)) - 32);
    } else if (e == 8 && sec == 0) {
        const_cast<uint8_t*>(q6.p[3])[blk * 2] = q3.p[3][blk * 2];
        const_cast<uint8_t*>(q6.p[3])[blk * 2 + 1] = q3.p[3][blk * 2 + 1];
    }
}

int ensure_q6_planes(b200q_ctx* ctx, const b200q_weight* cw) {
    b200q_weight* w = const_cast<b200q_weight*>(cw);
    if (w->q6_planes) return B200Q_OK;
    const int pbytes[4] = {128, 64, 16, 2};
    size_t off[4], total = 0;
    for (int j = 0; j < 4; j++) {
        off[j] = total;
        total += ((size_t)w->n_blocks * pbytes[j] + 64 + 255) & ~(size_t)255;   // slack: vector loads may over-read a tail
    }
    void* p = nullptr;
    B200Q_CUDA(cudaMalloc(&p, total), B200Q_ERR_ALLOC);
    WView v{};
    for (int j = 0; j < 4; j++) v.p[j] = static_cast<uint8_t*>(p) + off[j];
    cudaError_t e = cudaMemsetAsync(p, 0, total, ctx->stream);
    if (e == cudaSuccess) {
        const int64_t threads = w->n_blocks * 64;
        q3k_to_q6k_planes_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, ctx->stream>>>(w->view, v, w->n_blocks);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) {
        cudaFree(p);
        return cuda_fail(B200Q_ERR_LAUNCH, e, "gemm: Q6_K planes of a Q3_K tensor");
    }
    w->q6_planes = p;
    w->q6_view = v;
    return B200Q_OK;
}

int launch_gemm_core(b200q_ctx* ctx, const b200q_weight* w, const __half* d_x16, const float* d_scale, float* d_y, int64_t ldy,
                     int m, const char* who, bool may_allocate) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return fail(B200Q_ERR_INIT, "%s: cuTensorMapEncodeTiled is not available from this driver", who);
    const int bn = m >= 256 ? 256 : ((m + 15) / 16) * 16;
    CUtensorMap map;
    cuuint64_t gdim[2] = {(cuuint64_t)w->k, (cuuint64_t)m};
    cuuint64_t gstr[1] = {(cuuint64_t)w->k * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)bn};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(d_x16), gdim, gstr, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B200Q_ERR_INVALID, "%s: cuTensorMapEncodeTiled failed with code %d", who, (int)r);
    GemmArgs a{};
    a.v = w->view; a.xscale = d_scale; a.y = d_y; a.ldy = ldy;
    a.n_rows = (int)w->n_local; a.k = (int)w->k; a.m = m; a.bn = bn;
    a.status = ctx->d_status;
    a.n_extra = ctx->scatter_extra;
    for (int p = 0; p < ctx->scatter_extra; p++) a.y_extra[p] = ctx->scatter_y[p];
    dim3 grid((unsigned)((w->n_local + BM - 1) / BM), (unsigned)((m + bn - 1) / bn));
    // tile stores of the persistent kernel's staged epilogue: y as a [m, n_local] fp32 tensor with row pitch ldy
    CUtensorMap ymap = map;
    const bool y16 = ctx->scatter_bf16;   // outputs are bf16 (a scattered product with B200Q_MM_SCATTER_BF16)
    a.y_bf16 = y16 ? 1 : 0;
    bool y_tma_ok = (ldy % (y16 ? 8 : 4)) == 0 && (reinterpret_cast<uintptr_t>(d_y) & 15) == 0;
    if (y16 && !may_allocate) return fail(B200Q_ERR_UNSUPPORTED, "%s: bf16 outputs need the persistent kernel", who);
    for (int p = 0; p < ctx->scatter_extra; p++) y_tma_ok = y_tma_ok && (reinterpret_cast<uintptr_t>(ctx->scatter_y[p]) & 15) == 0;
    if (y16 && !y_tma_ok) return fail(B200Q_ERR_UNSUPPORTED, "%s: bf16 outputs must be 16-byte aligned with ldy %% 8 == 0", who);
    PeerMaps peers;
    for (int p = 0; p < 7; p++) peers.m[p] = map;
    if (y_tma_ok) {
        cuuint64_t ydim[2] = {(cuuint64_t)w->n_local, (cuuint64_t)m};
        cuuint64_t ystr[1] = {(cuuint64_t)ldy * (y16 ? 2 : 4)};
        // one epilogue warp's block (32 weight rows x 32 activation rows), or, for a scattered product, the tile of a
        // group of four warps (128 weight rows)
        cuuint32_t ybox[2] = {ctx->scatter_extra > 0 ? 128u : 32u, 32u};
        for (int p = -1; p < ctx->scatter_extra; p++) {   // this GPU's output, then the peers' (a scattered product)
            r = enc(p < 0 ? &ymap : &peers.m[p], y16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, p < 0 ? d_y : ctx->scatter_y[p], ydim, ystr, ybox,
                    estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return fail(B200Q_ERR_INVALID, "%s: cuTensorMapEncodeTiled (output %d) failed with code %d", who, p + 1, (int)r);
        }
    }
    constexpr size_t STAGE_EPI_BYTES = 64 * BM * sizeof(float) + 128 + 128;
    // the persistent kernel prefetches partial sums from its workspace: [slots * 256 activation rows, 128 weight rows] fp32
    CUtensorMap wsmap = map;
    auto make_wsmap = [&]() -> int {
        cuuint64_t sdim[2] = {(cuuint64_t)BM, (cuuint64_t)ctx->sk_ctas * 256};
        cuuint64_t sstr[1] = {(cuuint64_t)BM * 4};
        cuuint32_t sbox[2] = {(cuuint32_t)BM, 64u};
        CUresult e = enc(&wsmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, ctx->sk_ws, sdim, sstr, sbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (e != CUDA_SUCCESS) return fail(B200Q_ERR_INVALID, "%s: cuTensorMapEncodeTiled (workspace) failed with code %d", who, (int)e);
        return B200Q_OK;
    };
    if (may_allocate && w->f16_scales_ok && (w->fmt == fmt_of(Q6_K, GGUF) || w->fmt == fmt_of(Q3_K, GGUF)) && (w->k % 256) == 0 &&
        (int64_t)grid.x * grid.y * (w->k / 256) < (1ll << 30)) {
        // Q6_K with the weight operand in tensor memory (persistent kernel only): three planes by TMA, d by plain loads.
        // A Q3_K tensor runs the same kernel on Q6_K planes that hold its weights exactly.
        if (w->fmt == fmt_of(Q3_K, GGUF)) {
            int rc = ensure_q6_planes(ctx, w);
            if (rc != B200Q_OK) return rc;
            a.v = w->q6_view;
        }
        a.a_col0 = (bn + 31) & ~31;
        a.tmem_cols = 32;
        while (a.tmem_cols < a.a_col0 + A_SLOT_COLS * STAGES) a.tmem_cols <<= 1;
        const size_t smem = 1024 + (size_t)STAGES * bn * BK * 2 + (size_t)2 * BM * 208 +
                            (2 * STAGES + 2 * RAW_STAGES + 4) * 8 + 32 + STAGE_EPI_BYTES;   // raw ring of two stages
        a.staged_epilogue = y_tma_ok ? 1 : 0;
        const int nsb = (int)(w->k / 256);
        CUtensorMap pm[3];
        const int pbytes[3] = {128, 64, 16};
        for (int j = 0; j < 3; j++) {
            const cuuint64_t row_bytes = (cuuint64_t)nsb * pbytes[j];
            cuuint64_t wdim[2] = {row_bytes, (cuuint64_t)w->n_local};
            cuuint64_t wstr[1] = {row_bytes};
            cuuint32_t wbox[2] = {(cuuint32_t)pbytes[j], (cuuint32_t)BM};
            const CUtensorMapSwizzle sw = j == 0 ? CU_TENSOR_MAP_SWIZZLE_128B : j == 1 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE;
            r = enc(&pm[j], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(a.v.p[j]), wdim, wstr, wbox, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return fail(B200Q_ERR_INVALID, "%s: cuTensorMapEncodeTiled (Q6_K plane %d) failed with code %d", who, j, (int)r);
        }
        const int64_t units = (int64_t)grid.x * grid.y * nsb;
        const int ctas = (int)std::min<int64_t>(ctx->info.sm_count, units);
        int rc = ensure_sk_workspace(ctx, ctx->info.sm_count);
        if (rc != B200Q_OK) return rc;
        if ((rc = make_wsmap()) != B200Q_OK) return rc;
        static std::atomic<bool> configured_q6[64] = {};
        rc = configure_once(ctx, gemm_tmem_sk_kernel<2>, configured_q6);
        if (rc != B200Q_OK) return rc;
        SkArgs k{};
        k.a = a;
        k.tiles_x = (int)grid.x; k.nsb = nsb; k.total_units = (int)units;
        k.ws = static_cast<float*>(ctx->sk_ws);
        k.flags = reinterpret_cast<int*>(static_cast<uint8_t*>(ctx->sk_ws) + (size_t)ctx->sk_ctas * SK_SLOT_FLOATS * sizeof(float));
        if (++ctx->sk_epoch == 0x7FFFFFFF) ctx->sk_epoch = 1;
        k.epoch = ctx->sk_epoch;
        B200Q_CUDA(launch_sk(ctx, gemm_tmem_sk_kernel<2>, ctas, smem, map, pm[0], pm[1], pm[2], ymap, wsmap, peers, k), B200Q_ERR_LAUNCH);
        return B200Q_OK;
    }
    if (may_allocate && mx6_tmem_path(w, m)) {
        // MXFP6 E2M3 with the weight operand in tensor memory, read from the decode image (persistent kernel only)
        a.a_col0 = (bn + 31) & ~31;
        a.tmem_cols = 32;
        while (a.tmem_cols < a.a_col0 + A_SLOT_COLS * STAGES) a.tmem_cols <<= 1;
        const size_t smem = 1024 + (size_t)STAGES * bn * BK * 2 + (size_t)2 * BM * 256 + (2 * STAGES + 2 * RAW_STAGES + 4) * 8 + 32 + STAGE_EPI_BYTES;
        a.staged_epilogue = y_tma_ok ? 1 : 0;
        const int nsb = (int)(w->k / 256);
        const int64_t units = (int64_t)grid.x * grid.y * nsb;
        const int ctas = (int)std::min<int64_t>(ctx->info.sm_count, units);
        int rc = ensure_sk_workspace(ctx, ctx->info.sm_count);
        if (rc != B200Q_OK) return rc;
        if ((rc = make_wsmap()) != B200Q_OK) return rc;
        static std::atomic<bool> configured_mx6[64] = {};
        rc = configure_once(ctx, gemm_tmem_sk_kernel<6>, configured_mx6);
        if (rc != B200Q_OK) return rc;
        SkArgs k{};
        k.a = a;
        k.tiles_x = (int)grid.x; k.nsb = nsb; k.total_units = (int)units;
        k.ws = static_cast<float*>(ctx->sk_ws);
        k.flags = reinterpret_cast<int*>(static_cast<uint8_t*>(ctx->sk_ws) + (size_t)ctx->sk_ctas * SK_SLOT_FLOATS * sizeof(float));
        if (++ctx->sk_epoch == 0x7FFFFFFF) ctx->sk_epoch = 1;
        k.epoch = ctx->sk_epoch;
        if (w->fmt == fmt_of(MXFP6_E3M2, GGUF)) {
            b200q_weight* wm = const_cast<b200q_weight*>(w);
            if (!wm->pimg.base && (rc = build_e3m2_prefill_image(ctx, w, &wm->pimg)) != B200Q_OK) return rc;
            k.img = w->pimg.base; k.img_nh = w->pimg.nh; k.img_nrt = w->pimg.nrt; k.img_e3m2 = 1;
        } else {
            k.img = w->dimg.base; k.img_nh = w->dimg.nh; k.img_nrt = w->dimg.nrt;
        }
        B200Q_CUDA(launch_sk(ctx, gemm_tmem_sk_kernel<6>, ctas, smem, map, map, map, map, ymap, wsmap, peers, k), B200Q_ERR_LAUNCH);
        return B200Q_OK;
    }
    if (may_allocate && mx4_tmem_path(w, m)) {
        // MXFP4 with the weight operand in tensor memory (persistent kernel only)
        a.a_col0 = (bn + 31) & ~31;
        a.tmem_cols = 32;
        while (a.tmem_cols < a.a_col0 + A_SLOT_COLS * STAGES) a.tmem_cols <<= 1;
        const bool q80 = w->fmt == fmt_of(Q8_0, GGUF);   // 32 code bytes per block, raw ring of two 32 KB stages
        const size_t smem = 1024 + (size_t)STAGES * bn * BK * 2 + (q80 ? (size_t)2 * BM * 256 : (size_t)RAW_STAGES * BM * 128) +
                            (2 * STAGES + 2 * RAW_STAGES + 4) * 8 + 32 + STAGE_EPI_BYTES;
        a.staged_epilogue = y_tma_ok ? 1 : 0;
        CUtensorMap wmap;
        const cuuint64_t row_bytes = (cuuint64_t)(w->k / 32) * (q80 ? 32 : 16);
        cuuint64_t wdim[2] = {row_bytes, (cuuint64_t)w->n_local};
        cuuint64_t wstr[1] = {row_bytes};
        cuuint32_t wbox[2] = {128u, (cuuint32_t)BM};
        r = enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(w->view.p[1]), wdim, wstr, wbox, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(B200Q_ERR_INVALID, "%s: cuTensorMapEncodeTiled (codes) failed with code %d", who, (int)r);
        const int nsb = (int)(w->k / 256);
        const int64_t units = (int64_t)grid.x * grid.y * nsb;
        const int ctas = (int)std::min<int64_t>(ctx->info.sm_count, units);
        int rc = ensure_sk_workspace(ctx, ctx->info.sm_count);
        if (rc != B200Q_OK) return rc;
        if ((rc = make_wsmap()) != B200Q_OK) return rc;
        const bool q40 = w->fmt == fmt_of(Q4_0, GGUF);
        static std::atomic<bool> configured_mx[64] = {}, configured_q40[64] = {};
        static std::atomic<bool> configured_q80[64] = {};
        rc = q80 ? configure_once(ctx, gemm_tmem_sk_kernel<4>, configured_q80)
                 : q40 ? configure_once(ctx, gemm_tmem_sk_kernel<3>, configured_q40) : configure_once(ctx, gemm_tmem_sk_kernel<1>, configured_mx);
        if (rc != B200Q_OK) return rc;
        SkArgs k{};
        k.a = a;
        k.tiles_x = (int)grid.x; k.nsb = nsb; k.total_units = (int)units;
        k.ws = static_cast<float*>(ctx->sk_ws);
        k.flags = reinterpret_cast<int*>(static_cast<uint8_t*>(ctx->sk_ws) + (size_t)ctx->sk_ctas * SK_SLOT_FLOATS * sizeof(float));
        if (++ctx->sk_epoch == 0x7FFFFFFF) ctx->sk_epoch = 1;
        k.epoch = ctx->sk_epoch;
        if (q80) B200Q_CUDA(launch_sk(ctx, gemm_tmem_sk_kernel<4>, ctas, smem, map, wmap, wmap, wmap, ymap, wsmap, peers, k), B200Q_ERR_LAUNCH);
        else if (q40) B200Q_CUDA(launch_sk(ctx, gemm_tmem_sk_kernel<3>, ctas, smem, map, wmap, wmap, wmap, ymap, wsmap, peers, k), B200Q_ERR_LAUNCH);
        else B200Q_CUDA(launch_sk(ctx, gemm_tmem_sk_kernel<1>, ctas, smem, map, wmap, wmap, wmap, ymap, wsmap, peers, k), B200Q_ERR_LAUNCH);
        return B200Q_OK;
    }
    const bool q5k = w->fmt == fmt_of(Q5_K, GGUF);   // persistent kernel only (no one-CTA-per-tile variant)
    if (w->f16_scales_ok && (w->fmt == fmt_of(Q4_K, GGUF) || (q5k && may_allocate && (int64_t)grid.x * grid.y * (w->k / 256) < (1ll << 30))) && (w->k % 256) == 0) {
        // weight operand in tensor memory
        a.a_col0 = (bn + 31) & ~31;
        a.tmem_cols = 32;
        while (a.tmem_cols < a.a_col0 + A_SLOT_COLS * STAGES) a.tmem_cols <<= 1;
        const int raw_row = q5k ? 176 : RAW_ROW_BYTES;   // bytes of one super-block
        const size_t smem = 1024 + (size_t)STAGES * bn * BK * 2 +
                            (q5k ? (size_t)2 * BM * 176 : (size_t)RAW_STAGES * RAW_STAGE_BYTES) +   // Q5_K: raw ring of two stages
                            (2 * STAGES + 2 * RAW_STAGES + 1) * 8 + 16;
        static std::atomic<bool> configured[64] = {};
        int rc = q5k ? B200Q_OK : configure_once(ctx, gemm_q4k_tmem_kernel, configured);
        if (rc != B200Q_OK) return rc;
        CUtensorMap wmap;
        const cuuint64_t row_bytes = (cuuint64_t)(w->k / 256) * raw_row;
        cuuint64_t wdim[2] = {row_bytes, (cuuint64_t)w->n_local};
        cuuint64_t wstr[1] = {row_bytes};
        cuuint32_t wbox[2] = {(cuuint32_t)raw_row, (cuuint32_t)BM};
        r = enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(w->view.p[0]), wdim, wstr, wbox, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(B200Q_ERR_INVALID, "%s: cuTensorMapEncodeTiled (weights) failed with code %d", who, (int)r);
        const int nsb = (int)(w->k / 256);
        const int64_t units = (int64_t)grid.x * grid.y * nsb;
        if (may_allocate && units < (1ll << 30)) {
            // persistent kernel: one CTA per SM, all co-resident (one CTA fills an SM's shared memory)
            const int ctas = (int)std::min<int64_t>(ctx->info.sm_count, units);
            rc = ensure_sk_workspace(ctx, ctx->info.sm_count);
            if (rc != B200Q_OK) return rc;
            if ((rc = make_wsmap()) != B200Q_OK) return rc;
            static std::atomic<bool> configured_sk[64] = {}, configured_q5k[64] = {};
            rc = q5k ? configure_once(ctx, gemm_tmem_sk_kernel<5>, configured_q5k) : configure_once(ctx, gemm_tmem_sk_kernel<0>, configured_sk);
            if (rc != B200Q_OK) return rc;
            SkArgs k{};
            k.a = a;
            k.a.staged_epilogue = y_tma_ok ? 1 : 0;
            k.tiles_x = (int)grid.x; k.nsb = nsb; k.total_units = (int)units;
            k.ws = static_cast<float*>(ctx->sk_ws);
            k.flags = reinterpret_cast<int*>(static_cast<uint8_t*>(ctx->sk_ws) + (size_t)ctx->sk_ctas * SK_SLOT_FLOATS * sizeof(float));
            if (++ctx->sk_epoch == 0x7FFFFFFF) ctx->sk_epoch = 1;
            k.epoch = ctx->sk_epoch;
            if (q5k) B200Q_CUDA(launch_sk(ctx, gemm_tmem_sk_kernel<5>, ctas, smem + 32 + STAGE_EPI_BYTES, map, wmap, wmap, wmap, ymap, wsmap, peers, k), B200Q_ERR_LAUNCH);
            else B200Q_CUDA(launch_sk(ctx, gemm_tmem_sk_kernel<0>, ctas, smem + 32 + STAGE_EPI_BYTES, map, wmap, wmap, wmap, ymap, wsmap, peers, k), B200Q_ERR_LAUNCH);
            return B200Q_OK;
        }
        if (y16) return fail(B200Q_ERR_UNSUPPORTED, "%s: bf16 outputs need the persistent kernel", who);
        gemm_q4k_tmem_kernel<<<grid, NTHREADS, smem, ctx->stream>>>(map, wmap, a);
        B200Q_CUDA(cudaGetLastError(), B200Q_ERR_LAUNCH);
        return B200Q_OK;
    }
    if (y16) return fail(B200Q_ERR_UNSUPPORTED, "%s: bf16 outputs need a format of the tensor-memory kernel with k %% 256 == 0 and block scales in the f16 range", who);
    a.tmem_cols = 32;
    while (a.tmem_cols < bn) a.tmem_cols <<= 1;
    const size_t smem = 1024 + (size_t)STAGES * (A_STAGE_BYTES + (size_t)bn * BK * 2) + (3 * STAGES + 1) * 8 + 16;
    switch (w->fmt) {
#define X(F) \
    case F: return launch_fmt<F>(ctx, map, a, grid, smem);
        B200Q_FOR_EACH_FMT(X)
#undef X
    }
    return fail(B200Q_ERR_INVALID, "%s: unknown format %d", who, w->fmt);
}

}  // namespace

// The layouts whose block scales the upload does not scan on the host (f32 scales, f16 sub-block scales): one pass over
// the weights themselves, on the device, the first time the question is asked. Synchronises the stream once per tensor.
static bool weights_fit_f16(const b200q_weight* cw) {
    if (cw->range_scanned) return cw->f16_weights_ok;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    b200q_weight* w = const_cast<b200q_weight*>(cw);
    if (w->range_scanned) return w->f16_weights_ok;
    b200q_ctx* ctx = w->ctx;
    unsigned int* d_max = reinterpret_cast<unsigned int*>(ctx->d_status + 6);
    unsigned int bits = 0x7F800000u;   // any failure below reads as "out of range": the fp32 kernels take the tensor
    bool ok = cudaSetDevice(ctx->device) == cudaSuccess && cudaMemsetAsync(d_max, 0, sizeof(unsigned int), ctx->stream) == cudaSuccess &&
              launch_absmax(ctx, w->fmt, w->view, w->n_elements, d_max) == B200Q_OK &&
              cudaMemcpyAsync(&bits, d_max, sizeof(unsigned int), cudaMemcpyDeviceToHost, ctx->stream) == cudaSuccess &&
              cudaMemsetAsync(d_max, 0, sizeof(unsigned int), ctx->stream) == cudaSuccess &&
              cudaStreamSynchronize(ctx->stream) == cudaSuccess;
    float mx;
    memcpy(&mx, &bits, 4);
    // the same limits as the host scan of the GGUF layouts: nothing beyond the f16 range, the largest weight not a subnormal
    w->f16_weights_ok = ok && (mx == 0.0f || (mx <= 60000.0f && mx >= 6.2e-5f));
    w->range_scanned = true;
    return w->f16_weights_ok;
}

bool gemm_tc_supported(const b200q_weight* w, int m) {
    // weights beyond the f16 range (seen by the upload's scan of the block scales, or by a scan of the weights) stay on
    // the fp32 decode kernels
    return w->orient == B200Q_ORIENT_NK && m >= 1 && (w->k % BK) == 0 && w->n_local < 0x7FFFFF00ll && w->k < (1 << 30) &&
           weights_fit_f16(w);
}

// x: fp32 or bf16 [m, ldx] on the device. y: fp32 [m, ldy]. Uses the context's third scratch buffer for the
// f16 copy of the activations and their row scales.
int launch_gemm_tc(b200q_ctx* ctx, const b200q_weight* w, const void* d_x, int x_is_bf16, int64_t ldx, float* d_y, int64_t ldy, int m) {
    if (!gemm_tc_supported(w, m)) return fail(B200Q_ERR_UNSUPPORTED, "gemm: needs an NK tensor with k %% 64 == 0");
    const size_t x16_bytes = ((size_t)m * w->k * 2 + 255) & ~(size_t)255;
    // + 2 KB: the staged epilogue reads the scales of whole 32-row blocks, up to one tile past row m
    int rc = ensure_scratch(ctx, x16_bytes + (size_t)m * sizeof(float) + 2048, 2);
    if (rc != B200Q_OK) return rc;
    __half* d_x16 = static_cast<__half*>(ctx->scratch3);
    float* d_scale = reinterpret_cast<float*>(static_cast<uint8_t*>(ctx->scratch3) + x16_bytes);
    // the nibble-mask producers emit weights in the order 0,2,1,3 inside every group of four
    const int perm = (w->fmt == fmt_of(Q4_K, GGUF) || q5k_tmem_path(w, m) || (mx4_tmem_path(w, m) && w->fmt != fmt_of(Q8_0, GGUF))) ? 1 : 0;
    if (x_is_bf16) rc = launch_x_to_f16(ctx, static_cast<const __nv_bfloat16*>(d_x), ldx, d_x16, d_scale, m, (int)w->k, perm);
    else rc = launch_x_to_f16(ctx, static_cast<const float*>(d_x), ldx, d_x16, d_scale, m, (int)w->k, perm, ctx->act_mul);
    if (rc != B200Q_OK) return rc;
    return launch_gemm_core(ctx, w, d_x16, d_scale, d_y, ldy, m, "gemm", true);
}

// Two prefill products of ONE activation tensor (gate and up, or any pair with the same inner dimension and the
// same activation order): the f16 copy of the activations is made once and both tensor-core kernels read it.
int launch_gemm_tc_pair(b200q_ctx* ctx, const b200q_weight* w0, const b200q_weight* w1, const float* d_x, int64_t ldx,
                        float* d_y0, float* d_y1, int m) {
    auto perm_of = [&](const b200q_weight* w) {
        return (w->fmt == fmt_of(Q4_K, GGUF) || q5k_tmem_path(w, m) || (mx4_tmem_path(w, m) && w->fmt != fmt_of(Q8_0, GGUF))) ? 1 : 0;
    };
    if (!gemm_tc_supported(w0, m) || !gemm_tc_supported(w1, m) || w0->k != w1->k || perm_of(w0) != perm_of(w1)) {
        int rc = launch_gemm_tc(ctx, w0, d_x, 0, ldx, d_y0, w0->n_local, m);
        if (rc != B200Q_OK) return rc;
        return launch_gemm_tc(ctx, w1, d_x, 0, ldx, d_y1, w1->n_local, m);
    }
    const size_t x16_bytes = ((size_t)m * w0->k * 2 + 255) & ~(size_t)255;
    int rc = ensure_scratch(ctx, x16_bytes + (size_t)m * sizeof(float) + 2048, 2);
    if (rc != B200Q_OK) return rc;
    __half* d_x16 = static_cast<__half*>(ctx->scratch3);
    float* d_scale = reinterpret_cast<float*>(static_cast<uint8_t*>(ctx->scratch3) + x16_bytes);
    rc = launch_x_to_f16(ctx, d_x, ldx, d_x16, d_scale, m, (int)w0->k, perm_of(w0));
    if (rc != B200Q_OK) return rc;
    rc = launch_gemm_core(ctx, w0, d_x16, d_scale, d_y0, w0->n_local, m, "gemm", true);
    if (rc != B200Q_OK) return rc;
    // the second kernel's weight copies and conversion overlap the first kernel's tail; it reads the same f16
    // activations only after the first kernel has completed (griddepcontrol.wait), and both only read them
    return launch_gemm_core(ctx, w1, d_x16, d_scale, d_y1, w1->n_local, m, "gemm", true);
}

// ---------------------------------------------------------------------------------------------------
// Prefill product for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the moment they need a product: a serving process
// whose own pool has already claimed the rest of HBM (the allocation would simply fail), or a latency-
// critical loop that cannot afford cudaMalloc's implicit device-wide synchronisation. The ordinary entry
// points grow a per-context scratch buffer on demand (the f16 copy of the activations and their row
// scales); this variant keeps that scratch in a fixed array that is part of the library image instead.
// Every GPU that loads the library carries the array (16 MiB + 64 KiB) until the process exits.
constexpr size_t NOALLOC_X16_BYTES = 16u << 20;     // f16 copy of the activations: m * k <= 8,388,608
constexpr size_t NOALLOC_SCALE_BYTES = 64u << 10;   // one fp32 scale per activation row: m <= 16,384
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_X16_BYTES + NOALLOC_SCALE_BYTES];

// In host code the array's name is only a stand-in; the device address has to be asked for, once per
// device, with that device current.
static std::atomic<void*> g_noalloc_dev_ptr[64] = {};

int launch_gemm_tc_noalloc(b200q_ctx* ctx, const b200q_weight* w, const float* d_x, float* d_y, int m) {
    if (!gemm_tc_supported(w, m)) return fail(B200Q_ERR_UNSUPPORTED, "matmul_noalloc: needs an NK tensor with k %% 64 == 0");
    if (ctx->device < 0 || ctx->device >= 64) return fail(B200Q_ERR_INVALID, "matmul_noalloc: device index %d out of range", ctx->device);
    if ((size_t)m * (size_t)w->k * 2 > NOALLOC_X16_BYTES || (size_t)m * sizeof(float) > NOALLOC_SCALE_BYTES)
        return fail(B200Q_ERR_INVALID,
                    "matmul_noalloc: m=%d x k=%lld needs %zu bytes of scratch; the built-in scratch holds m*k <= %zu elements and m <= %zu rows",
                    m, (long long)w->k, (size_t)m * (size_t)w->k * 2, NOALLOC_X16_BYTES / 2, NOALLOC_SCALE_BYTES / sizeof(float));
    if (!g_noalloc_dev_ptr[ctx->device].load()) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) return cuda_fail(B200Q_ERR_INIT, e, "cudaGetSymbolAddress(built-in scratch)");
        g_noalloc_dev_ptr[ctx->device] = p;
    }
    __half* d_x16 = static_cast<__half*>(g_noalloc_dev_ptr[ctx->device].load());
    float* d_scale = reinterpret_cast<float*>(static_cast<unsigned char*>(g_noalloc_dev_ptr[ctx->device].load()) + NOALLOC_X16_BYTES);
    // nothing in the scratch has to start at zero: the conversion below rewrites every element the GEMM reads
    const int perm = w->fmt == fmt_of(Q4_K, GGUF) ? 1 : 0;
    int rc = launch_x_to_f16(ctx, d_x, w->k, d_x16, d_scale, m, (int)w->k, perm);
    if (rc != B200Q_OK) return rc;
    return launch_gemm_core(ctx, w, d_x16, d_scale, d_y, w->n_local, m, "matmul_noalloc", false);
}

int launch_bounded_wait_selftest(b200q_ctx* ctx, long long budget_cycles) {
    bounded_wait_selftest_kernel<<<1, 32, 0, ctx->stream>>>(ctx->d_status, budget_cycles);
    B200Q_CUDA(cudaGetLastError(), B200Q_ERR_LAUNCH);
    return B200Q_OK;
}

// Reads and clears the launch status words: [0] a bounded wait of a tensor-core kernel expired (site code),
// [1] token ids the embedding lookup found out of range.
int gemm_tc_check_status(b200q_ctx* ctx) {
    // one small copy into page-locked memory and ONE synchronise: the copy rides the stream behind the kernels
    int* h = ctx->h_status;
    B200Q_CUDA(cudaMemcpyAsync(h, ctx->d_status, 2 * sizeof(int), cudaMemcpyDeviceToHost, ctx->stream), B200Q_ERR_COPY);
    B200Q_CUDA(cudaStreamSynchronize(ctx->stream), B200Q_ERR_DEVICE);
    const int h0 = h[0], h1 = h[1];
    if (h0 != 0 || h1 != 0) cudaMemsetAsync(ctx->d_status, 0, 8 * sizeof(int), ctx->stream);   // the decode kernel's counters too
    if (h0 != 0)
        return fail(B200Q_ERR_TIMEOUT, "a bounded device-side wait expired (site %d); results of that launch are invalid", h0);
    if (h1 != 0)
        return fail(B200Q_ERR_INVALID, "get_rows: %d token id(s) exceed the vocabulary size; their output rows were zero-filled", h1);
    return B200Q_OK;
}

}  // namespace b200q
