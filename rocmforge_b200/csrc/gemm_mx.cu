// Native block-scaled prefill product for GGUF MXFP4 and MXFP6 (opt-in, B200Q_MM_MX_NATIVE): the 4-bit E2M1 (6-bit
// E2M3 / E3M2) codes go to the tensor cores AS THEY ARE, with their E8M0 block scales, through
// tcgen05.mma.kind::mxf8f6f4.block_scale; nothing is dequantised. The activations are quantised to MXFP8 (E4M3 codes, one E8M0 scale per 32 values) by a small
// kernel ahead of the product, so the result carries the rounding of a 4-bit mantissa per activation (relative
// error of a few 1e-2 on random data, against 2e-3 for the default f16 path): it is a throughput mode for callers
// that accept MX activations, never the default. Reference side: the tensors of src/loader/dequant.rs:85-132 /
// kernels/mxfp_dequant.hip:147, multiplied without their fp32 expansion.
//
// Operands (both K-major, 128-byte swizzle, 128 k per pipeline stage, one MMA per 32 k):
//   A  weights: the tensor's code plane [n, k/2] bytes, fetched by TMA as 16 x U4 -> 16-byte containers
//      (CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B: 8 code bytes followed by 8 bytes of padding), the layout the MMA reads
//      4-bit operands in. The hardware takes byte j of a block as elements (2j, 2j+1); a GGUF block keeps elements
//      (j, j+16) there, so hardware position h of a block holds element 8 (h/16) + (h%16)/2 + 16 (h%2). The
//      activation codes are written in the same order, so the products pair up. MXFP6: the code plane [n, 3k/4]
//      bytes as 16 x U6 -> 16-byte containers (12 code bytes + 4 of padding); its 6-bit fields are already in the
//      hardware's order (element i at bit 6 i), so the activations keep theirs.
//   B  activations: E4M3 bytes [m, k] in that order, plain tiled TMA.
//   Scales: one byte per row and 32 k, in tensor memory. The MMA wants them as 512-byte chunks of 128 rows x 4
//      k-blocks, byte (row % 32) * 16 + (row / 32) * 4 + kblock; both scale planes are kept in that order in global
//      memory (the weights' plane is built once per tensor from its exponent plane, the activations' by the
//      quantising kernel), a stage fetches its chunks with untiled bulk copies and the MMA thread moves them to
//      tensor memory with tcgen05.cp (32 x 128 bit, replicated to the four lane quarters).
// Persistent CTAs, one per SM, over whole 128 x BN output tiles (no partial sums): warp 0 issues the copies and runs
// ahead across tile boundaries, warp 1 the tensor-memory copies and MMAs, warps 2..5 read the accumulator and store
// fp32 while the ring refills for the next tile. Every wait is bounded.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <stdlib.h>

#include <algorithm>
#include <atomic>

#include "common.cuh"
#include "formats.cuh"

namespace b200q {

namespace {

constexpr int MX_BM = 128;
constexpr int MX_BK = 128;          // k per stage = one 128-byte swizzle row of 8-bit containers
constexpr int MX_STAGES = 4;
constexpr int MX_THREADS = 192;          // pair kernel: copies / MMA / 4 epilogue warps
constexpr int MX1_THREADS = 224;         // single-CTA kernel: one more warp moves the scales to tensor memory
constexpr long long MX_WAIT_BUDGET = 1ll << 31;
constexpr int MX_SFA_COL = 256;     // tensor-memory columns: accumulator 0..255, weight scales 4 per stage, activation scales 8 per stage
constexpr int MX_SFB_COL = 272;

__device__ __forceinline__ uint32_t mx_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mx_bar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mx_bar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mx_bar_try(uint32_t bar, uint32_t parity) {
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
// bounded: after about a second of SM clock the wait raises the CTA's abort flag and the launch's status word
__device__ __forceinline__ bool mx_bar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
    long long t0 = 0;
    for (uint32_t spin = 1;; spin++) {
        if (mx_bar_try(bar, parity)) return true;
        if ((spin & 4095u) == 0) {
            if (*abort_flag != 0) return false;
            const long long now = clock64();
            if (t0 == 0) t0 = now;
            if (now - t0 > MX_WAIT_BUDGET) {
                *abort_flag = 1;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ void mx_tma_2d(uint32_t dst, const CUtensorMap* map, int cx, int cy, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(cx), "r"(cy)
        : "memory");
}
__device__ __forceinline__ void mx_bulk(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void mx_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void mx_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void mx_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// K-major operand tile with 128-byte swizzle: rows at a 128-byte pitch, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t mx_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFFu);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;          // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;          // SWIZZLE_128B
    return d;
}
// 32 rows x 16 bytes, unswizzled: rows 16 bytes apart, 8-row groups 128 bytes apart (source of the scale copies)
__device__ __forceinline__ uint64_t mx_desc_sf(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFFu);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(128 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}
__device__ __forceinline__ void mx_cp_sf(uint32_t tmem_col, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_col), "l"(desc) : "memory");
}
__device__ __forceinline__ void mx_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate, uint32_t sfa,
                                       uint32_t sfb) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
}
__device__ __forceinline__ void mx_tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
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

struct MxArgs {
    const uint8_t* sfa;   // weight scales in chunk order: [row tiles][k / 128][512]
    const uint8_t* sfb;   // activation scales: [token tiles of 128][k / 128][512]
    float* y;
    int64_t ldy;
    int n_rows, m, k, bn;
    int a_format;         // operand format of the weights in the MMA: 5 = E2M1, 3 = E2M3, 4 = E3M2
    int a_tx;             // bytes a stage's code tile counts for on its barrier: the PACKED bytes (64 or 96 per row)
    int m_tiles, row_tiles;
    // The tiles of the last, partly filled wave are cut along the activation rows into `split` (1 or 2) pieces of
    // `sub_bn` rows each (work items >= full_tiles), so that the wave costs half a tile time instead of a whole one.
    int full_tiles, split, sub_bn, n_work;
    int* status;
};

// hardware position h (0..31) of a block -> element of the GGUF block
__host__ __device__ __forceinline__ int mx_elem_of_pos(int h) { return 8 * (h >> 4) + ((h & 15) >> 1) + 16 * (h & 1); }

// Weight scales: exponent plane [n, k/32] -> chunks. One thread per output byte.
__global__ void __launch_bounds__(256) mx_build_sfa_kernel(const uint8_t* __restrict__ e, uint8_t* __restrict__ out, int n_rows, int nkb, int64_t total) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int b = (int)(i & 511);
    const int64_t chunk = i >> 9;
    const int kb = (int)(chunk % nkb);
    const int64_t rt = chunk / nkb;
    const int r32 = b >> 4, q = (b >> 2) & 3, j = b & 3;
    const int64_t row = rt * 128 + q * 32 + r32;
    out[i] = row < n_rows ? e[row * ((int64_t)nkb * 4) + kb * 4 + j] : (uint8_t)127;
}

// Activations -> MXFP8: one thread per (row, block of 32). E8M0 scale = the smallest power of two that brings the
// block's largest magnitude inside E4M3's range (448), codes by round-to-nearest with saturation, written at the
// hardware positions of the weights' code order; the scale byte goes to its place in the chunk order.
template <typename T, bool PERM>
__global__ void __launch_bounds__(256) mx_quantize_x_kernel(const T* __restrict__ x, int64_t ldx, uint8_t* __restrict__ q, uint8_t* __restrict__ sfb,
                                                            int m, int k, int m_pad) {
    const int nb = k >> 5;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)m_pad * nb) return;
    const int tok = (int)(i / nb), blk = (int)(i - (int64_t)tok * nb);
    float v[32];
    float amax = 0.f;
    if (tok < m) {
        const T* xp = x + (int64_t)tok * ldx + (int64_t)blk * 32;
        if (sizeof(T) == 4 && (ldx & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
            const float4* x4 = reinterpret_cast<const float4*>(xp);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float4 t = __ldg(x4 + j);
                v[4 * j] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = (float)xp[j];
        }
#pragma unroll
        for (int j = 0; j < 32; j++) amax = fmaxf(amax, fabsf(v[j]));
    } else {
#pragma unroll
        for (int j = 0; j < 32; j++) v[j] = 0.f;
    }
    int e = 127;
    if (amax > 0.f && amax <= 3.0e38f) {
        // smallest e with amax / 2^(e-127) <= 448
        int ex;
        const float fr = frexpf(amax * (1.0f / 448.0f), &ex);   // amax / 448 = fr * 2^ex, fr in [0.5, 1)
        e = 127 + (fr == 0.5f ? ex - 1 : ex);
        e = min(max(e, 1), 254);
    }
    const float inv = __uint_as_float((uint32_t)(254 - e) << 23);   // 2^(127 - e)
    uint32_t w[8];
#pragma unroll
    for (int g = 0; g < 8; g++) {
        uint32_t word = 0;
#pragma unroll
        for (int p = 0; p < 4; p += 2) {
            const int h = 4 * g + p;
            const float2 pr = PERM ? make_float2(v[mx_elem_of_pos(h)] * inv, v[mx_elem_of_pos(h + 1)] * inv) : make_float2(v[h] * inv, v[h + 1] * inv);
            word |= (uint32_t)__nv_cvt_float2_to_fp8x2(pr, __NV_SATFINITE, __NV_E4M3) << (8 * p);
        }
        w[g] = word;
    }
    uint4* dst = reinterpret_cast<uint4*>(q + (int64_t)tok * k + (int64_t)blk * 32);
    dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
    dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
    const int nkb = k >> 7;
    const int64_t chunk = (int64_t)(tok >> 7) * nkb + (blk >> 2);
    const int r = tok & 127;
    sfb[chunk * 512 + (r & 31) * 16 + (r >> 5) * 4 + (blk & 3)] = (uint8_t)e;
}

struct MxWork {
    int row0, tok0, nb, row_tile;
};
__device__ __forceinline__ MxWork mx_work(const MxArgs& a, int w) {
    MxWork r;
    int tile = w, sub = 0;
    r.nb = a.bn;
    if (w >= a.full_tiles) {
        tile = a.full_tiles + (w - a.full_tiles) / a.split;
        sub = (w - a.full_tiles) % a.split;
        r.nb = a.sub_bn;
    }
    r.row_tile = tile / a.m_tiles;
    r.row0 = r.row_tile * MX_BM;
    r.tok0 = (tile - r.row_tile * a.m_tiles) * a.bn + sub * a.sub_bn;
    return r;
}

__global__ void __launch_bounds__(MX1_THREADS, 1)
gemm_mxf4_native_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                        const __grid_constant__ CUtensorMap tmap_xs, MxArgs a) {
    extern __shared__ uint8_t mx_smem_raw[];
    uint8_t* smem = mx_smem_raw + ((1024u - (mx_smem_u32(mx_smem_raw) & 1023u)) & 1023u);
    const int b_stage = a.bn * MX_BK;                 // bytes
    const int nsfb = (a.bn + 127) >> 7;               // activation-scale chunks per stage
    uint8_t* sA = smem;                                // [stages][128 rows][128 B]
    uint8_t* sB = sA + MX_STAGES * MX_BM * MX_BK;      // [stages][bn rows][128 B]
    uint8_t* sSFA = sB + MX_STAGES * b_stage;          // [stages][512]
    uint8_t* sSFB = sSFA + MX_STAGES * 512;            // [stages][2][512]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sSFB + MX_STAGES * 1024);
    uint64_t* full = bars;
    uint64_t* empty = bars + MX_STAGES;
    uint64_t* accum = empty + MX_STAGES;     // the MMAs of a tile are complete -> epilogue
    uint64_t* afree = accum + 1;             // the four epilogue warps have read the accumulator -> next tile's MMAs
    uint64_t* sfrdy = afree + 1;             // [stages] the stage's scales are in tensor memory -> its MMAs
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sfrdy + MX_STAGES);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nkb = a.k / MX_BK;
    // Persistent: CTA c takes tiles c, c + grid, ...; token tiles vary fastest, so the CTAs that run together share
    // the weight tiles (read from HBM once) and the activation tiles of all token tiles stay in L2.
    const int total_tiles = a.n_work;
    if (tid == 0) {
        for (int s = 0; s < MX_STAGES; s++) {
            mx_bar_init(mx_smem_u32(&full[s]), 1);
            mx_bar_init(mx_smem_u32(&empty[s]), 1);
            mx_bar_init(mx_smem_u32(&sfrdy[s]), 1);
        }
        mx_bar_init(mx_smem_u32(accum), 1);
        mx_bar_init(mx_smem_u32(afree), 4);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(mx_smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    mx_fence_before();
    __syncthreads();
    mx_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- copies: codes, activation codes, scales
        // (runs ahead of the MMAs by the depth of the ring, across tile boundaries: the ring is full again when the
        // accumulator of the previous tile has been read out)
        if (lane == 0) {
            // the code tile counts with its PACKED bytes (64 or 96 per row), although it fills 128 bytes per row of shared memory
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const MxWork wk = mx_work(a, tile);
                const int row0 = wk.row0, tok0 = wk.tok0;
                const bool piece = wk.nb != a.bn;            // a piece of a tile of the last wave: its own, smaller copy box
                const int nsf = piece ? 1 : nsfb;            // pieces are at most 128 rows inside one chunk of scales
                const uint32_t stage_tx = (uint32_t)(a.a_tx + wk.nb * MX_BK + 512 + 512 * nsf);
                const uint8_t* sfa_row = a.sfa + (int64_t)wk.row_tile * nkb * 512;
                for (int kb = 0; kb < nkb; kb++, it++) {
                    const int s = it & (MX_STAGES - 1);
                    const uint32_t ph = (uint32_t)(it / MX_STAGES) & 1;
                    if (!mx_bar_wait(mx_smem_u32(&empty[s]), ph ^ 1, abort_flag, a.status, 21)) { ok = false; break; }
                    const uint32_t fb = mx_smem_u32(&full[s]);
                    mx_bar_expect_tx(fb, stage_tx);
                    mx_tma_2d(mx_smem_u32(sA + s * MX_BM * MX_BK), &tmap_w, kb * MX_BK, row0, fb);
                    mx_tma_2d(mx_smem_u32(sB + s * b_stage), piece ? &tmap_xs : &tmap_x, kb * MX_BK, tok0, fb);
                    mx_bulk(mx_smem_u32(sSFA + s * 512), sfa_row + (int64_t)kb * 512, 512u, fb);
                    for (int c = 0; c < nsf; c++)
                        mx_bulk(mx_smem_u32(sSFB + s * 1024 + c * 512), a.sfb + ((int64_t)((tok0 >> 7) + c) * nkb + kb) * 512, 512u, fb);
                }
            }
            for (int j = max(0, it - MX_STAGES); j < it; j++) {   // nothing stays in flight behind this thread
                const int s = j & (MX_STAGES - 1);
                const uint32_t ph = (uint32_t)(j / MX_STAGES) & 1;
                const long long t0 = clock64();
                while (!mx_bar_try(mx_smem_u32(&full[s]), ph)) {
                    if (clock64() - t0 > MX_WAIT_BUDGET) { atomicCAS(a.status, 0, 22); break; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- scales to tensor memory, then the MMAs
        if (lane == 0) {
            // instruction descriptor (block-scaled form): A = E2M1 (5), E2M3 (3) or E3M2 (4) at bits 7..9, B = E4M3 (0) at 10..12, both K-major,
            // N / 8 at bits 17..22, scales E8M0 at bit 23, M / 16 at bits 24..28; the scale byte of an MMA's k-block
            // inside its 32-bit column goes to bits 4..5 (B) and 29..30 (A)
            const uint32_t idesc_base = ((uint32_t)a.a_format << 7) | (0u << 10) | (1u << 23) | ((uint32_t)(MX_BM >> 4) << 24);
            const uint64_t adesc0 = mx_desc_sw128(mx_smem_u32(sA)), bdesc0 = mx_desc_sw128(mx_smem_u32(sB));
            bool ok = true;
            int it = 0, n = 0;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, n++) {
                // the previous tile's accumulator must have been read out
                if (!mx_bar_wait(mx_smem_u32(afree), (uint32_t)(n & 1) ^ 1, abort_flag, a.status, 25)) break;
                mx_fence_after();
                const MxWork wk = mx_work(a, tile);
                const uint32_t idesc0 = idesc_base | ((uint32_t)(wk.nb >> 3) << 17);
                for (int kb = 0; kb < nkb; kb++, it++) {
                    const int s = it & (MX_STAGES - 1);
                    const uint32_t ph = (uint32_t)(it / MX_STAGES) & 1;
                    // the scale warp has seen the stage's bytes land and has moved its scales to tensor memory
                    if (!mx_bar_wait(mx_smem_u32(&sfrdy[s]), ph, abort_flag, a.status, 23)) { ok = false; break; }
                    mx_fence_after();
                    const uint32_t sfa_col = tmem_base + MX_SFA_COL + 4 * s, sfb_col = tmem_base + MX_SFB_COL + 8 * s;
                    const uint64_t ad = adesc0 + (uint64_t)((s * MX_BM * MX_BK) >> 4), bd = bdesc0 + (uint64_t)((s * b_stage) >> 4);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        // 32 k further: 32 bytes inside the swizzle row (+2 in the encoded address), next scale byte
                        const uint32_t idesc = idesc0 | ((uint32_t)j << 4) | ((uint32_t)j << 29);
                        mx_mma(tmem_base, ad + 2 * j, bd + 2 * j, idesc, (kb | j) != 0 ? 1u : 0u, sfa_col, sfb_col);   // a piece starts on a chunk of activation scales: same address
                    }
                    mx_commit(mx_smem_u32(&empty[s]));
                }
                if (ok) mx_commit(mx_smem_u32(accum));
            }
        }
    } else if (warp == 6) {
        // ---------------------------------------------------------------- scales to tensor memory, a stage ahead of the MMAs
        // (its own thread: the three copies per stage cost the MMA thread a fifth of its time when it issued them itself)
        if (lane == 0) {
            bool ok = true;
            int it = 0;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const MxWork wk = mx_work(a, tile);
                const int nsf = wk.nb != a.bn ? 1 : nsfb;
                for (int kb = 0; kb < nkb; kb++, it++) {
                    const int s = it & (MX_STAGES - 1);
                    const uint32_t ph = (uint32_t)(it / MX_STAGES) & 1;
                    if (!mx_bar_wait(mx_smem_u32(&full[s]), ph, abort_flag, a.status, 26)) { ok = false; break; }
                    mx_fence_after();
                    const uint32_t sfa_col = tmem_base + MX_SFA_COL + 4 * s, sfb_col = tmem_base + MX_SFB_COL + 8 * s;
                    mx_cp_sf(sfa_col, mx_desc_sf(mx_smem_u32(sSFA + s * 512)));
                    for (int c = 0; c < nsf; c++) mx_cp_sf(sfb_col + 4 * c, mx_desc_sf(mx_smem_u32(sSFB + s * 1024 + c * 512)));
                    mx_commit(mx_smem_u32(&sfrdy[s]));
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue: lane quarter warp % 4
        const int q = warp & 3;
        bool ok = true;
        int n = 0;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, n++) {
            const MxWork wk = mx_work(a, tile);
            const int row0 = wk.row0, tok0 = wk.tok0, nb = wk.nb;
            if (lane == 0) ok = mx_bar_wait(mx_smem_u32(accum), (uint32_t)(n & 1), abort_flag, a.status, 24);
            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
            if (!ok) break;
            mx_fence_after();
            const int row = row0 + q * 32 + lane;
            for (int c0 = 0; c0 < nb; c0 += 32) {
                uint32_t v[32];
                mx_tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
                if (c0 + 32 >= nb) {
                    // the last read of this warp: the accumulator may be overwritten once all four warps are here
                    mx_fence_before();
                    __syncwarp();
                    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(mx_smem_u32(afree)) : "memory");
                }
                if (row < a.n_rows) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int tok = tok0 + c0 + j;
                        if (tok < a.m && c0 + j < nb) a.y[(int64_t)tok * a.ldy + row] = __uint_as_float(v[j]);
                    }
                }
            }
        }
    }
    mx_fence_before();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------
// The same product on CTA PAIRS (tcgen05 cta_group::2): two CTAs of a cluster, one per SM, share a 256 x 256 output tile.
// Each CTA holds 128 of the tile's weight rows (its A operand and their scales) and HALF of the activation tile (128 of
// the 256 activation rows); one MMA issued by the pair's first CTA reads both halves, so every SM fetches and stages
// half the activation bytes per flop -- the shared-memory traffic that bounds the single-CTA form. All copies are
// tiled TMA loads in their pair form (their bytes count on the FIRST CTA's barrier); stages are handed back with one
// commit per CTA; the accumulator hand-over of the second CTA's epilogue warps arrives on the first CTA's barrier
// through its cluster address. Every wait is bounded; every thread of both CTAs reaches the cluster barrier at the end.
constexpr int PX_STAGES = 6;
constexpr int PX_SFA_COL = 256;   // 4 columns per stage
constexpr int PX_SFB_COL = 288;   // 8 columns per stage
constexpr int PX_STAGE_BYTES = MX_BM * MX_BK + 128 * MX_BK + 512 + 1024;

__device__ __forceinline__ uint32_t px_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t px_mapa(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void px_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// pair form of the tiled load: executed by both CTAs, the bytes count on the barrier of the pair's first CTA
__device__ __forceinline__ void px_tma_2d(uint32_t dst, const CUtensorMap* map, int cx, int cy, uint32_t bar_of_first) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar_of_first), "r"(cx), "r"(cy)
        : "memory");
}
__device__ __forceinline__ void px_commit(uint32_t bar_cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void px_cp_sf(uint32_t tmem_col, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_col), "l"(desc) : "memory");
}
__device__ __forceinline__ void px_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate, uint32_t sfa,
                                       uint32_t sfb) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
}
__device__ __forceinline__ void px_arrive_cluster(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

struct PxArgs {
    float* y;
    int64_t ldy;
    int n_rows, m, k;
    int a_format, a_tx;
    int m_tiles, pair_tiles;   // 256-row activation tiles, 256-row weight tiles
    int* status;
};

__global__ void __launch_bounds__(MX_THREADS, 1)
gemm_mxf4_pair_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                      const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb, PxArgs a) {
    extern __shared__ uint8_t mx_smem_raw[];
    uint8_t* smem = mx_smem_raw + ((1024u - (mx_smem_u32(mx_smem_raw) & 1023u)) & 1023u);
    uint8_t* sA = smem;                                 // [stages][128 rows][128 B]
    uint8_t* sB = sA + PX_STAGES * MX_BM * MX_BK;       // [stages][128 activation rows][128 B]
    uint8_t* sSFA = sB + PX_STAGES * 128 * MX_BK;       // [stages][512]
    uint8_t* sSFB = sSFA + PX_STAGES * 512;             // [stages][2][512]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sSFB + PX_STAGES * 1024);
    uint64_t* full = bars;                  // used in the pair's first CTA: the stage's bytes of BOTH CTAs have landed
    uint64_t* empty = bars + PX_STAGES;     // per CTA: the MMAs that read the stage are complete
    uint64_t* accum = empty + PX_STAGES;    // per CTA: the tile's MMAs are complete
    uint64_t* afree = accum + 1;            // first CTA: the eight epilogue warps of the pair have read their accumulators
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(afree + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = px_cta_rank();
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int nkb = a.k / MX_BK;
    const int total = a.m_tiles * a.pair_tiles;
    if (tid == 0) {
        for (int s = 0; s < PX_STAGES; s++) {
            mx_bar_init(mx_smem_u32(&full[s]), 1);
            mx_bar_init(mx_smem_u32(&empty[s]), 1);
        }
        mx_bar_init(mx_smem_u32(accum), 1);
        mx_bar_init(mx_smem_u32(afree), 8);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(mx_smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    mx_fence_before();
    __syncthreads();
    px_cluster_sync();     // both CTAs' barriers exist before anything arrives on them from the other CTA
    mx_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- copies (both CTAs: their own halves)
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int w = pair; w < total && ok; w += n_pairs) {
                const int pt = w / a.m_tiles, tt = w - pt * a.m_tiles;
                const int row_tile = 2 * pt + (int)rank, row0 = row_tile * MX_BM, tok0 = tt * 256;
                for (int kb = 0; kb < nkb; kb++, it++) {
                    const int s = it % PX_STAGES;
                    const uint32_t ph = (uint32_t)(it / PX_STAGES) & 1;
                    if (!mx_bar_wait(mx_smem_u32(&empty[s]), ph ^ 1, abort_flag, a.status, 31)) { ok = false; break; }
                    const uint32_t fb = mx_smem_u32(&full[s]) & 0xFEFFFFFFu;   // the first CTA's barrier
                    if (rank == 0) mx_bar_expect_tx(mx_smem_u32(&full[s]), 2u * (uint32_t)(a.a_tx + 128 * MX_BK + 512 + 1024));
                    px_tma_2d(mx_smem_u32(sA + s * MX_BM * MX_BK), &tmap_w, kb * MX_BK, row0, fb);
                    px_tma_2d(mx_smem_u32(sB + s * 128 * MX_BK), &tmap_x, kb * MX_BK, tok0 + (int)rank * 128, fb);
                    px_tma_2d(mx_smem_u32(sSFA + s * 512), &tmap_sfa, 0, row_tile * nkb + kb, fb);
                    px_tma_2d(mx_smem_u32(sSFB + s * 1024), &tmap_sfb, 0, (tok0 >> 7) * nkb + kb, fb);
                    px_tma_2d(mx_smem_u32(sSFB + s * 1024 + 512), &tmap_sfb, 0, ((tok0 >> 7) + 1) * nkb + kb, fb);
                }
            }
            if (!ok) {   // gave up: let copies that may still be in flight land before this CTA's shared memory goes away
                const long long t0 = clock64();
                while (clock64() - t0 < 400000) __nanosleep(1000);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- the pair's MMAs (first CTA only)
        if (lane == 0 && rank == 0) {
            const uint32_t idesc0 = ((uint32_t)a.a_format << 7) | (0u << 10) | ((uint32_t)(256 >> 3) << 17) | (1u << 23) | ((uint32_t)(256 >> 4) << 24);
            const uint64_t adesc0 = mx_desc_sw128(mx_smem_u32(sA)), bdesc0 = mx_desc_sw128(mx_smem_u32(sB));
            bool ok = true;
            int it = 0, n = 0;
            for (int w = pair; w < total && ok; w += n_pairs, n++) {
                if (!mx_bar_wait(mx_smem_u32(afree), (uint32_t)(n & 1) ^ 1, abort_flag, a.status, 35)) break;
                mx_fence_after();
                for (int kb = 0; kb < nkb; kb++, it++) {
                    const int s = it % PX_STAGES;
                    const uint32_t ph = (uint32_t)(it / PX_STAGES) & 1;
                    if (!mx_bar_wait(mx_smem_u32(&full[s]), ph, abort_flag, a.status, 33)) { ok = false; break; }
                    mx_fence_after();
                    const uint32_t sfa_col = tmem_base + PX_SFA_COL + 4 * s, sfb_col = tmem_base + PX_SFB_COL + 8 * s;
                    px_cp_sf(sfa_col, mx_desc_sf(mx_smem_u32(sSFA + s * 512)));
                    px_cp_sf(sfb_col, mx_desc_sf(mx_smem_u32(sSFB + s * 1024)));
                    px_cp_sf(sfb_col + 4, mx_desc_sf(mx_smem_u32(sSFB + s * 1024 + 512)));
                    const uint64_t ad = adesc0 + (uint64_t)((s * MX_BM * MX_BK) >> 4), bd = bdesc0 + (uint64_t)((s * 128 * MX_BK) >> 4);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const uint32_t idesc = idesc0 | ((uint32_t)j << 4) | ((uint32_t)j << 29);
                        px_mma(tmem_base, ad + 2 * j, bd + 2 * j, idesc, (kb | j) != 0 ? 1u : 0u, sfa_col, sfb_col);
                    }
                    // hand the stage back to the copy threads of both CTAs
                    const uint32_t eb = mx_smem_u32(&empty[s]);
                    px_commit(px_mapa(eb, 0));
                    px_commit(px_mapa(eb, 1));
                }
                if (ok) {
                    const uint32_t ab = mx_smem_u32(accum);
                    px_commit(px_mapa(ab, 0));
                    px_commit(px_mapa(ab, 1));
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (both CTAs): lane quarter warp % 4
        const int q = warp & 3;
        bool ok = true;
        int n = 0;
        const uint32_t afree_first = px_mapa(mx_smem_u32(afree), 0);
        for (int w = pair; w < total && ok; w += n_pairs, n++) {
            const int pt = w / a.m_tiles, tt = w - pt * a.m_tiles;
            const int row0 = (2 * pt + (int)rank) * MX_BM, tok0 = tt * 256;
            if (lane == 0) ok = mx_bar_wait(mx_smem_u32(accum), (uint32_t)(n & 1), abort_flag, a.status, 34);
            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
            if (!ok) break;
            mx_fence_after();
            const int row = row0 + q * 32 + lane;
            for (int c0 = 0; c0 < 256; c0 += 32) {
                uint32_t v[32];
                mx_tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
                if (c0 == 224) {
                    mx_fence_before();
                    __syncwarp();
                    if (lane == 0) px_arrive_cluster(afree_first);
                }
                if (row < a.n_rows) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int tok = tok0 + c0 + j;
                        if (tok < a.m) a.y[(int64_t)tok * a.ldy + row] = __uint_as_float(v[j]);
                    }
                }
            }
        }
    }
    mx_fence_before();
    __syncthreads();
    px_cluster_sync();     // the first CTA's MMAs read this CTA's shared memory: neither leaves before both are done
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

typedef CUresult (*MxEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                               const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

MxEncodeFn mx_encode_fn() {
    static std::atomic<MxEncodeFn> fn{nullptr};
    if (!fn.load()) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
            fn.store(reinterpret_cast<MxEncodeFn>(p));
    }
    return fn.load();
}

}  // namespace

bool gemm_mx_native_supported(const b200q_weight* w, int m) {
    return (w->fmt == fmt_of(MXFP4, GGUF) || w->fmt == fmt_of(MXFP6_E2M3, GGUF) || w->fmt == fmt_of(MXFP6_E3M2, GGUF)) && w->orient == B200Q_ORIENT_NK && m > 8 && (w->k % 128) == 0 && w->k < (1 << 30) &&
           w->n_local < 0x7FFFFF00ll;
}

// x: fp32 or bf16 [m, ldx] on the device; y: fp32 [m, ldy]. Uses the context's third scratch buffer for the activation
// codes and their scales; the weights' scale plane in chunk order is built on first use and kept with the tensor.
int launch_gemm_mx_native(b200q_ctx* ctx, const b200q_weight* w, const void* d_x, int x_is_bf16, int64_t ldx, float* d_y, int64_t ldy, int m) {
    if (!gemm_mx_native_supported(w, m)) return fail(B200Q_ERR_UNSUPPORTED, "matmul (native MX): needs a GGUF MXFP4 or MXFP6 NK tensor with k %% 128 == 0 and m > 8");
    MxEncodeFn enc = mx_encode_fn();
    if (!enc) return fail(B200Q_ERR_INIT, "matmul (native MX): cuTensorMapEncodeTiled is not available from this driver");
    const int k = (int)w->k, nkb = k / MX_BK;
    const bool fp4 = w->fmt == fmt_of(MXFP4, GGUF);
    const int bn = m >= 256 ? 256 : ((m + 15) / 16) * 16;
    const int m_tiles = (m + bn - 1) / bn;
    const int m_pad = ((m_tiles * bn + 127) / 128) * 128;   // whole chunks of 128 rows of scales; rows the copies may touch exist
    const int64_t row_tiles = (w->n_local + MX_BM - 1) / MX_BM;
    b200q_weight* wm = const_cast<b200q_weight*>(w);
    const int64_t sfa_row_tiles = (row_tiles + 1) & ~(int64_t)1;   // the pair kernel's second CTA may stand on a row tile past the end
    if (!wm->mx_sfa) {
        const int64_t total = sfa_row_tiles * nkb * 512;
        void* p = nullptr;
        B200Q_CUDA(cudaMalloc(&p, (size_t)total), B200Q_ERR_ALLOC);
        mx_build_sfa_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(w->view.p[0], static_cast<uint8_t*>(p), (int)w->n_local, nkb, total);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) {
            cudaFree(p);
            return cuda_fail(B200Q_ERR_LAUNCH, e, "matmul (native MX): weight scale plane");
        }
        wm->mx_sfa = p;
    }
    const size_t q_bytes = ((size_t)m_pad * k + 255) & ~(size_t)255;
    const size_t sfb_bytes = (size_t)(m_pad / 128) * nkb * 512;
    int rc = ensure_scratch(ctx, q_bytes + sfb_bytes, 2);
    if (rc != B200Q_OK) return rc;
    uint8_t* d_q = static_cast<uint8_t*>(ctx->scratch3);
    uint8_t* d_sfb = d_q + q_bytes;
    {
        const int64_t threads = (int64_t)m_pad * (k / 32);
        const unsigned grid = (unsigned)((threads + 255) / 256);
        if (fp4) {
            if (x_is_bf16) mx_quantize_x_kernel<__nv_bfloat16, true><<<grid, 256, 0, ctx->stream>>>(static_cast<const __nv_bfloat16*>(d_x), ldx, d_q, d_sfb, m, k, m_pad);
            else mx_quantize_x_kernel<float, true><<<grid, 256, 0, ctx->stream>>>(static_cast<const float*>(d_x), ldx, d_q, d_sfb, m, k, m_pad);
        } else {
            if (x_is_bf16) mx_quantize_x_kernel<__nv_bfloat16, false><<<grid, 256, 0, ctx->stream>>>(static_cast<const __nv_bfloat16*>(d_x), ldx, d_q, d_sfb, m, k, m_pad);
            else mx_quantize_x_kernel<float, false><<<grid, 256, 0, ctx->stream>>>(static_cast<const float*>(d_x), ldx, d_q, d_sfb, m, k, m_pad);
        }
        B200Q_CUDA(cudaGetLastError(), B200Q_ERR_LAUNCH);
    }
    CUtensorMap wmap, xmap, xsmap;
    cuuint32_t estr[2] = {1, 1};
    {
        // code plane as [n, k] 4-bit (6-bit) elements: 16 per 8 (12) bytes, unpacked to 16-byte containers in shared memory
        cuuint64_t gdim[2] = {(cuuint64_t)k, (cuuint64_t)w->n_local};
        cuuint64_t gstr[1] = {fp4 ? (cuuint64_t)k / 2 : (cuuint64_t)k / 4 * 3};
        cuuint32_t box[2] = {128u, (cuuint32_t)MX_BM};
        CUresult r = enc(&wmap, fp4 ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_16U6_ALIGN16B, 2, const_cast<uint8_t*>(w->view.p[1]), gdim, gstr, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(B200Q_ERR_INVALID, "matmul (native MX): cuTensorMapEncodeTiled (codes) failed with code %d", (int)r);
        cuuint64_t xdim[2] = {(cuuint64_t)k, (cuuint64_t)m_pad};
        cuuint64_t xstr[1] = {(cuuint64_t)k};
        cuuint32_t xbox[2] = {128u, (cuuint32_t)bn};
        r = enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, d_q, xdim, xstr, xbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(B200Q_ERR_INVALID, "matmul (native MX): cuTensorMapEncodeTiled (activations) failed with code %d", (int)r);
    }
    const int64_t total_tiles = row_tiles * m_tiles;
    if (total_tiles > 0x3FFFFFF0ll) return fail(B200Q_ERR_UNSUPPORTED, "matmul (native MX): too many tiles for one launch");
    {
        // CTA pairs (cta_group::2) for whole 256-row activation tiles: B200Q_MX_PAIR=1 (a tuning knob like
        // B200Q_DECODE_RING). Off by default: it measured the same as the single-CTA kernel on the shapes tried
        // ([28672 x 8192], M = 512 and 2048), so halving the activation bytes per SM is not what bounds this path.
        const char* pe = getenv("B200Q_MX_PAIR");
        const bool want_pair = pe && pe[0] == '1';
        if (want_pair && bn == 256 && (m % 256) == 0 && row_tiles >= 2) {
            const int64_t pair_tiles = (row_tiles + 1) / 2;
            CUtensorMap xh, sfam, sfbm;
            cuuint64_t xdim[2] = {(cuuint64_t)k, (cuuint64_t)m_pad};
            cuuint64_t xstr[1] = {(cuuint64_t)k};
            cuuint32_t xbox[2] = {128u, 128u};
            CUresult r = enc(&xh, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, d_q, xdim, xstr, xbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return fail(B200Q_ERR_INVALID, "matmul (native MX): cuTensorMapEncodeTiled (activation halves) failed with code %d", (int)r);
            // scale planes as [chunks, 128 words]: one 512-byte chunk per copy; the weights' plane holds an even number of row tiles
            cuuint64_t sdim[2] = {128u, (cuuint64_t)(sfa_row_tiles * nkb)};
            cuuint64_t sstr[1] = {512u};
            cuuint32_t sbox[2] = {128u, 1u};
            r = enc(&sfam, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, wm->mx_sfa, sdim, sstr, sbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return fail(B200Q_ERR_INVALID, "matmul (native MX): cuTensorMapEncodeTiled (weight scales) failed with code %d", (int)r);
            cuuint64_t bdim[2] = {128u, (cuuint64_t)((m_pad / 128) * nkb)};
            r = enc(&sfbm, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, d_sfb, bdim, sstr, sbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return fail(B200Q_ERR_INVALID, "matmul (native MX): cuTensorMapEncodeTiled (activation scales) failed with code %d", (int)r);
            PxArgs pa{};
            pa.y = d_y; pa.ldy = ldy;
            pa.n_rows = (int)w->n_local; pa.m = m; pa.k = k;
            pa.a_format = fp4 ? 5 : w->fmt == fmt_of(MXFP6_E2M3, GGUF) ? 3 : 4;
            pa.a_tx = MX_BM * (fp4 ? 64 : 96);
            pa.m_tiles = m / 256; pa.pair_tiles = (int)pair_tiles;
            pa.status = ctx->d_status;
            const size_t psmem = 1024 + (size_t)PX_STAGES * PX_STAGE_BYTES + (2 * PX_STAGES + 2) * 8 + 16;
            static std::atomic<bool> pconfigured[64] = {};
            if (!pconfigured[ctx->device & 63]) {
                B200Q_CUDA(cudaFuncSetAttribute(gemm_mxf4_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024), B200Q_ERR_LAUNCH);
                pconfigured[ctx->device & 63] = true;
            }
            const int64_t items = pair_tiles * pa.m_tiles;
            const int pairs = (int)std::min<int64_t>(items, ctx->info.sm_count / 2);
            cudaLaunchConfig_t cfg{};
            cfg.gridDim = dim3((unsigned)(2 * pairs));
            cfg.blockDim = dim3(MX_THREADS);
            cfg.dynamicSmemBytes = psmem;
            cfg.stream = ctx->stream;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            B200Q_CUDA(cudaLaunchKernelEx(&cfg, gemm_mxf4_pair_kernel, wmap, xh, sfam, sfbm, pa), B200Q_ERR_LAUNCH);
            return B200Q_OK;
        }
    }
    MxArgs a{};
    a.sfa = static_cast<const uint8_t*>(wm->mx_sfa);
    a.sfb = d_sfb;
    a.y = d_y; a.ldy = ldy;
    a.n_rows = (int)w->n_local; a.m = m; a.k = k; a.bn = bn;
    a.a_format = fp4 ? 5 : w->fmt == fmt_of(MXFP6_E2M3, GGUF) ? 3 : 4;
    a.a_tx = MX_BM * (fp4 ? 64 : 96);
    a.m_tiles = m_tiles; a.row_tiles = (int)row_tiles;
    a.full_tiles = (int)total_tiles; a.split = 1; a.sub_bn = bn; a.n_work = (int)total_tiles;
    {
        const int ctas = ctx->info.sm_count;
        const int rem = (int)(total_tiles % ctas);
        // Two pieces of 128 rows only: a piece must start on a whole 128-row chunk of activation scales, because the
        // scale address the MMA takes in tensor memory has to stay on the chunk's first column (an address 1..3
        // columns into a chunk raised a misaligned-address fault).
        if (total_tiles > ctas && bn == 256 && rem > 0 && rem * 2 <= ctas) {
            a.full_tiles = (int)(total_tiles - rem);
            a.split = 2;
            a.sub_bn = 128;
            a.n_work = a.full_tiles + rem * 2;
        }
    }
    xsmap = xmap;
    if (a.split > 1) {
        cuuint64_t xdim[2] = {(cuuint64_t)k, (cuuint64_t)m_pad};
        cuuint64_t xstr[1] = {(cuuint64_t)k};
        cuuint32_t xbox[2] = {128u, (cuuint32_t)a.sub_bn};
        CUresult r = enc(&xsmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, d_q, xdim, xstr, xbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(B200Q_ERR_INVALID, "matmul (native MX): cuTensorMapEncodeTiled (activation pieces) failed with code %d", (int)r);
    }
    a.status = ctx->d_status;
    const size_t smem = 1024 + (size_t)MX_STAGES * (MX_BM * MX_BK + (size_t)bn * MX_BK + 512 + 1024) + (3 * MX_STAGES + 2) * 8 + 16;
    static std::atomic<bool> configured[64] = {};
    if (!configured[ctx->device & 63]) {
        B200Q_CUDA(cudaFuncSetAttribute(gemm_mxf4_native_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024), B200Q_ERR_LAUNCH);
        configured[ctx->device & 63] = true;
    }
    dim3 grid((unsigned)std::min<int64_t>(a.n_work, ctx->info.sm_count));
    gemm_mxf4_native_kernel<<<grid, MX1_THREADS, smem, ctx->stream>>>(wmap, xmap, xsmap, a);
    B200Q_CUDA(cudaGetLastError(), B200Q_ERR_LAUNCH);
    return B200Q_OK;
}

}  // namespace b200q
