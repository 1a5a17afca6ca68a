// Prefill kernel: fused dequant + GEMM on the 5th-generation tensor cores (tcgen05, accumulators in TMEM).
//
// Replaces what the reference does for m > 1 today: dequantise the whole tensor to fp32 and call an fp32
// library GEMM with host-side transposes (src/kernels/matmul/quantized/q8_0.rs:69-106,
// src/tensor/matmul.rs:153-214). Here packed weights are expanded tile by tile, to bf16, straight into shared
// memory and never touch HBM as fp32.
// (Shared-memory operands are f16, not bf16: see the note on operand formats below.)
//
//   y[m, n] = x[m, k] * W[n, k]^T   computed as   D[128 weight rows, BN activation rows] += A * B^T
//
//   A (UMMA M side) : 128 weight rows x 64 k, f16, K-major, 128-byte swizzle, written by 4 dequant warps
//                     (decode8 gives the exact fp32 values; one round-to-nearest to f16, whose 11-bit
//                     mantissa keeps the result well inside the 2e-3 tolerance; bf16 weights do not)
//   B (UMMA N side) : BN <= 256 activation rows x 64 k, f16, loaded by TMA (cp.async.bulk.tensor, no
//                     multicast) with the same swizzle. Activations (fp32 or bf16 from the caller) are first
//                     copied to f16 with one power-of-two scale per row, so neither large nor small rows
//                     leave the f16 range; the scale is multiplied back in the epilogue
//   D               : fp32 in tensor memory, 128 lanes x BN columns; read back with tcgen05.ld by the four
//                     dequant warps (one lane quarter each) and stored to y, coalesced along n
//
// Warp roles (192 threads): warp 0 = TMA producer + TMEM allocator, warp 1 = MMA issuer (one elected
// thread), warps 2..5 = dequant producers, then epilogue. A 4-stage ring of {A, B} tiles is handed over
// with mbarriers: full_a (4 warp arrivals), full_b (TMA transaction bytes), empty (tcgen05.commit).
// Every wait is bounded by a clock budget; on expiry the kernel raises a status word, all roles leave
// their loops, outstanding copies are waited for (again bounded), TMEM is freed and the kernel returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace b200q {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int STAGES = 4;
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
// Waits for the phase with the given parity. Gives up after WAIT_BUDGET cycles or when another role already
// gave up; then raises the CTA's abort flag and the launch's status word and returns false.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = clock64();
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag != 0) return false;
        if (clock64() - t0 > WAIT_BUDGET) {
            *abort_flag = 1;
            atomicCAS(status, 0, code);
            return false;
        }
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int cx, int cy, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(cx), "r"(cy)
        : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

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

struct GemmArgs {
    WView v;
    const float* xscale;   // per activation row: the power of two its f16 copy was divided by
    float* y;
    int64_t ldy;
    int n_rows, k, m, bn, tmem_cols;
    int* status;
};

template <int F>
__global__ void __launch_bounds__(192, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, GemmArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
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
            mbar_init(smem_u32(&full_a[s]), 4);
            mbar_init(smem_u32(&full_b[s]), 1);
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

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer (activations)
        if (lane == 0) {
            int issued = 0;
            for (int kb = 0; kb < nkb; kb++) {
                const int s = kb % STAGES;
                const uint32_t ph = (kb / STAGES) & 1;
                if (!mbar_wait(smem_u32(&empty[s]), ph ^ 1, abort_flag, a.status, 1)) break;
                mbar_arrive_expect_tx(smem_u32(&full_b[s]), (uint32_t)b_stage_bytes);
                tma_load_2d(smem_u32(sB + s * b_stage_bytes), &tmap_x, kb * BK, tok0, smem_u32(&full_b[s]));
                issued = kb + 1;
            }
            // do not leave copies in flight behind: the last STAGES tiles issued must have landed
            for (int kb = max(0, issued - STAGES); kb < issued; kb++) {
                const int s = kb % STAGES;
                const uint32_t ph = (kb / STAGES) & 1;
                long long t0 = clock64();
                while (!mbar_try_wait(smem_u32(&full_b[s]), ph)) {
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
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; kb++) {
                const int s = kb % STAGES;
                const uint32_t ph = (kb / STAGES) & 1;
                ok = mbar_wait(smem_u32(&full_a[s]), ph, abort_flag, a.status, 2) &&
                     mbar_wait(smem_u32(&full_b[s]), ph, abort_flag, a.status, 3);
                if (!ok) break;
                tc_fence_after();
                const uint64_t adesc = umma_desc_sw128(smem_u32(sA + s * A_STAGE_BYTES));
                const uint64_t bdesc = umma_desc_sw128(smem_u32(sB + s * b_stage_bytes));
#pragma unroll
                for (int kk = 0; kk < BK / 16; kk++) {
                    // 16 bf16 = 32 bytes further along k inside the swizzle atom: +2 in the encoded address
                    umma_bf16(tmem_base, adesc + (uint64_t)(2 * kk), bdesc + (uint64_t)(2 * kk), idesc, (kb | kk) != 0);
                }
                umma_commit(smem_u32(&empty[s]));
            }
            umma_commit(smem_u32(accum));   // arrives once every MMA issued so far has completed
        }
    } else {
        // ---------------------------------------------------------------- dequant producers, then epilogue
        const int dt = tid - 64;   // 0..127
        bool ok = true;
        for (int kb = 0; kb < nkb && ok; kb++) {
            const int s = kb % STAGES;
            const uint32_t ph = (kb / STAGES) & 1;
            ok = mbar_wait(smem_u32(&empty[s]), ph ^ 1, abort_flag, a.status, 4);
            if (!ok) break;
            uint8_t* tile = sA + s * A_STAGE_BYTES;
#pragma unroll 2
            for (int it = 0; it < (BM * BK / 8) / 128; it++) {
                const int idx = it * 128 + dt;
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
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> tensor-core reads
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&full_a[s]));
        }
        if (ok) ok = mbar_wait(smem_u32(accum), 0, abort_flag, a.status, 6);
        if (ok) {
            tc_fence_after();
            const int q = warp & 3;                       // the lane quarter this warp may read
            const int row = row0 + q * 32 + lane;
            for (int c0 = 0; c0 < a.bn; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
                if (row < a.n_rows) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int tok = tok0 + c0 + j;
                        if (tok < a.m) a.y[(int64_t)tok * a.ldy + row] = __uint_as_float(v[j]) * __ldg(a.xscale + tok);
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

// Activation rows -> f16 with a power-of-two scale per row (max |x| of the row lands in [1, 2)).
template <typename T>
__global__ void __launch_bounds__(256) x_to_f16_kernel(const T* __restrict__ x, int64_t ldx, __half* __restrict__ out,
                                                       float* __restrict__ scale, int k) {
    const int row = blockIdx.x;
    const T* xr = x + (int64_t)row * ldx;
    float mx = 0.0f;
    for (int i = threadIdx.x; i < k; i += blockDim.x) mx = fmaxf(mx, fabsf((float)xr[i]));
    __shared__ float red[8];
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = red[0];
    for (int i = 1; i < 8; i++) mx = fmaxf(mx, red[i]);
    int e = (int)((__float_as_uint(mx) >> 23) & 255u);
    e = (mx == 0.0f || !(mx <= 3.0e38f)) ? 127 : min(max(e, 1), 253);
    const float sdown = __uint_as_float((uint32_t)(254 - e) << 23);
    for (int i = threadIdx.x; i < k; i += blockDim.x) out[(int64_t)row * k + i] = __float2half_rn((float)xr[i] * sdown);
    if (threadIdx.x == 0) scale[row] = __uint_as_float((uint32_t)e << 23);
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

template <int F>
int launch_fmt(b200q_ctx* ctx, const CUtensorMap& map, const GemmArgs& a, dim3 grid, size_t smem) {
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        B200Q_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<F>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024), B200Q_ERR_LAUNCH);
        configured[ctx->device & 63] = true;
    }
    gemm_tc_kernel<F><<<grid, 192, smem, ctx->stream>>>(map, a);
    B200Q_CUDA(cudaGetLastError(), B200Q_ERR_LAUNCH);
    return B200Q_OK;
}

}  // namespace

bool gemm_tc_supported(const b200q_weight* w, int m) {
    return w->orient == B200Q_ORIENT_NK && m >= 1 && (w->k % BK) == 0 && w->n_local < 0x7FFFFF00ll && w->k < (1 << 30);
}

// x: fp32 or bf16 [m, ldx] on the device. y: fp32 [m, ldy]. Uses the context's third scratch buffer for the
// f16 copy of the activations and their row scales.
int launch_gemm_tc(b200q_ctx* ctx, const b200q_weight* w, const void* d_x, int x_is_bf16, int64_t ldx, float* d_y, int64_t ldy, int m) {
    if (!gemm_tc_supported(w, m)) return fail(B200Q_ERR_UNSUPPORTED, "gemm: needs an NK tensor with k %% 64 == 0");
    const size_t x16_bytes = ((size_t)m * w->k * 2 + 255) & ~(size_t)255;
    int rc = ensure_scratch(ctx, x16_bytes + (size_t)m * sizeof(float), 2);
    if (rc != B200Q_OK) return rc;
    __half* d_x16 = static_cast<__half*>(ctx->scratch3);
    float* d_scale = reinterpret_cast<float*>(static_cast<uint8_t*>(ctx->scratch3) + x16_bytes);
    if (x_is_bf16) x_to_f16_kernel<__nv_bfloat16><<<m, 256, 0, ctx->stream>>>(static_cast<const __nv_bfloat16*>(d_x), ldx, d_x16, d_scale, (int)w->k);
    else x_to_f16_kernel<float><<<m, 256, 0, ctx->stream>>>(static_cast<const float*>(d_x), ldx, d_x16, d_scale, (int)w->k);
    B200Q_CUDA(cudaGetLastError(), B200Q_ERR_LAUNCH);
    const void* d_x_bf16 = d_x16;
    ldx = w->k;
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return fail(B200Q_ERR_INIT, "gemm: cuTensorMapEncodeTiled is not available from this driver");
    int bn = m >= 256 ? 256 : ((m + 15) / 16) * 16;
    int tmem_cols = 32;
    while (tmem_cols < bn) tmem_cols <<= 1;
    CUtensorMap map;
    cuuint64_t gdim[2] = {(cuuint64_t)w->k, (cuuint64_t)m};
    cuuint64_t gstr[1] = {(cuuint64_t)ldx * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)bn};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(d_x_bf16), gdim, gstr, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B200Q_ERR_INVALID, "gemm: cuTensorMapEncodeTiled failed with code %d", (int)r);
    GemmArgs a{};
    a.v = w->view; a.xscale = d_scale; a.y = d_y; a.ldy = ldy;
    a.n_rows = (int)w->n_local; a.k = (int)w->k; a.m = m; a.bn = bn; a.tmem_cols = tmem_cols;
    a.status = ctx->d_status;
    dim3 grid((unsigned)((w->n_local + BM - 1) / BM), (unsigned)((m + bn - 1) / bn));
    size_t smem = 1024 + (size_t)STAGES * (A_STAGE_BYTES + (size_t)bn * BK * 2) + (3 * STAGES + 1) * 8 + 16;
    switch (w->fmt) {
#define X(F) \
    case F: return launch_fmt<F>(ctx, map, a, grid, smem);
        B200Q_FOR_EACH_FMT(X)
#undef X
    }
    return fail(B200Q_ERR_INVALID, "gemm: unknown format %d", w->fmt);
}

// Reads and clears the status word the tensor-core kernel raises when a bounded wait expires.
int gemm_tc_check_status(b200q_ctx* ctx) {
    int h[1] = {0};
    B200Q_CUDA(cudaMemcpyAsync(h, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream), B200Q_ERR_COPY);
    B200Q_CUDA(cudaStreamSynchronize(ctx->stream), B200Q_ERR_DEVICE);
    if (h[0] != 0) {
        cudaMemsetAsync(ctx->d_status, 0, sizeof(int), ctx->stream);
        return fail(B200Q_ERR_TIMEOUT, "gemm: a bounded device-side wait expired (site %d); results of that launch are invalid", h[0]);
    }
    return B200Q_OK;
}

}  // namespace b200q
