// b200q_matmul*: argument checks and the choice of kernel for one fused dequant + matmul.
#include <chrono>
#include <cuda_bf16.h>
#include <vector>

#include "common.cuh"
#include <cstring>

#include "gemv_i8.cuh"

using namespace b200q;

struct b200q_batch {
    b200q_ctx* ctx = nullptr;
    int m = 0;
    std::vector<const b200q_weight*> w;
    std::vector<const float*> x;
    std::vector<float*> y;
    size_t weight_bytes = 0;
    // grouped launch of the decode kernel (every product has a decode image): device copies of the plan
    bool grouped = false;
    DOp* d_dops = nullptr;
    int2* d_ranges = nullptr;
    int n_ctas = 0, total_rt = 0, n_units = 0;
    DOp dsingle{};
    DecodeLaunch dl{};
    // host-output variant of the plan (b200q_batch_run_host with pinned, device-mapped outputs): the same
    // products with y pointing into the caller's host buffer
    std::vector<DOp> h_dops;
    DOp* d_dops_hosty = nullptr;
    const float* hosty_base = nullptr;
    DOp dsingle_hosty{};
};

static DOp make_dop(const b200q_weight* w, const float* x, int64_t ldx, float* y, int64_t ldy) {
    DOp op{};
    op.img = w->dimg.base;
    op.x = x; op.y = y; op.ldx = ldx; op.ldy = ldy;
    op.n_rows = (int)w->n_local; op.k = (int)w->k;
    op.kind = w->dimg.kind; op.item_bytes = w->dimg.item_bytes; op.nh = w->dimg.nh;
    op.rt0 = 0; op.nrt = w->dimg.nrt;
    op.n_extra = w->ctx->scatter_extra;
    for (int p = 0; p < op.n_extra; p++) op.y_extra[p] = w->ctx->scatter_y[p];
    return op;
}


static int check_matmul_args(b200q_ctx* ctx, const b200q_weight* w, const void* d_x, const void* d_y, int m) {
    if (!w) return fail(B200Q_ERR_INVALID, "matmul: weight handle is null");
    if (w->ctx->device != ctx->device) return fail(B200Q_ERR_INVALID, "matmul: weight lives on device %d, ctx on %d", w->ctx->device, ctx->device);
    if (m < 0) return fail(B200Q_ERR_INVALID, "matmul: m=%d is negative", m);
    if (m > 0 && (!d_x || !d_y)) return fail(B200Q_ERR_INVALID, "matmul: null activation or output pointer");
    return B200Q_OK;
}

// fp32 in, fp32 out; picks the kernel.
static int matmul_f32(b200q_ctx* ctx, const b200q_weight* w, const float* x, int64_t ldx, float* y, int64_t ldy, int m,
                      unsigned flags) {
    const bool scatter = ctx->scatter_extra > 0;
    if ((flags & B200Q_MM_SEQUENTIAL) || !gemv_fast_supported(w))
        return scatter ? fail(B200Q_ERR_UNSUPPORTED, "matmul_scatter: the sequential kernel writes one output only") : launch_matmul_seq(ctx, w, x, ldx, y, ldy, m);
    bool aligned = (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (ldx % 4) == 0;
    if (!aligned) return scatter ? fail(B200Q_ERR_UNSUPPORTED, "matmul_scatter: activations must be 16-byte aligned") : launch_matmul_seq(ctx, w, x, ldx, y, ldy, m);
    // integer decode kernel on the tensor's decode image: largest activation-row chunk whose image fits
    {
        int chunk = 8;
        while (chunk > 1 && !gemv_i8_supported(w, chunk)) chunk >>= 1;
        if (gemv_i8_supported(w, chunk)) {
            for (int i = 0; i < m; i += chunk) {
                const int mm = m - i < chunk ? m - i : chunk;
                DOp op = make_dop(w, x + (int64_t)i * ldx, ldx, y + (int64_t)i * ldy, ldy);
                for (int p = 0; p < op.n_extra; p++) op.y_extra[p] += (int64_t)i * ldy;
                DecodeLaunch L;
                gemv_i8_plan(op.item_bytes, op.k, 1 << op.kind, mm, &L);
                const int n_ctas = ctx->info.sm_count * L.ctas_per_sm;
                // the launch that stores the last rows raises the peers' flags itself
                PeerSignal sig{};
                const bool last = i + chunk >= m;
                if (last && ctx->scatter_sig_n > 0) {
                    sig.n = ctx->scatter_sig_n; sig.my = ctx->scatter_sig_my; sig.epoch = ctx->scatter_sig_epoch;
                    for (int p = 0; p < sig.n; p++) sig.flag[p] = ctx->scatter_flag[p];
                    ctx->scatter_signalled = true;
                }
                int rc = launch_gemv_i8(ctx, &op, nullptr, 1, nullptr, n_ctas, n_ctas, op.nrt, mm, L, &sig);
                if (rc != B200Q_OK) return rc;
            }
            return B200Q_OK;
        }
    }
    // no decode image (a format, orientation or k the decode kernel does not take): the CUDA-core kernel
    if (scatter) return fail(B200Q_ERR_UNSUPPORTED, "matmul_scatter: m <= 8 needs a tensor with a decode image (Q4_0, Q8_0, Q4_K, Q5_K, Q6_K, MXFP4, MXFP6 E2M3 in GGUF layout, NK, k %% 128 == 0)");
    for (int i = 0; i < m; i += 8) {
        const int mm = m - i < 8 ? m - i : 8;
        int rc = launch_gemv(ctx, w, x + (int64_t)i * ldx, ldx, y + (int64_t)i * ldy, ldy, mm);
        if (rc != B200Q_OK) return rc;
    }
    return B200Q_OK;
}

namespace {

struct PeerFlags {
    int* p[8];
};

// one lane per rank: the slice this GPU stored into rank p's output is complete (the kernel that stored it has ended)
__global__ void peer_signal_kernel(PeerFlags f, int n_ranks, int my_rank, int epoch) {
    const int p = threadIdx.x;
    if (p >= n_ranks || p == my_rank) return;
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(f.p[p] + my_rank), "r"(epoch) : "memory");
}

// One lane per rank: bounded wait until rank p has signalled this round. Launched programmatically behind the product
// whose stores it orders: it lets the kernel behind it become resident at once, polls while the product still runs,
// and completes only after the product has (griddepcontrol.wait), so that completion of this kernel still implies
// completion of everything ahead of it on the stream.
__global__ void peer_wait_kernel(const int* flags, int n_ranks, int my_rank, int epoch, long long budget, int* status) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int p = threadIdx.x;
    if (p < n_ranks && p != my_rank) {
        const long long t0 = clock64();
        for (;;) {
            int v;
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flags + p) : "memory");
            if (v - epoch >= 0) break;   // epochs only grow: a fast peer may already have signalled a later one
            if (clock64() - t0 > budget) {
                atomicExch(status, 300 + p);
                break;
            }
            __nanosleep(100);
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

}  // namespace

extern "C" {

int b200q_peer_signal(b200q_ctx* ctx, void* const* d_flags_of_ranks, int n_ranks, int my_rank, int epoch) {
    if (!ctx) return fail(B200Q_ERR_INVALID, "peer_signal: ctx is null");
    if (!d_flags_of_ranks || n_ranks < 1 || n_ranks > 8 || my_rank < 0 || my_rank >= n_ranks)
        return fail(B200Q_ERR_INVALID, "peer_signal: rank %d of %d (1..8 ranks)", my_rank, n_ranks);
    PeerFlags f{};
    for (int p = 0; p < n_ranks; p++) {
        if (!d_flags_of_ranks[p]) return fail(B200Q_ERR_INVALID, "peer_signal: flag array of rank %d is null", p);
        f.p[p] = static_cast<int*>(d_flags_of_ranks[p]);
    }
    B200Q_CUDA(cudaSetDevice(ctx->device), B200Q_ERR_DEVICE);
    if (n_ranks == 1) return B200Q_OK;
    peer_signal_kernel<<<1, 32, 0, ctx->stream>>>(f, n_ranks, my_rank, epoch);
    B200Q_CUDA(cudaGetLastError(), B200Q_ERR_LAUNCH);
    return B200Q_OK;
}

int b200q_peer_wait(b200q_ctx* ctx, const void* d_flags_own, int n_ranks, int my_rank, int epoch) {
    if (!ctx) return fail(B200Q_ERR_INVALID, "peer_wait: ctx is null");
    if (!d_flags_own || n_ranks < 1 || n_ranks > 8 || my_rank < 0 || my_rank >= n_ranks)
        return fail(B200Q_ERR_INVALID, "peer_wait: rank %d of %d (1..8 ranks)", my_rank, n_ranks);
    B200Q_CUDA(cudaSetDevice(ctx->device), B200Q_ERR_DEVICE);
    if (n_ranks == 1) return B200Q_OK;
    // programmatic launch: the one-warp kernel may become resident while the product ahead of it still runs (it reads
    // nothing that kernel writes); what follows it on the stream still waits for its completion
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    B200Q_CUDA(cudaLaunchKernelEx(&cfg, peer_wait_kernel, static_cast<const int*>(d_flags_own), n_ranks, my_rank, epoch, 2000000000ll, ctx->d_status),
               B200Q_ERR_LAUNCH);
    B200Q_CUDA(cudaGetLastError(), B200Q_ERR_LAUNCH);
    ctx->tc_pending = true;   // the next synchronise reads the status word
    return B200Q_OK;
}

int b200q_matmul_ex(b200q_ctx* ctx, const b200q_weight* w, const void* d_x, int x_dtype, int64_t ldx, void* d_y,
                    int y_dtype, int64_t ldy, int m, unsigned flags) {
    if (!ctx) return fail(B200Q_ERR_INVALID, "matmul: ctx is null");
    B200Q_CUDA(cudaSetDevice(ctx->device), B200Q_ERR_DEVICE);
    int rc = check_matmul_args(ctx, w, d_x, d_y, m);
    if (rc != B200Q_OK) return rc;
    if (x_dtype != B200Q_F32 && x_dtype != B200Q_BF16) return fail(B200Q_ERR_INVALID, "matmul: unknown activation dtype %d", x_dtype);
    if (y_dtype != B200Q_F32 && y_dtype != B200Q_BF16) return fail(B200Q_ERR_INVALID, "matmul: unknown output dtype %d", y_dtype);
    if (ldx == 0) ldx = w->k;
    if (ldy == 0) ldy = w->n_local;
    if (ldx < w->k || ldy < w->n_local) return fail(B200Q_ERR_INVALID, "matmul: ldx=%lld < k=%lld or ldy=%lld < n=%lld", (long long)ldx, (long long)w->k, (long long)ldy, (long long)w->n_local);
    if (m == 0) return B200Q_OK;
    float* y32 = static_cast<float*>(d_y);
    int64_t ldy32 = ldy;
    if (y_dtype == B200Q_BF16) {
        rc = ensure_scratch(ctx, (size_t)m * w->n_local * sizeof(float), 1);
        if (rc != B200Q_OK) return rc;
        y32 = static_cast<float*>(ctx->scratch2);
        ldy32 = w->n_local;
    }
    // A few activation rows on a small tensor: the decode kernel, 8 rows at a time, beats the prefill kernels, whose
    // launch pair, pipeline fill and partial-tile hand-over cost about 20 us whatever the size. Estimates from the
    // measured rates: decode 5 us + image bytes at 2.5 TB/s per 8 rows; prefill 20 us + the larger of flops at
    // 1.2 PFLOP/s and bytes at 5 TB/s.
    bool decode_rows = false;
    if (m > 8 && m <= 32 && x_dtype == B200Q_F32 && w->dimg.base && gemv_fast_supported(w) && gemv_i8_supported(w, 8) &&
        (reinterpret_cast<uintptr_t>(d_x) & 15) == 0 && (ldx % 4) == 0) {
        const double bytes = (double)w->dimg.bytes;
        const double t_dec = ((m + 7) / 8) * (5e-6 + bytes / 2.5e12);
        const double flops = 2.0 * m * (double)w->n_local * (double)w->k;
        const double t_pre = 20e-6 + (flops / 1.2e15 > bytes / 5e12 ? flops / 1.2e15 : bytes / 5e12);
        decode_rows = t_dec < t_pre;
    }
    if ((flags & B200Q_MM_MX_NATIVE) && m > 8) {
        // opt-in: 4-bit codes and their block scales straight into the block-scaled tensor-core MMA, activations as MXFP8
        if (flags & (B200Q_MM_SEQUENTIAL | B200Q_MM_NO_TENSOR)) return fail(B200Q_ERR_INVALID, "matmul: B200Q_MM_MX_NATIVE contradicts the other flags");
        if (ctx->scatter_extra > 0) return fail(B200Q_ERR_UNSUPPORTED, "matmul_scatter: the native MX kernel writes one output");
        rc = launch_gemm_mx_native(ctx, w, d_x, x_dtype == B200Q_BF16, ldx, y32, ldy32, m);
        if (rc != B200Q_OK) return rc;
        ctx->tc_pending = true;
        if (y_dtype == B200Q_BF16) rc = launch_convert_f32_to_bf16(ctx, y32, ldy32, d_y, ldy, m, w->n_local);
        return rc;
    }
    const bool tensor = m > 8 && !decode_rows && !(flags & (B200Q_MM_SEQUENTIAL | B200Q_MM_NO_TENSOR)) && gemm_tc_supported(w, m);
    if (tensor) {
        // tcgen05 path: activations are copied to f16 (row-scaled) and fetched by TMA
        rc = launch_gemm_tc(ctx, w, d_x, x_dtype == B200Q_BF16, ldx, y32, ldy32, m);
        if (rc != B200Q_OK) return rc;
        ctx->tc_pending = true;
    } else {
        const float* x32 = static_cast<const float*>(d_x);
        int64_t ldx32 = ldx;
        if (x_dtype == B200Q_BF16) {
            rc = ensure_scratch(ctx, (size_t)m * w->k * sizeof(float), 0);
            if (rc != B200Q_OK) return rc;
            rc = launch_convert_bf16_to_f32(ctx, d_x, ldx, static_cast<float*>(ctx->scratch), w->k, m, w->k);
            if (rc != B200Q_OK) return rc;
            x32 = static_cast<const float*>(ctx->scratch);
            ldx32 = w->k;
        }
        rc = matmul_f32(ctx, w, x32, ldx32, y32, ldy32, m, flags);
        if (rc != B200Q_OK) return rc;
    }
    if (y_dtype == B200Q_BF16) rc = launch_convert_f32_to_bf16(ctx, y32, ldy32, d_y, ldy, m, w->n_local);
    return rc;
}

// Sharded product with the gather fused into the kernels' epilogues: this GPU's output slice is stored into
// its column block of EVERY listed full output (its own and the peers', peer-mapped), so no collective copies
// the slices afterwards. The caller synchronises the GPUs before reading (a barrier, or one tiny collective
// on the same streams).
int b200q_matmul_scatter(b200q_ctx* ctx, const b200q_weight* w, const void* d_x, int x_dtype, void* const* d_y_full, int n_outputs,
                         int64_t ldy, int m, unsigned flags) {
    if (!ctx) return fail(B200Q_ERR_INVALID, "matmul_scatter: ctx is null");
    if (!w) return fail(B200Q_ERR_INVALID, "matmul_scatter: weight handle is null");
    if (!d_y_full || n_outputs < 1 || n_outputs > 8) return fail(B200Q_ERR_INVALID, "matmul_scatter: %d outputs (1..8 allowed)", n_outputs);
    if (ldy < w->row0 + w->n_local) return fail(B200Q_ERR_INVALID, "matmul_scatter: ldy=%lld is smaller than the end of this shard's columns (%lld)", (long long)ldy, (long long)(w->row0 + w->n_local));
    for (int p = 0; p < n_outputs; p++)
        if (!d_y_full[p] || (reinterpret_cast<uintptr_t>(d_y_full[p]) & 15)) return fail(B200Q_ERR_INVALID, "matmul_scatter: output %d is null or not 16-byte aligned", p);
    if (flags & B200Q_MM_SEQUENTIAL) return fail(B200Q_ERR_UNSUPPORTED, "matmul_scatter: the sequential kernel writes one output only");
    if (m > 8 && ((flags & B200Q_MM_NO_TENSOR) || !gemm_tc_supported(w, m)))
        return fail(B200Q_ERR_UNSUPPORTED, "matmul_scatter: m > 8 needs the tensor-core prefill kernels");
    if (flags & B200Q_MM_SCATTER_BF16) {
        // bf16 outputs: the prefill kernels' staged epilogue only
        if (m <= 8) return fail(B200Q_ERR_UNSUPPORTED, "matmul_scatter: bf16 outputs are for m > 8 (the decode kernel writes fp32)");
        if (x_dtype != B200Q_F32 && x_dtype != B200Q_BF16) return fail(B200Q_ERR_INVALID, "matmul_scatter: unknown activation dtype %d", x_dtype);
        if (w->ctx->device != ctx->device) return fail(B200Q_ERR_INVALID, "matmul_scatter: weight lives on device %d, ctx on %d", w->ctx->device, ctx->device);
        if (!d_x) return fail(B200Q_ERR_INVALID, "matmul_scatter: null activation pointer");
        B200Q_CUDA(cudaSetDevice(ctx->device), B200Q_ERR_DEVICE);
        ctx->scatter_extra = n_outputs - 1;
        ctx->scatter_bf16 = true;
        for (int p = 1; p < n_outputs; p++)
            ctx->scatter_y[p - 1] = reinterpret_cast<float*>(static_cast<__nv_bfloat16*>(d_y_full[p]) + w->row0);
        int rc = launch_gemm_tc(ctx, w, d_x, x_dtype == B200Q_BF16 ? 1 : 0, w->k,
                                reinterpret_cast<float*>(static_cast<__nv_bfloat16*>(d_y_full[0]) + w->row0), ldy, m);
        ctx->scatter_extra = 0;
        ctx->scatter_bf16 = false;
        if (rc == B200Q_OK) ctx->tc_pending = true;
        return rc;
    }
    ctx->scatter_extra = n_outputs - 1;
    for (int p = 1; p < n_outputs; p++) ctx->scatter_y[p - 1] = static_cast<float*>(d_y_full[p]) + w->row0;
    int rc = b200q_matmul_ex(ctx, w, d_x, x_dtype, 0, static_cast<float*>(d_y_full[0]) + w->row0, B200Q_F32, ldy, m, flags);
    ctx->scatter_extra = 0;
    return rc;
}

int b200q_matmul_scatter_signal(b200q_ctx* ctx, const b200q_weight* w, const void* d_x, int x_dtype, void* const* d_y_full, int n_outputs,
                                int64_t ldy, int m, unsigned flags, void* const* d_flags_of_ranks, int my_rank, int epoch) {
    if (!ctx) return fail(B200Q_ERR_INVALID, "matmul_scatter_signal: ctx is null");
    if (!d_flags_of_ranks || n_outputs < 1 || n_outputs > 8 || my_rank < 0 || my_rank >= n_outputs)
        return fail(B200Q_ERR_INVALID, "matmul_scatter_signal: rank %d of %d outputs", my_rank, n_outputs);
    for (int p = 0; p < n_outputs; p++) {
        if (!d_flags_of_ranks[p]) return fail(B200Q_ERR_INVALID, "matmul_scatter_signal: flag array of rank %d is null", p);
        ctx->scatter_flag[p] = static_cast<int*>(d_flags_of_ranks[p]);
    }
    ctx->scatter_sig_n = n_outputs; ctx->scatter_sig_my = my_rank; ctx->scatter_sig_epoch = epoch;
    ctx->scatter_signalled = false;
    int rc = b200q_matmul_scatter(ctx, w, d_x, x_dtype, d_y_full, n_outputs, ldy, m, flags);
    const bool done = ctx->scatter_signalled;
    ctx->scatter_sig_n = 0;
    ctx->scatter_signalled = false;
    if (rc != B200Q_OK) return rc;
    // kernels that do not raise the flags themselves (the prefill kernels): a one-warp kernel behind them does
    return done ? B200Q_OK : b200q_peer_signal(ctx, d_flags_of_ranks, n_outputs, my_rank, epoch);
}

int b200q_ipc_get_handle(b200q_ctx* ctx, const void* d_ptr, void* handle64) {
    if (!ctx || !d_ptr || !handle64) return fail(B200Q_ERR_INVALID, "ipc_get_handle: null argument");
    B200Q_CUDA(cudaSetDevice(ctx->device), B200Q_ERR_DEVICE);
    cudaIpcMemHandle_t h;
    B200Q_CUDA(cudaIpcGetMemHandle(&h, const_cast<void*>(d_ptr)), B200Q_ERR_DEVICE);
    static_assert(sizeof(h) == 64, "cudaIpcMemHandle_t is 64 bytes");
    memcpy(handle64, &h, 64);
    return B200Q_OK;
}

int b200q_ipc_open(b200q_ctx* ctx, const void* handle64, void** d_ptr_out) {
    if (!ctx || !handle64 || !d_ptr_out) return fail(B200Q_ERR_INVALID, "ipc_open: null argument");
    B200Q_CUDA(cudaSetDevice(ctx->device), B200Q_ERR_DEVICE);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    B200Q_CUDA(cudaIpcOpenMemHandle(d_ptr_out, h, cudaIpcMemLazyEnablePeerAccess), B200Q_ERR_DEVICE);
    return B200Q_OK;
}

int b200q_ipc_close(b200q_ctx* ctx, void* d_ptr) {
    if (!ctx || !d_ptr) return fail(B200Q_ERR_INVALID, "ipc_close: null argument");
    B200Q_CUDA(cudaSetDevice(ctx->device), B200Q_ERR_DEVICE);
    B200Q_CUDA(cudaIpcCloseMemHandle(d_ptr), B200Q_ERR_DEVICE);
    return B200Q_OK;
}

int b200q_matmul_noalloc(b200q_ctx* ctx, const b200q_weight* w, const float* d_x, float* d_y, int m) {
    if (!ctx) return fail(B200Q_ERR_INVALID, "matmul_noalloc: ctx is null");
    B200Q_CUDA(cudaSetDevice(ctx->device), B200Q_ERR_DEVICE);
    int rc = check_matmul_args(ctx, w, d_x, d_y, m);
    if (rc != B200Q_OK) return rc;
    if (m == 0) return B200Q_OK;
    rc = launch_gemm_tc_noalloc(ctx, w, d_x, d_y, m);
    if (rc == B200Q_OK) ctx->tc_pending = true;
    return rc;
}

int b200q_matmul(b200q_ctx* ctx, const b200q_weight* w, const void* d_x, int x_dtype, void* d_y, int y_dtype, int m,
                 unsigned flags) {
    return b200q_matmul_ex(ctx, w, d_x, x_dtype, 0, d_y, y_dtype, 0, m, flags);
}

int b200q_matmul_host(b200q_ctx* ctx, const b200q_weight* w, const float* h_x, float* h_y, int m, unsigned flags) {
    if (!ctx) return fail(B200Q_ERR_INVALID, "matmul_host: ctx is null");
    B200Q_CUDA(cudaSetDevice(ctx->device), B200Q_ERR_DEVICE);
    int rc = check_matmul_args(ctx, w, h_x, h_y, m);
    if (rc != B200Q_OK) return rc;
    if (m == 0) return B200Q_OK;
    size_t xb = (size_t)m * w->k * sizeof(float), yb = (size_t)m * w->n_local * sizeof(float);
    if ((rc = ensure_scratch(ctx, xb, 0)) != B200Q_OK) return rc;
    if ((rc = ensure_scratch(ctx, yb, 1)) != B200Q_OK) return rc;
    B200Q_CUDA(cudaMemcpyAsync(ctx->scratch, h_x, xb, cudaMemcpyHostToDevice, ctx->stream), B200Q_ERR_COPY);
    rc = b200q_matmul_ex(ctx, w, ctx->scratch, B200Q_F32, w->k, ctx->scratch2, B200Q_F32, w->n_local, m, flags);
    if (rc != B200Q_OK) return rc;
    B200Q_CUDA(cudaMemcpyAsync(h_y, ctx->scratch2, yb, cudaMemcpyDeviceToHost, ctx->stream), B200Q_ERR_COPY);
    return b200q_synchronize(ctx);
}

// Time per image byte of the decode kernel's item forms at m = 1, relative to Q6_K's: the formats differ in instructions
// per byte (a Q4_K item holds the same 2048 weights as a Q6_K item in 0.72 of its bytes), and the work units of a grouped
// launch are cut to equal TIME, not equal bytes. Q4_K's 1.2 is measured on the Q4_K_M decode step (61.1 us with 1.0,
// 58.0 us with 1.2, rising again above 1.25); the others follow the formats' single-product rates at [28672 x 8192].
// With several activation rows the kernel is bound by instruction issue in every format and equal bytes balance best.
// tuning knob: B200Q_DECODE_KIND_COST="q4k,q6k,q80,mx6,mx4,q40,q5k" (the order of the kernel's item kinds)
static double decode_kind_cost(int kind, int m) {
    static double table[DK_COUNT] = {1.2, 1.0, 0.95, 0.95, 1.6, 1.15, 1.15};
    static const bool parsed = [] {
        if (const char* e = getenv("B200Q_DECODE_KIND_COST")) {
            double v[DK_COUNT];
            if (sscanf(e, "%lf,%lf,%lf,%lf,%lf,%lf,%lf", &v[0], &v[1], &v[2], &v[3], &v[4], &v[5], &v[6]) == DK_COUNT) {
                bool ok = true;
                for (int i = 0; i < DK_COUNT; i++) ok = ok && v[i] >= 0.25 && v[i] <= 4.0;
                if (ok) for (int i = 0; i < DK_COUNT; i++) table[i] = v[i];
            }
        }
        return true;
    }();
    (void)parsed;
    return (m == 1 && kind >= 0 && kind < DK_COUNT) ? table[kind] : 1.0;
}

int b200q_batch_create(b200q_ctx* ctx, int count, const b200q_weight* const* w, const float* const* d_x,
                       float* const* d_y, int m, b200q_batch** out) {
    if (!ctx) return fail(B200Q_ERR_INVALID, "batch_create: ctx is null");
    if (!out) return fail(B200Q_ERR_INVALID, "batch_create: out is null");
    *out = nullptr;
    if (count < 0 || (count > 0 && (!w || !d_x || !d_y))) return fail(B200Q_ERR_INVALID, "batch_create: null array");
    if (m < 1 || m > 8) return fail(B200Q_ERR_INVALID, "batch_create: m=%d outside 1..8", m);
    b200q_batch* b = new b200q_batch();
    b->ctx = ctx;
    b->m = m;
    for (int i = 0; i < count; i++) {
        int rc = check_matmul_args(ctx, w[i], d_x[i], d_y[i], m);
        if (rc == B200Q_OK && !gemv_fast_supported(w[i])) rc = fail(B200Q_ERR_UNSUPPORTED, "batch_create: op %d is not an NK tensor with k %% 8 == 0", i);
        if (rc == B200Q_OK && (reinterpret_cast<uintptr_t>(d_x[i]) & 15) != 0) rc = fail(B200Q_ERR_INVALID, "batch_create: activations of op %d are not 16-byte aligned", i);
        if (rc != B200Q_OK) { delete b; return rc; }
        b->w.push_back(w[i]);
        b->x.push_back(d_x[i]);
        b->y.push_back(d_y[i]);
        b->weight_bytes += w[i]->packed_bytes;
    }
    // one grouped launch of the integer decode kernel when every product has a decode image
    bool all_i8 = count > 0;
    for (int i = 0; i < count; i++) all_i8 = all_i8 && gemv_i8_supported(w[i], m);
    if (all_i8) {
        int max_item = 0, kmax = 0, mask = 0;
        for (int i = 0; i < count; i++) {
            if (w[i]->dimg.item_bytes > max_item) max_item = w[i]->dimg.item_bytes;
            if (w[i]->k > kmax) kmax = (int)w[i]->k;
            mask |= 1 << w[i]->dimg.kind;
        }
        all_i8 = gemv_i8_plan(max_item, kmax, mask, m, &b->dl);
    }
    if (all_i8) {
        std::vector<DOp> ops(count);
        std::vector<double> tile_cost;
        std::vector<int> tile_op;
        int total = 0;
        for (int i = 0; i < count; i++) {
            ops[i] = make_dop(w[i], d_x[i], w[i]->k, d_y[i], w[i]->n_local);
            ops[i].rt0 = total;
            total += ops[i].nrt;
            const double c = (double)ops[i].nh * ops[i].item_bytes * decode_kind_cost(ops[i].kind, m);
            for (int t = 0; t < ops[i].nrt; t++) { tile_cost.push_back(c); tile_op.push_back(i); }
        }
        int n_ctas = ctx->info.sm_count * b->dl.ctas_per_sm;
        std::vector<int2> ranges;
        gemv_i8_make_units(tile_cost, tile_op, n_ctas, &ranges);
        b->n_units = (int)ranges.size();
        if (n_ctas > b->n_units) n_ctas = b->n_units;
        cudaError_t e = cudaSetDevice(ctx->device);
        if (e == cudaSuccess) e = cudaMalloc(&b->d_dops, sizeof(DOp) * count);
        if (e == cudaSuccess) e = cudaMalloc(&b->d_ranges, sizeof(int2) * ranges.size());
        if (e == cudaSuccess) e = cudaMemcpyAsync(b->d_dops, ops.data(), sizeof(DOp) * count, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(b->d_ranges, ranges.data(), sizeof(int2) * ranges.size(), cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) {
            if (b->d_dops) cudaFree(b->d_dops);
            if (b->d_ranges) cudaFree(b->d_ranges);
            delete b;
            return cuda_fail(B200Q_ERR_ALLOC, e, "batch_create");
        }
        b->grouped = true;
        b->h_dops = ops;
        b->n_ctas = n_ctas;
        b->total_rt = total;
        b->dsingle = ops[0];
        *out = b;
        return B200Q_OK;
    }
    *out = b;
    return B200Q_OK;
}

int b200q_batch_run(b200q_ctx* ctx, b200q_batch* batch, float* ms_out) {
    if (!ctx || !batch) return fail(B200Q_ERR_INVALID, "batch_run: null argument");
    B200Q_CUDA(cudaSetDevice(ctx->device), B200Q_ERR_DEVICE);
    if (ms_out) B200Q_CUDA(cudaEventRecord(ctx->ev0, ctx->stream), B200Q_ERR_DEVICE);
    if (batch->grouped) {
        int n = (int)batch->w.size();
        int rc = launch_gemv_i8(ctx, &batch->dsingle, batch->d_dops, n, batch->d_ranges, batch->n_units, batch->n_ctas,
                                batch->total_rt, batch->m, batch->dl);
        if (rc != B200Q_OK) return rc;
    } else {
        for (size_t i = 0; i < batch->w.size(); i++) {
            int rc = launch_gemv(ctx, batch->w[i], batch->x[i], batch->w[i]->k, batch->y[i], batch->w[i]->n_local, batch->m);
            if (rc != B200Q_OK) return rc;
        }
    }
    if (ms_out) {
        B200Q_CUDA(cudaEventRecord(ctx->ev1, ctx->stream), B200Q_ERR_DEVICE);
        B200Q_CUDA(cudaEventSynchronize(ctx->ev1), B200Q_ERR_DEVICE);
        B200Q_CUDA(cudaEventElapsedTime(ms_out, ctx->ev0, ctx->ev1), B200Q_ERR_DEVICE);
    }
    return B200Q_OK;
}

int b200q_batch_run_host(b200q_ctx* ctx, b200q_batch* batch, const float* h_x_all, float* h_y_all) {
    if (!ctx || !batch) return fail(B200Q_ERR_INVALID, "batch_run_host: null argument");
    B200Q_CUDA(cudaSetDevice(ctx->device), B200Q_ERR_DEVICE);
    const size_t cnt = batch->w.size();
    if (cnt == 0) return B200Q_OK;
    if (!h_x_all || !h_y_all) return fail(B200Q_ERR_INVALID, "batch_run_host: null host buffer");
    // one copy each way when the device buffers of the batch are laid out back to back, else one per product
    bool xc = true, yc = true;
    size_t xtot = 0, ytot = 0;
    for (size_t i = 0; i < cnt; i++) {
        size_t xb = (size_t)batch->m * batch->w[i]->k, yb = (size_t)batch->m * batch->w[i]->n_local;
        if (batch->x[i] != batch->x[0] + xtot) xc = false;
        if (batch->y[i] != batch->y[0] + ytot) yc = false;
        xtot += xb; ytot += yb;
    }
    if (xc) {
        B200Q_CUDA(cudaMemcpyAsync(const_cast<float*>(batch->x[0]), h_x_all, xtot * sizeof(float), cudaMemcpyHostToDevice, ctx->stream), B200Q_ERR_COPY);
    } else {
        size_t off = 0;
        for (size_t i = 0; i < cnt; i++) {
            size_t xb = (size_t)batch->m * batch->w[i]->k;
            B200Q_CUDA(cudaMemcpyAsync(const_cast<float*>(batch->x[i]), h_x_all + off, xb * sizeof(float), cudaMemcpyHostToDevice, ctx->stream), B200Q_ERR_COPY);
            off += xb;
        }
    }
    // Outputs in pinned host memory the device can address: the grouped kernel stores its results straight into
    // them (posted writes over PCIe, overlapped with the rest of the launch) instead of a device buffer + a copy.
    if (batch->grouped && batch->w[0]->ctx->scatter_extra == 0) {
        cudaPointerAttributes pa{};
        if (cudaPointerGetAttributes(&pa, h_y_all) == cudaSuccess && pa.type == cudaMemoryTypeHost && pa.devicePointer) {
            float* dy = static_cast<float*>(pa.devicePointer);
            {
                if (batch->hosty_base != h_y_all) {
                    std::vector<DOp> ops = batch->h_dops;
                    size_t off = 0;
                    for (size_t i = 0; i < cnt; i++) {
                        ops[i].y = dy + off;
                        off += (size_t)batch->m * batch->w[i]->n_local;
                    }
                    cudaError_t e = cudaSuccess;
                    if (!batch->d_dops_hosty) e = cudaMalloc(&batch->d_dops_hosty, sizeof(DOp) * cnt);
                    if (e == cudaSuccess) e = cudaMemcpyAsync(batch->d_dops_hosty, ops.data(), sizeof(DOp) * cnt, cudaMemcpyHostToDevice, ctx->stream);
                    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);   // `ops` is pageable and local
                    if (e != cudaSuccess) return cuda_fail(B200Q_ERR_ALLOC, e, "batch_run_host");
                    batch->dsingle_hosty = ops[0];
                    batch->hosty_base = h_y_all;
                }
                int n = (int)cnt;
                // The kernel's last CTA, once every CTA's results are on their way (system-scope fences), stores the
                // launch's status word and then a sequence number into a host-visible word; the host polls that word
                // instead of synchronising the stream and copying the status back (two round trips less per step).
                PeerSignal sig{};
                if (ctx->h_done) {
                    if (++ctx->done_seq == 0x7FFFFFFF) ctx->done_seq = 1;
                    sig.n = 2; sig.my = 0; sig.epoch = ctx->done_seq;
                    sig.flag[0] = ctx->d_done; sig.flag[1] = ctx->d_done;   // slot [1][my = 0] = word 0
                    sig.status_out = ctx->d_done + 1;
                }
                int rc = launch_gemv_i8(ctx, &batch->dsingle_hosty, batch->d_dops_hosty, n, batch->d_ranges, batch->n_units,
                                        batch->n_ctas, batch->total_rt, batch->m, batch->dl, ctx->h_done ? &sig : nullptr);
                if (rc != B200Q_OK) return rc;
                if (ctx->h_done) {
                    const auto t0 = std::chrono::steady_clock::now();
                    bool seen = false;
                    for (unsigned spin = 1; !seen; spin++) {
                        seen = ctx->h_done[0] == ctx->done_seq;
                        if (!seen && (spin & 1023u) == 0) {
                            if (cudaStreamQuery(ctx->stream) != cudaErrorNotReady) break;          // finished (or failed) without the word
                            if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(5)) break;
                        }
                    }
                    if (seen && ctx->h_done[1] == 0) return B200Q_OK;   // results are in host memory, nothing to report
                }
                return b200q_synchronize(ctx);
            }
        }
        cudaGetLastError();   // pageable host memory: not an error, take the copy path
    }
    int rc = b200q_batch_run(ctx, batch, nullptr);
    if (rc != B200Q_OK) return rc;
    if (yc) {
        B200Q_CUDA(cudaMemcpyAsync(h_y_all, batch->y[0], ytot * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream), B200Q_ERR_COPY);
    } else {
        size_t off = 0;
        for (size_t i = 0; i < cnt; i++) {
            size_t yb = (size_t)batch->m * batch->w[i]->n_local;
            B200Q_CUDA(cudaMemcpyAsync(h_y_all + off, batch->y[i], yb * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream), B200Q_ERR_COPY);
            off += yb;
        }
    }
    B200Q_CUDA(cudaStreamSynchronize(ctx->stream), B200Q_ERR_DEVICE);
    return B200Q_OK;
}

int b200q_batch_free(b200q_batch* batch) {
    if (!batch) return B200Q_OK;
    if (batch->d_ranges || batch->d_dops) {
        cudaSetDevice(batch->ctx->device);
        cudaStreamSynchronize(batch->ctx->stream);
        if (batch->d_dops) cudaFree(batch->d_dops);
        if (batch->d_ranges) cudaFree(batch->d_ranges);
        if (batch->d_dops_hosty) cudaFree(batch->d_dops_hosty);
        cudaGetLastError();
    }
    delete batch;
    return B200Q_OK;
}

int b200q_batch_launches(const b200q_batch* batch) { return batch ? (batch->grouped ? 1 : (int)batch->w.size()) : 0; }

size_t b200q_batch_weight_bytes(const b200q_batch* batch) { return batch ? batch->weight_bytes : 0; }

}  // extern "C"
