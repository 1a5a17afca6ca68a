// b200q_matmul*: argument checks and the choice of kernel for one fused dequant + matmul.
#include <vector>

#include "common.cuh"

using namespace b200q;

struct b200q_batch {
    b200q_ctx* ctx = nullptr;
    int m = 0;
    std::vector<const b200q_weight*> w;
    std::vector<const float*> x;
    std::vector<float*> y;
    size_t weight_bytes = 0;
};

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
    if ((flags & B200Q_MM_SEQUENTIAL) || !gemv_fast_supported(w)) return launch_matmul_seq(ctx, w, x, ldx, y, ldy, m);
    bool aligned = (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (ldx % 4) == 0;
    if (!aligned) return launch_matmul_seq(ctx, w, x, ldx, y, ldy, m);
    for (int i = 0; i < m; i += 8) {
        int mm = m - i < 8 ? m - i : 8;
        int rc = launch_gemv(ctx, w, x + (int64_t)i * ldx, ldx, y + (int64_t)i * ldy, ldy, mm);
        if (rc != B200Q_OK) return rc;
    }
    return B200Q_OK;
}

extern "C" {

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
    float* y32 = static_cast<float*>(d_y);
    int64_t ldy32 = ldy;
    if (y_dtype == B200Q_BF16) {
        rc = ensure_scratch(ctx, (size_t)m * w->n_local * sizeof(float), 1);
        if (rc != B200Q_OK) return rc;
        y32 = static_cast<float*>(ctx->scratch2);
        ldy32 = w->n_local;
    }
    rc = matmul_f32(ctx, w, x32, ldx32, y32, ldy32, m, flags);
    if (rc != B200Q_OK) return rc;
    if (y_dtype == B200Q_BF16) rc = launch_convert_f32_to_bf16(ctx, y32, ldy32, d_y, ldy, m, w->n_local);
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
    rc = matmul_f32(ctx, w, static_cast<const float*>(ctx->scratch), w->k, static_cast<float*>(ctx->scratch2), w->n_local, m, flags);
    if (rc != B200Q_OK) return rc;
    B200Q_CUDA(cudaMemcpyAsync(h_y, ctx->scratch2, yb, cudaMemcpyDeviceToHost, ctx->stream), B200Q_ERR_COPY);
    B200Q_CUDA(cudaStreamSynchronize(ctx->stream), B200Q_ERR_DEVICE);
    return B200Q_OK;
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
        if (rc != B200Q_OK) { delete b; return rc; }
        b->w.push_back(w[i]);
        b->x.push_back(d_x[i]);
        b->y.push_back(d_y[i]);
        b->weight_bytes += w[i]->packed_bytes;
    }
    *out = b;
    return B200Q_OK;
}

int b200q_batch_run(b200q_ctx* ctx, b200q_batch* batch, float* ms_out) {
    if (!ctx || !batch) return fail(B200Q_ERR_INVALID, "batch_run: null argument");
    B200Q_CUDA(cudaSetDevice(ctx->device), B200Q_ERR_DEVICE);
    if (ms_out) B200Q_CUDA(cudaEventRecord(ctx->ev0, ctx->stream), B200Q_ERR_DEVICE);
    for (size_t i = 0; i < batch->w.size(); i++) {
        int rc = launch_gemv(ctx, batch->w[i], batch->x[i], batch->w[i]->k, batch->y[i], batch->w[i]->n_local, batch->m);
        if (rc != B200Q_OK) return rc;
    }
    if (ms_out) {
        B200Q_CUDA(cudaEventRecord(ctx->ev1, ctx->stream), B200Q_ERR_DEVICE);
        B200Q_CUDA(cudaEventSynchronize(ctx->ev1), B200Q_ERR_DEVICE);
        B200Q_CUDA(cudaEventElapsedTime(ms_out, ctx->ev0, ctx->ev1), B200Q_ERR_DEVICE);
    }
    return B200Q_OK;
}

int b200q_batch_free(b200q_batch* batch) {
    delete batch;
    return B200Q_OK;
}

size_t b200q_batch_weight_bytes(const b200q_batch* batch) { return batch ? batch->weight_bytes : 0; }

}  // extern "C"
