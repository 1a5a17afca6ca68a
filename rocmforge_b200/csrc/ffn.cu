// Projection-site operators on packed weights: the SwiGLU MLP block, the row bias add, and the shared-input
// projection group (Q, K, V) — the callers either side of the fused dequant + matmul products.
//
// Replaces HipBackend::mlp_swiglu (src/backend/hip_backend/backend.rs:1153-1276: two fp32 hipBLAS products on
// dequantised weights, a synchronise, kernels/swiglu.hip:37-63, a synchronise, a third product) and
// HipBackend::add_row_bias (backend.rs:924-975: one saxpy per row). Here the weights stay packed; at m <= 8 the
// gate and up projections are ONE grouped launch of the tensor-core decode kernel (they share the activations),
// the activation kernel runs in stream order with no host synchronisation in between, and the down projection
// follows on the same stream. At m > 8 the three products are the prefill kernels; at m > 32 the activation is formed
// by the down projection's own activation conversion instead of a kernel of its own.
#include "common.cuh"

namespace b200q {

// out[i] = gate[i] * swish(up[i]), swish(u) = u * 1 / (1 + expf(-u))   (kernels/swiglu.hip:55-62: the
// activation is applied to the UP projection, and the operation order below is that kernel's)
__global__ void __launch_bounds__(256) swiglu_kernel(const float* __restrict__ gate, const float* __restrict__ up,
                                                     float* __restrict__ out, int64_t total) {
    // the product that follows may start its CTAs and stream its weights while this kernel runs; it waits for
    // this kernel's completion (griddepcontrol.wait) before it reads the activations written here
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // launched with programmatic stream serialisation itself: gate and up come from the kernel ahead of it
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int64_t i4 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i4 >= total) return;
    if (i4 + 4 <= total) {
        const float4 g = *reinterpret_cast<const float4*>(gate + i4);
        const float4 u = *reinterpret_cast<const float4*>(up + i4);
        float4 o;
        o.x = g.x * (u.x * (1.0f / (1.0f + expf(-u.x))));
        o.y = g.y * (u.y * (1.0f / (1.0f + expf(-u.y))));
        o.z = g.z * (u.z * (1.0f / (1.0f + expf(-u.z))));
        o.w = g.w * (u.w * (1.0f / (1.0f + expf(-u.w))));
        *reinterpret_cast<float4*>(out + i4) = o;
    } else {
        for (int64_t i = i4; i < total; i++) {
            const float u = up[i];
            out[i] = gate[i] * (u * (1.0f / (1.0f + expf(-u))));
        }
    }
}

// y[r, c] += bias[c]: saxpy(alpha = 1) per row, i.e. one fp32 add per element
__global__ void __launch_bounds__(256) add_row_bias_kernel(float* __restrict__ y, int64_t ldy, const float* __restrict__ bias,
                                                           int64_t cols) {
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    float* p = y + (int64_t)blockIdx.y * ldy + c;
    *p = __fadd_rn(1.0f * __ldg(bias + c), *p);
}

}  // namespace b200q

using namespace b200q;

struct b200q_mlp {
    b200q_ctx* ctx = nullptr;
    const b200q_weight *gate = nullptr, *up = nullptr, *down = nullptr;
    const float* x = nullptr;
    float* out = nullptr;
    int m = 0;
    float *d_gate = nullptr, *d_up = nullptr;   // [m, n_ff] each; the activation overwrites d_gate
    b200q_batch* gate_up = nullptr;             // grouped decode launch (m <= 8), else null
};

extern "C" {

int b200q_swiglu(b200q_ctx* ctx, const float* d_gate, const float* d_up, float* d_out, int64_t seq_len, int64_t intermediate_size) {
    if (!ctx) return fail(B200Q_ERR_INVALID, "swiglu: ctx is null");
    B200Q_CUDA(cudaSetDevice(ctx->device), B200Q_ERR_DEVICE);
    if (seq_len < 0 || intermediate_size < 0) return fail(B200Q_ERR_INVALID, "swiglu: negative size");
    const int64_t total = seq_len * intermediate_size;
    if (total == 0) return B200Q_OK;
    if (!d_gate || !d_up || !d_out) return fail(B200Q_ERR_INVALID, "swiglu: null device pointer");
    if ((reinterpret_cast<uintptr_t>(d_gate) | reinterpret_cast<uintptr_t>(d_up) | reinterpret_cast<uintptr_t>(d_out)) & 15)
        return fail(B200Q_ERR_INVALID, "swiglu: buffers must be 16-byte aligned");
    const int64_t grid = (total + 1023) / 1024;
    if (grid > 0x7FFFFFFF) return fail(B200Q_ERR_INVALID, "swiglu: tensor too large for one launch");
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(256);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    B200Q_CUDA(cudaLaunchKernelEx(&cfg, swiglu_kernel, d_gate, d_up, d_out, total), B200Q_ERR_LAUNCH);
    return B200Q_OK;
}

int b200q_add_row_bias(b200q_ctx* ctx, float* d_y, int64_t ldy, const float* d_bias, int64_t rows, int64_t cols) {
    if (!ctx) return fail(B200Q_ERR_INVALID, "add_row_bias: ctx is null");
    B200Q_CUDA(cudaSetDevice(ctx->device), B200Q_ERR_DEVICE);
    if (rows < 0 || cols < 0) return fail(B200Q_ERR_INVALID, "add_row_bias: negative size");
    if (rows == 0 || cols == 0) return B200Q_OK;   // backend.rs:944-946
    if (!d_y || !d_bias) return fail(B200Q_ERR_INVALID, "add_row_bias: null device pointer");
    if (ldy == 0) ldy = cols;
    if (ldy < cols) return fail(B200Q_ERR_INVALID, "add_row_bias: row pitch %lld smaller than %lld columns", (long long)ldy, (long long)cols);
    if (rows > 65535) return fail(B200Q_ERR_INVALID, "add_row_bias: more than 65535 rows in one call");
    dim3 grid((unsigned)((cols + 255) / 256), (unsigned)rows);
    add_row_bias_kernel<<<grid, 256, 0, ctx->stream>>>(d_y, ldy, d_bias, cols);
    B200Q_CUDA(cudaGetLastError(), B200Q_ERR_LAUNCH);
    return B200Q_OK;
}

int b200q_mlp_create(b200q_ctx* ctx, const b200q_weight* w_gate, const b200q_weight* w_up, const b200q_weight* w_down,
                     const float* d_hidden_states, float* d_output, int m, b200q_mlp** out) {
    if (!ctx) return fail(B200Q_ERR_INVALID, "mlp_create: ctx is null");
    if (!out) return fail(B200Q_ERR_INVALID, "mlp_create: out is null");
    *out = nullptr;
    if (!w_gate || !w_up || !w_down) return fail(B200Q_ERR_INVALID, "mlp_create: null weight handle");
    if (!d_hidden_states || !d_output) return fail(B200Q_ERR_INVALID, "mlp_create: null device pointer");
    if (m < 1) return fail(B200Q_ERR_INVALID, "mlp_create: seq_len %d < 1", m);
    // the reference's shape checks (backend.rs:1169-1207), on [out_features, in_features] packed tensors
    const int64_t hidden = w_gate->k, n_ff = w_gate->n_local;
    if (w_up->k != hidden) return fail(B200Q_ERR_INVALID, "up_weight must be 2D [hidden_size, intermediate_size]");
    if (w_down->n_local != hidden) return fail(B200Q_ERR_INVALID, "down_weight must be 2D [intermediate_size, hidden_size]");
    if (w_up->n_local != n_ff || w_down->k != n_ff) return fail(B200Q_ERR_INVALID, "All intermediate dimensions must match");
    B200Q_CUDA(cudaSetDevice(ctx->device), B200Q_ERR_DEVICE);
    b200q_mlp* p = new b200q_mlp();
    p->ctx = ctx; p->gate = w_gate; p->up = w_up; p->down = w_down;
    p->x = d_hidden_states; p->out = d_output; p->m = m;
    const size_t bytes = ((size_t)m * n_ff * sizeof(float) + 255) & ~(size_t)255;
    void* base = nullptr;
    cudaError_t e = cudaMalloc(&base, 2 * bytes);
    if (e != cudaSuccess) { delete p; return cuda_fail(B200Q_ERR_ALLOC, e, "mlp_create"); }
    p->d_gate = static_cast<float*>(base);
    p->d_up = reinterpret_cast<float*>(static_cast<uint8_t*>(base) + bytes);
    if (m <= 8) {
        const b200q_weight* w[2] = {w_gate, w_up};
        const float* x[2] = {d_hidden_states, d_hidden_states};
        float* y[2] = {p->d_gate, p->d_up};
        int rc = b200q_batch_create(ctx, 2, w, x, y, m, &p->gate_up);
        if (rc != B200Q_OK) p->gate_up = nullptr;   // formats without a grouped kernel: two single launches below
    }
    *out = p;
    return B200Q_OK;
}

int b200q_mlp_run(b200q_ctx* ctx, b200q_mlp* p) {
    if (!ctx || !p) return fail(B200Q_ERR_INVALID, "mlp_run: null argument");
    if (p->ctx != ctx) return fail(B200Q_ERR_INVALID, "mlp_run: plan belongs to another context");
    int rc;
    if (p->gate_up) {
        rc = b200q_batch_run(ctx, p->gate_up, nullptr);
        if (rc != B200Q_OK) return rc;
    } else if (p->m > 8 && gemm_tc_supported(p->gate, p->m) && gemm_tc_supported(p->up, p->m)) {
        // prefill: one f16 copy of the activations serves both tensor-core products
        B200Q_CUDA(cudaSetDevice(ctx->device), B200Q_ERR_DEVICE);
        rc = launch_gemm_tc_pair(ctx, p->gate, p->up, p->x, p->gate->k, p->d_gate, p->d_up, p->m);
        if (rc != B200Q_OK) return rc;
        ctx->tc_pending = true;
    } else {
        rc = b200q_matmul(ctx, p->gate, p->x, B200Q_F32, p->d_gate, B200Q_F32, p->m, 0);
        if (rc != B200Q_OK) return rc;
        rc = b200q_matmul(ctx, p->up, p->x, B200Q_F32, p->d_up, B200Q_F32, p->m, 0);
        if (rc != B200Q_OK) return rc;
    }
    // prefill: gate * swish(up) is formed by the down projection's activation conversion, the pass that reads those
    // rows anyway (five launches for the block instead of six, one pass over [m, intermediate] less)
    if (p->m > 32 && gemm_tc_supported(p->down, p->m)) {
        B200Q_CUDA(cudaSetDevice(ctx->device), B200Q_ERR_DEVICE);
        ctx->act_mul = p->d_up;
        rc = launch_gemm_tc(ctx, p->down, p->d_gate, 0, p->down->k, p->out, p->down->n_local, p->m);
        ctx->act_mul = nullptr;
        if (rc == B200Q_OK) ctx->tc_pending = true;
        return rc;
    }
    rc = b200q_swiglu(ctx, p->d_gate, p->d_up, p->d_gate, p->m, p->gate->n_local);
    if (rc != B200Q_OK) return rc;
    return b200q_matmul(ctx, p->down, p->d_gate, B200Q_F32, p->out, B200Q_F32, p->m, 0);
}

int b200q_mlp_free(b200q_mlp* p) {
    if (!p) return B200Q_OK;
    if (p->gate_up) b200q_batch_free(p->gate_up);
    if (p->d_gate) {
        cudaSetDevice(p->ctx->device);
        cudaStreamSynchronize(p->ctx->stream);
        cudaFree(p->d_gate);
        cudaGetLastError();
    }
    delete p;
    return B200Q_OK;
}

}  // extern "C"
