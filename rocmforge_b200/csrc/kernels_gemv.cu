// Decode-side fused dequant + matmul kernels on CUDA cores (any format, m <= 8 per launch).
//
// Replaces kernels/q4_0_matmul.hip:153, q4_k_matmul.hip:216 and q6_k_matmul.hip:216 of the reference,
// which run ONE thread block per activation row and fetch one 4-bit code per inner iteration. Here the
// output features are spread over the whole GPU: a group of L lanes (L = 4..32, a power of two) owns
// one weight row, every lane decodes 8 weights at a time straight from the packed planes, multiplies
// them with up to 8 activation rows held in L1, and the group reduces with warp shuffles.
//
// matmul_seq_kernel is the parity kernel: one thread per output, ascending k, multiply then add,
// which reproduces cpu_matmul_f32 (src/tensor/matmul.rs:219-233) bit for bit in either orientation.
#include <cuda_bf16.h>

#include "common.cuh"

namespace b200q {

template <int F, int MT>
__global__ void __launch_bounds__(256)
gemv_piece_kernel(WView v, const float* __restrict__ x, int64_t ldx, float* __restrict__ y, int64_t ldy,
                  int64_t n_rows, int64_t k, int m, int lanes_log2) {
    const int L = 1 << lanes_log2;
    const int lane = threadIdx.x & 31;
    const int sub = lane & (L - 1);
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t row = warp * (32 >> lanes_log2) + (lane >> lanes_log2);
    const int64_t pieces = k >> 3;
    float acc[MT];
#pragma unroll
    for (int i = 0; i < MT; i++) acc[i] = 0.0f;
    if (row < n_rows) {
        const int64_t base = row * pieces;
#pragma unroll 2
        for (int64_t p = sub; p < pieces; p += L) {
            float w[8];
            int64_t gp = base + p;
            decode8<F>(v, gp >> 2, (int)(gp & 3), w);
#pragma unroll
            for (int mi = 0; mi < MT; mi++) {
                if (mi < m) {
                    const float4* xp = reinterpret_cast<const float4*>(x + mi * ldx + p * 8);
                    float4 a = __ldg(xp), b = __ldg(xp + 1);
                    float s = acc[mi];
                    s = fmaf(w[0], a.x, s); s = fmaf(w[1], a.y, s); s = fmaf(w[2], a.z, s); s = fmaf(w[3], a.w, s);
                    s = fmaf(w[4], b.x, s); s = fmaf(w[5], b.y, s); s = fmaf(w[6], b.z, s); s = fmaf(w[7], b.w, s);
                    acc[mi] = s;
                }
            }
        }
    }
#pragma unroll
    for (int mi = 0; mi < MT; mi++) {
        float s = acc[mi];
        for (int o = L >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
        if (sub == 0 && row < n_rows && mi < m) y[mi * ldy + row] = s;
    }
}

bool gemv_fast_supported(const b200q_weight* w) {
    // rows must start on an 8-weight piece and activations must allow 16-byte loads
    return w->orient == B200Q_ORIENT_NK && (w->k % 8) == 0;
}

template <int F>
static int launch_gemv_fmt(b200q_ctx* ctx, const b200q_weight* w, const float* d_x, int64_t ldx, float* d_y,
                           int64_t ldy, int m) {
    int64_t pieces = w->k / 8;
    int lanes_log2 = 2;
    while (lanes_log2 < 5 && (1 << lanes_log2) < pieces) lanes_log2++;
    int rows_per_warp = 32 >> lanes_log2;
    int64_t warps = (w->n_local + rows_per_warp - 1) / rows_per_warp;
    int64_t grid = (warps + 7) / 8;
    if (grid > 0x7FFFFFFF) return fail(B200Q_ERR_INVALID, "matmul: too many rows for one launch");
    dim3 g((unsigned)grid), b(256);
    if (m == 1) gemv_piece_kernel<F, 1><<<g, b, 0, ctx->stream>>>(w->view, d_x, ldx, d_y, ldy, w->n_local, w->k, m, lanes_log2);
    else if (m == 2) gemv_piece_kernel<F, 2><<<g, b, 0, ctx->stream>>>(w->view, d_x, ldx, d_y, ldy, w->n_local, w->k, m, lanes_log2);
    else if (m <= 4) gemv_piece_kernel<F, 4><<<g, b, 0, ctx->stream>>>(w->view, d_x, ldx, d_y, ldy, w->n_local, w->k, m, lanes_log2);
    else gemv_piece_kernel<F, 8><<<g, b, 0, ctx->stream>>>(w->view, d_x, ldx, d_y, ldy, w->n_local, w->k, m, lanes_log2);
    B200Q_CUDA(cudaGetLastError(), B200Q_ERR_LAUNCH);
    return B200Q_OK;
}

int launch_gemv(b200q_ctx* ctx, const b200q_weight* w, const float* d_x, int64_t ldx, float* d_y, int64_t ldy, int m) {
    if (m < 1 || m > 8) return fail(B200Q_ERR_INVALID, "gemv: m=%d outside 1..8", m);
    if ((reinterpret_cast<uintptr_t>(d_x) & 15) != 0 || (ldx % 4) != 0)
        return fail(B200Q_ERR_INVALID, "gemv: activations must be 16-byte aligned with ldx a multiple of 4");
    if (w->n_local == 0) return B200Q_OK;
    switch (w->fmt) {
#define X(F) \
    case F: return launch_gemv_fmt<F>(ctx, w, d_x, ldx, d_y, ldy, m);
        B200Q_FOR_EACH_FMT(X)
#undef X
    }
    return fail(B200Q_ERR_INVALID, "gemv: unknown format %d", w->fmt);
}

// ---------------------------------------------------------------------------------------------
template <int F>
__global__ void __launch_bounds__(128)
matmul_seq_kernel(WView v, const float* __restrict__ x, int64_t ldx, float* __restrict__ y, int64_t ldy,
                  int64_t n, int64_t k, int m, int orient_kn) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n * m) return;
    int64_t j = idx % n;
    int mi = (int)(idx / n);
    float sum = 0.0f;
    int64_t cur = -1;
    float w[8];
    for (int64_t l = 0; l < k; l++) {
        int64_t e = orient_kn ? l * n + j : j * k + l;
        int64_t piece = e >> 3;
        if (piece != cur) {
            decode8<F>(v, piece >> 2, (int)(piece & 3), w);
            cur = piece;
        }
        float wv = w[0];
#pragma unroll
        for (int t = 1; t < 8; t++)
            if ((int)(e & 7) == t) wv = w[t];
        sum = __fadd_rn(sum, __fmul_rn(x[mi * ldx + l], wv));
    }
    y[mi * ldy + j] = sum;
}

int launch_matmul_seq(b200q_ctx* ctx, const b200q_weight* w, const float* d_x, int64_t ldx, float* d_y, int64_t ldy, int m) {
    int64_t total = w->n_local * (int64_t)m;
    if (total == 0) return B200Q_OK;
    int64_t grid = (total + 127) / 128;
    if (grid > 0x7FFFFFFF) return fail(B200Q_ERR_INVALID, "matmul: too many outputs for one launch");
    switch (w->fmt) {
#define X(F)                                                                                                        \
    case F:                                                                                                         \
        matmul_seq_kernel<F><<<(unsigned)grid, 128, 0, ctx->stream>>>(w->view, d_x, ldx, d_y, ldy, w->n_local, w->k, m, \
                                                                      w->orient == B200Q_ORIENT_KN);                \
        break;
        B200Q_FOR_EACH_FMT(X)
#undef X
        default: return fail(B200Q_ERR_INVALID, "matmul: unknown format %d", w->fmt);
    }
    B200Q_CUDA(cudaGetLastError(), B200Q_ERR_LAUNCH);
    return B200Q_OK;
}

// ---------------------------------------------------------------------------------------------
__global__ void bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ in, int64_t ld_in, float* __restrict__ out,
                                   int64_t ld_out, int rows, int64_t cols) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)rows * cols) return;
    int64_t r = i / cols, c = i % cols;
    out[r * ld_out + c] = __bfloat162float(in[r * ld_in + c]);
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ in, int64_t ld_in, __nv_bfloat16* __restrict__ out,
                                   int64_t ld_out, int rows, int64_t cols) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)rows * cols) return;
    int64_t r = i / cols, c = i % cols;
    out[r * ld_out + c] = __float2bfloat16_rn(in[r * ld_in + c]);
}

int launch_convert_bf16_to_f32(b200q_ctx* ctx, const void* d_in, int64_t ld_in, float* d_out, int64_t ld_out, int rows, int64_t cols) {
    int64_t total = (int64_t)rows * cols;
    if (total == 0) return B200Q_OK;
    bf16_to_f32_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(
        static_cast<const __nv_bfloat16*>(d_in), ld_in, d_out, ld_out, rows, cols);
    B200Q_CUDA(cudaGetLastError(), B200Q_ERR_LAUNCH);
    return B200Q_OK;
}

int launch_convert_f32_to_bf16(b200q_ctx* ctx, const float* d_in, int64_t ld_in, void* d_out, int64_t ld_out, int rows, int64_t cols) {
    int64_t total = (int64_t)rows * cols;
    if (total == 0) return B200Q_OK;
    f32_to_bf16_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(
        d_in, ld_in, static_cast<__nv_bfloat16*>(d_out), ld_out, rows, cols);
    B200Q_CUDA(cudaGetLastError(), B200Q_ERR_LAUNCH);
    return B200Q_OK;
}

}  // namespace b200q
