// Dequantise-to-fp32 kernels and the upload-time plane split.
//
// Replaces kernels/q4_0_dequant.hip:72, q8_0_dequant.hip:40, q4_k_dequant.hip:81, q6_k_dequant.hip:82 and
// mxfp_dequant.hip:85,147 of the reference (one thread per ELEMENT there). Here one thread decodes 8
// consecutive weights and writes one 32-byte sector, so a warp writes 1 KB of contiguous fp32: the
// kernel is bound by the 4 B/weight it writes to HBM.
#include "common.cuh"

#include <algorithm>

namespace b200q {

template <int F>
__global__ void __launch_bounds__(256) dequant_kernel(WView v, float* __restrict__ out, int64_t n, int64_t valid_bytes) {
    int64_t piece = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t e0 = piece * 8;
    if (e0 >= n) return;
    float w[8];
    decode8<F>(v, piece >> 2, (int)(piece & 3), w);
    if (need_end<F>(e0 + 7) > valid_bytes || need_end<F>(e0) > valid_bytes) {
        // the file stream ends inside or before this piece: uncovered elements stay 0.0
#pragma unroll
        for (int i = 0; i < 8; i++)
            if (need_end<F>(e0 + i) > valid_bytes) w[i] = 0.0f;
    }
    float* o = out + e0;
    if (e0 + 8 <= n && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
        reinterpret_cast<float4*>(o)[0] = make_float4(w[0], w[1], w[2], w[3]);
        reinterpret_cast<float4*>(o)[1] = make_float4(w[4], w[5], w[6], w[7]);
    } else {
#pragma unroll
        for (int i = 0; i < 8; i++)
            if (e0 + i < n) o[i] = w[i];
    }
}

int launch_dequant(b200q_ctx* ctx, int fmt, const WView& v, float* d_out, int64_t n, int64_t valid_bytes) {
    if (n <= 0) return B200Q_OK;
    int64_t pieces = (n + 7) / 8;
    int64_t grid = (pieces + 255) / 256;
    if (grid > 0x7FFFFFFF) return fail(B200Q_ERR_INVALID, "dequantize: tensor too large for one launch");
    switch (fmt) {
#define X(F) \
    case F: dequant_kernel<F><<<(unsigned)grid, 256, 0, ctx->stream>>>(v, d_out, n, valid_bytes); break;
        B200Q_FOR_EACH_FMT(X)
#undef X
        default: return fail(B200Q_ERR_INVALID, "dequantize: unknown format %d", fmt);
    }
    B200Q_CUDA(cudaGetLastError(), B200Q_ERR_LAUNCH);
    return B200Q_OK;
}

// Largest |weight| of a tensor, as float bits raised into *out with an atomic maximum (bits of non-negative floats
// order like the floats). NaN counts as infinity. The same decode8 as the dequantise kernel.
template <int F>
__global__ void __launch_bounds__(256) absmax_kernel(WView v, int64_t n, unsigned int* __restrict__ out) {
    const int64_t pieces = (n + 7) / 8;
    float mx = 0.0f;
    for (int64_t piece = (int64_t)blockIdx.x * 256 + threadIdx.x; piece < pieces; piece += (int64_t)gridDim.x * 256) {
        float w[8];
        decode8<F>(v, piece >> 2, (int)(piece & 3), w);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            if (piece * 8 + i < n) {
                const float a = fabsf(w[i]);
                mx = (a != a) ? INFINITY : fmaxf(mx, a);
            }
        }
    }
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    if ((threadIdx.x & 31) == 0) atomicMax(out, __float_as_uint(mx));
}

int launch_absmax(b200q_ctx* ctx, int fmt, const WView& v, int64_t n, unsigned int* d_out) {
    if (n <= 0) return B200Q_OK;
    const int64_t pieces = (n + 7) / 8;
    const unsigned grid = (unsigned)std::min<int64_t>((pieces + 255) / 256, 148 * 8);
    switch (fmt) {
#define X(F) \
    case F: absmax_kernel<F><<<grid, 256, 0, ctx->stream>>>(v, n, d_out); break;
        B200Q_FOR_EACH_FMT(X)
#undef X
        default: return fail(B200Q_ERR_INVALID, "absmax: unknown format %d", fmt);
    }
    B200Q_CUDA(cudaGetLastError(), B200Q_ERR_LAUNCH);
    return B200Q_OK;
}

// Fused dequantise + RMSNorm (replaces kernels/fused_dequant_rmsnorm.hip:87-165): one CTA per row of a packed
// [rows, hidden] tensor, every thread decodes 8 consecutive weights at a time (the same decode8 as everywhere
// else, so the normalised values start from bit-exact weights), sum of squares reduced by shuffles, then a
// second pass over the packed bytes (served by L1/L2) writes val * rsqrt(mean + eps) * weight as 32-byte
// sectors. The fp32 row never exists in memory; the kernel is bound by the 4 B/weight it writes.
template <int F>
__global__ void __launch_bounds__(256) fused_dequant_rmsnorm_kernel(WView v, const float* __restrict__ weight,
                                                                    float* __restrict__ out, int hidden, float eps) {
    const int64_t row = blockIdx.x;
    const int64_t piece0 = row * (hidden >> 3);
    float ss = 0.0f;
    for (int p = threadIdx.x; p < (hidden >> 3); p += 256) {
        float w[8];
        const int64_t piece = piece0 + p;
        decode8<F>(v, piece >> 2, (int)(piece & 3), w);
#pragma unroll
        for (int i = 0; i < 8; i++) ss = fmaf(w[i], w[i], ss);
    }
    __shared__ float red[8];
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) total += red[i];
    const float rms = 1.0f / sqrtf(__fadd_rn(__fdiv_rn(total, (float)hidden), eps));
    for (int p = threadIdx.x; p < (hidden >> 3); p += 256) {
        float w[8];
        const int64_t piece = piece0 + p;
        decode8<F>(v, piece >> 2, (int)(piece & 3), w);
        const float4 g0 = __ldg(reinterpret_cast<const float4*>(weight) + 2 * p);
        const float4 g1 = __ldg(reinterpret_cast<const float4*>(weight) + 2 * p + 1);
        float4* o = reinterpret_cast<float4*>(out + row * hidden) + 2 * p;
        o[0] = make_float4(w[0] * rms * g0.x, w[1] * rms * g0.y, w[2] * rms * g0.z, w[3] * rms * g0.w);
        o[1] = make_float4(w[4] * rms * g1.x, w[5] * rms * g1.y, w[6] * rms * g1.z, w[7] * rms * g1.w);
    }
}

int launch_fused_dequant_rmsnorm(b200q_ctx* ctx, int fmt, const WView& v, const float* d_weight, float* d_out, int64_t rows,
                                 int hidden, float eps) {
    if (rows <= 0) return B200Q_OK;
    if (rows > 0x7FFFFFFF) return fail(B200Q_ERR_INVALID, "fused_dequant_rmsnorm: too many rows for one launch");
    switch (fmt) {
#define X(F) \
    case F: fused_dequant_rmsnorm_kernel<F><<<(unsigned)rows, 256, 0, ctx->stream>>>(v, d_weight, d_out, hidden, eps); break;
        B200Q_FOR_EACH_FMT(X)
#undef X
        default: return fail(B200Q_ERR_INVALID, "fused_dequant_rmsnorm: unknown format %d", fmt);
    }
    B200Q_CUDA(cudaGetLastError(), B200Q_ERR_LAUNCH);
    return B200Q_OK;
}

// Quantised embedding lookup (the GetRows op on a packed token_embd, replaces the per-token device copies of
// src/ggml/hip_backend/ops/get_rows.rs:24-78 that need the table as fp32): one CTA per token id, the row is
// decoded with the same decode8 as everywhere else (bit-exact against the dequantised table) and written as
// 32-byte sectors. A token id outside [0, n_rows) never touches the table: its output row is zero-filled and
// the launch's status word counts it, so the host can report it the way validate_token_ids does.
template <int F>
__global__ void __launch_bounds__(256) get_rows_kernel(WView v, const int32_t* __restrict__ ids, float* __restrict__ out,
                                                       int64_t ldo, int hidden, int64_t n_rows, int* __restrict__ bad_ids) {
    const int64_t t = blockIdx.x;
    const int64_t id = ids[t];
    const bool valid = id >= 0 && id < n_rows;
    if (!valid && threadIdx.x == 0) atomicAdd(bad_ids, 1);
    const int64_t piece0 = (valid ? id : 0) * (hidden >> 3);
    for (int p = threadIdx.x; p < (hidden >> 3); p += 256) {
        float w[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
        const int64_t piece = piece0 + p;
        if (valid) decode8<F>(v, piece >> 2, (int)(piece & 3), w);
        float4* o = reinterpret_cast<float4*>(out + t * ldo) + 2 * p;
        o[0] = make_float4(w[0], w[1], w[2], w[3]);
        o[1] = make_float4(w[4], w[5], w[6], w[7]);
    }
}

int launch_get_rows(b200q_ctx* ctx, int fmt, const WView& v, const int32_t* d_ids, int64_t n_ids, float* d_out, int64_t ldo,
                    int hidden, int64_t n_rows) {
    if (n_ids <= 0) return B200Q_OK;
    if (n_ids > 0x7FFFFFFF) return fail(B200Q_ERR_INVALID, "get_rows: too many token ids for one launch");
    switch (fmt) {
#define X(F) \
    case F: get_rows_kernel<F><<<(unsigned)n_ids, 256, 0, ctx->stream>>>(v, d_ids, d_out, ldo, hidden, n_rows, ctx->d_status + 1); break;
        B200Q_FOR_EACH_FMT(X)
#undef X
        default: return fail(B200Q_ERR_INVALID, "get_rows: unknown format %d", fmt);
    }
    B200Q_CUDA(cudaGetLastError(), B200Q_ERR_LAUNCH);
    return B200Q_OK;
}

// File blocks (header and codes interleaved) -> planes. The block sizes are not word multiples, so
// this moves single bytes; it runs once per tensor at load time.
struct RepackArgs {
    uint8_t* dst[4];
    int plane_bytes[4];
    int plane_off[4];
    int nplanes;
    int block_bytes;
};

__global__ void __launch_bounds__(256) repack_kernel(const uint8_t* __restrict__ raw, int64_t total_bytes, RepackArgs a) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total_bytes) return;
    int64_t b = i / a.block_bytes;
    int o = (int)(i - b * a.block_bytes);
    int j = 0;
#pragma unroll
    for (int t = 1; t < 4; t++)
        if (t < a.nplanes && o >= a.plane_off[t]) j = t;
    a.dst[j][b * a.plane_bytes[j] + (o - a.plane_off[j])] = raw[i];
}

int launch_repack(b200q_ctx* ctx, int fmt, const uint8_t* d_raw, int64_t n_blocks, const WView& v) {
    FmtInfo I = fmt_info(fmt);
    RepackArgs a{};
    a.nplanes = I.nplanes;
    a.block_bytes = I.block_bytes;
    int off = 0;
    for (int j = 0; j < I.nplanes; j++) {
        a.dst[j] = const_cast<uint8_t*>(v.p[j]);
        a.plane_bytes[j] = I.plane_bytes[j];
        a.plane_off[j] = off;
        off += I.plane_bytes[j];
    }
    int64_t total = n_blocks * I.block_bytes;
    if (total == 0) return B200Q_OK;
    int64_t grid = (total + 255) / 256;
    if (grid > 0x7FFFFFFF) return fail(B200Q_ERR_INVALID, "upload: tensor too large for one repack launch");
    repack_kernel<<<(unsigned)grid, 256, 0, ctx->stream>>>(d_raw, total, a);
    B200Q_CUDA(cudaGetLastError(), B200Q_ERR_LAUNCH);
    return B200Q_OK;
}

}  // namespace b200q
