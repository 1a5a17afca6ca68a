// C ABI of the library (include/b200q.h): context, memory, upload, dequantise, matmul dispatch.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>
#include <math.h>
#include <stdlib.h>

#include <vector>

#include "common.cuh"
#include "gemv_i8.cuh"

namespace b200q {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int cuda_fail(int code, cudaError_t e, const char* what) {
    // a failed launch leaves a sticky "last error"; clear it so later calls report their own
    cudaGetLastError();
    if (e == cudaErrorMemoryAllocation) code = B200Q_ERR_ALLOC;
    return fail(code, "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
}

int ensure_scratch(b200q_ctx* ctx, size_t bytes, int which) {
    void** p = which == 0 ? &ctx->scratch : which == 1 ? &ctx->scratch2 : &ctx->scratch3;
    size_t* sz = which == 0 ? &ctx->scratch_bytes : which == 1 ? &ctx->scratch2_bytes : &ctx->scratch3_bytes;
    if (*sz >= bytes) return B200Q_OK;
    if (*p) {
        B200Q_CUDA(cudaStreamSynchronize(ctx->stream), B200Q_ERR_DEVICE);
        cudaFree(*p);
        *p = nullptr;
        *sz = 0;
    }
    size_t want = (bytes + (1u << 20) - 1) & ~((size_t)(1u << 20) - 1);
    B200Q_CUDA(cudaMalloc(p, want), B200Q_ERR_ALLOC);
    *sz = want;
    return B200Q_OK;
}

static bool valid_qtype(int q) { return q >= 0 && q < NUM_QTYPES; }
static bool valid_layout(int l) { return l == RF || l == GGUF; }

// Carve the planes of `n_blocks` blocks out of one allocation (256-byte aligned sub-allocations).
static size_t plane_layout(int fmt, int64_t n_blocks, size_t off[4]) {
    FmtInfo I = fmt_info(fmt);
    size_t total = 0;
    for (int j = 0; j < I.nplanes; j++) {
        off[j] = total;
        size_t sz = (size_t)n_blocks * I.plane_bytes[j] + 64;  // slack: vector loads may over-read a tail
        total += (sz + 255) & ~(size_t)255;
    }
    return total ? total : 256;
}

}  // namespace b200q

using namespace b200q;

extern "C" {

const char* b200q_last_error(void) { return g_err; }

int b200q_is_recoverable(int status) {
    return status == B200Q_ERR_ALLOC || status == B200Q_ERR_COPY || status == B200Q_ERR_LAUNCH ||
           status == B200Q_ERR_DEVICE || status == B200Q_ERR_TIMEOUT;
}

int b200q_init_on_stream(int device, void* cuda_stream, b200q_ctx** out) {
    if (!out) return fail(B200Q_ERR_INVALID, "init: out is null");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        return fail(B200Q_ERR_NO_DEVICE, "init: no CUDA device (%s)", e == cudaSuccess ? "count is 0" : cudaGetErrorString(e));
    }
    if (device < 0 || device >= count) return fail(B200Q_ERR_NO_DEVICE, "init: device %d of %d", device, count);
    B200Q_CUDA(cudaSetDevice(device), B200Q_ERR_INIT);
    b200q_ctx* ctx = new b200q_ctx();
    ctx->device = device;
    if (cuda_stream == (void*)(intptr_t)-1) {
        e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
        if (e != cudaSuccess) { delete ctx; return cuda_fail(B200Q_ERR_INIT, e, "cudaStreamCreate"); }
        ctx->own_stream = true;
    } else {
        ctx->stream = static_cast<cudaStream_t>(cuda_stream);
    }
    cudaEventCreate(&ctx->ev0);
    cudaEventCreate(&ctx->ev1);
    cudaDeviceProp p{};
    e = cudaGetDeviceProperties(&p, device);
    if (e != cudaSuccess) { b200q_destroy(ctx); return cuda_fail(B200Q_ERR_INIT, e, "cudaGetDeviceProperties"); }
    snprintf(ctx->info.name, sizeof(ctx->info.name), "%.127s", p.name);
    ctx->info.sm_count = p.multiProcessorCount;
    ctx->info.cc_major = p.major;
    ctx->info.cc_minor = p.minor;
    ctx->info.total_mem = p.totalGlobalMem;
    ctx->info.smem_per_block_optin = p.sharedMemPerBlockOptin;
    ctx->info.l2_bytes = p.l2CacheSize;
    if (p.major != 10) {
        int maj = p.major, min = p.minor;
        b200q_destroy(ctx);
        return fail(B200Q_ERR_INIT, "init: device is sm_%d%d; this library is built for sm_100a only", maj, min);
    }
    e = cudaMalloc(&ctx->d_status, sizeof(int) * 8);
    if (e != cudaSuccess) { b200q_destroy(ctx); return cuda_fail(B200Q_ERR_ALLOC, e, "cudaMalloc(status)"); }
    cudaMemsetAsync(ctx->d_status, 0, sizeof(int) * 8, ctx->stream);
    {
        void* hd = nullptr;
        if (cudaHostAlloc(&hd, sizeof(int) * 4, cudaHostAllocMapped) == cudaSuccess) {
            void* dd = nullptr;
            if (cudaHostGetDevicePointer(&dd, hd, 0) == cudaSuccess) {
                memset(hd, 0, sizeof(int) * 4);
                ctx->h_done = static_cast<volatile int*>(hd);
                ctx->d_done = static_cast<int*>(dd);
            } else {
                cudaFreeHost(hd);
            }
        }
        cudaGetLastError();   // without the word the host-buffer path synchronises the stream as before
    }
    e = cudaHostAlloc(reinterpret_cast<void**>(&ctx->h_status), sizeof(int) * 4, cudaHostAllocDefault);
    if (e != cudaSuccess) { b200q_destroy(ctx); return cuda_fail(B200Q_ERR_ALLOC, e, "cudaHostAlloc(status)"); }
    *out = ctx;
    return B200Q_OK;
}

int b200q_init(int device, b200q_ctx** out) { return b200q_init_on_stream(device, (void*)(intptr_t)-1, out); }

void b200q_destroy(b200q_ctx* ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->scratch2) cudaFree(ctx->scratch2);
    if (ctx->scratch3) cudaFree(ctx->scratch3);
    if (ctx->sk_ws) cudaFree(ctx->sk_ws);
    if (ctx->d_status) cudaFree(ctx->d_status);
    if (ctx->h_status) cudaFreeHost(ctx->h_status);
    if (ctx->h_done) cudaFreeHost(const_cast<int*>(ctx->h_done));
    if (ctx->ev0) cudaEventDestroy(ctx->ev0);
    if (ctx->ev1) cudaEventDestroy(ctx->ev1);
    if (ctx->own_stream && ctx->stream) cudaStreamDestroy(ctx->stream);
    cudaGetLastError();
    delete ctx;
}

#define CTX_GUARD(name)                                              \
    if (!ctx) return fail(B200Q_ERR_INVALID, name ": ctx is null");  \
    B200Q_CUDA(cudaSetDevice(ctx->device), B200Q_ERR_DEVICE)

int b200q_get_device_info(b200q_ctx* ctx, b200q_device_info* out) {
    CTX_GUARD("get_device_info");
    if (!out) return fail(B200Q_ERR_INVALID, "get_device_info: out is null");
    size_t fr = 0, tot = 0;
    B200Q_CUDA(cudaMemGetInfo(&fr, &tot), B200Q_ERR_DEVICE);
    *out = ctx->info;
    out->free_mem = fr;
    out->total_mem = tot;
    return B200Q_OK;
}

int b200q_malloc(b200q_ctx* ctx, size_t bytes, void** d_out) {
    CTX_GUARD("malloc");
    if (!d_out) return fail(B200Q_ERR_INVALID, "malloc: d_out is null");
    *d_out = nullptr;
    if (bytes == 0) bytes = 1;
    B200Q_CUDA(cudaMalloc(d_out, bytes), B200Q_ERR_ALLOC);
    return B200Q_OK;
}

int b200q_free(b200q_ctx* ctx, void* d_ptr) {
    CTX_GUARD("free");
    if (!d_ptr) return B200Q_OK;
    B200Q_CUDA(cudaStreamSynchronize(ctx->stream), B200Q_ERR_DEVICE);
    B200Q_CUDA(cudaFree(d_ptr), B200Q_ERR_DEVICE);
    return B200Q_OK;
}

int b200q_memcpy_h2d(b200q_ctx* ctx, void* d_dst, const void* h_src, size_t bytes) {
    CTX_GUARD("memcpy_h2d");
    if (bytes == 0) return B200Q_OK;
    if (!d_dst || !h_src) return fail(B200Q_ERR_INVALID, "memcpy_h2d: null pointer");
    B200Q_CUDA(cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, ctx->stream), B200Q_ERR_COPY);
    B200Q_CUDA(cudaStreamSynchronize(ctx->stream), B200Q_ERR_COPY);
    return B200Q_OK;
}

int b200q_memcpy_d2h(b200q_ctx* ctx, void* h_dst, const void* d_src, size_t bytes) {
    CTX_GUARD("memcpy_d2h");
    if (bytes == 0) return B200Q_OK;
    if (!h_dst || !d_src) return fail(B200Q_ERR_INVALID, "memcpy_d2h: null pointer");
    B200Q_CUDA(cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, ctx->stream), B200Q_ERR_COPY);
    if (ctx->tc_pending) {   // a caller that fetches results this way must still learn of an expired device-side wait
        ctx->tc_pending = false;
        return gemm_tc_check_status(ctx);
    }
    B200Q_CUDA(cudaStreamSynchronize(ctx->stream), B200Q_ERR_COPY);
    return B200Q_OK;
}

int b200q_memset(b200q_ctx* ctx, void* d_dst, int value, size_t bytes) {
    CTX_GUARD("memset");
    if (bytes == 0) return B200Q_OK;
    if (!d_dst) return fail(B200Q_ERR_INVALID, "memset: null pointer");
    B200Q_CUDA(cudaMemsetAsync(d_dst, value, bytes, ctx->stream), B200Q_ERR_COPY);
    return B200Q_OK;
}

int b200q_synchronize(b200q_ctx* ctx) {
    CTX_GUARD("synchronize");
    if (ctx->tc_pending) {   // kernels that can report through the status words ran: read them behind the work
        ctx->tc_pending = false;
        return gemm_tc_check_status(ctx);
    }
    B200Q_CUDA(cudaStreamSynchronize(ctx->stream), B200Q_ERR_DEVICE);
    return B200Q_OK;
}

int b200q_selftest_bounded_wait(b200q_ctx* ctx, int64_t budget_cycles) {
    CTX_GUARD("selftest_bounded_wait");
    if (budget_cycles < 1 || budget_cycles > (1ll << 31))
        return fail(B200Q_ERR_INVALID, "selftest_bounded_wait: budget %lld outside 1..2^31 cycles", (long long)budget_cycles);
    int rc = launch_bounded_wait_selftest(ctx, budget_cycles);
    if (rc == B200Q_OK) ctx->tc_pending = true;
    return rc;
}

void* b200q_stream(b200q_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

int b200q_timer_start(b200q_ctx* ctx) {
    CTX_GUARD("timer_start");
    B200Q_CUDA(cudaEventRecord(ctx->ev0, ctx->stream), B200Q_ERR_DEVICE);
    return B200Q_OK;
}

int b200q_timer_stop_ms(b200q_ctx* ctx, float* ms_out) {
    CTX_GUARD("timer_stop_ms");
    B200Q_CUDA(cudaEventRecord(ctx->ev1, ctx->stream), B200Q_ERR_DEVICE);
    B200Q_CUDA(cudaEventSynchronize(ctx->ev1), B200Q_ERR_DEVICE);
    float ms = 0;
    B200Q_CUDA(cudaEventElapsedTime(&ms, ctx->ev0, ctx->ev1), B200Q_ERR_DEVICE);
    if (ms_out) *ms_out = ms;
    return B200Q_OK;
}

int b200q_block_elems(int qtype) { return valid_qtype(qtype) ? fmt_info(fmt_of(qtype, 0)).block_elems : 0; }

size_t b200q_block_bytes(int qtype, int layout) {
    return (valid_qtype(qtype) && valid_layout(layout)) ? (size_t)fmt_info(fmt_of(qtype, layout)).block_bytes : 0;
}

size_t b200q_tensor_bytes(int qtype, int layout, int64_t n_elements) {
    if (!valid_qtype(qtype) || !valid_layout(layout) || n_elements < 0) return 0;
    FmtInfo I = fmt_info(fmt_of(qtype, layout));
    return (size_t)((n_elements + I.block_elems - 1) / I.block_elems) * I.block_bytes;
}

static float half_bits_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 31u, man = h & 1023u;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            int e = -1;
            uint32_t mm = man;
            do { mm <<= 1; e++; } while (!(mm & 1024u));
            bits = sign | ((uint32_t)(112 - e) << 23) | ((mm & 1023u) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
    else bits = sign | ((exp + 112u) << 23) | (man << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

// Scan of the block scales in the file bytes (GGUF layouts with a tensor-core prefill kernel). The prefill kernels
// hold weights as f16: `weights_ok` says every weight fits the f16 range (and the largest block is not lost to
// underflow), `scales_ok` the same for the products "scale x sub-scale" the tensor-memory kernels' converters form
// in f16. A tensor that fails takes the next more careful kernel; one that fails both is multiplied by the fp32
// decode kernels, eight activation rows at a time.
static void scan_f16_ranges(int fmt, const uint8_t* blocks, int64_t n_blocks, bool* scales_ok, bool* weights_ok) {
    *scales_ok = *weights_ok = true;
    auto ld16h = [](const uint8_t* p) { return half_bits_to_float((uint16_t)(p[0] | (p[1] << 8))); };
    auto mag = [](float d) { return d != d ? INFINITY : (d < 0 ? -d : d); };
    FmtInfo I = fmt_info(fmt);
    // per block: s = the f16 (or power-of-two) scale; the format's largest "s x sub-scale" and largest weight follow
    float sub = 0.f, top = 0.f;   // multipliers of s
    switch (fmt) {
        case fmt_of(MXFP4, GGUF): sub = 1.f; top = 12.f; break;        // s = 2^(E-127) / 2, codes are 2 x value
        case fmt_of(MXFP6_E2M3, GGUF): sub = 8.f; top = 7.5f; break;    // the prefill converter forms (8 x value) x (s / 8)
        case fmt_of(MXFP6_E3M2, GGUF): sub = 4096.f; top = 28.f; break; // the prefill converter forms (value / 4096) x (4096 s)
        case fmt_of(Q4_K, GGUF): sub = 63.f; top = 63.f * 16.f; break; // d sc q - dmin m
        case fmt_of(Q5_K, GGUF): sub = 63.f; top = 63.f * 32.f; break;
        case fmt_of(Q6_K, GGUF): sub = 128.f; top = 128.f * 32.f; break;
        case fmt_of(Q8_0, GGUF): sub = 128.f; top = 128.f; break;
        case fmt_of(Q4_0, GGUF): sub = 8.f; top = 8.f; break;
        case fmt_of(Q3_K, GGUF): sub = 32.f; top = 32.f * 4.f; break;  // d (sc - 32) (q - 4)
        case fmt_of(Q2_K, GGUF): sub = 15.f; top = 15.f * 4.f; break;  // d sc q - dmin m, q <= 3
        default: return;
    }
    float smax = 0.f;
    bool small_block = false;   // MXFP6: a block with codes and a scale below 2^-21 (E2M3) / 2^-20 (E3M2): its f16 products would round
    for (int64_t b = 0; b < n_blocks; b++) {
        const uint8_t* p = blocks + b * I.block_bytes;
        float s;
        if ((fmt == fmt_of(MXFP6_E2M3, GGUF) && p[0] < 106) || (fmt == fmt_of(MXFP6_E3M2, GGUF) && p[0] < 107)) {
            for (int j = 1; j < 25 && !small_block; j++) small_block = p[j] != 0;
        }
        switch (fmt) {
            case fmt_of(MXFP4, GGUF): s = p[0] == 255 ? INFINITY : ldexpf(0.5f, (int)p[0] - 127); break;
            case fmt_of(MXFP6_E2M3, GGUF):
            case fmt_of(MXFP6_E3M2, GGUF): s = p[0] == 255 ? INFINITY : ldexpf(1.0f, (int)p[0] - 127); break;
            case fmt_of(Q4_K, GGUF):
            case fmt_of(Q5_K, GGUF): s = fmaxf(mag(ld16h(p)), mag(ld16h(p + 2))); break;
            case fmt_of(Q6_K, GGUF): s = mag(ld16h(p + 208)); break;
            case fmt_of(Q3_K, GGUF): s = mag(ld16h(p + 108)); break;
            case fmt_of(Q2_K, GGUF): s = fmaxf(mag(ld16h(p + 80)), mag(ld16h(p + 82))); break;
            default: s = mag(ld16h(p)); break;
        }
        if (s > smax) smax = s;
    }
    if (!(smax * sub <= 60000.f) || smax * sub < 6.2e-5f) *scales_ok = false;
    if (!(smax * top <= 60000.f) || smax < 6.2e-5f) *weights_ok = false;
    if (small_block) *scales_ok = false;
    if (smax == 0.f) *scales_ok = *weights_ok = true;   // an all-zero tensor is exact on every path
}

// Allocates the planes for n_blocks blocks, copies `avail` bytes of file blocks from the host (zero
// filling the rest) and splits them into planes. Used by upload and by dequantize_bytes.
// With `place` (plane_layout() bytes inside an arena) and `stage_buf` (room for the file blocks) nothing is allocated
// and the stream is not synchronised: copies and kernels of consecutive tensors queue up behind one another.
static int make_planes(b200q_ctx* ctx, int fmt, const uint8_t* h_bytes, size_t avail, int64_t n_blocks, void** base_out,
                       WView* view_out, uint8_t* place = nullptr, void* stage_buf = nullptr) {
    FmtInfo I = fmt_info(fmt);
    size_t off[4] = {0, 0, 0, 0};
    size_t total = plane_layout(fmt, n_blocks, off);
    void* base = place;
    if (!place) B200Q_CUDA(cudaMalloc(&base, total), B200Q_ERR_ALLOC);
    WView v{};
    for (int j = 0; j < I.nplanes; j++) v.p[j] = static_cast<uint8_t*>(base) + off[j];
    size_t raw_bytes = (size_t)n_blocks * I.block_bytes;
    if (avail > raw_bytes) avail = raw_bytes;
    cudaError_t e = cudaSuccess;
    int rc = B200Q_OK;
    if (I.nplanes == 1) {
        // the file layout is the device layout
        e = cudaMemsetAsync(static_cast<uint8_t*>(base) + avail, 0, total - avail, ctx->stream);
        if (e == cudaSuccess && avail) e = cudaMemcpyAsync(base, h_bytes, avail, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess && !place) e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) rc = cuda_fail(B200Q_ERR_COPY, e, "upload copy");
    } else {
        void* stage = stage_buf;
        if (!stage) e = cudaMalloc(&stage, raw_bytes ? raw_bytes : 1);
        if (e != cudaSuccess) {
            if (!place) cudaFree(base);
            return cuda_fail(B200Q_ERR_ALLOC, e, "upload staging");
        }
        e = cudaMemsetAsync(base, 0, total, ctx->stream);
        if (e == cudaSuccess && avail < raw_bytes)
            e = cudaMemsetAsync(static_cast<uint8_t*>(stage) + avail, 0, raw_bytes - avail, ctx->stream);
        if (e == cudaSuccess && avail) e = cudaMemcpyAsync(stage, h_bytes, avail, cudaMemcpyHostToDevice, ctx->stream);
        if (e != cudaSuccess) rc = cuda_fail(B200Q_ERR_COPY, e, "upload copy");
        if (rc == B200Q_OK) rc = launch_repack(ctx, fmt, static_cast<const uint8_t*>(stage), n_blocks, v);
        if (!stage_buf) {
            e = cudaStreamSynchronize(ctx->stream);
            if (rc == B200Q_OK && e != cudaSuccess) rc = cuda_fail(B200Q_ERR_DEVICE, e, "upload repack");
            cudaFree(stage);
        }
    }
    if (rc != B200Q_OK) {
        if (!place) cudaFree(base);
        return rc;
    }
    *base_out = base;
    *view_out = v;
    return B200Q_OK;
}

static size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

static bool image_enabled() {
    const char* no_img = getenv("B200Q_NO_DECODE_IMAGE");
    return !(no_img && no_img[0] == '1');
}

static int weight_upload_impl(b200q_ctx* ctx, b200q_arena* arena, const void* h_bytes, size_t nbytes, int qtype, int layout, int orient,
                              int64_t n, int64_t k, int shard_rank, int shard_count, b200q_weight** out) {
    CTX_GUARD("weight_upload");
    if (!out) return fail(B200Q_ERR_INVALID, "weight_upload: out is null");
    *out = nullptr;
    if (!valid_qtype(qtype) || !valid_layout(layout)) return fail(B200Q_ERR_INVALID, "weight_upload: unknown qtype %d / layout %d", qtype, layout);
    if (orient != B200Q_ORIENT_NK && orient != B200Q_ORIENT_KN) return fail(B200Q_ERR_INVALID, "weight_upload: unknown orientation %d", orient);
    if (n <= 0 || k <= 0) return fail(B200Q_ERR_INVALID, "weight_upload: n=%lld k=%lld must be positive", (long long)n, (long long)k);
    if (!h_bytes) return fail(B200Q_ERR_INVALID, "weight_upload: h_bytes is null");
    if (shard_count < 1 || shard_rank < 0 || shard_rank >= shard_count)
        return fail(B200Q_ERR_INVALID, "weight_upload: shard %d of %d", shard_rank, shard_count);
    int fmt = fmt_of(qtype, layout);
    FmtInfo I = fmt_info(fmt);
    size_t need = b200q_tensor_bytes(qtype, layout, n * k);
    // same check as execute_matmul_q4_0 (src/ggml/hip_backend/op_dispatch.rs:973-979): byte count must match the shape
    if (nbytes != need)
        return fail(B200Q_ERR_INVALID, "weight_upload: %zu bytes given, %lld x %lld weights need %zu", nbytes, (long long)n, (long long)k, need);
    int64_t row0 = 0, n_local = n;
    if (shard_count > 1) {
        if (orient != B200Q_ORIENT_NK) return fail(B200Q_ERR_UNSUPPORTED, "weight_upload: only NK tensors can be sharded by output feature");
        if (n % shard_count) return fail(B200Q_ERR_INVALID, "weight_upload: n=%lld does not divide into %d shards", (long long)n, shard_count);
        n_local = n / shard_count;
        row0 = n_local * shard_rank;
        if ((n_local * k) % I.block_elems)
            return fail(B200Q_ERR_INVALID, "weight_upload: a shard of %lld rows x %lld does not end on a %d-weight block", (long long)n_local, (long long)k, I.block_elems);
    }
    int64_t n_el = n_local * k;
    int64_t n_blocks = (n_el + I.block_elems - 1) / I.block_elems;
    const uint8_t* src = static_cast<const uint8_t*>(h_bytes) + (size_t)((row0 * k) / I.block_elems) * I.block_bytes;
    b200q_weight* w = new b200q_weight();
    w->ctx = ctx;
    w->qtype = qtype; w->layout = layout; w->orient = orient; w->fmt = fmt;
    w->n_local = n_local; w->k = k; w->row0 = row0; w->n_total = n;
    w->n_elements = n_el; w->n_blocks = n_blocks;
    w->packed_bytes = (size_t)n_blocks * I.block_bytes;
    if (layout == GGUF) scan_f16_ranges(fmt, src, n_blocks, &w->f16_scales_ok, &w->f16_weights_ok);
    else w->range_scanned = false;   // f32 and per-sub-block scales: the weights themselves are scanned, on the device, on first use
    const bool image = image_enabled() && decode_image_wanted(fmt, orient, n_local, k);
    uint8_t *place = nullptr, *img_place = nullptr;
    if (arena) {
        // bump allocation, 256-byte aligned (ModelWeightArena, src/memory/arena.rs:82,206); the staging buffer grows to
        // the largest tensor seen (a growth waits for the copies queued on the old one)
        size_t off[4];
        const size_t planes = align256(plane_layout(fmt, n_blocks, off));
        const size_t img = image ? align256(decode_image_bytes(fmt, n_local, k)) : 0;
        if (arena->used + planes + img > arena->capacity) {
            delete w;
            return fail(B200Q_ERR_ALLOC, "arena_upload: tensor needs %zu bytes, arena has %zu of %zu left", planes + img,
                        arena->capacity - arena->used, arena->capacity);
        }
        if (I.nplanes > 1 && arena->stage_bytes < w->packed_bytes) {
            cudaStreamSynchronize(ctx->stream);
            if (arena->stage) cudaFree(arena->stage);
            arena->stage = nullptr;
            arena->stage_bytes = 0;
            cudaError_t e = cudaMalloc(&arena->stage, w->packed_bytes);
            if (e != cudaSuccess) { delete w; return cuda_fail(B200Q_ERR_ALLOC, e, "arena staging"); }
            arena->stage_bytes = w->packed_bytes;
        }
        place = arena->base + arena->used;
        img_place = image ? place + planes : nullptr;
        arena->used += planes + img;
    }
    int rc = make_planes(ctx, fmt, src, w->packed_bytes, n_blocks, &w->base, &w->view, place, arena ? arena->stage : nullptr);
    if (rc != B200Q_OK) { delete w; return rc; }
    // second, decode-ordered copy for the m <= 8 kernel (B200Q_NO_DECODE_IMAGE=1 keeps only the stream layout)
    if (image) {
        rc = build_decode_image(ctx, w, &w->dimg, img_place);
        if (rc != B200Q_OK) { if (!arena) cudaFree(w->base); delete w; return rc; }
    }
    if (arena) {
        w->arena = arena;
        arena->tensors++;
        arena->live++;
    }
    *out = w;
    return B200Q_OK;
}

int b200q_weight_upload(b200q_ctx* ctx, const void* h_bytes, size_t nbytes, int qtype, int layout, int orient,
                        int64_t n, int64_t k, int shard_rank, int shard_count, b200q_weight** out) {
    return weight_upload_impl(ctx, nullptr, h_bytes, nbytes, qtype, layout, orient, n, k, shard_rank, shard_count, out);
}

int b200q_arena_tensor_bytes(int qtype, int layout, int orient, int64_t n_local, int64_t k, size_t* bytes) {
    if (!bytes) return fail(B200Q_ERR_INVALID, "arena_tensor_bytes: bytes is null");
    if (!valid_qtype(qtype) || !valid_layout(layout) || n_local <= 0 || k <= 0)
        return fail(B200Q_ERR_INVALID, "arena_tensor_bytes: qtype %d / layout %d / %lld x %lld", qtype, layout, (long long)n_local, (long long)k);
    const int fmt = fmt_of(qtype, layout);
    FmtInfo I = fmt_info(fmt);
    const int64_t n_blocks = (n_local * k + I.block_elems - 1) / I.block_elems;
    size_t off[4];
    size_t total = align256(plane_layout(fmt, n_blocks, off));
    if (image_enabled() && decode_image_wanted(fmt, orient, n_local, k)) total += align256(decode_image_bytes(fmt, n_local, k));
    *bytes = total;
    return B200Q_OK;
}

int b200q_arena_create(b200q_ctx* ctx, size_t capacity, b200q_arena** out) {
    CTX_GUARD("arena_create");
    if (!out) return fail(B200Q_ERR_INVALID, "arena_create: out is null");
    *out = nullptr;
    if (capacity == 0) return fail(B200Q_ERR_INVALID, "arena_create: capacity is 0");
    b200q_arena* a = new b200q_arena();
    a->ctx = ctx;
    a->capacity = align256(capacity);
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, a->capacity);
    if (e != cudaSuccess) {
        delete a;
        return cuda_fail(B200Q_ERR_ALLOC, e, "arena_create");
    }
    a->base = static_cast<uint8_t*>(p);
    *out = a;
    return B200Q_OK;
}

int b200q_arena_upload(b200q_ctx* ctx, b200q_arena* arena, const void* h_bytes, size_t nbytes, int qtype, int layout, int orient,
                       int64_t n, int64_t k, int shard_rank, int shard_count, b200q_weight** out) {
    if (!arena) return fail(B200Q_ERR_INVALID, "arena_upload: arena is null");
    if (ctx && arena->ctx != ctx) return fail(B200Q_ERR_INVALID, "arena_upload: the arena belongs to another context");
    return weight_upload_impl(ctx, arena, h_bytes, nbytes, qtype, layout, orient, n, k, shard_rank, shard_count, out);
}

int b200q_arena_info(const b200q_arena* arena, size_t* capacity, size_t* used, int64_t* tensors, int64_t* live) {
    if (!arena) return fail(B200Q_ERR_INVALID, "arena_info: arena is null");
    if (capacity) *capacity = arena->capacity;
    if (used) *used = arena->used;
    if (tensors) *tensors = arena->tensors;
    if (live) *live = arena->live;
    return B200Q_OK;
}

int b200q_arena_free(b200q_arena* arena) {
    if (!arena) return B200Q_OK;
    if (arena->live != 0) return fail(B200Q_ERR_INVALID, "arena_free: %lld weight handles of this arena are still alive", (long long)arena->live);
    cudaSetDevice(arena->ctx->device);
    cudaStreamSynchronize(arena->ctx->stream);
    if (arena->stage) cudaFree(arena->stage);
    cudaFree(arena->base);
    cudaGetLastError();
    delete arena;
    return B200Q_OK;
}

int b200q_weight_free(b200q_weight* w) {
    if (!w) return B200Q_OK;
    b200q_ctx* ctx = w->ctx;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (w->mx_sfa) cudaFree(w->mx_sfa);
    if (w->q6_planes) cudaFree(w->q6_planes);
    if (w->pimg.base) cudaFree(w->pimg.base);
    if (w->arena) {
        w->arena->live--;   // the memory goes back with the arena
    } else {
        cudaFree(w->base);
        if (w->dimg.base) cudaFree(w->dimg.base);
    }
    cudaGetLastError();
    delete w;
    return B200Q_OK;
}

int b200q_weight_info(const b200q_weight* w, int* qtype, int* layout, int* orient, int64_t* n_local, int64_t* k,
                      int64_t* row0, int64_t* n_total, size_t* packed_bytes) {
    if (!w) return fail(B200Q_ERR_INVALID, "weight_info: handle is null");
    if (qtype) *qtype = w->qtype;
    if (layout) *layout = w->layout;
    if (orient) *orient = w->orient;
    if (n_local) *n_local = w->n_local;
    if (k) *k = w->k;
    if (row0) *row0 = w->row0;
    if (n_total) *n_total = w->n_total;
    if (packed_bytes) *packed_bytes = w->packed_bytes;
    return B200Q_OK;
}

int b200q_dequantize(b200q_ctx* ctx, const b200q_weight* w, float* d_out, int64_t n_elements) {
    CTX_GUARD("dequantize");
    if (!w) return fail(B200Q_ERR_INVALID, "dequantize: weight handle is null");
    if (w->ctx->device != ctx->device) return fail(B200Q_ERR_INVALID, "dequantize: weight lives on device %d, ctx on %d", w->ctx->device, ctx->device);
    if (n_elements < 0 || n_elements > w->n_elements)
        return fail(B200Q_ERR_INVALID, "dequantize: %lld elements asked, tensor holds %lld", (long long)n_elements, (long long)w->n_elements);
    if (n_elements == 0) return B200Q_OK;
    if (!d_out) return fail(B200Q_ERR_INVALID, "dequantize: d_out is null");
    return launch_dequant(ctx, w->fmt, w->view, d_out, n_elements, (int64_t)w->packed_bytes);
}

int b200q_fused_dequant_rmsnorm(b200q_ctx* ctx, const b200q_weight* w, const float* d_norm_weight, float* d_out, float eps) {
    CTX_GUARD("fused_dequant_rmsnorm");
    if (!w) return fail(B200Q_ERR_INVALID, "fused_dequant_rmsnorm: weight handle is null");
    if (w->ctx->device != ctx->device) return fail(B200Q_ERR_INVALID, "fused_dequant_rmsnorm: tensor lives on device %d, ctx on %d", w->ctx->device, ctx->device);
    if (w->orient != B200Q_ORIENT_NK) return fail(B200Q_ERR_UNSUPPORTED, "fused_dequant_rmsnorm: needs a tensor stored as rows of hidden_size values");
    if (w->k % 8 || w->k > 0x7FFFFFF8ll) return fail(B200Q_ERR_UNSUPPORTED, "fused_dequant_rmsnorm: hidden_size %lld must be a multiple of 8", (long long)w->k);
    if (!d_norm_weight || !d_out) return fail(B200Q_ERR_INVALID, "fused_dequant_rmsnorm: null device pointer");
    if ((reinterpret_cast<uintptr_t>(d_norm_weight) & 15) || (reinterpret_cast<uintptr_t>(d_out) & 15))
        return fail(B200Q_ERR_INVALID, "fused_dequant_rmsnorm: weight and output must be 16-byte aligned");
    return launch_fused_dequant_rmsnorm(ctx, w->fmt, w->view, d_norm_weight, d_out, w->n_local, (int)w->k, eps);
}

int b200q_get_rows(b200q_ctx* ctx, const b200q_weight* w, const int32_t* d_ids, int64_t n_ids, float* d_out, int64_t ldo) {
    CTX_GUARD("get_rows");
    if (!w) return fail(B200Q_ERR_INVALID, "get_rows: weight handle is null");
    if (w->ctx->device != ctx->device) return fail(B200Q_ERR_INVALID, "get_rows: tensor lives on device %d, ctx on %d", w->ctx->device, ctx->device);
    if (w->orient != B200Q_ORIENT_NK) return fail(B200Q_ERR_UNSUPPORTED, "get_rows: needs a table stored as rows of n_embd values");
    if (w->k % 8 || w->k > 0x7FFFFFF8ll) return fail(B200Q_ERR_UNSUPPORTED, "get_rows: n_embd %lld must be a multiple of 8", (long long)w->k);
    if (n_ids < 0) return fail(B200Q_ERR_INVALID, "get_rows: negative token count");
    if (n_ids == 0) return B200Q_OK;
    if (!d_ids || !d_out) return fail(B200Q_ERR_INVALID, "get_rows: null device pointer");
    if (ldo < w->k || (ldo % 4) || (reinterpret_cast<uintptr_t>(d_out) & 15))
        return fail(B200Q_ERR_INVALID, "get_rows: output rows must be 16-byte aligned and at least n_embd wide");
    ctx->tc_pending = true;   // the next synchronize reads the status words
    return launch_get_rows(ctx, w->fmt, w->view, d_ids, n_ids, d_out, ldo, (int)w->k, w->n_local);
}

int b200q_get_rows_host(b200q_ctx* ctx, const b200q_weight* w, const uint32_t* h_ids, int64_t n_ids, float* d_out, int64_t ldo) {
    CTX_GUARD("get_rows_host");
    if (!w) return fail(B200Q_ERR_INVALID, "get_rows: weight handle is null");
    if (n_ids < 0) return fail(B200Q_ERR_INVALID, "get_rows: negative token count");
    if (n_ids == 0) return B200Q_OK;
    if (!h_ids) return fail(B200Q_ERR_INVALID, "get_rows: token ids are null");
    for (int64_t i = 0; i < n_ids; i++)   // validate_token_ids: nothing is launched for a bad id
        if ((int64_t)h_ids[i] >= w->n_local)
            return fail(B200Q_ERR_INVALID, "Token ID %u exceeds vocab size %lld", h_ids[i], (long long)w->n_local);
    int rc = ensure_scratch(ctx, (size_t)n_ids * sizeof(int32_t), 0);
    if (rc != B200Q_OK) return rc;
    B200Q_CUDA(cudaMemcpyAsync(ctx->scratch, h_ids, (size_t)n_ids * sizeof(int32_t), cudaMemcpyHostToDevice, ctx->stream), B200Q_ERR_COPY);
    rc = b200q_get_rows(ctx, w, static_cast<const int32_t*>(ctx->scratch), n_ids, d_out, ldo);
    if (rc != B200Q_OK) return rc;
    return b200q_synchronize(ctx);   // the ids are pageable host memory: the call returns when they have been read
}

int b200q_dequantize_bytes(b200q_ctx* ctx, const void* h_bytes, size_t nbytes, int qtype, int layout, float* d_out,
                           int64_t n_elements) {
    CTX_GUARD("dequantize_bytes");
    if (!valid_qtype(qtype) || !valid_layout(layout)) return fail(B200Q_ERR_INVALID, "dequantize_bytes: unknown qtype %d / layout %d", qtype, layout);
    if (n_elements < 0) return fail(B200Q_ERR_INVALID, "dequantize_bytes: negative element count");
    if (n_elements == 0) return B200Q_OK;
    if (!d_out) return fail(B200Q_ERR_INVALID, "dequantize_bytes: d_out is null");
    if (!h_bytes && nbytes) return fail(B200Q_ERR_INVALID, "dequantize_bytes: h_bytes is null");
    int fmt = fmt_of(qtype, layout);
    FmtInfo I = fmt_info(fmt);
    int64_t n_blocks = (n_elements + I.block_elems - 1) / I.block_elems;
    void* base = nullptr;
    WView v{};
    int rc = make_planes(ctx, fmt, static_cast<const uint8_t*>(h_bytes), nbytes, n_blocks, &base, &v);
    if (rc != B200Q_OK) return rc;
    rc = launch_dequant(ctx, fmt, v, d_out, n_elements, (int64_t)nbytes);
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    cudaFree(base);
    if (rc != B200Q_OK) return rc;
    if (e != cudaSuccess) return cuda_fail(B200Q_ERR_DEVICE, e, "dequantize_bytes");
    return B200Q_OK;
}

}  // extern "C"
