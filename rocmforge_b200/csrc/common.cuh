// Shared host-side declarations of the library: context, weight handle, error plumbing.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/b200q.h"
#include "formats.cuh"

struct b200q_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    b200q_device_info info{};
    // grow-only device scratch (activation conversion, host staging of matmul_host, split buffers)
    void* scratch = nullptr;
    size_t scratch_bytes = 0;
    void* scratch2 = nullptr;
    size_t scratch2_bytes = 0;
    int* d_status = nullptr;  // device words: [0] bounded-wait failures, [1] bad token ids, [2..4] counters of the decode kernel
    int* h_status = nullptr;  // page-locked landing place of [0..1] when a synchronise reads them
    // Completion word of launches whose results go straight to host memory: [0] the sequence number the kernel's
    // last CTA stores when every CTA's results are out, [1] the launch's status word (page-locked, device-mapped)
    volatile int* h_done = nullptr;
    int* d_done = nullptr;    // the same words as the device sees them
    int done_seq = 0;
    bool tc_pending = false;  // a tensor-core launch has not had its status word read yet
    void* scratch3 = nullptr; // f16 copy of the activations + row scales for the tensor-core path
    size_t scratch3_bytes = 0;
    // split-tile workspace of the persistent prefill kernel: one partial accumulator tile per CTA, then one
    // flag word per CTA; a flag holds the number of the launch that last published the slot
    void* sk_ws = nullptr;
    int sk_ctas = 0;
    int sk_epoch = 0;
    // while b200q_matmul_scatter runs: the same output slice in the other GPUs' full outputs (peer-mapped)
    // set around the down projection of a SwiGLU block at m > 32: the activation conversion of the prefill product
    // forms x * swish(act_mul) as it reads the rows (fp32, same shape and pitch as x)
    const float* act_mul = nullptr;
    int scatter_extra = 0;
    bool scatter_bf16 = false;   // the outputs of the scattered product are bf16
    float* scatter_y[7] = {};
    // ... and the peers' flag arrays when the product's last CTA is to signal them (scatter_sig_n == 0: no signal)
    int* scatter_flag[8] = {};
    int scatter_sig_n = 0, scatter_sig_my = 0, scatter_sig_epoch = 0;
    bool scatter_signalled = false;   // the kernel that ran took care of the signal
};

namespace b200q {
// Decode image of one NK tensor (built at upload, streamed by the integer tensor-core decode kernel): the
// packed weights re-arranged into the order that kernel's threads consume them. An ITEM is 16 weight rows x
// 128 weights (half a super-block per row) stored contiguously; item (row tile T, half h) sits at
// (T * nh + h) * item_bytes with nh = k / 128, so any run of row tiles is one contiguous byte range. Rows
// past the tensor's last row are zero items.
struct DImage {
    uint8_t* base = nullptr;   // device allocation (nullptr: the tensor has no decode image)
    int kind = -1;
    int item_bytes = 0;
    int nh = 0;                // items per row tile
    int nrt = 0;               // row tiles
    size_t bytes = 0;
};
}  // namespace b200q

// One device allocation that holds the planes and decode images of many tensors (256-byte aligned sub-allocations),
// plus the staging buffer their file bytes pass through.
struct b200q_arena {
    b200q_ctx* ctx = nullptr;
    uint8_t* base = nullptr;
    size_t capacity = 0, used = 0;
    void* stage = nullptr;
    size_t stage_bytes = 0;
    int64_t tensors = 0;   // handles handed out
    int64_t live = 0;      // ... and not yet freed
};

struct b200q_weight {
    b200q_ctx* ctx = nullptr;
    b200q_arena* arena = nullptr;   // set when base and dimg.base are sub-allocations of an arena
    int qtype = 0, layout = 0, orient = 0, fmt = 0;
    int64_t n_local = 0, k = 0, row0 = 0, n_total = 0;
    int64_t n_elements = 0;  // n_local * k
    int64_t n_blocks = 0;
    size_t packed_bytes = 0;  // bytes of the file blocks this handle holds
    void* base = nullptr;     // one allocation holding every plane
    b200q::WView view{};
    // From a scan of the scale bytes at upload. f16_scales_ok: the products "scale x sub-scale" the tensor-memory
    // prefill kernels form in f16 stay in range; f16_weights_ok: every weight does (the kernel that decodes in fp32
    // and rounds each weight once to f16). A tensor that fails both is multiplied by the fp32 decode kernels.
    bool f16_scales_ok = true, f16_weights_ok = true;
    b200q::DImage dimg{};     // second, decode-ordered copy for m <= 8 (formats of the integer decode kernel)
    void* mx_sfa = nullptr;   // MXFP4: block scales in the chunk order of the block-scaled MMA (built on first use, own allocation)
    // GGUF Q3_K: the same weights re-encoded, exactly, as Q6_K planes for the tensor-memory prefill kernel (built on
    // first use, own allocation)
    b200q::DImage pimg{};     // GGUF MXFP6 E3M2: image for the tensor-memory prefill kernel (built on first use, own allocation)
    void* q6_planes = nullptr;
    b200q::WView q6_view{};
    // false for the layouts whose scales the upload does not scan on the host: f16_weights_ok is then settled by a
    // device scan of the weights on first use
    bool range_scanned = true;
};

namespace b200q {

int fail(int code, const char* fmt, ...);
int cuda_fail(int code, cudaError_t e, const char* what);
int ensure_scratch(b200q_ctx* ctx, size_t bytes, int which = 0);

#define B200Q_CUDA(call, code)                                        \
    do {                                                              \
        cudaError_t e__ = (call);                                     \
        if (e__ != cudaSuccess) return b200q::cuda_fail((code), e__, #call); \
    } while (0)

// Expands `X(F)` for every format index (qtype*2+layout).
#define B200Q_FOR_EACH_FMT(X) \
    X(0) X(1) X(2) X(3) X(4) X(5) X(6) X(7) X(8) X(9) X(10) X(11) X(12) X(13) X(14) X(15) X(16) X(17) X(18) X(19)

// kernels_dequant.cu
int launch_fused_dequant_rmsnorm(b200q_ctx* ctx, int fmt, const WView& v, const float* d_weight, float* d_out, int64_t rows,
                                 int hidden, float eps);
int launch_dequant(b200q_ctx* ctx, int fmt, const WView& v, float* d_out, int64_t n, int64_t valid_bytes);
int launch_get_rows(b200q_ctx* ctx, int fmt, const WView& v, const int32_t* d_ids, int64_t n_ids, float* d_out, int64_t ldo,
                    int hidden, int64_t n_rows);
int launch_repack(b200q_ctx* ctx, int fmt, const uint8_t* d_raw, int64_t n_blocks, const WView& v);
int launch_absmax(b200q_ctx* ctx, int fmt, const WView& v, int64_t n, unsigned int* d_out);
// kernels_gemv.cu
int launch_gemv(b200q_ctx* ctx, const b200q_weight* w, const float* d_x, int64_t ldx, float* d_y, int64_t ldy, int m);
int launch_matmul_seq(b200q_ctx* ctx, const b200q_weight* w, const float* d_x, int64_t ldx, float* d_y, int64_t ldy, int m);
int launch_convert_bf16_to_f32(b200q_ctx* ctx, const void* d_in, int64_t ld_in, float* d_out, int64_t ld_out, int rows, int64_t cols);
int launch_convert_f32_to_bf16(b200q_ctx* ctx, const float* d_in, int64_t ld_in, void* d_out, int64_t ld_out, int rows, int64_t cols);
bool gemv_fast_supported(const b200q_weight* w);
// gemm_mx.cu
bool gemm_mx_native_supported(const b200q_weight* w, int m);
int launch_gemm_mx_native(b200q_ctx* ctx, const b200q_weight* w, const void* d_x, int x_is_bf16, int64_t ldx, float* d_y, int64_t ldy, int m);
// gemm_tc.cu
bool gemm_tc_supported(const b200q_weight* w, int m);
int launch_gemm_tc(b200q_ctx* ctx, const b200q_weight* w, const void* d_x, int x_is_bf16, int64_t ldx, float* d_y, int64_t ldy, int m);
int gemm_tc_check_status(b200q_ctx* ctx);
int launch_bounded_wait_selftest(b200q_ctx* ctx, long long budget_cycles);
int launch_gemm_tc_pair(b200q_ctx* ctx, const b200q_weight* w0, const b200q_weight* w1, const float* d_x, int64_t ldx,
                        float* d_y0, float* d_y1, int m);
int launch_gemm_tc_noalloc(b200q_ctx* ctx, const b200q_weight* w, const float* d_x, float* d_y, int m);

}  // namespace b200q
