// Declarations of the grouped decode kernel (gemv_mma.cu).
#pragma once
#include "common.cuh"

namespace b200q {

// One fused dequant + matmul product inside a grouped launch.
struct GOp {
    WView v;
    const float* x;   // [m, ldx] fp32 activations
    float* y;         // [m, ldy] fp32 outputs
    int64_t ldx, ldy;
    int n_rows;       // output features of this product (rows of W)
    int k;            // inner dimension
    int fmt;
    int kw_log2;      // log2 of the warps that split k for one 16-row tile (8 >> kw_log2 row tiles per CTA tile)
    int tile0;        // index of this product's first CTA tile in the launch
    int ntiles;       // CTA tiles of this product
    int n_extra;      // further copies of y to write (outputs of a sharded product gathered by peer stores)
    float* y_extra[7];
};

bool gemv_mma_supported(const b200q_weight* w, int m);
size_t gemv_mma_smem_bytes(int fmt, int k, int m);
// Fills kw_log2 / ntiles of `op` from its shape; `few_tiles` trades tile size for parallelism (single launches).
void gemv_mma_plan(GOp* op, bool few_tiles);
// ops/ranges are device pointers when n_ops > 1; for n_ops == 1 the product travels as a kernel argument.
// Depth (2 or 4 items) of the per-warp weight ring for inner dimension k and m activation rows, and the
// dynamic shared memory of a launch with that depth whose largest product has inner dimension kmax.
int gemv_mma_ring_depth(int k, int m);
size_t gemv_mma_smem_for(int ring_d, int kmax, int m);
int launch_gemv_mma(b200q_ctx* ctx, const GOp* h_single, const GOp* d_ops, int n_ops, const int2* d_ranges, int n_ctas,
                    int total_tiles, int m, size_t smem_bytes, int ring_d, bool has_q4_0);
// true when the product needs the kernel instantiation that carries the GGUF Q4_0 path
bool gemv_mma_is_q4_0(int fmt);

}  // namespace b200q
