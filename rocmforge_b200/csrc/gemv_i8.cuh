// Declarations of the integer tensor-core decode kernel and of the decode image it streams (gemv_i8.cu).
#pragma once
#include <vector>

#include "common.cuh"

namespace b200q {

// Formats the kernel has an item layout for.
enum : int { DK_NONE = -1, DK_Q4K = 0, DK_Q6K = 1, DK_Q80 = 2, DK_MX6 = 3, DK_MX4 = 4, DK_Q40 = 5, DK_Q5K = 6, DK_COUNT = 7 };

// kind for a format index (fmt_of(qtype, layout)), or DK_NONE
int decode_kind_of(int fmt);
int decode_item_bytes(int kind);
// true when the tensor can carry a decode image (NK, a format of the kernel, k a multiple of 128)
bool decode_image_wanted(int fmt, int orient, int64_t n_rows, int64_t k);
// Builds the image of `w` (its stream-layout planes are already on the device) into a new allocation, or at `place`
// (decode_image_bytes() bytes, 256-byte aligned) without synchronising the stream.
int build_decode_image(b200q_ctx* ctx, const b200q_weight* w, DImage* out, uint8_t* place = nullptr);
size_t decode_image_bytes(int fmt, int64_t n_rows, int64_t k);
int build_e3m2_prefill_image(b200q_ctx* ctx, const b200q_weight* w, DImage* out);

// One fused dequant + matmul product inside a grouped launch of the integer decode kernel.
struct DOp {
    const uint8_t* img;
    const float* x;   // [m, ldx] fp32 activations
    float* y;         // [m, ldy] fp32 outputs
    int64_t ldx, ldy;
    int n_rows;       // output features (rows of W)
    int k;
    int kind;
    int item_bytes;
    int nh;           // items per row tile
    int rt0;          // index of this product's first row tile in the launch
    int nrt;          // row tiles of this product
    int n_extra;      // further copies of y to write (outputs of a sharded product gathered by peer stores)
    float* y_extra[7];
};

// Signal raised at the end of a launch whose products were scattered to peer GPUs: the last CTA stores `epoch` into
// slot `my` of every other rank's flag array (n == 0: no signal).
struct PeerSignal {
    int* flag[8];
    int n, my, epoch;
    int* status_out;   // when set: the launch's status word is copied there ahead of the flags (a host-visible word)
};

struct DecodeLaunch {
    int chunk_items;   // items per bulk copy
    int depth;         // ring slots per warp
    int slot_bytes;
    size_t smem_bytes;
    int ctas_per_sm;
    int nw;            // warps per CTA
    bool many;         // activation rows on the MMA's N side (m >= 2)
};

bool gemv_i8_supported(const b200q_weight* w, int m);
// Ring geometry and shared memory of a launch whose products have at most `max_item_bytes` per item, inner
// dimension at most kmax and kinds in `kind_mask`; returns false when the activation image does not fit.
bool gemv_i8_plan(int max_item_bytes, int kmax, int kind_mask, int m, DecodeLaunch* out);
size_t gemv_i8_image_smem(int kind, int k, int m);
// Work units: d_ranges lists n_units contiguous row-tile ranges (device array), or is null and the total_rt row
// tiles are cut into n_units equal ranges. The first n_ctas units start on their own CTA, the rest are handed out
// as CTAs finish. d_ops is a device array when n_ops > 1; a single product travels as a kernel argument.
int launch_gemv_i8(b200q_ctx* ctx, const DOp* h_single, const DOp* d_ops, int n_ops, const int2* d_ranges, int n_units, int n_ctas,
                   int total_rt, int m, const DecodeLaunch& L, const PeerSignal* sig = nullptr);
// Cuts the row tiles of a launch (byte cost and product index per tile) into work units: n_ctas ranges of equal
// cost, optionally followed by smaller units that are handed out as CTAs finish.
void gemv_i8_make_units(const std::vector<double>& tile_cost, const std::vector<int>& tile_op, int n_ctas, std::vector<int2>* units);

}  // namespace b200q
