/*
 * CPU oracle for the quantized-weight matmul path -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the reference's CPU dequantisation and CPU matmul
 * (ROCmForge, Rust). It exists so the CUDA path can be checked against it and so
 * the benchmark can time the reference's CPU algorithm beside the GPU. Nothing in
 * the shipped library links, imports or calls it.
 *
 * Two layout families are restated:
 *   rf_*    the byte layouts the reference's own CPU code parses ("RF layout"),
 *   gguf_*  the llama.cpp/GGUF layouts the benchmark configurations describe. The
 *           reference has no code for those; they are checked against the
 *           third-party `gguf` python package (0.19.0) in the CPU tests, except
 *           MXFP6 which no available implementation covers ("parity unpinned").
 *
 * Pinning: rf_* functions are checked against every known-answer vector the
 * reference's unit tests hold for this path (tests/golden/reference_vectors.json).
 * The reference itself (Rust 1.82 + crates half 2.7.1 / rayon 1.11.0) cannot be
 * compiled here, so there is no oracle/_ref build.
 *
 * Compile with -ffp-contract=off: Rust never fuses a*b+c, and neither may this.
 */
#ifndef B200Q_ORACLE_H
#define B200Q_ORACLE_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* IEEE binary16 -> binary32, exact, subnormals kept (half::f16::to_f32). */
float orc_f16_to_f32(uint16_t h);
/* f32::powi(2.0, e) as compiler-rt's __powisf2 evaluates it (e = -128 gives 0). */
float orc_pow2i(int e);

/* ---- RF layout: what the reference CPU code parses ------------------------- */
void rf_dequant_q4_0(const uint8_t* data, size_t nbytes, size_t n, float* out);   /* src/kernels/quant/q4_0.rs:266-310 */
void rf_dequant_q8_0(const uint8_t* data, size_t nbytes, size_t n, float* out);   /* src/kernels/quant/q8_0.rs:23-71   */
void rf_dequant_q8_0_i8(const uint8_t* data, size_t nbytes, size_t n, float* out);/* src/kernels/matmul/quantized/q8_0.rs:18-54 (variant) */
void rf_dequant_q4_k(const uint8_t* data, size_t nbytes, size_t n, float* out);   /* src/kernels/quant/q4_k.rs:201-273 */
void rf_dequant_q6_k(const uint8_t* data, size_t nbytes, size_t n, float* out);   /* src/kernels/quant/q6_k.rs:201-266 */
void rf_dequant_mxfp4(const uint8_t* data, size_t nbytes, size_t n, float* out);  /* src/loader/dequant.rs:41-82       */
void rf_dequant_mxfp6(const uint8_t* data, size_t nbytes, size_t n, float* out);  /* src/loader/dequant.rs:85-132      */
float rf_decode_e2m1(uint8_t bits);                                               /* src/loader/mxfp.rs:234-244 */
float rf_decode_e2m3(uint8_t bits);                                               /* src/loader/mxfp.rs:283-293 */
/* MxfpBlock helpers the reference's round-trip tests use (src/loader/mxfp.rs). */
uint8_t rf_encode_e2m1(float v);                                                  /* :200-231 */
uint8_t rf_encode_e2m3(float v);                                                  /* :249-280 */
int8_t  rf_e8m0_from_f32(float v);                                                /* :29-43   */
void rf_pack_6bit(const uint8_t* vals, size_t count, uint8_t* packed);            /* :297-320 */
void rf_unpack_6bit(const uint8_t* packed, size_t nbytes, size_t count, uint8_t* vals); /* :324-353 */
void rf_mxfpblock_pack_mxfp4(const float* v32, int8_t* exp_out, uint8_t* elems16);   /* :77-117  */
void rf_mxfpblock_unpack_mxfp4(int8_t e, const uint8_t* elems16, float* out32);      /* :120-139 */
void rf_mxfpblock_pack_mxfp6(const float* v32, int8_t* exp_out, uint8_t* elems24);   /* :142-174 */
void rf_mxfpblock_unpack_mxfp6(int8_t e, const uint8_t* elems24, float* out32);      /* :177-190 */

/* ---- GGUF layout: what the benchmark configurations describe ---------------- */
void gguf_dequant_q4_0(const uint8_t* data, size_t nbytes, size_t n, float* out);
void gguf_dequant_q8_0(const uint8_t* data, size_t nbytes, size_t n, float* out);
void rf_dequant_q5_k(const uint8_t* data, size_t nbytes, size_t n, float* out);   /* src/loader/dequant.rs:150-233 */
void rf_dequant_q3_k(const uint8_t* data, size_t nbytes, size_t n, float* out);   /* src/loader/dequant.rs:243-322 */
void rf_dequant_q2_k(const uint8_t* data, size_t nbytes, size_t n, float* out);   /* src/loader/dequant.rs:326-419 */
void gguf_dequant_q2_k(const uint8_t* data, size_t nbytes, size_t n, float* out);
void gguf_dequant_q3_k(const uint8_t* data, size_t nbytes, size_t n, float* out);
void gguf_dequant_q5_k(const uint8_t* data, size_t nbytes, size_t n, float* out);
void gguf_dequant_q4_k(const uint8_t* data, size_t nbytes, size_t n, float* out);
void gguf_dequant_q6_k(const uint8_t* data, size_t nbytes, size_t n, float* out);
void gguf_dequant_mxfp4(const uint8_t* data, size_t nbytes, size_t n, float* out);
void gguf_dequant_mxfp6_e2m3(const uint8_t* data, size_t nbytes, size_t n, float* out);
void gguf_dequant_mxfp6_e3m2(const uint8_t* data, size_t nbytes, size_t n, float* out);

/* Dispatcher in the shape of loader::dequantize (src/loader/dequant.rs:673-700).
 * qtype: 0 Q4_0, 1 Q8_0, 2 Q4_K, 3 Q6_K, 4 MXFP4, 5 MXFP6_E2M3, 6 MXFP6_E3M2.
 * layout: 0 RF, 1 GGUF. Returns 0, or -1 for an unknown pair. */
int orc_dequantize(int qtype, int layout, const uint8_t* data, size_t nbytes, size_t n, float* out);
size_t orc_block_bytes(int qtype, int layout);
size_t orc_block_elems(int qtype);

/* ---- matmul ------------------------------------------------------------------ */
/* cpu_matmul_f32, src/tensor/matmul.rs:219-233: c[i,j] = sum_l a[i,l]*b[l,j], fp32,
 * ascending l, multiply then add; b is [k,n] row-major. */
void orc_matmul_f32(const float* a, const float* b, int m, int n, int k, float* c);
/* Same sums with b stored as n rows of k ("[N,K]" orientation): c[i,j] = sum_l a[i,l]*w[j,l]. */
void orc_matmul_f32_nk(const float* a, const float* w, int m, int n, int k, float* c);
/* fp64 accumulation of the same products, to show which side is nearer the exact sum. */
void orc_matmul_f64_nk(const float* a, const float* w, int m, int n, int k, double* c);
void orc_matmul_f64(const float* a, const float* b, int m, int n, int k, double* c);
/* The same loops split over output rows with OpenMP (the "all cores" CPU baseline).
 * threads <= 0 means omp_get_max_threads(). Returns the thread count used. */
int orc_matmul_f32_nk_omp(const float* a, const float* w, int m, int n, int k, float* c, int threads);
int orc_matmul_f32_omp(const float* a, const float* b, int m, int n, int k, float* c, int threads);
int orc_dequantize_omp(int qtype, int layout, const uint8_t* data, size_t nbytes, size_t n, float* out, int threads);
int orc_max_threads(void);

/* kernels/fused_dequant_rmsnorm.hip:87-165 (launched by src/ggml/hip_backend/ops/fused_ops.rs:149-215):
 * per row of a packed [seq_len, hidden] tensor: dequantise, sum of squares accumulated the way the kernel's
 * 256 threads do (thread t takes j = t, t+256, ...; tree reduction with halving strides), rms = 1/sqrt(mean + eps),
 * out = val * rms * weight[j]. Parity unpinned: the reference has no test vector for this kernel. */
int orc_fused_dequant_rmsnorm(int qtype, int layout, const uint8_t* data, size_t nbytes, int seq_len, int hidden,
                              const float* weight, float eps, float* out);

/* kernels/swiglu.hip:37-63: out[i] = gate[i] * (up[i] * (1 / (1 + expf(-up[i])))), fp32, that operation order.
 * Parity unpinned: the reference's test for it (src/mlp/swiglu_tests.rs) compares its GPU kernel with the same
 * formula on the CPU at 1e-4; libm's expf stands in for the device's. */
void orc_swiglu(const float* gate, const float* up, float* out, size_t n);
/* HipBackend::add_row_bias (src/backend/hip_backend/backend.rs:924-975): saxpy(alpha = 1) of the bias onto every row */
void orc_add_row_bias(float* y, const float* bias, size_t rows, size_t cols);

#ifdef __cplusplus
}
#endif
#endif
