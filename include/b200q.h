/*
 * b200q -- C ABI of the B200 (sm_100a) quantized-weight matmul library.
 *
 * This is the boundary a ROCmForge backend binds instead of the HIP runtime + HSACO
 * kernels it uses today for its quantized-weight path. Every entry point returns an
 * int status (0 = success, negative = b200q_status) the way the reference's FFI
 * returns HIP status codes (src/backend/hip_backend/ffi.rs:10-72, HIP_SUCCESS = 0);
 * the text of the last failure on the calling thread is b200q_last_error(). Nothing
 * throws, aborts or traps. File:line citations name the reference interface each
 * entry point replaces, by path inside the ROCmForge tree.
 *
 * Pointers named d_* are device pointers on the context's device, h_* are host
 * pointers. All work of a context is ordered on its one stream (the reference backend
 * is a single-stream singleton, src/backend/hip_backend/backend.rs:83-105).
 */
#ifndef B200Q_H
#define B200Q_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b200q_ctx b200q_ctx;       /* device + stream + scratch; replaces HipBackend (backend.rs:83-105) */
typedef struct b200q_weight b200q_weight; /* device-resident packed tensor; replaces Arc<DeviceTensor> of a quantized weight */

/* Status codes; names follow HipError (src/backend/hip_backend/error.rs:6-28). */
typedef enum {
    B200Q_OK = 0,
    B200Q_ERR_INIT = -1,          /* InitializationFailed */
    B200Q_ERR_NO_DEVICE = -2,     /* DeviceNotFound */
    B200Q_ERR_ALLOC = -3,         /* MemoryAllocationFailed (recoverable) */
    B200Q_ERR_COPY = -4,          /* MemoryCopyFailed (recoverable) */
    B200Q_ERR_LAUNCH = -5,        /* KernelLaunchFailed (recoverable) */
    B200Q_ERR_DEVICE = -6,        /* DeviceError (recoverable) */
    B200Q_ERR_INVALID = -7,       /* GenericError: bad argument, size or shape; nothing was launched */
    B200Q_ERR_UNSUPPORTED = -8,   /* GenericError: valid request this build has no kernel for */
    B200Q_ERR_TIMEOUT = -9        /* a bounded device-side wait gave up; the context stays usable */
} b200q_status;

/* Tensor types. Values in comments are GgufTensorType ids (src/loader/tensor_type.rs:16-32). */
typedef enum {
    B200Q_Q4_0 = 0,        /* 2  */
    B200Q_Q8_0 = 1,        /* 8  */
    B200Q_Q4_K = 2,        /* 12 */
    B200Q_Q6_K = 3,        /* 14 */
    B200Q_MXFP4 = 4,       /* 20 */
    B200Q_MXFP6_E2M3 = 5,  /* 21 */
    B200Q_MXFP6_E3M2 = 6,  /* 22 */
    B200Q_Q2_K = 7,        /* 10 */
    B200Q_Q3_K = 8,        /* 11 */
    B200Q_Q5_K = 9         /* 13 */
} b200q_qtype;

/* Byte layout of the blocks.
 * RF   = what the reference's CPU dequant parses: Q4_0 20 B (f32 scale), Q8_0 36 B, Q4_K 256 B,
 *        Q6_K 256 B, MXFP4 17 B (int8 exponent, high nibble first), MXFP6 25 B
 *        (src/kernels/quant/{q4_0,q8_0,q4_k,q6_k}.rs, src/loader/dequant.rs:41-132).
 * GGUF = llama.cpp blocks: 18 / 34 / 144 / 210 / 17 / 25 bytes.
 * Q2_K / Q3_K / Q5_K: RF = 256-byte blocks of 16 sub-blocks (src/loader/dequant.rs:150-419), GGUF = 84 / 110 /
 * 176 bytes. They have the dequantise kernel and the CUDA-core / shared-memory-operand matmul kernels. */
typedef enum { B200Q_LAYOUT_RF = 0, B200Q_LAYOUT_GGUF = 1 } b200q_layout;

/* How the flat element stream maps to the [n, k] weight matrix.
 * NK: n rows of k contiguous weights (blocks run along k) -- the documented operand of matmul_q4_0
 *     (src/kernels/matmul/quantized/q4_0.rs:139-148).
 * KN: flat [k, n] stream, W[l*n + j], as the reference kernels and its CPU composition index it
 *     (kernels/q4_0_matmul.hip:242, src/tensor/matmul.rs:219-233). */
typedef enum { B200Q_ORIENT_NK = 0, B200Q_ORIENT_KN = 1 } b200q_orient;

typedef enum { B200Q_F32 = 0, B200Q_BF16 = 1 } b200q_dtype;

/* b200q_matmul flags */
#define B200Q_MM_DEFAULT 0u
#define B200Q_MM_SEQUENTIAL 1u /* one thread per output, ascending k, multiply then add: bit-identical to cpu_matmul_f32 */
#define B200Q_MM_NO_TENSOR 2u  /* never take the tcgen05 path (CUDA-core kernels only) */
#define B200Q_MM_MX_NATIVE 8u  /* m > 8, GGUF MXFP4 / MXFP6 NK tensors with k % 128 == 0 only (B200Q_ERR_UNSUPPORTED otherwise): the 4- or 6-bit codes
                                  * and their E8M0 block scales go to tcgen05.mma.kind::mxf8f6f4.block_scale as they are, the
                                  * activations are quantised to MXFP8 (E4M3, one E8M0 scale per 32) on the way in. About twice
                                  * the throughput of the default path; the result carries the activations' 4-bit mantissa
                                  * (relative error of a few 1e-2 on random data, against 2e-3). Ignored at m <= 8. */
#define B200Q_MM_SCATTER_BF16 4u /* b200q_matmul_scatter[_signal] only, m > 8: every output is bf16 [m, ldy] (half the
                                  * bytes over NVLink), rounded once from the fp32 accumulators */

typedef struct {
    char name[128];
    int sm_count;
    int cc_major, cc_minor;
    size_t total_mem, free_mem;
    size_t smem_per_block_optin;
    int l2_bytes;
} b200q_device_info;

/* ---- context: replaces HipBackend::new / the hip* runtime calls of ffi.rs:10-72 ---------------- */
int b200q_init(int device, b200q_ctx** out);                         /* hipInit+hipSetDevice+hipStreamCreate */
int b200q_init_on_stream(int device, void* cuda_stream, b200q_ctx** out); /* run on a stream the caller owns */
void b200q_destroy(b200q_ctx* ctx);
const char* b200q_last_error(void);                                  /* hipGetErrorString(hipGetLastError()) */
int b200q_is_recoverable(int status);                                /* HipError::is_recoverable, error.rs:67-76 */
int b200q_get_device_info(b200q_ctx* ctx, b200q_device_info* out);   /* hipGetDeviceProperties, hipMemGetInfo */
int b200q_malloc(b200q_ctx* ctx, size_t bytes, void** d_out);        /* hipMalloc (HipBackend::allocate_buffer, backend.rs:704) */
int b200q_free(b200q_ctx* ctx, void* d_ptr);                         /* hipFree */
int b200q_memcpy_h2d(b200q_ctx* ctx, void* d_dst, const void* h_src, size_t bytes); /* hipMemcpyHtoD (HipBuffer::copy_from_host) */
int b200q_memcpy_d2h(b200q_ctx* ctx, void* h_dst, const void* d_src, size_t bytes); /* hipMemcpyDtoH (HipBuffer::copy_to_host) */
int b200q_memset(b200q_ctx* ctx, void* d_dst, int value, size_t bytes);             /* hipMemset */
int b200q_synchronize(b200q_ctx* ctx);                               /* HipBackend::synchronize, backend.rs:753 */
void* b200q_stream(b200q_ctx* ctx);                                  /* the cudaStream_t work is ordered on */
/* CUDA-event timing on the context's stream (KernelTimer, src/profiling/kernel_timer.rs:58-340). */
int b200q_timer_start(b200q_ctx* ctx);
int b200q_timer_stop_ms(b200q_ctx* ctx, float* ms_out);              /* synchronises; elapsed since timer_start */

/* ---- sizes: GgufTensorType::block_size, calculate_tensor_size (src/loader/gguf/tensor_info.rs:104-133) */
int b200q_block_elems(int qtype);
size_t b200q_block_bytes(int qtype, int layout);
size_t b200q_tensor_bytes(int qtype, int layout, int64_t n_elements);

/* ---- upload: replaces GgufLoader::load_tensor_to_gpu / gpu_dequantize_upload
 *      (src/loader/gguf/types.rs:199-254, src/loader/gguf/gpu_upload.rs:22-125). The packed bytes stay
 *      packed on the device (re-arranged into 16-byte-aligned planes of the same total size).
 *      shard_count > 1 keeps only rows [shard_rank*n/shard_count, (shard_rank+1)*n/shard_count) of an NK
 *      tensor; n must divide evenly and the slice must start and end on a block boundary. */
int b200q_weight_upload(b200q_ctx* ctx, const void* h_bytes, size_t nbytes, int qtype, int layout, int orient,
                        int64_t n, int64_t k, int shard_rank, int shard_count, b200q_weight** out);
int b200q_weight_free(b200q_weight* w);
int b200q_weight_info(const b200q_weight* w, int* qtype, int* layout, int* orient, int64_t* n_local, int64_t* k,
                      int64_t* row0, int64_t* n_total, size_t* packed_bytes);

/* ---- dequantise to fp32 on the device, bit-exact with the reference CPU dequant. Replaces
 *      dequantize_q4_0_kernel_cached (src/kernels/quant/q4_0.rs:107-153), dequantize_q4_k_gpu_kernel
 *      (q4_k.rs:99-148), dequantize_q6_k_gpu_kernel (q6_k.rs:102-149) and the HIP kernels under them
 *      (kernels/q4_0_dequant.hip:72, q8_0_dequant.hip:40, q4_k_dequant.hip:81, q6_k_dequant.hip:82,
 *      mxfp_dequant.hip:85,147). n_elements may stop inside a block. */
int b200q_dequantize(b200q_ctx* ctx, const b200q_weight* w, float* d_out, int64_t n_elements);
/* Host bytes in, device fp32 out (the exact shape of the reference wrappers: &[u8] -> HipBuffer). A byte
 * stream shorter than n_elements needs leaves the uncovered outputs 0.0, as the CPU functions do. */
int b200q_dequantize_bytes(b200q_ctx* ctx, const void* h_bytes, size_t nbytes, int qtype, int layout,
                           float* d_out, int64_t n_elements);

/* ---- fused dequant + matmul: y[m, n_local] = x[m, k] * W^T. Replaces matmul_q4_0 / matmul_q4_k /
 *      matmul_q6_k / matmul_q8_0 (src/kernels/matmul/quantized/q4_0.rs:153, q4_k.rs:173, q6_k.rs:163,
 *      q8_0.rs:69), their kernels (kernels/q4_0_matmul.hip:153, q4_k_matmul.hip:216, q6_k_matmul.hip:216)
 *      and the IR ops MatMulQ4_0 / MatMulQ8_0 (src/ggml/hip_backend/op_dispatch.rs:951-1082).
 *      m <= 8 takes the HBM-bound decode kernels, larger m the tensor-core kernel. x is [m, ldx] and y is
 *      [m, ldy] row-major (ld in elements; 0 means dense: k and n_local). */
int b200q_matmul(b200q_ctx* ctx, const b200q_weight* w, const void* d_x, int x_dtype, void* d_y, int y_dtype,
                 int m, unsigned flags);
int b200q_matmul_ex(b200q_ctx* ctx, const b200q_weight* w, const void* d_x, int x_dtype, int64_t ldx, void* d_y,
                    int y_dtype, int64_t ldy, int m, unsigned flags);
/* No counterpart in the reference: y[m, n_local] = x[m, k] * W^T (fp32 in, fp32 out, dense, tensor-core
 * kernel) for callers that cannot allocate device memory when they need the product -- a server whose own
 * pool already holds the rest of HBM, or a loop that cannot take cudaMalloc's device-wide synchronisation.
 * The call performs no cudaMalloc / cudaFree: its scratch (the f16 copy of the activations) is a fixed
 * 16 MiB + 64 KiB array inside the library image, held by every GPU that loads the library until exit.
 * Limits: m * k <= 8,388,608, m <= 16,384, NK tensor with k a multiple of 64; anything larger is refused
 * with B200Q_ERR_INVALID before any launch. The first call on a device looks up the array's device address;
 * make that first call before any stream capture begins. All calls share the one array, which keeps the
 * previous call's contents (every element a call reads is rewritten by that call first): two such calls
 * that overlap on the same GPU (different streams or contexts) race. */
int b200q_matmul_noalloc(b200q_ctx* ctx, const b200q_weight* w, const float* d_x, float* d_y, int m);
/* Host activations in, host result out; copies ride the context's stream (pinned or pageable memory). */
int b200q_matmul_host(b200q_ctx* ctx, const b200q_weight* w, const float* h_x, float* h_y, int m, unsigned flags);

/* ---- batch front end: replaces BatchQuantizedMatmul::process_batch / process_batch_profiled
 *      (src/ggml/hip_backend/ops/batch_quantized.rs:147-190). One launch covers every op of the batch.
 *      d_x[i] is op i's [m, k_i] fp32 input (the reference shares one input; pass the same pointer),
 *      d_y[i] its [m, n_i] fp32 output. ms_out (optional) receives the device time of the batch. */
typedef struct b200q_batch b200q_batch;
int b200q_batch_create(b200q_ctx* ctx, int count, const b200q_weight* const* w, const float* const* d_x,
                       float* const* d_y, int m, b200q_batch** out);
int b200q_batch_run(b200q_ctx* ctx, b200q_batch* batch, float* ms_out);
/* Host activations in, host results out for the whole batch: h_x_all is the [m, k_i] inputs of the products
 * back to back in batch order, h_y_all receives the [m, n_i] outputs the same way. Copies ride the context's
 * stream (one copy each way when the batch's device buffers are contiguous) and the call returns after the
 * results have landed. When h_y_all is page-locked host memory the device can address (cudaHostAlloc /
 * cudaHostRegister, a pinned torch tensor) and the batch is one grouped launch, the kernel stores its results
 * straight into h_y_all — posted writes that overlap the launch — and the batch's device output buffers are
 * left untouched by that call. The reference's process_batch takes a device input and returns device buffers
 * (batch_quantized.rs:147-161); this is the same call for a caller whose tensors live on the host. */
int b200q_batch_run_host(b200q_ctx* ctx, b200q_batch* batch, const float* h_x_all, float* h_y_all);
int b200q_batch_free(b200q_batch* batch);
/* Bytes of packed weights one run of the batch streams (BatchQuantizedMatmul::calculate_throughput, :277-289). */
size_t b200q_batch_weight_bytes(const b200q_batch* batch);
/* Kernel launches one run of the batch issues (1 when every product has a grouped decode kernel). */
int b200q_batch_launches(const b200q_batch* batch);

/* ---- multi-GPU (no counterpart in the reference, which is single-GPU): a tensor sharded by output feature
 *      (shard_rank / shard_count of b200q_weight_upload) produces y[:, row0 : row0 + n_local]. matmul_scatter
 *      fuses the gather into the product: d_y_full lists the FULL outputs [m, ldy] of every GPU that needs the
 *      result (this GPU's own first or anywhere; the others peer-mapped through b200q_ipc_open), and the
 *      kernels' epilogues store the slice into its column block of each of them over NVLink (plain stores in the
 *      decode kernel, TMA stores from shared memory in the persistent prefill kernel; nothing is ever loaded from a peer).
 *      fp32 outputs; the decode kernel's formats for m <= 8, the prefill kernels for m > 8. The caller
 *      synchronises the GPUs (a barrier or any collective on the same streams) before reading.
 *      ipc_*: cudaIpcGetMemHandle / OpenMemHandle / CloseMemHandle on a b200q_malloc'ed buffer; the 64 handle
 *      bytes travel between the processes by whatever channel the host has. */
int b200q_matmul_scatter(b200q_ctx* ctx, const b200q_weight* w, const void* d_x, int x_dtype, void* const* d_y_full,
                         int n_outputs, int64_t ldy, int m, unsigned flags);
/* Ordering the GPUs after a scattered product without a collective: every rank owns a flag array of n_ranks ints
 * (b200q_malloc + b200q_memset to 0, exported like the outputs). b200q_peer_signal, enqueued behind the product,
 * stores `epoch` into slot my_rank of every other rank's array (release stores over NVLink; the product's own peer
 * stores are complete by then because the kernel has ended). b200q_peer_wait, enqueued on the same stream, holds the
 * stream until every other slot of THIS rank's array holds `epoch` or a later value (a peer that runs ahead may
 * already have signalled its next product); whatever follows it on the stream may read the full output. The wait
 * is bounded (about a second of SM clock): on expiry the next b200q_synchronize returns B200Q_ERR_TIMEOUT and the
 * context stays usable. Epochs must grow by one per product (a counter). A peer that runs ahead also stores its
 * NEXT product's rows while this rank may still read the current ones: alternate two output buffers when both
 * products write the same one. */
int b200q_peer_signal(b200q_ctx* ctx, void* const* d_flags_of_ranks, int n_ranks, int my_rank, int epoch);
/* b200q_matmul_scatter followed by b200q_peer_signal in one call (d_y_full[p] and d_flags_of_ranks[p] belong to rank p,
 * n_outputs ranks). The decode kernel raises the flags itself when its last CTA has stored its rows, so m <= 8 costs
 * no extra launch. */
int b200q_matmul_scatter_signal(b200q_ctx* ctx, const b200q_weight* w, const void* d_x, int x_dtype, void* const* d_y_full,
                                int n_outputs, int64_t ldy, int m, unsigned flags, void* const* d_flags_of_ranks, int my_rank,
                                int epoch);
int b200q_peer_wait(b200q_ctx* ctx, const void* d_flags_own, int n_ranks, int my_rank, int epoch);
int b200q_ipc_get_handle(b200q_ctx* ctx, const void* d_ptr, void* handle64);
int b200q_ipc_open(b200q_ctx* ctx, const void* handle64, void** d_ptr_out);
int b200q_ipc_close(b200q_ctx* ctx, void* d_ptr);

/* ---- failure-path self test (no counterpart in the reference, whose kernels have no device-side waits):
 *      launches one thread that waits, for at most budget_cycles SM clock cycles, on a barrier nothing ever
 *      arrives on, and gives up the way the prefill kernels do. The next b200q_synchronize returns
 *      B200Q_ERR_TIMEOUT (recoverable); the context stays usable. Nothing faults, traps or hangs. */
int b200q_selftest_bounded_wait(b200q_ctx* ctx, int64_t budget_cycles);

/* ---- fused dequantise + RMSNorm: replaces fused_q4_0_rmsnorm (src/ggml/hip_backend/ops/fused_ops.rs:149-215,
 *      kernels/fused_dequant_rmsnorm.hip:87-165). w is a packed [seq_len, hidden_size] tensor uploaded as NK
 *      (n = seq_len, k = hidden_size; any qtype/layout, the reference has Q4_0 RF only);
 *      out[r, j] = deq(w)[r, j] * rsqrt(mean_j(deq(w)[r, :]^2) + eps) * norm_weight[j], fp32 [seq_len, hidden_size]. */
int b200q_fused_dequant_rmsnorm(b200q_ctx* ctx, const b200q_weight* w, const float* d_norm_weight, float* d_out, float eps);

/* ---- projection-site operators on packed weights (the callers of the fused products:
 *      src/model/execution_plan/execute.rs:300,403,456-458,585,601).
 *      b200q_swiglu: out[i] = gate[i] * swish(up[i]), swish(u) = u / (1 + expf(-u)) computed as
 *        u * (1 / (1 + expf(-u))) — kernels/swiglu.hip:37-63 (the activation is on the UP projection there);
 *        fp32 [seq_len, intermediate_size], out may alias gate.
 *      b200q_add_row_bias: y[r, c] += bias[c] — HipBackend::add_row_bias (src/backend/hip_backend/backend.rs:924-975,
 *        one saxpy per row); ldy = 0 means cols; rows == 0 or cols == 0 is a successful no-op as there.
 *      b200q_mlp_*: HipBackend::mlp_swiglu (backend.rs:1153-1276) with the three weights PACKED
 *        ([intermediate, hidden] gate and up, [hidden, intermediate] down, NK): out[m, hidden] =
 *        (gate(x) * swish(up(x))) . down. A plan binds the buffers once (scratch for the two [m, intermediate]
 *        projections); at m <= 8 gate and up are one grouped launch that reads x once. Errors carry the
 *        reference's shape messages. Q, K, V projections sharing one input are the same grouped launch through
 *        b200q_batch_create with three products. */
typedef struct b200q_mlp b200q_mlp;
int b200q_swiglu(b200q_ctx* ctx, const float* d_gate, const float* d_up, float* d_out, int64_t seq_len, int64_t intermediate_size);
int b200q_add_row_bias(b200q_ctx* ctx, float* d_y, int64_t ldy, const float* d_bias, int64_t rows, int64_t cols);
int b200q_mlp_create(b200q_ctx* ctx, const b200q_weight* w_gate, const b200q_weight* w_up, const b200q_weight* w_down,
                     const float* d_hidden_states, float* d_output, int m, b200q_mlp** out);
int b200q_mlp_run(b200q_ctx* ctx, b200q_mlp* plan);
int b200q_mlp_free(b200q_mlp* plan);

/* ---- quantised embedding lookup: replaces the GetRows op (execute_get_rows, src/ggml/hip_backend/op_dispatch.rs:13-102;
 *      get_rows + validate_token_ids, src/ggml/hip_backend/ops/get_rows.rs:24-94), which copies fp32 rows of a
 *      dequantised table. w is the packed [vocab_size, n_embd] token_embd uploaded as NK (any qtype/layout);
 *      out[i, :] = deq(w)[ids[i], :], fp32, row pitch ldo >= n_embd floats, bit-exact against b200q_dequantize.
 *      b200q_get_rows takes device ids and is asynchronous: an id outside [0, vocab_size) never reads the table,
 *      its row is zero-filled and the next b200q_synchronize returns B200Q_ERR_INVALID.
 *      b200q_get_rows_host takes host ids, validates them BEFORE any launch (the reference's order and message,
 *      "Token ID {} exceeds vocab size {}") and returns when the rows are written. */
int b200q_get_rows(b200q_ctx* ctx, const b200q_weight* w, const int32_t* d_ids, int64_t n_ids, float* d_out, int64_t ldo);
int b200q_get_rows_host(b200q_ctx* ctx, const b200q_weight* w, const uint32_t* h_ids, int64_t n_ids, float* d_out, int64_t ldo);

/* ---- GGUF container: replaces the parser and lazy loader in front of load_tensor_to_gpu
 *      (src/loader/gguf/header.rs:28-79 magic + version-3-only check, src/loader/gguf/metadata.rs:20-269
 *      key/value pairs, src/loader/gguf/tensor_info.rs:37-101 tensor directory -> LazyTensor,
 *      src/loader/mmap.rs:38-100 read-only mapping with bounds-checked slices). Host-only except
 *      b200q_gguf_upload_tensor. The file stays mapped until b200q_gguf_close; name and data pointers
 *      returned below live as long as the handle. */
typedef struct b200q_gguf b200q_gguf;

/* flags of b200q_gguf_open. Default (0) reads files the way ggml writes them: tensor offsets relative to the
 * data section (aligned to general.alignment, default 32), the contiguous dimension first, llama.cpp block
 * sizes. B200Q_GGUF_REFERENCE_FIXTURE reads files the way the reference's own fixtures are written and its
 * loader reads them (tests/common/fixtures.rs:125-183, src/loader/gguf/gpu_upload.rs:37): absolute offsets,
 * rows first, RF block sizes. */
enum { B200Q_GGUF_REFERENCE_FIXTURE = 1 };

typedef struct {
    const char* name;
    int n_dims;
    int64_t dims[4];      /* as stored in the file; unused entries are 1 */
    int ggml_type;        /* id in the file (GgufTensorType, src/loader/tensor_type.rs:16-32; 39 = ggml's MXFP4) */
    int qtype;            /* b200q_qtype, or -1 when this library has no packed kernel for the type (F32, F16) */
    int layout;           /* b200q_layout the bytes are in */
    int64_t n, k;         /* rows x row length as b200q_weight_upload wants them */
    int64_t file_offset;  /* absolute */
    size_t nbytes;        /* calculate_tensor_size (src/loader/gguf/tensor_info.rs:104-133) with this library's block sizes */
} b200q_gguf_tensor;

int b200q_gguf_open(const char* path, int flags, b200q_gguf** out);
void b200q_gguf_close(b200q_gguf* file);
int64_t b200q_gguf_tensor_count(const b200q_gguf* file);
int64_t b200q_gguf_kv_count(const b200q_gguf* file);
int64_t b200q_gguf_find_tensor(const b200q_gguf* file, const char* name);   /* index, or -1 */
int b200q_gguf_tensor_info(const b200q_gguf* file, int64_t index, b200q_gguf_tensor* out);
int b200q_gguf_kv_key(const b200q_gguf* file, int64_t index, const char** key, int* value_type);
/* Value of a key as text, the way the reference keeps every value (metadata.rs:56-143): numbers in decimal,
 * bools "true"/"false", strings verbatim, arrays "" (they are skipped). needed = length + 1. */
int b200q_gguf_meta_string(const b200q_gguf* file, const char* key, char* buf, size_t buflen, size_t* needed);
/* LazyTensor -> mapped bytes (MmapGguf::get_slice) */
int b200q_gguf_tensor_data(const b200q_gguf* file, int64_t index, const void** h_ptr, size_t* nbytes);
/* GgufLoader::load_tensor_to_gpu (src/loader/gguf/types.rs:199-254) for a quantized tensor: the mapped
 * bytes go to b200q_weight_upload as an NK tensor and stay packed. */
int b200q_gguf_upload_tensor(b200q_ctx* ctx, const b200q_gguf* file, int64_t index, int shard_rank, int shard_count,
                             b200q_weight** out);

/* ---- bulk upload into one allocation --------------------------------------------------------------------
 * Replaces GgufLoader::load_to_gpu_async / arena_upload_phase (src/loader/gguf/types.rs:326,
 * src/loader/gguf/gpu_upload.rs:413-594) and ModelWeightArena (src/memory/arena.rs:82,206): ONE device allocation
 * for all tensors of a model, bump-allocated in 256-byte aligned pieces. Unlike the reference's arena the tensors
 * stay packed (their planes, plus the decode image where the format has one). Uploads into an arena are queued on
 * the context's stream without waiting for one another (file bytes -> staging buffer -> plane split -> image
 * build); b200q_synchronize, or any product on the same context, orders behind them. Handles are freed with
 * b200q_weight_free as usual (their memory returns with the arena); b200q_arena_free refuses while handles live. */
typedef struct b200q_arena b200q_arena;
/* bytes one tensor (or one rank's shard of n_local rows) takes in an arena */
int b200q_arena_tensor_bytes(int qtype, int layout, int orient, int64_t n_local, int64_t k, size_t* bytes);
int b200q_arena_create(b200q_ctx* ctx, size_t capacity, b200q_arena** out);
/* b200q_weight_upload into the arena; B200Q_ERR_ALLOC when the arena is full */
int b200q_arena_upload(b200q_ctx* ctx, b200q_arena* arena, const void* h_packed, size_t nbytes, int qtype, int layout,
                       int orient, int64_t n, int64_t k, int shard_rank, int shard_count, b200q_weight** out);
int b200q_arena_info(const b200q_arena* arena, size_t* capacity, size_t* used, int64_t* tensors, int64_t* live);
int b200q_arena_free(b200q_arena* arena);
/* Every tensor of the file this library has packed kernels for, into a new arena sized for exactly them.
 * handles[i] (i < n_handles = b200q_gguf_tensor_count) receives tensor i's handle, or NULL for a tensor type
 * without packed kernels (F32/F16 norms and the like stay with the caller). A tensor whose row count does not
 * divide by shard_count is uploaded whole on every rank. Returns after the last copy is queued. */
int b200q_gguf_upload_all(b200q_ctx* ctx, const b200q_gguf* file, int shard_rank, int shard_count, b200q_arena** arena_out,
                          b200q_weight** handles, int64_t n_handles);

#ifdef __cplusplus
}
#endif
#endif
