/* simp_gpu.h -- C ABI of the B200 (sm_100a) runtime library for SimpLang's tensor hot path.
 *
 * One shared library, libsimp_gpu.so.  Every entry point returns an int status
 * (SIMP_OK == 0, negative on error, text via simp_gpu_last_error()) and never
 * aborts, traps or throws across the boundary.  Pointers named *_dev are device
 * pointers obtained from simp_gpu_alloc(); ops are enqueued on the library's
 * stream of the calling thread's current library device and are asynchronous:
 * call simp_gpu_sync() (or download) before reading results on the host.
 *
 * Each declaration cites the reference interface it replaces (paths relative
 * to the reference project root).  The reference has no run-time library for
 * these ops -- its compiler expands each `simp` dialect op into loops -- so
 * "replaces" means: the call a GPU lowering pattern emits in place of the
 * expansion cited.
 */
#ifndef SIMP_GPU_H_
#define SIMP_GPU_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SIMP_OK 0
#define SIMP_ERR_ARG (-1)         /* null pointer, negative size, bad flag              */
#define SIMP_ERR_SHAPE (-2)       /* shape outside what the op supports                 */
#define SIMP_ERR_CUDA (-3)        /* a CUDA runtime/driver call failed                  */
#define SIMP_ERR_STATE (-4)       /* library not initialised / wrong call order         */
#define SIMP_ERR_TIMEOUT (-5)     /* a bounded device-side wait gave up                 */
#define SIMP_ERR_COMM (-6)        /* NCCL / multi-GPU set-up or collective failed       */
#define SIMP_ERR_UNSUPPORTED (-7) /* valid request this build cannot serve              */

/* ---- life cycle, memory, stream ------------------------------------------------------------
 * Replaces: nothing in the op lowering; the reference hosts own all buffers as std::vector and
 * pass host pointers (examples/llama2/generate_stories110M.cpp:236-251).  The loader they use is
 * KernelRunner (runtime/include/kernel_runner.hpp:27-103). */
int simp_gpu_init(int device);          /* select `device`, create the stream; idempotent      */
int simp_gpu_shutdown(void);            /* free library-owned memory, destroy stream           */
const char* simp_gpu_last_error(void);  /* message of the calling thread's last failure        */
int simp_gpu_device_count(int* count);
int simp_gpu_alloc(void** dptr, size_t bytes);
int simp_gpu_free(void* dptr);
int simp_gpu_upload(void* dst_dev, const void* src_host, size_t bytes);   /* async on the stream */
int simp_gpu_download(void* dst_host, const void* src_dev, size_t bytes); /* synchronises        */
int simp_gpu_memset(void* dptr, int value, size_t bytes);
int simp_gpu_sync(void);
void* simp_gpu_stream(void);            /* the cudaStream_t ops are enqueued on                 */
/* Polls the device-side error word that bounded waits write; SIMP_OK or SIMP_ERR_TIMEOUT.      */
int simp_gpu_check_device_status(void);

/* ---- simp.matmul / tensor_matmul (f32) -----------------------------------------------------
 * C[coff + i*n + j] (+)= sum_p A[aoff + i*k + p] * B[boff + p*n + j], row-major, element offsets.
 * accumulate != 0: simp.matmul, C += A.B (MatMulOpLowering,
 *   src/mlir/lowering/ConvertSimpToMemRef.cpp:1794-1920; callers zero C, stories110M.sl:66-83).
 * accumulate == 0: tensor_matmul / tensor_matmul_into / tensor_matvecmul on f32, C = A.B
 *   (ConvertSimpToMemRef.cpp:2884-2950, 3280-3291, 3490-3627, 3632-3792).
 * b_transposed != 0: tensor_matmul_nt, B given as [n,k] (ConvertSimpToMemRef.cpp:3373-3486).
 * n == 1 runs the streaming GEMV kernel, a skinny left operand (m <= 64) the k-split streaming kernel, small shapes
 * the FFMA tile kernel: f32 FMA arithmetic.  GEMM-sized shapes (m, n >= 128, k >= 32, n % 4 == 0, m*n*k >= 2^26) run
 * on the tensor cores as 3 x TF32 (each operand split into two TF32 numbers, three products per step, f32
 * accumulation: error at f32 level, never a single TF32 product); that path keeps the split operands in library
 * scratch (2 x the operand bytes; grown on first use -- inside a recording it falls back to the FFMA kernel if the
 * scratch would have to grow), and for shapes with fewer than 37 tiles of 256 x 256 it splits K over the SMs and adds
 * the parts into C in no fixed order (results may differ in the last bits from run to run). */
int simp_gpu_matmul_f32(const float* A_dev, int64_t aoff, const float* B_dev, int64_t boff,
                        float* C_dev, int64_t coff, int64_t m, int64_t k, int64_t n,
                        int accumulate, int b_transposed);
/* The 3-D (batched) form of tensor_matmul on f32: C[b] = A[b] . B[b], A [batch, m, k], B [batch, k, n] (b_transposed:
 * [batch, n, k]), C [batch, m, n] fresh -- linalg.batch_matmul in TensorMatMulOpLowering
 * (ConvertSimpToMemRef.cpp:3286-3291). */
int simp_gpu_matmul_f32_batched(const float* A_dev, const float* B_dev, float* C_dev, int64_t batch, int64_t m,
                                int64_t k, int64_t n, int b_transposed);

/* ---- tensor_matmul on i8 -> i32 ------------------------------------------------------------
 * C[M,N] (i32, wrap-around) = A[M,K] . B, bit-exact.
 * a_unsigned == 0: signed x signed, the op as lowered (ConvertSimpToMemRef.cpp:3136-3279 and the
 *   VNNI rewrite src/mlir/passes/VNNIPass.cpp:597-999).
 * a_unsigned != 0: A is uint8 -- the raw vpdpbusd form
 *   (simptensor/tests/test_vnni_correctness.cpp:28-42).
 * b_transposed == 0: B is [K,N] (tensor_matmul / _into / tensor_matvecmul);
 * b_transposed != 0: B is [N,K] (tensor_matmul_nt, ConvertSimpToMemRef.cpp:3373-3486).
 * Shapes whose operand rows are 16-byte aligned run on the tcgen05 kind::i8 tensor-core kernel;
 * any other shape runs an integer dot-product kernel with the same result. */
int simp_gpu_matmul_i8(const void* A_dev, const int8_t* B_dev, int32_t* C_dev, int64_t M,
                       int64_t K, int64_t N, int a_unsigned, int b_transposed);

/* tensor_matmul on packed signed i4 operands, fresh i16 result.
 * Replaces: TensorMatMulOpLowering, packed-i4 branch (src/mlir/lowering/ConvertSimpToMemRef.cpp:2953-3133;
 * timed by simptensor/benchmarks/bench_int4_matmul.sl:16-47).  Two 4-bit two's-complement values per byte along
 * the LAST dimension of each operand, low nibble = even index: A is [M, ceil(K/2)] bytes, B is [K, ceil(N/2)]
 * bytes; C[i,j] = low 16 bits of sum_k a[i,k] * b[k,j] (the i32 sum is exact), row-major [M, N]. */
int simp_gpu_matmul_i4(const uint8_t* A_packed, const uint8_t* B_packed, int16_t* C, int64_t M, int64_t K, int64_t N);

/* tensor_gather: result[..., n, ...] = source[..., indices[n], ...] along one axis.
 * Replaces: TensorGatherOpLowering (src/mlir/lowering/ConvertSimpToMemRef.cpp:2625-2776).  The source is passed as
 * its [outer, axis_dim, inner] view (outer = product of the dimensions before the axis, inner = product of those
 * after it), elements are opaque (elem_size bytes), indices are i64 on the device.  An index outside
 * [0, axis_dim) is undefined in the reference; here that row is skipped and simp_gpu_check_device_status()
 * reports it. */
int simp_gpu_tensor_gather(const void* src_dev, const int64_t* indices_dev, void* dst_dev, int64_t outer,
                           int64_t axis_dim, int64_t inner, int64_t n_idx, int64_t elem_size);

/* conv2d on f32: NHWC input, weights [OC, KH, KW, IC], bias [OC], NHWC output (caller-allocated,
 * out_h = (in_h + 2*pad_h - kernel_h) / stride_h + 1, same for w), zero padding.
 * Replaces: Conv2DOpLowering (src/mlir/lowering/ConvertSimpToMemRef.cpp:1924-2150); argument order as the op's
 * operands (:1934-1948).  Taps accumulate in (kh, kw, ic) order starting from the bias, multiply and add
 * separately, so results equal the CPU loop bit for bit. */
int simp_gpu_conv2d_f32(const float* input_dev, const float* weights_dev, const float* bias_dev, float* output_dev,
                        int64_t batch, int64_t in_h, int64_t in_w, int64_t in_c, int64_t out_c, int64_t kernel_h,
                        int64_t kernel_w, int64_t stride_h, int64_t stride_w, int64_t pad_h, int64_t pad_w);

/* ---- matmul_quant / dequant_w4 (W4) --------------------------------------------------------
 * out[rows] = W4[rows,cols] . x[cols]; nibbles packed two per byte, low nibble = even flat index,
 * w = q*scale + zero (MatMulQuantOpLowering, ConvertSimpToMemRef.cpp:3853-4013;
 * DequantW4OpLowering :2367-2429).  `offset` is in weights (elements) into qweights.
 * scale_mode 0 ("reference"): scale index (i*cols)/gs + g, 128 weights visited per group -- the
 *   lowering exactly as written (:3916-3936).
 * scale_mode 1 ("per_matrix"): scale index (offset + i*cols)/gs + g, gs weights per group;
 *   requires cols % gs == 0.
 * zeros_dev == NULL: symmetric weights, zero = -8*scale (no zeros array is read). */
int simp_gpu_matmul_w4(const uint8_t* qweights_dev, const float* scales_dev, const float* zeros_dev,
                       const float* x_dev, float* out_dev, int64_t rows, int64_t cols,
                       int64_t group_size, int64_t offset, int scale_mode);
int simp_gpu_dequant_w4(const uint8_t* qweights_dev, const float* scales_dev,
                        const float* zeros_dev, int64_t first_index, int64_t count,
                        int64_t group_size, float* out_dev);
/* Same result as simp_gpu_matmul_w4, for callers that must not allocate device memory (a host that gave its
 * whole memory budget to its own pool at start-up, or code running where the runtime forbids allocation).
 * This entry point has no counterpart in the reference.  The streaming kernel packs x in shared memory, so the
 * call needs no scratch in global memory; it differs from simp_gpu_matmul_w4 in what it refuses:
 *   - cols may not exceed SIMP_W4_NOALLOC_MAX_COLS (larger shapes are rejected with SIMP_ERR_SHAPE);
 *   - the library must already be initialised (simp_gpu_init allocates; this call returns SIMP_ERR_STATE
 *     rather than initialising on demand);
 *   - the first call with a given tile shape sets a kernel attribute: make that first call before starting
 *     any stream capture. */
#define SIMP_W4_NOALLOC_MAX_COLS 16384
int simp_gpu_matmul_w4_noalloc(const uint8_t* qweights_dev, const float* scales_dev,
                               const float* zeros_dev, const float* x_dev, float* out_dev, int64_t rows,
                               int64_t cols, int64_t group_size, int64_t offset, int scale_mode);

/* ---- rmsnorm / softmax / silu --------------------------------------------------------------
 * rmsnorm: y[r,i] = (x[r,i] / sqrt(mean_i(x[r,:]^2) + eps)) * w[woff + i]
 *   (RMSNormOpLowering, ConvertSimpToMemRef.cpp:2157-2236).  The op is single-row; `rows` with
 *   `row_stride` (elements) batches independent rows.  residual_dev != NULL fuses the preceding
 *   residual add of the models (stories110M.sl:177-185): x[r,i] += residual[r,i] is written back
 *   to x before normalising.
 * softmax: per row, y[yoff + r*row_stride + i] = softmax(x[xoff + r*row_stride + i], i < n)
 *   (SoftmaxOpLowering, ConvertSimpToMemRef.cpp:2239-2322).
 * silu: y[i] = x[i] / (1 + expf(-x[i])), times mul[i] when mul_dev != NULL
 *   (SiLUOpLowering, ConvertSimpToMemRef.cpp:2325-2360; the product is stories110M.sl:202-212). */
int simp_gpu_rmsnorm_f32(float* x_dev, const float* w_dev, float* y_dev, int64_t rows, int64_t n,
                         float eps, int64_t woff, int64_t row_stride, const float* residual_dev);
int simp_gpu_softmax_f32(const float* x_dev, float* y_dev, int64_t rows, int64_t n, int64_t xoff,
                         int64_t yoff, int64_t row_stride);
int simp_gpu_silu_f32(const float* x_dev, const float* mul_dev, float* y_dev, int64_t n);

/* ---- int8 quantise / dequantise ------------------------------------------------------------
 * Scalar model code in the reference, not ops: y = (int8) trunc(clamp(x*scale, -128, 127))
 * (examples/llama2/llama32_1b_int8_tensor.sl:96-103; without the clamp in
 * llama32_1b_int8_prefill.sl:48) and y = float(acc) / divisor (llama32_1b_int8_tensor.sl:227). */
int simp_gpu_quantize_i8(const float* x_dev, int8_t* y_dev, int64_t n, float scale, int clamp);
int simp_gpu_dequantize_i32(const int32_t* acc_dev, float* y_dev, int64_t n, float divisor);

/* ---- pinned host memory, resident operands, timing -----------------------------------------
 * Replaces: the hosts' std::vector buffers and chrono timing (runtime/src/host.cpp:96-148).
 * simp_gpu_register_host uploads [host, host+bytes) once; afterwards any simp_host_* call that is
 * given a pointer inside that range uses the device copy instead of copying again (how the model
 * weights of examples/llama2/generate_stories110M.cpp:142-202 stay resident between tokens). */
int simp_gpu_host_alloc(void** hptr, size_t bytes);
int simp_gpu_host_free(void* hptr);
int simp_gpu_register_host(const void* host, size_t bytes);
int simp_gpu_unregister_host(const void* host);
int simp_gpu_event_create(void** event);
int simp_gpu_event_record(void* event);                      /* on the library stream          */
int simp_gpu_event_elapsed_ms(void* start, void* stop, float* ms);
int simp_gpu_event_destroy(void* event);

/* Record-and-replay of a sequence of device-pointer calls (no counterpart in the reference: its hosts call a
 * compiled CPU function in a loop, e.g. simptensor/benchmarks/bench_int8_matmul_omp_runner.cpp:150-175; on a GPU a
 * call of a few microseconds is dominated by its launch unless the sequence is replayed as one unit).
 * Between record_begin and record_end the calls are recorded, not executed; only the simp_gpu_* compute entry
 * points with device pointers may be called (no alloc / upload / download / sync, no first call of an op
 * family -- run the sequence once before recording it).  Pointers and shapes are frozen into the recording,
 * library scratch included: simp_gpu_matmul_i4 and simp_gpu_conv2d_f32 use it, so a recorded call of those that
 * would need MORE scratch than any earlier call fails with SIMP_ERR_STATE (run it once first); scratch that a
 * live recording uses is kept until the recording is destroyed, whatever later calls need.  Destroy every
 * recording before simp_gpu_shutdown. */
int simp_gpu_record_begin(void);
int simp_gpu_record_end(void** recording);
int simp_gpu_replay(void* recording, int64_t times);       /* enqueued on the library stream */
int simp_gpu_recording_destroy(void* recording);

/* ---- the same ops on HOST pointers ---------------------------------------------------------
 * What a compiled .sl kernel's host sees today: plain host arrays in, results in host arrays on
 * return (hosts: simptensor/benchmarks/bench_prefill_matmul_runner.cpp:18-23, 77-120;
 * examples/llama2/bench_llama_quant.cpp:10-28).  Each call copies operands that are not registered
 * to the device, runs the device op declared above with the same arguments, and copies the result
 * back.  The int8 GEMM pipelines upload / compute / download over row chunks of A. */
int simp_host_tensor_matmul_i8(const void* A, const int8_t* B, int32_t* C, int64_t M, int64_t K,
                               int64_t N, int a_unsigned, int b_transposed);
int simp_host_matmul_f32(const float* A, int64_t aoff, const float* B, int64_t boff, float* C,
                         int64_t coff, int64_t m, int64_t k, int64_t n, int accumulate,
                         int b_transposed);
int simp_host_matmul_quant(const uint8_t* qweights, size_t qweights_bytes, const float* scales,
                           const float* zeros, size_t n_groups, const float* x, float* out,
                           int64_t rows, int64_t cols, int64_t group_size, int64_t offset,
                           int scale_mode);
int simp_host_rmsnorm_f32(const float* x, const float* w, float* y, int64_t rows, int64_t n,
                          float eps, int64_t woff);
int simp_host_softmax_f32(const float* x, float* y, int64_t rows, int64_t n, int64_t xoff,
                          int64_t yoff, int64_t row_stride);
int simp_host_silu_f32(const float* x, const float* mul, float* y, int64_t n);

/* ---- whole-token LLaMA decode --------------------------------------------------------------
 * Replaces: the compiled model kernels stories110M_forward (examples/llama2/stories110M.sl:5-247)
 * and llama2_quant_forward (examples/llama2/llama2_quant.sl:7-198) together with the host loop
 * around them (examples/llama2/generate_stories110M.cpp:236-260, greedy argmax :73-83).
 * Tensors are loaded by the .sl argument names: token_embedding, rms_att_w, rms_ffn_w, rms_final_w,
 * wcls, and either wq wk wv wo w1 w2 w3 (f32, stacked [n_layers, rows, cols]) or qweights, scales
 * [, zeros] plus the seven element offsets of wq wk wv wo w1 w2 w3 inside qweights
 * (examples/llama2/bench_llama_quant.cpp:189-209).  KV cache and activations stay on the device;
 * one CUDA graph is replayed per token. */
typedef struct simp_llama_config {
  int64_t dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len;
  int64_t w4;          /* 0: f32 projections, 1: W4 projections (scale_mode 1) */
  int64_t group_size;  /* W4 only: 32, 64, ... 1024 */
  /* Tensor parallelism over the ranks of simp_dist_init (W4 model only; 0 or 1 = single GPU).  Every
   * projection is split by output rows (q/k/v by heads, gate/up/down/wo and the classifier by rows); each
   * rank keeps the KV cache of its heads; the row slices are exchanged with in-place NCCL all-gathers
   * (four per layer + one for the logits), so every output element is still computed by one rank with
   * the single-GPU reduction order.  simp_llama_load takes the FULL tensors on every rank and keeps
   * this rank's rows; call simp_llama_set_w4_offsets before loading qweights / scales / zeros. */
  int64_t tp_size;
} simp_llama_config;
int simp_llama_create(const simp_llama_config* cfg, void** model);
int simp_llama_load(void* model, const char* name, const void* host, size_t bytes);
int simp_llama_set_w4_offsets(void* model, const int64_t* offsets7);
/* One token at `pos`; logits_host (vocab floats) may be NULL. */
int simp_llama_forward(void* model, int64_t token, int64_t pos, float* logits_host);
/* Teacher-forces prompt[0..n_prompt), then greedily generates n_new tokens into tokens_out.
 * logits_trace (optional) receives (n_prompt + n_new - 1) x vocab logits; ms_out (optional) the
 * device time of the whole generation in milliseconds. */
int simp_llama_generate(void* model, const int32_t* prompt, int64_t n_prompt, int64_t n_new,
                        int32_t* tokens_out, float* logits_trace, float* ms_out);
/* Number of kernel launches one token costs (kernel nodes of the captured token graph; valid after the first
 * forward / generate).  A measurement aid: the reference's hosts count calls of the compiled forward function. */
int simp_llama_kernels_per_token(void* model, int64_t* kernels);
int simp_llama_destroy(void* model);

/* ---- int8 LLaMA-3.2-1B-style token forward ---------------------------------------------------
 * Replaces: the exported function `llama32_forward` of examples/llama2/llama32_1b_int8_tensor.sl:16-305
 * as the host examples/llama2/bench_llama32_1b_int8.cpp:200-318 drives it: an int8 input vector, a position,
 * f32 logits out; f32 residual stream and norms, int8 activations, int8 weights pre-transposed [N, K]
 * (tensor_matmul_nt, i32 accumulation), int8 KV cache (acc / 256), grouped-query attention, f32 classifier.
 * The .sl text applies no RoPE and divides scores by the literal 8.0; both are kept.
 * Tensors (simp_llama_i8_load names): rms_att_w, rms_ffn_w [n_layers, dim], rms_final_w [dim], wcls
 * [vocab, dim] (f32); wq_t, wo_t [n_layers, dim, dim], wk_t, wv_t [n_layers, kv_dim, dim], w1_t, w3_t
 * [n_layers, hidden, dim], w2_t [n_layers, dim, hidden] (int8).  dim and hidden_dim must be multiples of 16,
 * head_dim 16, 32, 64 or 128.  The KV cache lives on the device and is zeroed at creation. */
typedef struct simp_llama_i8_config {
  int64_t dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, max_seq_len, head_dim;
} simp_llama_i8_config;
int simp_llama_i8_create(const simp_llama_i8_config* cfg, void** model);
int simp_llama_i8_load(void* model, const char* name, const void* host, size_t bytes);
/* One token: x_i8_host holds dim int8 values; logits_host (vocab floats) may be NULL. */
int simp_llama_i8_forward(void* model, const int8_t* x_i8_host, int64_t pos, float* logits_host);
/* The host's decode loop (bench_llama32_1b_int8.cpp:283-318): n_tokens forwards of the same input at
 * positions start_pos, start_pos + 1, ...; ms_out receives the device time of the whole loop.  The position
 * lives in device memory, so the loop runs without host synchronisation. */
int simp_llama_i8_decode_loop(void* model, const int8_t* x_i8_host, int64_t start_pos, int64_t n_tokens,
                              float* logits_host, float* ms_out);
/* Prefill of seq_len <= min(256, max_seq_len) tokens at once: the exported functions llama32_prefill_8 ... _256 of
 * examples/llama2/llama32_1b_int8_prefill.sl:11-232 (host: bench_llama32_1b_int8_prefill.cpp:180-215).  The seven
 * projections of a layer run as int8 GEMMs on the tensor cores.  x_i8_host is [seq_len, dim]; outputs (each may be
 * NULL): the residual stream x_fp32 [seq_len, dim] and the K / V cache rows [n_layers, seq_len, kv_dim].  The rows
 * also stay in the model's device cache (positions 0 .. seq_len-1), so decoding can continue at seq_len.  As in
 * the .sl text there is no clamp in the quantisation steps, no final norm and no classifier. */
int simp_llama_i8_prefill(void* model, const int8_t* x_i8_host, int64_t seq_len, float* x_fp32_host,
                          int8_t* k_cache_host, int8_t* v_cache_host, float* ms_out);
int simp_llama_i8_reset_cache(void* model);
int simp_llama_i8_destroy(void* model);

/* ---- multi-GPU (one process per GPU, NCCL over NVLink / NVSwitch) ---------------------------
 * Replaces: the reference's only parallel schemes, OpenMP row tiles (src/mlir/mlir_pipeline.cpp:265-364)
 * and host-side row chunks sharing B (simptensor/benchmarks/bench_int8_parallel_runner.cpp:70-91).
 * Rank 0 creates the NCCL unique id (128 bytes); the host carries it to the other ranks.  Collectives run
 * on the library stream.  With world == 1 every call degenerates to a local copy / no-op. */
#define SIMP_DIST_ID_BYTES 128
int simp_dist_unique_id(void* id_out, size_t bytes);
int simp_dist_init(int rank, int world, const void* id, size_t bytes);
int simp_dist_shutdown(void);
int simp_dist_rank(void);
int simp_dist_world(void);
int simp_dist_allgather(const void* send_dev, void* recv_dev, size_t bytes_per_rank);
/* In-place all-gather inside a buffer from simp_dist_symm_alloc, without NCCL: every rank stores its slice
 * (already at offset + rank * slice) straight into the peers' copies over NVLink and waits, bounded, for theirs.
 * For kilobyte-sized exchanges (tensor-parallel decode) this costs a launch and one NVLink round trip.
 * Collective and ordered like the NCCL calls; the first call allocates its flag words (not inside a capture). */
int simp_dist_allgather_peer(void* symm_local, size_t offset, size_t slice);
int simp_dist_allreduce_f32(float* buf_dev, size_t count);
/* N-sharded tensor_matmul on i8: A[M,K] replicated, this rank's column block of B ([K,N_local], or
 * [N_local,K] when b_transposed); C_blocks_dev receives world blocks of M x N_local i32, block r being
 * columns [r*N_local, (r+1)*N_local) of C.  One all-gather, no reduction: results stay bit-exact. */
int simp_dist_matmul_i8_nsharded(const void* A_dev, const int8_t* B_local_dev, int32_t* C_blocks_dev,
                                 int64_t M, int64_t K, int64_t N_local, int a_unsigned,
                                 int b_transposed);
/* The same GEMM with the exchange fused into the tensor-core kernel: every C tile is staged once in shared
 * memory and written into every rank's copy of the full row-major C[M, N_local*world] (own HBM by TMA store; the
 * peers', over NVLink, by plain stores paced at the link's rate), so the all-gather overlaps the main loop tile by
 * tile and C arrives in the layout tensor_matmul defines.  C_symm_dev must come from simp_dist_symm_alloc (a collective that allocates
 * `bytes` on every rank and maps all ranks' buffers through CUDA IPC).  N_local must be a multiple of 32 (whole
 * 32-column boxes are stored; a narrower block would spill into the neighbour's).  The call ends with a rendezvous
 * of all ranks on the library stream (epoch words exchanged by peer stores, bounded waits), which orders every
 * rank's stores before later work on the stream; its first use allocates the epoch words (a collective): make the
 * first call outside any stream capture.  Buffer re-use: a rank may overwrite C_symm (or anything a peer stores
 * into) only after a rendezvous that follows its own last read of it. */
int simp_dist_symm_alloc(size_t bytes, void** local_ptr);
int simp_dist_symm_free(void* local_ptr);
int simp_dist_barrier(void);
int simp_dist_matmul_i8_nsharded_fused(const void* A_dev, const int8_t* B_local_dev, int32_t* C_symm_dev,
                                       int64_t M, int64_t K, int64_t N_local, int a_unsigned,
                                       int b_transposed);

/* ---- memref-ABI shims ----------------------------------------------------------------------
 * What a GPU lowering pattern calls from compiled .sl code.  Arguments follow MLIR 14's std->LLVM
 * expansion of memref operands: a 1-D dynamic memref (what `!simp.array<T>` becomes,
 * src/mlir/lowering/ConvertSimpToMemRef.cpp:43-46) is (allocated, aligned, offset, size, stride); a
 * static rank-2 memref (a `!simp.tensor`) is (allocated, aligned, offset, size0, size1, stride0, stride1) --
 * the expansion the reference hosts write by hand (examples/llama2/generate_stories110M.cpp:12-22).
 * Data pointers are HOST pointers; each shim forwards to the simp_host_* entry point of the op.  Scalars
 * after the memrefs are the op's own operands in the order of the .sl builtin
 * (src/mlir/mlir_codegen.cpp:1388-1530, 2068-2260).  Return value: status as above. */
#define SIMP_MEMREF1(T, n) T* n##_allocated, T* n##_aligned, int64_t n##_offset, int64_t n##_size, int64_t n##_stride
#define SIMP_MEMREF2(T, n)                                                                        \
  T* n##_allocated, T* n##_aligned, int64_t n##_offset, int64_t n##_size0, int64_t n##_size1, \
      int64_t n##_stride0, int64_t n##_stride1
int32_t simp_rt_matmul_f32(SIMP_MEMREF1(float, lhs), SIMP_MEMREF1(float, rhs), SIMP_MEMREF1(float, out),
                           int64_t m, int64_t k, int64_t n, int64_t lhs_off, int64_t rhs_off, int64_t out_off);
int32_t simp_rt_rmsnorm_f32(SIMP_MEMREF1(float, x), SIMP_MEMREF1(float, w), SIMP_MEMREF1(float, y), int64_t n,
                            float eps, int64_t weight_offset);
int32_t simp_rt_softmax_f32(SIMP_MEMREF1(float, x), SIMP_MEMREF1(float, y), int64_t n, int64_t input_offset,
                            int64_t output_offset);
int32_t simp_rt_silu_f32(SIMP_MEMREF1(float, x), SIMP_MEMREF1(float, y), int64_t n);
int32_t simp_rt_matmul_quant(SIMP_MEMREF1(int8_t, qweights), SIMP_MEMREF1(float, scales),
                             SIMP_MEMREF1(float, zeros), SIMP_MEMREF1(float, x), SIMP_MEMREF1(float, out),
                             int64_t rows, int64_t cols, int64_t group_size, int64_t offset);
int32_t simp_rt_tensor_matmul_i8(SIMP_MEMREF2(int8_t, a), SIMP_MEMREF2(int8_t, b), SIMP_MEMREF2(int32_t, c));
int32_t simp_rt_tensor_matmul_nt_i8(SIMP_MEMREF2(int8_t, a), SIMP_MEMREF2(int8_t, bt), SIMP_MEMREF2(int32_t, c));
int32_t simp_rt_tensor_matmul_f32(SIMP_MEMREF2(float, a), SIMP_MEMREF2(float, b), SIMP_MEMREF2(float, c));

#ifdef __cplusplus
}
#endif
#endif /* SIMP_GPU_H_ */
