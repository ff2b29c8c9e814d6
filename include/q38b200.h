/*
 * q38b200.h -- C ABI of the B200 quantized matvec / prefill-GEMM library (libq38b200.so).
 *
 * Drop-in boundary for the decode / prefill linear algebra of the q38rt runtime (ahmed-bensaad/QWENgine).
 * Each entry point names the reference interface it replaces (file:line inside the reference project).
 * Conventions, all taken from the reference:
 *   - `type` is the ggml type id the reference's QuantFormat enum carries verbatim
 *     (include/q38rt/q38rt_types.h:36-67): Q8_0 = 8, Q2_K = 10, Q4_K = 12, Q5_K = 13, Q6_K = 14, IQ2_XXS = 16,
 *     IQ2_XS = 17, IQ3_XXS = 18, IQ1_S = 19, IQ3_S = 21, IQ2_S = 22, IQ4_XS = 23, IQ1_M = 29 (the last six of the
 *     list: one-column kernel, exact dequantizer and prefill GEMM; several columns run as one launch per column);
 *   - weights are row-major GGUF blocks exactly as in the file, `row_bytes` apart (src/cuda/gemv.cuh:26-29);
 *     M counts output rows, K the row length (a multiple of 256);
 *   - output column c of a multi-column call is y + c * y_ld (src/cuda/gemv.cuh:31-34);
 *   - the caller owns every buffer, kernels allocate nothing and only enqueue work on the caller's stream
 *     (`stream` is a cudaStream_t passed as void*); all pointers named *_dev are device pointers.
 * Activations are ggml Q8_K blocks (float d, int8 qs[256], int16 bsums[16]; src/quant/quant_formats.h:95), the format
 * the reference's CPU kernels consume (src/cpu/cpu_kernels.h:13-22), produced on the device bit-identically to
 * quantize_row_q8_K_ref (src/quant/quant_ref.cpp:353-381); the *_act_q8 entry points take the reference GPU path's
 * per-32 format instead (ActQ8, src/cuda/gemv.cuh:14-21).
 * Every function returns 0 on success or a negative q38b_status; nothing calls exit().
 */
#ifndef Q38B200_H
#define Q38B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct q38b_ctx q38b_ctx;

enum q38b_status {
    Q38B_OK = 0,
    Q38B_ERR_ARG = -1,          /* null pointer, K not a multiple of 256, nb outside 1..8, ... */
    Q38B_ERR_UNSUPPORTED = -2,  /* format without a kernel (the reference returns false: src/cuda/gemv.cu:217,225) */
    Q38B_ERR_ALIGN = -3,        /* pointer or stride not aligned as the format needs */
    Q38B_ERR_CUDA = -4,         /* a CUDA runtime call failed; q38b_last_cuda_error() has the code */
    Q38B_ERR_DEVICE_WAIT = -5,  /* a bounded wait inside a kernel ran out; results of that launch are invalid */
    Q38B_ERR_NOMEM = -6,        /* shape does not fit the shared-memory plan or a fixed-size scratch */
    Q38B_ERR_NO_DEVICE = -7     /* no CUDA device; there is no CPU fallback */
};

enum q38b_out_kind { Q38B_OUT_F32 = 0, Q38B_OUT_F16 = 1, Q38B_OUT_BF16 = 2 };

/* One context per process and GPU.  Holds the device codebooks, the device status word, launch attributes and the work
 * areas of the top-k and of the multi-column matvec (64 MB: the K-part sums of rows longer than 8192).  The work areas
 * serve one launch at a time: issue a context's calls on one stream, or order the streams yourself. */
int q38b_ctx_create(int device, q38b_ctx** out);
void q38b_ctx_destroy(q38b_ctx* ctx);
/* Reads (and clears) the device status word after synchronising `stream`; Q38B_ERR_DEVICE_WAIT if a kernel gave up. */
int q38b_ctx_check(q38b_ctx* ctx, void* stream);
int q38b_last_cuda_error(const q38b_ctx* ctx);
const char* q38b_status_string(int status);
/* Bounded waits: a kernel that waits for another GPU (the cross-GPU barrier of the peer-store gather) gives up after
 * this many SM clocks, sets a status bit that q38b_ctx_check reports as Q38B_ERR_DEVICE_WAIT, and runs to its end; the
 * context stays usable.  Default 4e9 (about two seconds).  Waits inside one GPU (shared-memory barriers) keep a fixed
 * budget of about a second. */
int q38b_ctx_set_wait_budget_cycles(q38b_ctx* ctx, long long cycles);

/* Programmatic dependent launch lets a matvec start (and prefetch) while the previous KERNEL of the stream drains.  It
 * is always used between the kernels of a recorded pass.  For direct calls it is off by default, because a direct call
 * may follow a memcpy that fills its operands, which a programmatic launch does not wait for; 1 turns it on for
 * direct calls too (only when every matvec follows a kernel), 0 turns it off everywhere. */
int q38b_ctx_set_pdl(q38b_ctx* ctx, int enabled);
/* With programmatic dependent launch a matvec may start while the previous kernel of the stream is still running.  Its
 * activations always wait for that kernel; its weight stream waits too unless this option is 1, which promises that
 * the weights were written long before (resident model weights).  Passes (q38b_pass_run) stream resident matrices and
 * set it themselves.  Default 0. */
int q38b_ctx_set_static_weights(q38b_ctx* ctx, int enabled);
/* Single-column calls (nb = 1) normally run a dedicated dp4a kernel whose float summation order differs from the
 * tensor-core kernel used for nb >= 2 (both are exact in their integer parts and agree to ~1e-7).  With this option
 * set to 1, nb = 1 also runs the tensor-core kernel, so that every column of an nb-column call is bit-identical to
 * the one-column call, as gemv_q8n promises (src/cuda/gemv.cuh:31-34).  Columns of calls with nb >= 2 are always
 * bit-identical to each other across nb. */
int q38b_ctx_set_uniform_columns(q38b_ctx* ctx, int enabled);

/* Replaces gemv_q8_supported (src/cuda/gemv.cu:206-213): 1 if `type` has a matvec kernel here. */
int q38b_format_supported(uint32_t type);
/* Bytes of one row of K weights (quant_row_bytes, include/q38rt/q38rt_types.h), 0 if unsupported. */
size_t q38b_row_bytes(uint32_t type, int K);
/* Bytes of the Q8_K blocks of one activation vector of length K (292 per 256). */
size_t q38b_q8k_bytes(int K);

/* Replaces the Q8_K producers cpu::quantize_q8_K (src/cpu/cpu_kernels.cpp:785-828) and q8k_block_store
 * (src/cuda/ops.cu:43-76): n_rows vectors x_dev[r * x_ld .. + K) -> blocks q8k_dev + r * q8k_stride * 292. */
int q38b_quantize_q8k(q38b_ctx* ctx, const float* x_dev, long long x_ld, int K, int n_rows, void* q8k_dev,
                      long long q8k_stride, void* stream);

/* Replaces gemv_q8n / gemv_q8 (src/cuda/gemv.cu:215-233) with Q8_K activations as the CPU kernels take them
 * (vec_dot_n_fn, src/cpu/cpu_kernels.h:19-22): y_dev[c * y_ld + r] (+)= W[r,:] . x_c for r < M, c < nb (1..8).
 * Column c of the activations starts q8k_stride blocks after column c - 1.  Column results do not depend on nb for
 * nb >= 2 (and for nb = 1 too after q38b_ctx_set_uniform_columns).  W_dev must be 16-byte aligned. */
int q38b_gemv_q8k(q38b_ctx* ctx, uint32_t type, const void* W_dev, size_t row_bytes, int K, int M, const void* q8k_dev,
                  long long q8k_stride, int nb, float* y_dev, long long y_ld, int accumulate, void* stream);

/* Single-column matvec of up to three matrices of one format, K and row stride that read the SAME column, in one
 * launch: y[i][0..M[i]) = W[i] x.  The column comes either as Q8_K blocks (q8k, x_f32 = NULL) or as K floats
 * (x_f32, 16-byte aligned, q8k = NULL), which every CTA quantizes itself with the arithmetic of q38b_quantize_q8k:
 * results equal the separate quantize + q38b_gemv_q8k calls bit for bit.  Replaces runs of gemv_q8 calls on one
 * activation vector (q / k / v, gate / up: src/runtime/engine.cpp:1646, 1770-1849) and the quantize kernel before them
 * (src/cuda/gemv.cu:31-47).  Q38B_ERR_UNSUPPORTED when the shape runs only on the multi-column kernel (call
 * q38b_gemv_q8k per matrix then). */
int q38b_gemv_group(q38b_ctx* ctx, uint32_t type, int n_mats, const void* const* W, size_t row_bytes, int K, const int* M,
                    const void* q8k, const float* x_f32, float* const* y, void* stream);
/* Matvec straight from fp32 activations x_dev[c * x_ld .. + K), the form in which the reference's engine holds them
 * before quantize_act_q8 + gemv_q8n (src/cuda/gemv.cu:200-204, 215-228): quantizes the nb columns to Q8_K into
 * `q8k_scratch_dev` (caller-owned device scratch of at least nb * q38b_q8k_bytes(K) bytes) and runs q38b_gemv_q8k. */
int q38b_gemv_f32(q38b_ctx* ctx, uint32_t type, const void* W_dev, size_t row_bytes, int K, int M, const float* x_dev,
                  long long x_ld, int nb, float* y_dev, long long y_ld, int accumulate, void* q8k_scratch_dev,
                  size_t scratch_bytes, void* stream);

/* The reference GPU path's own activation format (ActQ8, src/cuda/gemv.cuh:14-21): int8 q[K], one scale d per 32 values
 * and s = d * sum(q) per 32 values; n_rows rows of K values, row r at q + r * K, d + r * K / 32, s + r * K / 32.
 * Replaces quantize_act_q8 (src/cuda/gemv.cu:31-47, 200-204), same arithmetic: d = amax / 127, q = round-half-even(v / d).
 * K must be a multiple of 32. */
int q38b_quantize_act_q8(q38b_ctx* ctx, const float* x_dev, int K, int n_rows, int8_t* q_dev, float* d_dev, float* s_dev,
                         void* stream);

/* Replaces gemv_q8n / gemv_q8 on ActQ8 activations (src/cuda/gemv.cuh:23-34, src/cuda/gemv.cu:206-233):
 * y_dev[c * y_ld + r] (+)= W[r,:] . x_c for c < nb, where x_c is the per-32 quantized column at q_dev + c * act_ld with
 * its scales at d_dev + c * act_ld / 32 (act_ld a multiple of 32, >= K).  The integer sums per 32 weights are exact and
 * each is scaled by its own activation scale.  Every column is computed by the one-column kernel, so column c equals
 * the nb = 1 call on that column bit for bit (the promise of src/cuda/gemv.cuh:31-34) and the cost grows linearly
 * with nb; the Q8_K entry points above are the fast path for several columns. */
int q38b_gemv_act_q8(q38b_ctx* ctx, uint32_t type, const void* W_dev, size_t row_bytes, int K, int M, const int8_t* q_dev,
                     const float* d_dev, int nb, int act_ld, float* y_dev, int y_ld, int accumulate, void* stream);

/* No counterpart in the reference.  q38b_gemv_f32 for callers that may not allocate device memory (an engine that
 * sized its arena at start-up, code running during stream capture, a loop that must not synchronise): the Q8_K
 * scratch is a fixed array inside the library, q38b_gemv_f32_static_capacity() bytes (158,848: up to 8 columns of
 * K = 17408, in general nb * K / 256 <= 544).  Larger requests return Q38B_ERR_NOMEM.  The call allocates nothing.  The
 * first call on a device looks the array's address up (make it before any stream capture, with the context's device
 * current).  All calls on a device share the array: calls that may overlap on the GPU (different streams) race, and
 * the array keeps the last call's blocks. */
int q38b_gemv_f32_static(q38b_ctx* ctx, uint32_t type, const void* W_dev, size_t row_bytes, int K, int M, const float* x_dev,
                         long long x_ld, int nb, float* y_dev, long long y_ld, int accumulate, void* stream);
size_t q38b_gemv_f32_static_capacity(void);

/* The same matvec with a fused all-gather for row-sharded matrices: every result is also stored at the same position
 * of n_peers (0..7) output buffers that live on other GPUs (peer-mapped pointers, see q38b_peer_*), so that after
 * q38b_peer_barrier every GPU holds the outputs of all shards.  No counterpart in the reference (single GPU). */
int q38b_gemv_q8k_scatter(q38b_ctx* ctx, uint32_t type, const void* W_dev, size_t row_bytes, int K, int M,
                          const void* q8k_dev, long long q8k_stride, int nb, float* y_dev, long long y_ld, int accumulate,
                          float* const* y_peers, int n_peers, void* stream);

/* Replaces swiglu_rows + the requantisation for the down projection (src/cuda/ops.cu:126-141, 946-949; CPU:
 * src/runtime/engine.cpp:177-182, 1646): h = silu(g) * u for n_rows rows of n (row stride ld floats), written as
 * fp32 to h_dev (may be NULL) and as Q8_K blocks to q8k_dev (may be NULL). n must be a multiple of 256. */
int q38b_swiglu_q8k(q38b_ctx* ctx, const float* g_dev, const float* u_dev, long long ld, int n, int n_rows, float* h_dev,
                    void* q8k_dev, long long q8k_stride, void* stream);

/* Replaces add_rmsnorm / add_rmsnorm_rows in front of the matvecs (src/cuda/ops.cuh:35-42, src/cuda/ops.cu:78-123): for
 * n_rows rows of n values (row stride ld floats) x += a (+ b) is written back when a or b is given (either may be NULL),
 * then xn = x * rsqrt(mean(x^2) + eps) * w is written as fp32 to xn_dev (may be NULL) and as Q8_K blocks to q8k_dev (may
 * be NULL; row r at q8k_dev + r * q8k_stride * 292): the residual add, the norm and the activation quantizer of the next
 * matvecs in one pass over the row.  n a multiple of 256, at most 8192; pointers 16-byte aligned. */
int q38b_add_rmsnorm_q8k(q38b_ctx* ctx, float* x_dev, const float* a_dev, const float* b_dev, const float* w_dev, int n,
                         long long ld, int n_rows, float eps, float* xn_dev, void* q8k_dev, long long q8k_stride, void* stream);

/* Replaces gemv_bf16 (src/cuda/gemv.cuh:27-28, src/cuda/gemv.cu:127-146): y[r] = W[r,:] . x for dense bf16 weights
 * W [N][K] (row-major, 16-byte aligned, K a multiple of 8), fp32 x and y, fp32 accumulation. */
int q38b_gemv_bf16(q38b_ctx* ctx, const void* W_bf16_dev, int K, int N, const float* x_dev, float* y_dev, void* stream);

/* Replaces topk (src/cuda/ops.cuh:142-144, src/cuda/ops.cu:823-903,1037-1044; called on the head's logits,
 * src/runtime/engine.cpp:1680,1910): for each of n_rows vectors of n logits (ld floats apart) the k largest values,
 * descending, equal values by ascending position, and their positions + index_offset; NaN ranks below everything; slots
 * past n get position -1.  vals_dev / idx_dev: [n_rows][out_ld].  1 <= k <= 64, n <= 393216, n_rows <= 8; no work buffer
 * argument (the context owns it), nothing allocated by the call. */
int q38b_topk(q38b_ctx* ctx, const float* logits_dev, long long ld, int n, int n_rows, int k, int index_offset, float* vals_dev,
              int* idx_dev, int out_ld, void* stream);

/* Replaces swiglu_rows_inplace (src/cuda/prefill.cuh:33-35, src/cuda/prefill.cu:132-151): for B rows of n values (row
 * stride ld floats) silu(G) * U is written IN PLACE over the first 2 n bytes of each row of G, as fp16
 * (out_kind = Q38B_OUT_F16, the reference's choice) or bf16 (Q38B_OUT_BF16, for q38b_gemm_prefill): the next GEMM reads
 * G as a 16-bit matrix with row stride 2 ld.  n a multiple of 8, ld a multiple of 4, 2 n bytes of shared memory. */
int q38b_swiglu_rows_inplace(q38b_ctx* ctx, float* G_dev, const float* U_dev, int B, int n, long long ld, int out_kind,
                             void* stream);

/* Replaces dequant_rows_f16 (src/cuda/prefill.cu:802-822): rows of GGUF blocks -> dense [rows][K] values, each the
 * exact dequantize_row_ref value (src/quant/quant_ref.cpp:323-351) as fp32, or rounded once to fp16 / bf16. */
int q38b_dequant_rows(q38b_ctx* ctx, uint32_t type, const void* W_dev, size_t row_bytes, int K, int rows, void* out_dev,
                      int out_kind, void* stream);

/* Replaces dequant_rows_f16 + gemm_f16 (src/cuda/prefill.cu:802-851; call site Engine::gemm_split,
 * src/runtime/engine.cpp:2308-2354) by one kernel: Y_dev[t * ldy + r] (+)= sum_k X[t][k] * W[r][k] for t < B tokens,
 * r < M rows; X_dev is bf16 [B][ldx] (16-byte aligned, ldx a multiple of 8), weights are GGUF blocks dequantized on
 * the fly to bf16 in shared memory and multiplied on tcgen05 tensor cores with fp32 accumulation in tensor memory.
 * What the tensor core multiplies, per format: Q8_0, IQ3_XXS, IQ3_S, IQ4_XS: the exact dequantize_row_ref value
 * (src/quant/quant_ref.cpp:323-351) rounded once to bf16; Q4_K, Q5_K, Q6_K: scale (d * sc) and minimum (dmin * m) are
 * rounded to bf16 first and applied to the exact integer by one bf16 fused multiply-add, so a weight may differ from
 * the rounded exact value by 2^-8 of its magnitude (outputs stay within 4e-3 of sum |w x|; the path's bound is 1e-2). */
int q38b_gemm_prefill(q38b_ctx* ctx, uint32_t type, const void* W_dev, size_t row_bytes, int K, int M, const void* X_dev,
                      long long ldx, int B, float* Y_dev, long long ldy, int accumulate, void* stream);

/* The same with fp16 operands, which is what the reference's own prefill path multiplies (dequant_rows_f16 writes fp16
 * weights, gemm_f16 takes fp16 activations: src/cuda/prefill.cuh:17-24): X_dev is fp16 [B][ldx]; weights are
 * dequantized to fp16 (the codebook formats and Q8_0: the exact value rounded once, i.e. dequant_rows_f16's output; the
 * K-quants: scale and minimum rounded to fp16 first, 2^-11 relative).  Y differs from dequant_rows_f16 + gemm_f16 only
 * by the order of the fp32 additions (and that scale rounding for the K-quants). */
int q38b_gemm_prefill_f16(q38b_ctx* ctx, uint32_t type, const void* W_dev, size_t row_bytes, int K, int M, const void* X_dev,
                          long long ldx, int B, float* Y_dev, long long ldy, int accumulate, void* stream);

/* ------------------------------------------------------------------------------------------------------------
 * All-HBM planner.  Replaces the reference's residency planner and split upload (plan_residency,
 * src/runtime/planner.cpp:91-163; SplitMat / upload_split, src/runtime/engine.h:55-85, engine.cpp:594-629): every
 * matrix is resident in HBM, row-sharded over the ranks (one process per GPU): rank g of G owns rows
 * [g*M/G, (g+1)*M/G).  A pass is a recorded sequence of quantize / matvec / SwiGLU / all-gather steps over
 * activation buffers that the pass owns; it replays as one CUDA graph (the decode_batch loop of
 * src/runtime/engine.cpp:1770-1849 reduced to its linear algebra).
 * ------------------------------------------------------------------------------------------------------------ */
typedef struct q38b_pass q38b_pass;

/* Multi-GPU: rank 0 makes a 128-byte id, every rank passes it to q38b_comm_init (NCCL underneath). */
int q38b_comm_unique_id(void* id128);
int q38b_comm_init(q38b_ctx* ctx, int n_ranks, int rank, const void* id128);

/* Peer-store gather (low-latency alternative to the NCCL all-gather; no counterpart in the single-GPU reference).
 * Device memory of one process is made visible to the others with CUDA IPC handles (64 bytes each, exchanged by the
 * caller, e.g. over torch.distributed).  q38b_peer_arena_create allocates this rank's arena (flag words plus room for
 * the fp32 buffers of passes created afterwards: every rank must create the same buffers in the same order) and
 * exports it; q38b_peer_connect takes the handles of all ranks (64 * n_ranks bytes, rank order);
 * q38b_peer_barrier enqueues a one-warp kernel that signals every peer and waits (bounded) for all of them. */
int q38b_peer_export(q38b_ctx* ctx, const void* dev_ptr, void* handle64);
int q38b_peer_import(q38b_ctx* ctx, const void* handle64, void** dev_ptr);
int q38b_peer_arena_create(q38b_ctx* ctx, size_t bytes, void* handle64);
int q38b_peer_connect(q38b_ctx* ctx, int n_ranks, int rank, const void* handles);
int q38b_peer_barrier(q38b_ctx* ctx, void* stream);

int q38b_pass_create(q38b_ctx* ctx, int max_nb, q38b_pass** out);
void q38b_pass_destroy(q38b_pass* pass);
/* Activation buffers owned by the pass; both return a buffer id >= 0 or a negative q38b_status. */
int q38b_pass_buffer_f32(q38b_pass* pass, int n);     /* fp32 [max_nb][n] */
int q38b_pass_buffer_q8k(q38b_pass* pass, int K);     /* Q8_K blocks [max_nb][K/256] */
void* q38b_pass_buffer_ptr(q38b_pass* pass, int buffer);
/* Resident matrices; return a matrix id >= 0.  _upload copies this rank's row shard of a host matrix of M rows into
 * HBM, packed (M divisible by n_shards);
 * _device adopts rows that are already on the device (M_local rows, not copied, not freed). */
int q38b_pass_matrix_upload(q38b_pass* pass, uint32_t type, const void* W_host, size_t row_bytes, int K, int M, int shard,
                            int n_shards);
int q38b_pass_matrix_device(q38b_pass* pass, uint32_t type, const void* W_dev, size_t row_bytes, int K, int M_local);
/* Steps, appended in execution order.  Offsets and counts are in floats per column. */
int q38b_pass_op_quantize(q38b_pass* pass, int src_f32, int src_off, int K, int dst_q8k);
int q38b_pass_op_gemv(q38b_pass* pass, int matrix, int src_q8k, int dst_f32, int dst_off);
int q38b_pass_op_swiglu(q38b_pass* pass, int g_f32, int g_off, int u_f32, int u_off, int n, int dst_q8k);
/* q38b_pass_op_gemv whose output stays on this GPU even in a peer-connected pass: for matrices that every rank holds
 * whole (replicated) because streaming them costs less than exchanging their outputs. */
int q38b_pass_op_gemv_local(q38b_pass* pass, int matrix, int src_q8k, int dst_f32, int dst_off);
/* The k best of n logits of buffer src_f32 (from float offset off) per column: dst_f32 gets k values followed by k
 * positions (int32 bit patterns), so that a run can return 8 k bytes per column instead of all logits. */
int q38b_pass_op_topk(q38b_pass* pass, int src_f32, int off, int n, int k, int dst_f32);
/* After q38b_peer_connect the fp32 buffers of a pass live in the arena and matvec steps push their outputs to every
 * peer; q38b_pass_op_barrier then makes them usable on all ranks.  One barrier may cover several matvecs. */
int q38b_pass_op_barrier(q38b_pass* pass);
/* 0: matvec steps of this pass keep their outputs local even when the context is peer-connected (default 1). */
int q38b_pass_set_peer_store(q38b_pass* pass, int enabled);
/* In-place all-gather over the ranks: rank g holds [off + g*count, off + (g+1)*count) of every column. */
int q38b_pass_op_allgather(q38b_pass* pass, int buf_f32, int off, int count_per_rank);
/* Runs the recorded steps for nb columns (1..max_nb) on `stream`; the first run for each nb captures the graph. */
int q38b_pass_run(q38b_pass* pass, int nb, void* stream);
/* End to end with host buffers: copies x_host [nb][x_len] into buffer `in_f32`, runs, copies [nb][y_len] of buffer
 * `out_f32` (from float offset out_off) back to y_host and synchronises. */
int q38b_pass_run_host(q38b_pass* pass, int nb, int in_f32, const float* x_host, int x_len, int out_f32, int out_off,
                       float* y_host, int y_len, void* stream);
/* Weight bytes one run streams from HBM on this rank (sum over the matvec steps). */
long long q38b_pass_weight_bytes(const q38b_pass* pass);
/* Kernels one single-column run launches on this rank (after merging, see q38b_pass_set_merge). */
int q38b_pass_kernel_count(const q38b_pass* pass);
/* Single-column runs on one GPU merge steps by default: matvecs of one format and shape class that read the same
 * column share a launch (q38b_gemv_group), and a quantize step whose output only feeds the matvecs right after it is
 * folded into them.  Results are bit-identical either way; enabled = 0 replays one kernel per recorded step. */
int q38b_pass_set_merge(q38b_pass* pass, int enabled);
/* ------------------------------------------------------------------------------------------------------------
 * GGUF files -> planner.  Replaces, for this path, the reference's GGUF v3 parser and split upload
 * (src/runtime/gguf_parser.h:70-146, src/runtime/engine.cpp:594-629): the file is memory-mapped, the key-value table
 * is skipped (general.alignment is honoured), the tensor-info table is read with bounds checks, and a 2-D weight
 * tensor goes to the pass row-sharded exactly like q38b_pass_matrix_upload.  GGUF stores dims[0] = row length K first.
 * ------------------------------------------------------------------------------------------------------------ */
typedef struct q38b_gguf q38b_gguf;
int q38b_gguf_open(const char* path, q38b_gguf** out);      /* Q38B_ERR_UNSUPPORTED: not GGUF v2/v3; Q38B_ERR_ARG: malformed */
void q38b_gguf_close(q38b_gguf* file);
int q38b_gguf_tensor_count(const q38b_gguf* file);
int q38b_gguf_find(const q38b_gguf* file, const char* name);   /* index, or -1 */
/* Any out pointer may be NULL.  type: ggml type id; dims: 4 entries, unused ones 1; data: inside the read-only mapping;
 * nbytes: 0 for a type whose block size this library does not know. */
int q38b_gguf_tensor(const q38b_gguf* file, int index, const char** name, uint32_t* type, int* n_dims, long long dims[4],
                     const void** data, size_t* nbytes);
/* Rows [shard * M / n_shards, (shard + 1) * M / n_shards) of tensor `index` (2-D, a supported format) -> matrix id. */
int q38b_pass_matrix_from_gguf(q38b_pass* pass, const q38b_gguf* file, int index, int shard, int n_shards);

#ifdef __cplusplus
}
#endif
#endif /* Q38B200_H */
