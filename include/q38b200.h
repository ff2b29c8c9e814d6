/*
 * q38b200.h -- C ABI of the B200 quantized matvec / prefill-GEMM library (libq38b200.so).
 *
 * Drop-in boundary for the decode / prefill linear algebra of the q38rt runtime (ahmed-bensaad/QWENgine).
 * Each entry point names the reference interface it replaces (file:line inside the reference project).
 * Conventions, all taken from the reference:
 *   - `type` is the ggml type id the reference's QuantFormat enum carries verbatim
 *     (include/q38rt/q38rt_types.h:36-67): Q8_0 = 8, Q4_K = 12, Q5_K = 13, Q6_K = 14, IQ3_XXS = 18,
 *     IQ3_S = 21, IQ4_XS = 23;
 *   - weights are row-major GGUF blocks exactly as in the file, `row_bytes` apart (src/cuda/gemv.cuh:26-29);
 *     M counts output rows, K the row length (a multiple of 256);
 *   - output column c of a multi-column call is y + c * y_ld (src/cuda/gemv.cuh:31-34);
 *   - the caller owns every buffer, kernels allocate nothing and only enqueue work on the caller's stream
 *     (`stream` is a cudaStream_t passed as void*); all pointers named *_dev are device pointers.
 * Activations are ggml Q8_K blocks (float d, int8 qs[256], int16 bsums[16]; src/quant/quant_formats.h:95), the format
 * the reference's CPU kernels consume (src/cpu/cpu_kernels.h:13-22), produced on the device bit-identically to
 * quantize_row_q8_K_ref (src/quant/quant_ref.cpp:353-381).
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

/* One context per process and GPU.  Holds the device codebooks, the device status word and launch attributes. */
int q38b_ctx_create(int device, q38b_ctx** out);
void q38b_ctx_destroy(q38b_ctx* ctx);
/* Reads (and clears) the device status word after synchronising `stream`; Q38B_ERR_DEVICE_WAIT if a kernel gave up. */
int q38b_ctx_check(q38b_ctx* ctx, void* stream);
int q38b_last_cuda_error(const q38b_ctx* ctx);
const char* q38b_status_string(int status);
/* Enable (1, default) or disable (0) programmatic dependent launch between consecutive kernels of a stream. */
int q38b_ctx_set_pdl(q38b_ctx* ctx, int enabled);

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
 * Column c of the activations starts q8k_stride blocks after column c - 1.  Each column's result is bit-identical
 * to a one-column call.  W_dev must be 16-byte aligned. */
int q38b_gemv_q8k(q38b_ctx* ctx, uint32_t type, const void* W_dev, size_t row_bytes, int K, int M, const void* q8k_dev,
                  long long q8k_stride, int nb, float* y_dev, long long y_ld, int accumulate, void* stream);

/* Replaces swiglu_rows + the requantisation for the down projection (src/cuda/ops.cu:126-141, 946-949; CPU:
 * src/runtime/engine.cpp:177-182, 1646): h = silu(g) * u for n_rows rows of n (row stride ld floats), written as
 * fp32 to h_dev (may be NULL) and as Q8_K blocks to q8k_dev (may be NULL). n must be a multiple of 256. */
int q38b_swiglu_q8k(q38b_ctx* ctx, const float* g_dev, const float* u_dev, long long ld, int n, int n_rows, float* h_dev,
                    void* q8k_dev, long long q8k_stride, void* stream);

/* Replaces dequant_rows_f16 (src/cuda/prefill.cu:802-822): rows of GGUF blocks -> dense [rows][K] values, each the
 * exact dequantize_row_ref value (src/quant/quant_ref.cpp:323-351) as fp32, or rounded once to fp16 / bf16. */
int q38b_dequant_rows(q38b_ctx* ctx, uint32_t type, const void* W_dev, size_t row_bytes, int K, int rows, void* out_dev,
                      int out_kind, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* Q38B200_H */
