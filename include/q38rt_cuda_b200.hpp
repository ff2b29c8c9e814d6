// q38rt_cuda_b200.hpp -- the q38rt runtime's GPU entry points for the quantized matvec and the prefill GEMM,
// implemented on libq38b200.so.
//
// The reference runtime calls these functions of namespace q38rt::cuda (declared in src/cuda/gemv.cuh:14-37 and
// src/cuda/prefill.cuh:17-28 of the reference project, defined in src/cuda/gemv.cu:200-238 and
// src/cuda/prefill.cu:802-851):
//
//     gemv_q8_supported   quantize_act_q8   gemv_q8   gemv_q8n          (decode: Engine::gemv_gpu, engine.cpp:1450-1454)
//     dequant_rows_f16    gemm_f16    cublas_create / cublas_bind / cublas_destroy   (prefill: Engine::gemm_split, :2308-2354)
//
// This header DEFINES them (external linkage, like the reference's own definitions), with the reference's exact
// signatures, on top of the C ABI of include/q38b200.h.  Compile exactly ONE translation unit of the runtime with it
// (for instance a file q38rt_b200.cpp that only includes this header), drop src/cuda/gemv.cu from the build, delete the
// five prefill functions above from src/cuda/prefill.cu, and link libq38b200.so: src/runtime/engine.cpp and every
// other caller compile and run unchanged.
//
// Inside the reference tree (the include path holds "cuda/gemv.cuh") the reference's own declarations are used; anywhere
// else the header declares QuantFormat and ActQ8 itself, identically, so that it can be tested without the reference.
//
// Behaviour kept from the reference: formats without a kernel make gemv_q8 / gemv_q8n / dequant_rows_f16 return false
// (src/cuda/gemv.cu:217,225); every call is enqueued on the caller's stream and returns; nothing is allocated on the
// decode path (the per-device context is created by the first call, so make one call before any stream capture); a
// failed GEMM ends the process like the reference's cuBLAS error path (src/cuda/prefill.cu:847-850).
//
// Differences, all invisible to engine.cpp:
//  * The prefill pair is fused.  dequant_rows_f16 does not write the fp16 scratch: it records (format, rows, stride)
//    under the scratch pointer, and the gemm_f16 call that receives that pointer as W runs one tcgen05 kernel that
//    dequantizes the GGUF rows to fp16 in shared memory (q38b_gemm_prefill_f16).  The weights must still be valid when
//    gemm_f16 runs, which holds for the reference's call sites (the GEMM directly follows its dequantization on the same
//    stream).  Define Q38RT_B200_EAGER_DEQUANT to make dequant_rows_f16 also write the fp16 rows (callers that read
//    the scratch themselves, like the reference's kernel tests).  gemm_f16 on fp16 rows that no dequant_rows_f16 call
//    recorded (the reference's BF16 projections, Engine::gemm_bf16) is not provided and ends the process with a message.
//  * gemv_q8n runs one launch per column (each column is the gemv_q8 result bit for bit, as src/cuda/gemv.cuh:31-34
//    promises); the multi-column tensor-core kernel takes Q8_K activations (q38b_gemv_q8k).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include "q38b200.h"

#if defined(__has_include)
#if __has_include("cuda/gemv.cuh") && __has_include("q38rt/q38rt_types.h")
#define Q38RT_B200_IN_REFERENCE_TREE 1
#endif
#endif

#if defined(Q38RT_B200_IN_REFERENCE_TREE)
#include "cuda/gemv.cuh"
#include "q38rt/q38rt_types.h"
// src/cuda/prefill.cuh also declares attention and DeltaNet kernels and pulls in their headers; only these five
// declarations of it (lines 17-28) are needed here
namespace q38rt {
namespace cuda {
bool dequant_rows_f16(QuantFormat type, const void* W, size_t row_bytes, int K, int rows, __half* out, cudaStream_t st);
void gemm_f16(void* cublas, const __half* W, int N, int K, const __half* X, int ldx, int B, float* Y, int ldy,
              bool accumulate, cudaStream_t st);
void* cublas_create();
bool cublas_bind(void* cublas, cudaStream_t st, void* workspace, size_t bytes);
void cublas_destroy(void* h);
}  // namespace cuda
}  // namespace q38rt
#else
namespace q38rt {
// the ggml type ids the reference keeps verbatim (include/q38rt/q38rt_types.h:36-67); only the ones the path names
enum class QuantFormat : uint32_t {
    FP32 = 0, FP16 = 1, Q8_0 = 8, Q2_K = 10, Q4_K = 12, Q5_K = 13, Q6_K = 14, IQ2_XXS = 16, IQ2_XS = 17, IQ3_XXS = 18,
    IQ1_S = 19, IQ3_S = 21, IQ2_S = 22, IQ4_XS = 23, IQ1_M = 29, BF16 = 30, INVALID = 0xFFFFFFFFu,
};
namespace cuda {
struct ActQ8 {             // src/cuda/gemv.cuh:14-21
    int8_t* q = nullptr;   // [K]
    float* d = nullptr;    // [K/32]
    float* s = nullptr;    // [K/32]
};
void quantize_act_q8(const float* x, int K, int n_rows, ActQ8 out, cudaStream_t st);
bool gemv_q8(QuantFormat type, const void* W, size_t row_bytes, int K, int N, const ActQ8& act, float* y, cudaStream_t st,
             bool accumulate = false);
bool gemv_q8n(QuantFormat type, const void* W, size_t row_bytes, int K, int N, const ActQ8& act, int nb, int act_ld, float* y,
              int y_ld, cudaStream_t st, bool accumulate = false);
bool gemv_q8_supported(QuantFormat type);
bool dequant_rows_f16(QuantFormat type, const void* W, size_t row_bytes, int K, int rows, __half* out, cudaStream_t st);
void gemm_f16(void* cublas, const __half* W, int N, int K, const __half* X, int ldx, int B, float* Y, int ldy,
              bool accumulate, cudaStream_t st);
void* cublas_create();
bool cublas_bind(void* cublas, cudaStream_t st, void* workspace, size_t bytes);
void cublas_destroy(void* h);
}  // namespace cuda
}  // namespace q38rt
#endif

namespace q38rt {
namespace cuda {
namespace b200 {

// One library context per device, created by the first call on that device (the reference's launchers keep their
// per-process state the same way, src/cuda/gemv.cu:148,157-166).  One thread issues the runtime's GPU work.
inline q38b_ctx* context() {
    static q38b_ctx* per_device[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!per_device[dev] && q38b_ctx_create(dev, &per_device[dev]) != Q38B_OK) per_device[dev] = nullptr;
    return per_device[dev];
}

[[noreturn]] inline void fatal(const char* what, int status) {
    std::fprintf(stderr, "q38rt/b200: %s failed: %s\n", what, q38b_status_string(status));
    std::exit(1);
}

// What the last dequant_rows_f16 calls stood for: fp16 scratch pointer -> the GGUF rows it would hold.
struct PendingRows { const __half* out; QuantFormat type; const void* W; size_t row_bytes; int K, rows; };
inline PendingRows* pending(const __half* out, bool claim) {
    static PendingRows slots[8] = {};
    PendingRows* free_slot = &slots[0];
    for (PendingRows& p : slots) {
        if (p.out == out) return &p;
        if (!p.out) free_slot = &p;
    }
    if (!claim) return nullptr;
    return free_slot;   // all slots taken: the oldest convention does not matter, the runtime uses one scratch buffer
}

}  // namespace b200

bool gemv_q8_supported(QuantFormat type) { return q38b_format_supported((uint32_t)type) != 0; }

void quantize_act_q8(const float* x, int K, int n_rows, ActQ8 out, cudaStream_t st) {
    const int rc = q38b_quantize_act_q8(b200::context(), x, K, n_rows, out.q, out.d, out.s, (void*)st);
    if (rc != Q38B_OK) b200::fatal("quantize_act_q8", rc);
}

bool gemv_q8n(QuantFormat type, const void* W, size_t row_bytes, int K, int N, const ActQ8& act, int nb, int act_ld, float* y,
              int y_ld, cudaStream_t st, bool accumulate) {
    if (nb < 1 || nb > 7 || !gemv_q8_supported(type)) return false;   // the reference's limits (src/cuda/gemv.cu:217)
    const int rc = q38b_gemv_act_q8(b200::context(), (uint32_t)type, W, row_bytes, K, N, act.q, act.d, nb, act_ld, y, y_ld,
                                    accumulate ? 1 : 0, (void*)st);
    if (rc != Q38B_OK) b200::fatal("gemv_q8n", rc);
    return true;
}

bool gemv_q8(QuantFormat type, const void* W, size_t row_bytes, int K, int N, const ActQ8& act, float* y, cudaStream_t st,
                    bool accumulate) {
    return gemv_q8n(type, W, row_bytes, K, N, act, 1, K, y, N, st, accumulate);
}

bool dequant_rows_f16(QuantFormat type, const void* W, size_t row_bytes, int K, int rows, __half* out, cudaStream_t st) {
    if (!q38b_format_supported((uint32_t)type)) return false;
    b200::PendingRows* p = b200::pending(out, true);
    *p = b200::PendingRows{out, type, W, row_bytes, K, rows};
#if defined(Q38RT_B200_EAGER_DEQUANT)
    const int rc = q38b_dequant_rows(b200::context(), (uint32_t)type, W, row_bytes, K, rows, out, Q38B_OUT_F16, (void*)st);
    if (rc != Q38B_OK) b200::fatal("dequant_rows_f16", rc);
#else
    (void)st;
#endif
    return true;
}

void gemm_f16(void* cublas, const __half* W, int N, int K, const __half* X, int ldx, int B, float* Y, int ldy, bool accumulate,
                     cudaStream_t st) {
    (void)cublas;
    const b200::PendingRows* p = b200::pending(W, false);
    if (!p || p->K != K || p->rows < N) {
        std::fprintf(stderr, "q38rt/b200: gemm_f16 on fp16 rows that no dequant_rows_f16 call produced (N=%d K=%d) is not provided\n", N, K);
        std::exit(1);
    }
    const int rc = q38b_gemm_prefill_f16(b200::context(), (uint32_t)p->type, p->W, p->row_bytes, K, N, X, ldx, B, Y, ldy,
                                         accumulate ? 1 : 0, (void*)st);
    if (rc != Q38B_OK) b200::fatal("gemm_f16", rc);
}

#if defined(Q38RT_B200_WITH_TOPK)
// topk of the sampling step (src/cuda/ops.cuh:142-144 of the reference project), for builds that also drop it from
// src/cuda/ops.cu: the same result (values descending, equal values by ascending position); `work` is not used.
void topk(const float* logits, int n, int k, int index_offset, float* vals, int* idx, void* work, cudaStream_t st) {
    (void)work;
    const int rc = q38b_topk(b200::context(), logits, n, n, 1, k, index_offset, vals, idx, k, (void*)st);
    if (rc != Q38B_OK) b200::fatal("topk", rc);
}
size_t topk_work_bytes(int) { return 16; }
#endif

// The GEMM needs no library handle or workspace here; the runtime still gets a non-null token to pass around.
void* cublas_create() { return b200::context(); }
bool cublas_bind(void* cublas, cudaStream_t, void*, size_t) { return cublas != nullptr; }
void cublas_destroy(void*) {}

}  // namespace cuda
}  // namespace q38rt
