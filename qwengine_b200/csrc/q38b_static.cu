// q38b_static.cu -- matvec from fp32 activations for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc on the decode path: a runtime that sized one arena at start-up
// and hands out nothing afterwards (the q38rt engine works that way), code that runs while a stream is being
// captured, or a latency-critical loop in which an allocation would synchronise the device.  q38b_gemv_f32 asks such a
// caller for a scratch buffer; this variant brings its own: the Q8_K blocks of the activations go into a fixed
// array in the library's device image.  Every GPU that loads the library holds that array (155 KB) until exit.
#include <cuda_runtime.h>

#include "../../include/q38b200.h"
#include "q38b_internal.h"

namespace {

constexpr int STATIC_MAX_BLOCKS = 8 * 68;                    // 8 columns of K = 17408, or any nb * K/256 <= 544
constexpr size_t STATIC_SCRATCH_BYTES = (size_t)STATIC_MAX_BLOCKS * 292;

// Scratch of the entry point below.  In host code this name is only a handle for the runtime, never a device
// address: the address is looked up once per device with cudaGetSymbolAddress and that pointer goes to the kernels.
static __device__ __align__(256) unsigned char g_q8k_scratch[STATIC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
void* g_scratch_ptr[MAX_DEVICES] = {};

}  // namespace

extern "C" size_t q38b_gemv_f32_static_capacity(void) { return STATIC_SCRATCH_BYTES; }

extern "C" int q38b_gemv_f32_static(q38b_ctx* ctx, uint32_t type, const void* W, size_t row_bytes, int K, int M, const float* x,
                                    long long x_ld, int nb, float* y, long long y_ld, int accumulate, void* stream) {
    if (!ctx || nb < 1 || nb > 8 || K <= 0 || K % 256) return Q38B_ERR_ARG;
    if ((size_t)nb * q38b_q8k_bytes(K) > STATIC_SCRATCH_BYTES) return Q38B_ERR_NOMEM;   // beyond the built-in scratch
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev != ctx->device || dev < 0 || dev >= MAX_DEVICES) return Q38B_ERR_ARG;
    if (!g_scratch_ptr[dev]) {
        // set-up, first call on this device (the context's device is current): resolve the array's device address
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_q8k_scratch);
        if (e != cudaSuccess || !p) { ctx->last_cuda = (int)e; return Q38B_ERR_CUDA; }
        g_scratch_ptr[dev] = p;
    }
    // the quantizer overwrites every byte the matvec reads, so nothing has to be cleared between calls
    return q38b_gemv_f32(ctx, type, W, row_bytes, K, M, x, x_ld, nb, y, y_ld, accumulate, g_scratch_ptr[dev], STATIC_SCRATCH_BYTES,
                         stream);
}
