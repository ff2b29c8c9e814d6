// Calls the reference runtime's GPU entry points (namespace q38rt::cuda) the way src/runtime/engine.cpp does
// (gemv_gpu: engine.cpp:1450-1454; gemm_split: engine.cpp:2308-2354), through include/q38rt_cuda_b200.hpp.  Built by the
// tests into a small shared library; all pointers are device pointers.
#include "q38rt_cuda_b200.hpp"

using namespace q38rt;
using namespace q38rt::cuda;

extern "C" int probe_decode(uint32_t type, const void* W, size_t row_bytes, int K, int N, const float* x, int nb, int8_t* q, float* d,
                            float* s, float* y) {
    if (!gemv_q8_supported((QuantFormat)type)) return 1;
    ActQ8 act;
    act.q = q;
    act.d = d;
    act.s = s;
    quantize_act_q8(x, K, nb, act, nullptr);
    if (nb == 1) return gemv_q8((QuantFormat)type, W, row_bytes, K, N, act, y, nullptr) ? 0 : 2;
    return gemv_q8n((QuantFormat)type, W, row_bytes, K, N, act, nb, K, y, N, nullptr) ? 0 : 2;
}

extern "C" int probe_prefill(uint32_t type, const void* W, size_t row_bytes, int K, int rows, __half* scratch, const __half* X, int ldx,
                             int B, float* Y, int ldy) {
    void* handle = cublas_create();
    if (!handle || !cublas_bind(handle, nullptr, nullptr, 0)) return 3;
    // rows per dequant + GEMM block as in Engine::gemm_split: two blocks through the same scratch
    const int R = (rows + 1) / 2;
    for (int r0 = 0; r0 < rows; r0 += R) {
        const int n = rows - r0 < R ? rows - r0 : R;
        if (!dequant_rows_f16((QuantFormat)type, (const uint8_t*)W + (size_t)r0 * row_bytes, row_bytes, K, n, scratch, nullptr)) return 1;
        gemm_f16(handle, scratch, n, K, X, ldx, B, Y + r0, ldy, false, nullptr);
    }
    cublas_destroy(handle);
    return 0;
}
