// ref_shim.cpp -- TEST INFRASTRUCTURE, not product code.
//
// C entry points around the reference's OWN sources (src/quant/quant_ref.cpp and
// src/cpu/cpu_kernels.cpp of ahmed-bensaad/QWENgine), which oracle/Makefile compiles where they
// lie in the reference checkout and links with this file into oracle/_ref/libq38ref.so.  Nothing
// of the reference is copied: this file only includes its headers and forwards calls.  The
// library pins oracle_port.c and serves as the timed CPU baseline of the benchmark.
#include <chrono>
#include <cstdint>
#include <cstring>
#include <memory>
#include <vector>

#include "cpu/cpu_kernels.h"      // cpu::get_vec_dot_n, cpu::quantize_q8_K   (src/cpu/cpu_kernels.h:13-36)
#include "cpu/thread_pool.h"      // cpu::ThreadPool                          (src/cpu/thread_pool.h:17-86)
#include "quant/quant_formats.h"  // dequantize_row_ref, quantize_row_q8_K_ref (src/quant/quant_formats.h:123-137)

using namespace q38rt;

namespace {
struct GemvCtx {
    cpu::vec_dot_n_fn fn;
    const uint8_t* W;
    size_t rb;
    int K;
    int64_t rows;
    const block_q8_K* x;
    size_t xs;
    int nb;
    float* y;
    int64_t y_ld;
    int reps;
};

// Static row split, one multi-column call per row: the drive pattern of bench_task_n in
// tests/kernels/test_cpu_gemv.cpp:52-60.
void gemv_task(void* vc, int tid, int n) {
    const GemvCtx& c = *(const GemvCtx*)vc;
    const int64_t r0 = c.rows * tid / n, r1 = c.rows * (tid + 1) / n;
    float yr[8];
    for (int rep = 0; rep < c.reps; rep++)
        for (int64_t r = r0; r < r1; r++) {
            c.fn(c.K, c.W + (size_t)r * c.rb, c.x, c.xs, yr);
            for (int b = 0; b < c.nb; b++) c.y[(size_t)b * c.y_ld + r] = yr[b];
        }
}

std::unique_ptr<cpu::ThreadPool> g_pool;
int g_pool_n = 0;
cpu::ThreadPool& pool(int n) {
    if (!g_pool || g_pool_n != n) {
        g_pool.reset();
        g_pool.reset(new cpu::ThreadPool(n));
        g_pool_n = n;
    }
    return *g_pool;
}
}  // namespace

extern "C" {

int q38ref_dequantize_row(uint32_t t, const void* src, float* dst, int64_t n) {
    return dequantize_row_ref((QuantFormat)t, src, dst, n) ? 0 : -1;
}

void q38ref_quantize_q8_K_scalar(const float* x, void* y, int64_t n) { quantize_row_q8_K_ref(x, (block_q8_K*)y, n); }
void q38ref_quantize_q8_K_avx2(const float* x, void* y, int K) { cpu::quantize_q8_K(x, (block_q8_K*)y, K); }

int q38ref_has_vec_dot(uint32_t t) { return cpu::get_vec_dot((QuantFormat)t) != nullptr; }

int q38ref_vec_dot_n(uint32_t t, int K, const void* w_row, const void* xq, size_t x_stride, int nb, float* y) {
    cpu::vec_dot_n_fn fn = cpu::get_vec_dot_n((QuantFormat)t, nb);
    if (!fn) return -1;
    fn(K, w_row, (const block_q8_K*)xq, x_stride, y);
    return 0;
}

// y[c*y_ld + r] = W[r,:] . x_c on `threads` pinned workers; returns seconds for `reps` passes (<0: unsupported).
double q38ref_gemv(uint32_t t, const void* W, size_t row_bytes, int K, int64_t M, const void* xq, size_t x_stride,
                   int nb, float* y, int64_t y_ld, int threads, int reps) {
    cpu::vec_dot_n_fn fn = cpu::get_vec_dot_n((QuantFormat)t, nb);
    if (!fn || threads < 1) return -1.0;
    GemvCtx c{fn, (const uint8_t*)W, row_bytes, K, M, (const block_q8_K*)xq, x_stride, nb, y, y_ld, reps};
    cpu::ThreadPool& p = pool(threads);
    const auto t0 = std::chrono::steady_clock::now();
    p.run(gemv_task, &c);
    return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
}

void q38ref_pool_release() { g_pool.reset(); g_pool_n = 0; }

float q38ref_fp16_to_fp32(uint16_t h) { return fp16_to_fp32(h); }
uint16_t q38ref_fp32_to_fp16(float f) { return fp32_to_fp16(f); }

}  // extern "C"
