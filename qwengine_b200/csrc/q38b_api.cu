// q38b_api.cu -- host side of libq38b200.so: context, launch planning, C ABI (include/q38b200.h).
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <new>

#include "../../include/q38b200.h"
#include "q38b_act.cuh"
#include "q38b_internal.h"
#include "q38b_gemv.cuh"

using namespace q38b;

namespace {

constexpr int NGROUPS = 2;
constexpr int GEMV_THREADS = 32 * (1 + NGROUPS * GROUP_WARPS);

#define Q38B_CUDA(ctx, call)                                   \
    do {                                                       \
        cudaError_t e_ = (call);                               \
        if (e_ != cudaSuccess) {                               \
            (ctx)->last_cuda = (int)e_;                        \
            return Q38B_ERR_CUDA;                              \
        }                                                      \
    } while (0)

int align_up(int v, int a) { return (v + a - 1) / a * a; }

bool known_format(uint32_t t) {
    switch (t) {
        case T_Q8_0: case T_Q4_K: case T_Q5_K: case T_Q6_K: case T_IQ3_XXS: case T_IQ3_S: case T_IQ4_XS: return true;
        default: return false;
    }
}

// alignment (bytes) the shared-memory loads of a format need from W and row_bytes
int format_alignment(uint32_t t) {
    switch (t) {
        case T_Q4_K: case T_Q5_K: return 16;
        case T_IQ4_XS: return 8;
        default: return 2;
    }
}

struct Plan {
    GemvArgs a;
    int grid;
    int smem;
};

// Carves the 227 KB of shared memory of one CTA: barriers | activation scales | activations | codebook |
// reduction buffers | NGROUPS rings of n_stages stages of 16 row slots.
int plan_gemv(const q38b_ctx* ctx, uint32_t type, int K, int M, int nb, Plan* p) {
    const int bb = block_bytes((int)type);
    const int nsb = K / 256;
    int cb_entries = type == T_IQ3_XXS ? 256 : type == T_IQ3_S ? 512 : 0;
    const int budget = ctx->smem_optin - 128;   // base is aligned up to 128 inside the kernel
    GemvArgs& a = p->a;
    a.nsb = nsb;
    a.n_tiles = (M + TILE_ROWS - 1) / TILE_ROWS;
    a.off_actd = 256;
    a.off_actq = a.off_actd + align_up(nsb * 32, 16);
    a.off_cb = a.off_actq + align_up(nb * K, 128);
    // rows of a group land 16 bytes (32 for the formats read with 64-bit loads) further round the 32 banks
    const int bank_skew = (type == T_Q4_K || type == T_Q5_K) ? 32 : 16;
    for (int rep_log2 = cb_entries ? 5 : 0; rep_log2 >= 0; rep_log2 -= (rep_log2 == 5 ? 2 : 3)) {
        a.cb_rep_log2 = rep_log2;
        a.off_red = a.off_cb + align_up(cb_entries * 4 << rep_log2, 128);
        a.off_stage = a.off_red + NGROUPS * 2 * GROUP_THREADS * 16;
        const int avail = budget - a.off_stage;
        // K-chunk sizes to try: the whole row, then fewer super-blocks, multiples of 4 first (8 half super-blocks
        // per 4 keep the 8 warps of a group evenly loaded)
        for (int pass = 0; pass < 2; pass++)
            for (int cs = nsb; cs >= 1; cs--) {
                const bool even = cs == nsb || cs % 4 == 0;
                if (even != (pass == 0)) continue;
                int slot = align_up(cs * bb + 32, 16);
                while (slot % 128 != bank_skew) slot += 16;
                const int stage = TILE_ROWS * slot;
                if (stage > 56 * 1024 && cs > 1) continue;
                const int stages = avail / (NGROUPS * stage);
                if (stages < 2) continue;
                a.chunk_sb = cs;
                a.n_chunks = (nsb + cs - 1) / cs;
                a.n_stages = std::min(stages, 4);
                a.slot_stride = slot;
                a.stage_bytes = stage;
                p->smem = a.off_stage + NGROUPS * a.n_stages * stage + 128;
                const int ctas_needed = (a.n_tiles + NGROUPS - 1) / NGROUPS;
                p->grid = std::max(1, std::min(ctx->sm_count, ctas_needed));
                return Q38B_OK;
            }
        if (!cb_entries) break;
    }
    return Q38B_ERR_NOMEM;
}

template <int FMT>
int launch_gemv(q38b_ctx* ctx, const Plan& p, cudaStream_t st) {
    auto kern = gemv_kernel<FMT, NGROUPS>;
    static int configured_device = -1;   // one opt-in per process and device is enough
    if (configured_device != ctx->device) {
        Q38B_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ctx->smem_optin));
        configured_device = ctx->device;
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)p.grid);
    cfg.blockDim = dim3(GEMV_THREADS);
    cfg.dynamicSmemBytes = (size_t)p.smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->pdl ? 1 : 0;
    Q38B_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, p.a));
    return Q38B_OK;
}

template <int KIND>
int launch_dequant(q38b_ctx* ctx, uint32_t type, const uint8_t* W, long long rb, int K, int rows, void* out, cudaStream_t st) {
    const long long n = (long long)rows * (K / 32);
    const unsigned blocks = (unsigned)((n + 127) / 128);
    switch (type) {
        case T_Q8_0: dequant_rows_kernel<T_Q8_0, KIND><<<blocks, 128, 0, st>>>(W, rb, K, rows, out); break;
        case T_Q4_K: dequant_rows_kernel<T_Q4_K, KIND><<<blocks, 128, 0, st>>>(W, rb, K, rows, out); break;
        case T_Q5_K: dequant_rows_kernel<T_Q5_K, KIND><<<blocks, 128, 0, st>>>(W, rb, K, rows, out); break;
        case T_Q6_K: dequant_rows_kernel<T_Q6_K, KIND><<<blocks, 128, 0, st>>>(W, rb, K, rows, out); break;
        case T_IQ3_XXS: dequant_rows_kernel<T_IQ3_XXS, KIND><<<blocks, 128, 0, st>>>(W, rb, K, rows, out); break;
        case T_IQ3_S: dequant_rows_kernel<T_IQ3_S, KIND><<<blocks, 128, 0, st>>>(W, rb, K, rows, out); break;
        case T_IQ4_XS: dequant_rows_kernel<T_IQ4_XS, KIND><<<blocks, 128, 0, st>>>(W, rb, K, rows, out); break;
        default: return Q38B_ERR_UNSUPPORTED;
    }
    Q38B_CUDA(ctx, cudaGetLastError());
    return Q38B_OK;
}

}  // namespace

extern "C" {

int q38b_ctx_create(int device, q38b_ctx** out) {
    if (!out) return Q38B_ERR_ARG;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0 || device < 0 || device >= n) return Q38B_ERR_NO_DEVICE;
    q38b_ctx* c = new (std::nothrow) q38b_ctx;
    if (!c) return Q38B_ERR_NOMEM;
    c->device = device;
    int rc = Q38B_OK;
    do {
        if (cudaSetDevice(device) != cudaSuccess) { rc = Q38B_ERR_CUDA; break; }
        cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, device);
        cudaDeviceGetAttribute(&c->smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
        if (cudaMalloc(&c->d_status, sizeof(int)) != cudaSuccess) { rc = Q38B_ERR_CUDA; break; }
        cudaMemset(c->d_status, 0, sizeof(int));
        const void *xxs = nullptr, *s = nullptr;
        if (cudaGetSymbolAddress((void**)&xxs, q38b_iq3xxs_grid) != cudaSuccess ||
            cudaGetSymbolAddress((void**)&s, q38b_iq3s_grid) != cudaSuccess) { rc = Q38B_ERR_CUDA; break; }
        c->d_cb_iq3xxs = (uint32_t*)xxs;
        c->d_cb_iq3s = (uint32_t*)s;
    } while (0);
    if (rc != Q38B_OK) {
        c->last_cuda = (int)cudaGetLastError();
        if (c->d_status) cudaFree(c->d_status);
        delete c;
        return rc;
    }
    *out = c;
    return Q38B_OK;
}

void q38b_ctx_destroy(q38b_ctx* ctx) {
    if (!ctx) return;
    if (ctx->d_status) cudaFree(ctx->d_status);
    delete ctx;
}

int q38b_ctx_check(q38b_ctx* ctx, void* stream) {
    if (!ctx) return Q38B_ERR_ARG;
    int bits = 0;
    Q38B_CUDA(ctx, cudaMemcpyAsync(&bits, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    Q38B_CUDA(ctx, cudaStreamSynchronize((cudaStream_t)stream));
    if (bits) {
        Q38B_CUDA(ctx, cudaMemsetAsync(ctx->d_status, 0, sizeof(int), (cudaStream_t)stream));
        return Q38B_ERR_DEVICE_WAIT;
    }
    return Q38B_OK;
}

int q38b_last_cuda_error(const q38b_ctx* ctx) { return ctx ? ctx->last_cuda : 0; }

int q38b_ctx_set_pdl(q38b_ctx* ctx, int enabled) {
    if (!ctx) return Q38B_ERR_ARG;
    ctx->pdl = enabled ? 1 : 0;
    return Q38B_OK;
}

const char* q38b_status_string(int s) {
    switch (s) {
        case Q38B_OK: return "ok";
        case Q38B_ERR_ARG: return "invalid argument";
        case Q38B_ERR_UNSUPPORTED: return "format has no kernel";
        case Q38B_ERR_ALIGN: return "pointer or stride misaligned for the format";
        case Q38B_ERR_CUDA: return "CUDA runtime error";
        case Q38B_ERR_DEVICE_WAIT: return "a bounded device-side wait ran out";
        case Q38B_ERR_NOMEM: return "shape does not fit the shared-memory plan";
        case Q38B_ERR_NO_DEVICE: return "no CUDA device (there is no CPU fallback)";
        default: return "unknown status";
    }
}

int q38b_format_supported(uint32_t type) { return known_format(type) ? 1 : 0; }

size_t q38b_row_bytes(uint32_t type, int K) {
    if (!known_format(type) || K <= 0 || K % 256) return 0;
    return (size_t)(K / 256) * (size_t)block_bytes((int)type);
}

size_t q38b_q8k_bytes(int K) { return K > 0 && K % 256 == 0 ? (size_t)(K / 256) * Q8K_BYTES : 0; }

int q38b_quantize_q8k(q38b_ctx* ctx, const float* x, long long x_ld, int K, int n_rows, void* q8k, long long q8k_stride,
                      void* stream) {
    if (!ctx || !x || !q8k || K <= 0 || K % 256 || n_rows < 1 || x_ld < K || q8k_stride < K / 256) return Q38B_ERR_ARG;
    if (((uintptr_t)x | (uintptr_t)q8k) & 3) return Q38B_ERR_ALIGN;
    const long long blocks = (long long)n_rows * (K / 256);
    quantize_q8k_kernel<<<(unsigned)((blocks + ACT_WARPS - 1) / ACT_WARPS), ACT_WARPS * 32, 0, (cudaStream_t)stream>>>(
        x, x_ld, K, n_rows, (uint8_t*)q8k, q8k_stride);
    Q38B_CUDA(ctx, cudaGetLastError());
    return Q38B_OK;
}

int q38b_swiglu_q8k(q38b_ctx* ctx, const float* g, const float* u, long long ld, int n, int n_rows, float* h, void* q8k,
                    long long q8k_stride, void* stream) {
    if (!ctx || !g || !u || n <= 0 || n % 256 || n_rows < 1 || ld < n || (q8k && q8k_stride < n / 256)) return Q38B_ERR_ARG;
    if (((uintptr_t)g | (uintptr_t)u | (uintptr_t)h | (uintptr_t)q8k) & 3) return Q38B_ERR_ALIGN;
    const long long blocks = (long long)n_rows * (n / 256);
    swiglu_q8k_kernel<<<(unsigned)((blocks + ACT_WARPS - 1) / ACT_WARPS), ACT_WARPS * 32, 0, (cudaStream_t)stream>>>(
        g, u, ld, n, n_rows, h, (uint8_t*)q8k, q8k_stride);
    Q38B_CUDA(ctx, cudaGetLastError());
    return Q38B_OK;
}

int q38b_gemv_q8k(q38b_ctx* ctx, uint32_t type, const void* W, size_t row_bytes, int K, int M, const void* q8k,
                  long long q8k_stride, int nb, float* y, long long y_ld, int accumulate, void* stream) {
    if (!ctx || !W || !q8k || !y) return Q38B_ERR_ARG;
    if (!known_format(type)) return Q38B_ERR_UNSUPPORTED;
    if (K <= 0 || K % 256 || M < 1 || nb < 1 || nb > 8 || y_ld < M || q8k_stride < K / 256) return Q38B_ERR_ARG;
    if (row_bytes < q38b_row_bytes(type, K)) return Q38B_ERR_ARG;
    const int al = format_alignment(type);
    if (((uintptr_t)W & 15) || (row_bytes % al) || ((uintptr_t)q8k & 3) || ((uintptr_t)y & 3)) return Q38B_ERR_ALIGN;
    Plan p;
    memset(&p, 0, sizeof(p));
    int rc = plan_gemv(ctx, type, K, M, nb, &p);
    if (rc != Q38B_OK) return rc;
    GemvArgs& a = p.a;
    a.W = (const uint8_t*)W;
    a.row_bytes = (long long)row_bytes;
    a.xq = (const uint8_t*)q8k;
    a.x_stride = q8k_stride;
    a.y = y;
    a.y_ld = y_ld;
    a.status = ctx->d_status;
    a.codebook = type == T_IQ3_XXS ? ctx->d_cb_iq3xxs : type == T_IQ3_S ? ctx->d_cb_iq3s : nullptr;
    a.K = K;
    a.M = M;
    a.nb = nb;
    a.accumulate = accumulate ? 1 : 0;
    cudaStream_t st = (cudaStream_t)stream;
    switch (type) {
        case T_Q8_0: return launch_gemv<T_Q8_0>(ctx, p, st);
        case T_Q4_K: return launch_gemv<T_Q4_K>(ctx, p, st);
        case T_Q5_K: return launch_gemv<T_Q5_K>(ctx, p, st);
        case T_Q6_K: return launch_gemv<T_Q6_K>(ctx, p, st);
        case T_IQ3_XXS: return launch_gemv<T_IQ3_XXS>(ctx, p, st);
        case T_IQ3_S: return launch_gemv<T_IQ3_S>(ctx, p, st);
        case T_IQ4_XS: return launch_gemv<T_IQ4_XS>(ctx, p, st);
        default: return Q38B_ERR_UNSUPPORTED;
    }
}

int q38b_dequant_rows(q38b_ctx* ctx, uint32_t type, const void* W, size_t row_bytes, int K, int rows, void* out, int out_kind,
                      void* stream) {
    if (!ctx || !W || !out || K <= 0 || K % 256 || rows < 1) return Q38B_ERR_ARG;
    if (!known_format(type)) return Q38B_ERR_UNSUPPORTED;
    if (row_bytes < q38b_row_bytes(type, K)) return Q38B_ERR_ARG;
    if (((uintptr_t)W & 1) || (row_bytes & 1) || ((uintptr_t)out & 3)) return Q38B_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    switch (out_kind) {
        case Q38B_OUT_F32: return launch_dequant<0>(ctx, type, (const uint8_t*)W, (long long)row_bytes, K, rows, out, st);
        case Q38B_OUT_F16: return launch_dequant<1>(ctx, type, (const uint8_t*)W, (long long)row_bytes, K, rows, out, st);
        case Q38B_OUT_BF16: return launch_dequant<2>(ctx, type, (const uint8_t*)W, (long long)row_bytes, K, rows, out, st);
        default: return Q38B_ERR_ARG;
    }
}

}  // extern "C"
