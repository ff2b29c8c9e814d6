// q38b_act.cuh -- activation-side kernels (Q8_K quantizer, SwiGLU) and the exact row dequantizer.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

#include "q38b_decode.cuh"
#include "q38b_pipe.cuh"

namespace q38b {

#define Q38B_CODEBOOK_QUALIFIER __device__ const
#include "codebooks.inc"
#undef Q38B_CODEBOOK_QUALIFIER

// Two and four int32 values saturated to int8 and packed (cvt.pack: low byte = the last operand of each pair).
__device__ __forceinline__ uint32_t pack_s8x4(int q0, int q1, int q2, int q3) {
    uint32_t hi, w;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(q3), "r"(q2), "r"(0));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(w) : "r"(q1), "r"(q0), "r"(hi));
    return w;
}

// One warp turns 256 floats, eight per lane (lane l: elements 8l .. 8l+7), into the values of a ggml Q8_K block.
// Arithmetic of quantize_row_q8_K_ref (src/quant/quant_ref.cpp:353-381): the FIRST element of largest magnitude, with
// its sign, maps to -127 (iscale = -127 / that element); q = min(127, round-half-even(iscale * x)); d = 1 / iscale; a
// block of zeros stays all zero.  Outputs: this lane's eight int8 values packed in w0 | w1, their sum s8, and d (the
// same in every lane).
__device__ __forceinline__ void q8k_block_core(const float (&v)[8], uint32_t& w0, uint32_t& w1, int& s8, float& d) {
    // Magnitudes compare like their bit patterns, so the block maximum is an integer maximum: one REDUX over the warp.
    uint32_t mag[8], lane_top = 0;
#pragma unroll
    for (int e = 0; e < 8; e++) {
        mag[e] = __float_as_uint(v[e]) & 0x7FFFFFFFu;
        lane_top = max(lane_top, mag[e]);
    }
    const uint32_t top = __reduce_max_sync(0xffffffffu, lane_top);
    w0 = 0u; w1 = 0u; s8 = 0; d = 0.0f;
    if (top == 0u) return;
    // First occurrence: the lowest lane that holds the maximum (ballot + find-first-set), its lowest such element.
    float lead = 0.0f;
    bool have = false;
#pragma unroll
    for (int e = 0; e < 8; e++) {
        const bool hit = !have && mag[e] == top;
        lead = hit ? v[e] : lead;
        have = have || hit;
    }
    const int owner = __ffs((int)__ballot_sync(0xffffffffu, have)) - 1;
    const float iscale = __fdiv_rn(-127.0f, __shfl_sync(0xffffffffu, lead, owner));
    int qv[8];
#pragma unroll
    for (int e = 0; e < 8; e++) qv[e] = __float2int_rn(__fmul_rn(iscale, v[e]));   // >= -127; the pack clamps at +127
    w0 = pack_s8x4(qv[0], qv[1], qv[2], qv[3]);
    w1 = pack_s8x4(qv[4], qv[5], qv[6], qv[7]);
    s8 = __dp4a((int)w0, 0x01010101, __dp4a((int)w1, 0x01010101, 0));
    d = __fdiv_rn(1.0f, iscale);
}

// The block as ggml lays it out (float d | int8 qs[256] | int16 bsums[16], 292 bytes, 4-byte aligned) from the core's
// outputs: lane l owns qs[8l .. 8l+7]; a bsum covers 16 values, i.e. a pair of lanes.
__device__ __forceinline__ void q8k_block_from_regs(const float (&v)[8], uint8_t* blk) {
    const int lane = threadIdx.x & 31;
    uint32_t w0, w1;
    int s8;
    float d;
    q8k_block_core(v, w0, w1, s8, d);
    uint32_t* words = (uint32_t*)blk;
    words[1 + 2 * lane] = w0;
    words[2 + 2 * lane] = w1;
    const int pair_sum = s8 + __shfl_down_sync(0xffffffffu, s8, 1);
    int16_t* bsums = (int16_t*)(blk + 4 + 256);
    if (!(lane & 1)) bsums[lane >> 1] = (int16_t)pair_sum;
    if (lane == 0) words[0] = __float_as_uint(d);
}

constexpr int ACT_WARPS = 8;

// One warp quantizes 256 floats at `src` (lane l holds elements 8l..8l+7) into the Q8_K block at `blk`.
// COHERENT: read through L2 only (the floats were written by another SM during this kernel).
template <bool COHERENT>
__device__ __forceinline__ void quantize_block(const float* src, uint8_t* blk) {
    const int lane = threadIdx.x & 31;
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; e++) v[e] = COHERENT ? __ldcg(src + 8 * lane + e) : src[8 * lane + e];
    q8k_block_from_regs(v, blk);
}

// h = silu(g) * u, the CPU formula of the reference (src/runtime/engine.cpp:177-182): g / (1 + expf(-g)) * u
__device__ __forceinline__ float swiglu_value(float gv, float uv) { return __fmul_rn(__fdiv_rn(gv, __fadd_rn(1.0f, expf(-gv))), uv); }

// one warp, 256 values
template <bool COHERENT>
__device__ __forceinline__ void swiglu_block(const float* g, const float* u, float* h, uint8_t* blk) {
    const int lane = threadIdx.x & 31;
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; e++) {
        const float gv = COHERENT ? __ldcg(g + 8 * lane + e) : g[8 * lane + e];
        const float uv = COHERENT ? __ldcg(u + 8 * lane + e) : u[8 * lane + e];
        v[e] = swiglu_value(gv, uv);
    }
    if (h) {
#pragma unroll
        for (int e = 0; e < 8; e++) h[8 * lane + e] = v[e];
    }
    if (blk) q8k_block_from_regs(v, blk);
}

static __global__ void __launch_bounds__(ACT_WARPS * 32) quantize_q8k_kernel(const float* __restrict__ x, long long x_ld, int K,
                                                                       int n_rows, uint8_t* __restrict__ out,
                                                                       long long out_stride) {
    const int nsb = K >> 8;
    const long long blk = (long long)blockIdx.x * ACT_WARPS + (threadIdx.x >> 5);
    if (blk >= (long long)n_rows * nsb) return;
    const int r = (int)(blk / nsb), sb = (int)(blk % nsb);
    quantize_block<false>(x + (size_t)r * x_ld + (size_t)sb * 256, out + ((size_t)r * out_stride + sb) * 292);
}

// The reference GPU path's activation format (ActQ8, src/cuda/gemv.cuh:14-21; quantizer src/cuda/gemv.cu:31-47): one
// warp per 32 values, d = amax / 127, q = round-half-even(v / d) (an all-zero block stays zero), s = d * sum q.
static __global__ void __launch_bounds__(ACT_WARPS * 32) quantize_act_q8_kernel(const float* __restrict__ x, long long n_blocks,
                                                                          int8_t* __restrict__ q, float* __restrict__ d,
                                                                          float* __restrict__ s) {
    const long long blk = (long long)blockIdx.x * ACT_WARPS + (threadIdx.x >> 5);
    if (blk >= n_blocks) return;
    const int lane = threadIdx.x & 31;
    const float v = x[blk * 32 + lane];
    const float amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(v) & 0x7FFFFFFFu));
    const float dd = __fdiv_rn(amax, 127.0f);
    const int qi = dd > 0.0f ? __float2int_rn(__fdiv_rn(v, dd)) : 0;
    q[blk * 32 + lane] = (int8_t)qi;
    const int sum = __reduce_add_sync(0xffffffffu, qi);
    if (lane == 0) {
        d[blk] = dd;
        s[blk] = __fmul_rn(dd, (float)sum);
    }
}

static __global__ void __launch_bounds__(ACT_WARPS * 32) swiglu_q8k_kernel(const float* __restrict__ g, const float* __restrict__ u,
                                                                     long long ld, int n, int n_rows, float* __restrict__ h,
                                                                     uint8_t* __restrict__ out, long long out_stride,
                                                                     const PeerSync sync, int* status) {
    if (sync.n > 0) {   // gate and up were completed by the other GPUs: cross-GPU barrier first
        peer_sync_wait(sync, blockIdx.x == 0, (int)threadIdx.x, status);
        __syncthreads();
    }
    const int nsb = n >> 8;
    const long long blk = (long long)blockIdx.x * ACT_WARPS + (threadIdx.x >> 5);
    if (blk >= (long long)n_rows * nsb) return;
    const int r = (int)(blk / nsb), sb = (int)(blk % nsb);
    const size_t off = (size_t)r * ld + (size_t)sb * 256;
    swiglu_block<false>(g + off, u + off, h ? h + off : nullptr, out ? out + ((size_t)r * out_stride + sb) * 292 : nullptr);
}

// Residual add + RMSNorm + Q8_K in one pass over the row (replaces k_add_rmsnorm feeding the matvecs,
// src/cuda/ops.cu:78-123): x += a (+ b) is written back (the residual stream), xn = x * rsqrt(mean(x^2) + eps) * w goes
// out as fp32 (optional) and as the Q8_K blocks the next matvecs read.  One CTA per row, one warp per 256 values: every
// value stays in a register from the load to the quantizer.  n a multiple of 256, at most 32 * 256.
static __global__ void __launch_bounds__(1024) add_rmsnorm_q8k_kernel(float* __restrict__ x, const float* __restrict__ a,
                                                                      const float* __restrict__ b, const float* __restrict__ w, int n,
                                                                      long long ld, float eps, float* __restrict__ xn,
                                                                      uint8_t* __restrict__ q8k, long long q8k_stride) {
    __shared__ float part[32];
    __shared__ float s_scale;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const size_t ro = (size_t)blockIdx.x * ld, at = ro + (size_t)warp * 256 + 8 * lane;
    float v[8];
    {
        const float4 lo = *(const float4*)(x + at), hi = *(const float4*)(x + at + 4);
        v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
    }
    if (a) {
#pragma unroll
        for (int e = 0; e < 8; e++) v[e] = __fadd_rn(v[e], a[at + e]);
    }
    if (b) {
#pragma unroll
        for (int e = 0; e < 8; e++) v[e] = __fadd_rn(v[e], b[at + e]);
    }
    if (a || b) {
        *(float4*)(x + at) = make_float4(v[0], v[1], v[2], v[3]);
        *(float4*)(x + at + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    float ss = 0.0f;
#pragma unroll
    for (int e = 0; e < 8; e++) ss = fmaf(v[e], v[e], ss);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) part[warp] = ss;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? part[lane] : 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) s_scale = rsqrtf(t / (float)n + eps);
    }
    __syncthreads();
    const float scale = s_scale;
    const float4 wl = *(const float4*)(w + (size_t)warp * 256 + 8 * lane), wh = *(const float4*)(w + (size_t)warp * 256 + 8 * lane + 4);
    const float ww[8] = {wl.x, wl.y, wl.z, wl.w, wh.x, wh.y, wh.z, wh.w};
#pragma unroll
    for (int e = 0; e < 8; e++) v[e] = __fmul_rn(__fmul_rn(v[e], scale), ww[e]);
    if (xn) {
        *(float4*)(xn + at) = make_float4(v[0], v[1], v[2], v[3]);
        *(float4*)(xn + at + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    if (q8k) q8k_block_from_regs(v, q8k + ((size_t)blockIdx.x * q8k_stride + warp) * 292);
}

// y[r] = W[r,:] . x for dense bf16 weights (the model's two small per-layer projections, 48 x 5120; replaces gemv_bf16,
// src/cuda/gemv.cu:127-146, 235-238).  One CTA of BF16_THREADS per row: every thread takes 16-byte pieces (eight bf16) of
// the row, fp32 multiply-adds, a shuffle tree per warp and a last add over the warps in shared memory.
constexpr int BF16_THREADS = 128;
static __global__ void __launch_bounds__(BF16_THREADS) gemv_bf16_kernel(const uint16_t* __restrict__ W, int K, int N,
                                                                       const float* __restrict__ x, float* __restrict__ y) {
    __shared__ float part[BF16_THREADS / 32];
    const int row = blockIdx.x, tid = threadIdx.x;
    const uint4* w = (const uint4*)(W + (size_t)row * K);
    float acc = 0.0f;
    for (int i = tid; i < K / 8; i += BF16_THREADS) {
        const uint4 p = w[i];
        const float4 xa = *(const float4*)(x + 8 * i), xb = *(const float4*)(x + 8 * i + 4);
        // a bf16 is the upper half of an fp32
        acc = fmaf(__uint_as_float(p.x << 16), xa.x, acc); acc = fmaf(__uint_as_float(p.x & 0xFFFF0000u), xa.y, acc);
        acc = fmaf(__uint_as_float(p.y << 16), xa.z, acc); acc = fmaf(__uint_as_float(p.y & 0xFFFF0000u), xa.w, acc);
        acc = fmaf(__uint_as_float(p.z << 16), xb.x, acc); acc = fmaf(__uint_as_float(p.z & 0xFFFF0000u), xb.y, acc);
        acc = fmaf(__uint_as_float(p.w << 16), xb.z, acc); acc = fmaf(__uint_as_float(p.w & 0xFFFF0000u), xb.w, acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((tid & 31) == 0) part[tid >> 5] = acc;
    __syncthreads();
    if (tid == 0) {
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < BF16_THREADS / 32; i++) s += part[i];
        y[row] = s;
    }
}

// Prefill SwiGLU in place (replaces swiglu_rows_inplace, src/cuda/prefill.cu:132-151): row b of silu(G) * U, n values,
// overwrites the first 2 n bytes of G's row b as 16-bit floats (fp16 like the reference, or bf16 for the bf16 GEMM).
// One CTA per row: the whole result row is formed in shared memory first (2 n bytes), then copied over the row's start,
// so no read of G can see a half written earlier.  n, ld multiples of 8; 2 n bytes of shared memory.
template <bool BF16>
static __global__ void __launch_bounds__(256) swiglu_rows_inplace_kernel(float* G, const float* __restrict__ U, int n, long long ld) {
    extern __shared__ __align__(16) uint8_t row_smem[];
    uint32_t* h2 = (uint32_t*)row_smem;
    float* g = G + (size_t)blockIdx.x * ld;
    const float* u = U + (size_t)blockIdx.x * ld;
    for (int i = threadIdx.x; i < n / 2; i += 256) {
        const float2 a = *(const float2*)(g + 2 * i), b = *(const float2*)(u + 2 * i);
        const float h0 = a.x / (1.0f + __expf(-a.x)) * b.x, h1 = a.y / (1.0f + __expf(-a.y)) * b.y;
        if (BF16) { const __nv_bfloat162 v = __floats2bfloat162_rn(h0, h1); h2[i] = *(const uint32_t*)&v; }
        else { const __half2 v = __floats2half2_rn(h0, h1); h2[i] = *(const uint32_t*)&v; }
    }
    __syncthreads();
    uint4* dst = (uint4*)g;
    const uint4* src = (const uint4*)row_smem;
    for (int i = threadIdx.x; i < n / 8; i += 256) dst[i] = src[i];
}

// ---------------------------------------------------------------------------------------------
// Exact dequantizer: one thread per 32-weight sub-block.  Float operations are the ones of
// dequantize_row_ref (src/quant/quant_ref.cpp:57-103, 165-225, 284-308) in the same order, each
// individually rounded (no fused multiply-add), so fp32 outputs are bit-identical to it.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t g_u16(const uint8_t* p) { return *(const uint16_t*)p; }
__device__ __forceinline__ uint32_t g_u32a2(const uint8_t* p) { return g_u16(p) | (g_u16(p + 2) << 16); }
__device__ __forceinline__ float g_f16(const uint8_t* p) { return __half2float(__ushort_as_half((unsigned short)g_u16(p))); }

template <int FMT>
__device__ __forceinline__ void dequant_sub(const uint8_t* b, int s, float (&y)[32]) {
    if (FMT == T_Q8_0) {
        const uint8_t* q = b + 34 * s;
        const float d = g_f16(q);
#pragma unroll
        for (int j = 0; j < 32; j++) y[j] = __fmul_rn((float)(int8_t)q[2 + j], d);
    } else if (FMT == T_Q4_K || FMT == T_Q5_K) {
        const float d = g_f16(b), mn = g_f16(b + 2);
        const uint8_t* sc = b + 4;
        int scv, mv;
        if (s < 4) { scv = sc[s] & 63; mv = sc[s + 4] & 63; }
        else { scv = (sc[s + 4] & 0xF) | ((sc[s - 4] >> 6) << 4); mv = (sc[s + 4] >> 4) | ((sc[s] >> 6) << 4); }
        const float d1 = __fmul_rn(d, (float)scv), m1 = __fmul_rn(mn, (float)mv);
        const uint8_t* q = b + (FMT == T_Q5_K ? 48 : 16) + 32 * (s >> 1);
#pragma unroll
        for (int l = 0; l < 32; l++) {
            int v = (s & 1) ? (q[l] >> 4) : (q[l] & 0xF);
            if (FMT == T_Q5_K) v += ((b[16 + l] >> s) & 1) << 4;
            y[l] = __fsub_rn(__fmul_rn(d1, (float)v), m1);
        }
    } else if (FMT == T_Q6_K) {
        const float d = g_f16(b + 208);
        const int h = s >> 2, j = s & 3;
        const uint8_t* ql = b + 64 * h + 32 * (j & 1);
        const uint8_t* qh = b + 128 + 32 * h;
        const int8_t* sc = (const int8_t*)(b + 192 + 8 * h + 2 * j);
#pragma unroll
        for (int l = 0; l < 32; l++) {
            const int q = (int)(((ql[l] >> (4 * (j >> 1))) & 0xF) | (((qh[l] >> (2 * j)) & 3) << 4)) - 32;
            y[l] = __fmul_rn(__fmul_rn(d, (float)sc[l >> 4]), (float)q);
        }
    } else if (FMT == T_IQ3_XXS) {
        const float d = g_f16(b);
        const uint32_t aux = g_u32a2(b + 66 + 4 * s);
        const float db = __fmul_rn(__fmul_rn(d, __fadd_rn(0.5f, (float)(aux >> 28))), 0.5f);
#pragma unroll
        for (int l = 0; l < 4; l++) {
            const uint32_t s7 = (aux >> (7 * l)) & 127u;
            const uint32_t sg = s7 | ((uint32_t)(__popc(s7) & 1) << 7);
#pragma unroll
            for (int hh = 0; hh < 2; hh++) {
                const uint32_t gw = q38b_iq3xxs_grid[b[2 + 8 * s + 2 * l + hh]];
#pragma unroll
                for (int j = 0; j < 4; j++)
                    y[8 * l + 4 * hh + j] = __fmul_rn(__fmul_rn(db, (float)((gw >> (8 * j)) & 0xFF)), ((sg >> (4 * hh + j)) & 1) ? -1.f : 1.f);
            }
        }
    } else if (FMT == T_IQ3_S) {
        const float d = g_f16(b);
        const uint32_t ls = (b[106 + (s >> 1)] >> (4 * (s & 1))) & 0xF;
        const float db = __fmul_rn(d, (float)(1 + 2 * (int)ls));
        const uint32_t qh = b[66 + s];
#pragma unroll
        for (int l = 0; l < 4; l++) {
            const uint32_t sg = b[74 + 4 * s + l];
#pragma unroll
            for (int hh = 0; hh < 2; hh++) {
                const uint32_t idx = b[2 + 8 * s + 2 * l + hh] | (((qh >> (2 * l + hh)) & 1u) << 8);
                const uint32_t gw = q38b_iq3s_grid[idx];
#pragma unroll
                for (int j = 0; j < 4; j++)
                    y[8 * l + 4 * hh + j] = __fmul_rn(__fmul_rn(db, (float)((gw >> (8 * j)) & 0xFF)), ((sg >> (4 * hh + j)) & 1) ? -1.f : 1.f);
            }
        }
    } else if (FMT == T_Q2_K) {            // src/quant/quant_ref.cpp:33-55
        const float d = g_f16(b + 80), mn = g_f16(b + 82);
        const int n = s >> 2, j = s & 3;
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const uint32_t sc = b[2 * s + half];
            const float dl = __fmul_rn(d, (float)(sc & 0xF)), ml = __fmul_rn(mn, (float)(sc >> 4));
#pragma unroll
            for (int l = 0; l < 16; l++)
                y[16 * half + l] = __fsub_rn(__fmul_rn(dl, (float)((b[16 + 32 * n + 16 * half + l] >> (2 * j)) & 3)), ml);
        }
    } else if (FMT == T_IQ2_XXS || FMT == T_IQ2_XS || FMT == T_IQ2_S) {   // src/quant/quant_ref.cpp:105-168
        const float d = g_f16(b);
        const uint32_t a1 = FMT == T_IQ2_XXS ? g_u32a2(b + 6 + 8 * s) : 0u;
        const uint32_t scb = FMT == T_IQ2_XXS ? 0u : b[(FMT == T_IQ2_XS ? 66 : 74) + s];
#pragma unroll
        for (int l = 0; l < 4; l++) {
            uint32_t code, sg;
            float db;
            if (FMT == T_IQ2_XXS) {
                code = q38b_iq2xxs_codes[b[2 + 8 * s + l]];
                const uint32_t s7 = (a1 >> (7 * l)) & 127u;
                sg = s7 | ((uint32_t)(__popc(s7) & 1) << 7);
                db = __fmul_rn(__fmul_rn(d, __fadd_rn(0.5f, (float)(a1 >> 28))), 0.25f);
            } else if (FMT == T_IQ2_XS) {
                const uint32_t qv = g_u16(b + 2 + 2 * (4 * s + l));
                code = q38b_iq2xs_codes[qv & 511u];
                const uint32_t s7 = qv >> 9;
                sg = s7 | ((uint32_t)(__popc(s7) & 1) << 7);
                db = __fmul_rn(__fmul_rn(d, __fadd_rn(0.5f, (float)((l < 2 ? scb : scb >> 4) & 0xF))), 0.25f);
            } else {
                code = q38b_iq2s_codes[b[2 + 4 * s + l] | (((uint32_t)b[66 + s] << (8 - 2 * l)) & 0x300u)];
                sg = b[34 + 4 * s + l];
                db = __fmul_rn(__fmul_rn(d, __fadd_rn(0.5f, (float)((l < 2 ? scb : scb >> 4) & 0xF))), 0.25f);
            }
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const uint32_t lv = (code >> (2 * j)) & 3u;
                const float g = lv == 0 ? 8.f : lv == 1 ? 25.f : 43.f;
                y[8 * l + j] = __fmul_rn(__fmul_rn(db, g), ((sg >> j) & 1) ? -1.f : 1.f);
            }
        }
    } else if (FMT == T_IQ1_S) {           // src/quant/quant_ref.cpp:227-245
        const float d = g_f16(b);
        const uint32_t qh = g_u16(b + 34 + 2 * s);
        const float dl = __fmul_rn(d, (float)(2 * (int)((qh >> 12) & 7) + 1));
        const float delta = (qh & 0x8000u) ? -0.125f : 0.125f;
#pragma unroll
        for (int l = 0; l < 4; l++) {
            const uint32_t code = q38b_iq1s_codes[b[2 + 4 * s + l] | (((qh >> (3 * l)) & 7u) << 8)];
#pragma unroll
            for (int j = 0; j < 8; j++) y[8 * l + j] = __fmul_rn(dl, __fadd_rn((float)((int)((code >> (2 * j)) & 3u) - 1), delta));
        }
    } else if (FMT == T_IQ1_M) {           // src/quant/quant_ref.cpp:247-283
        const uint32_t s0 = g_u16(b + 48), s1 = g_u16(b + 50), s2 = g_u16(b + 52), s3 = g_u16(b + 54);
        const uint32_t su = (s0 >> 12) | ((s1 >> 8) & 0x00F0u) | ((s2 >> 4) & 0x0F00u) | (s3 & 0xF000u);
        const float d = __half2float(__ushort_as_half((unsigned short)su));
        const uint32_t scw = (s >> 1) == 0 ? s0 : (s >> 1) == 1 ? s1 : (s >> 1) == 2 ? s2 : s3;
        const uint32_t t = scw >> (6 * (s & 1));
        const float dl[2] = {__fmul_rn(d, (float)(2 * (int)(t & 7) + 1)), __fmul_rn(d, (float)(2 * (int)((t >> 3) & 7) + 1))};
#pragma unroll
        for (int l = 0; l < 4; l++) {
            const uint32_t hn = (b[32 + 2 * s + (l >> 1)] >> (4 * (l & 1))) & 0xFu;
            const uint32_t code = q38b_iq1s_codes[b[4 * s + l] | ((hn & 7u) << 8)];
            const float delta = (hn & 8u) ? -0.125f : 0.125f;
#pragma unroll
            for (int j = 0; j < 8; j++) y[8 * l + j] = __fmul_rn(dl[l >> 1], __fadd_rn((float)((int)((code >> (2 * j)) & 3u) - 1), delta));
        }
    } else if (FMT == T_IQ4_XS) {
        const float d = g_f16(b);
        const uint32_t sh = g_u16(b + 2);
        const int ls = (int)(((b[4 + (s >> 1)] >> (4 * (s & 1))) & 0xF) | (((sh >> (2 * s)) & 3) << 4));
        const float dl = __fmul_rn(d, (float)(ls - 32));
        const uint8_t* q = b + 8 + 16 * s;
#pragma unroll
        for (int j = 0; j < 16; j++) {
            y[j] = __fmul_rn(dl, (float)q38b_iq4nl_levels[q[j] & 0xF]);
            y[j + 16] = __fmul_rn(dl, (float)q38b_iq4nl_levels[q[j] >> 4]);
        }
    }
}

template <int FMT, int KIND>
__global__ void __launch_bounds__(128) dequant_rows_kernel(const uint8_t* __restrict__ W, long long row_bytes, int K, int rows,
                                                            void* __restrict__ out) {
    const int nsub = K >> 5;
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (id >= (long long)rows * nsub) return;
    const int r = (int)(id / nsub), sub = (int)(id % nsub);
    const uint8_t* blk = W + (size_t)r * row_bytes + (size_t)(sub >> 3) * Unit<FMT>::BLOCK_BYTES;
    float y[32];
    dequant_sub<FMT>(blk, sub & 7, y);
    const size_t o = (size_t)r * K + (size_t)sub * 32;
#pragma unroll
    for (int j = 0; j < 32; j++) {
        if (KIND == 0) ((float*)out)[o + j] = y[j];
        else if (KIND == 1) ((__half*)out)[o + j] = __float2half_rn(y[j]);
        else ((__nv_bfloat16*)out)[o + j] = __float2bfloat16_rn(y[j]);
    }
}

}  // namespace q38b
