// q38b_prefill.cu -- dequant-on-the-fly prefill GEMM on the 5th-generation tensor cores (tcgen05 + TMEM).
//
//   Y[t][r] (+)= sum_k X[t][k] * W[r][k]      X bf16 [B][ldx], W GGUF blocks [M rows], Y fp32 [B][ldy]
//
// Replaces dequant_rows_f16 + gemm_f16 (cuBLAS) of the reference (src/cuda/prefill.cu:30-85, 802-851) by one kernel:
// the weights never exist dequantized in global memory.  One CTA owns a 128-row weight tile and up to 512 tokens:
//   * warps 0-7 (256 threads) decode one 32-weight sub-block each per K-slab of 64 (the exact dequantize_row_ref value,
//     rounded once to bf16) and store it K-major with the 128-byte swizzle the tensor core expects (operand A);
//   * one thread streams the matching activation tiles (operand B, 2 x [256 tokens x 64]) with tiled TMA loads
//     (hardware swizzle, zero fill past the last token; no multicast);
//   * one thread issues tcgen05.mma (cta_group::1, kind::f16, M = 128, N = 256, K = 16) into two fp32 accumulators
//     in tensor memory (2 x 256 columns) and commits each slab to the stage's "empty" mbarrier;
//   * warps 0-3 read the accumulators back (tcgen05.ld 32x32b) and store Y, 32 consecutive rows per warp and token.
// All mbarrier waits are bounded; tensor memory is released before the kernel returns, also after a timeout.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstring>
#include <type_traits>

#include "../../include/q38b200.h"
#include "q38b_act.cuh"
#include "q38b_internal.h"
#include "q38b_pipe.cuh"

using namespace q38b;

namespace {

constexpr int PF_ROWS = 128;       // weight rows per CTA (MMA M)
constexpr int PF_NTILE = 256;      // tokens per accumulator (MMA N)
constexpr int PF_KSLAB = 64;       // K elements per stage: one 128-byte swizzle row of bf16
// The two operands have rings of their own: the dequantized weights (16 KB per slab) four deep, so that the decoders,
// whose loads come straight from L2 / HBM, run well ahead of the tensor core; the activation tiles (64 KB per slab) two.
constexpr int PF_A_STAGES = 4, PF_B_STAGES = 2;
constexpr int PF_A_BYTES = PF_ROWS * PF_KSLAB * 2;        // 16 KB
constexpr int PF_B_BYTES = PF_NTILE * PF_KSLAB * 2;       // 32 KB per accumulator
constexpr int PF_B_STAGE_BYTES = 2 * PF_B_BYTES;
// two groups of 8 decode warps (group g takes the slabs with slab % 2 == g: each thread has two slab times for the load
// and the decode of its 32 weights) + TMA warp + MMA warp
constexpr int PF_DECODE_GROUPS = 2, PF_DECODE_WARPS = 8 * PF_DECODE_GROUPS;
constexpr int PF_THREADS = 32 * (PF_DECODE_WARPS + 2);
constexpr int PF_SMEM = 1024 + PF_A_STAGES * PF_A_BYTES + PF_B_STAGES * PF_B_STAGE_BYTES + 256;

struct PrefillArgs {
    const uint8_t* W;
    long long row_bytes;
    float* Y;
    long long ldy;
    int* status;
    int K, M, B, accumulate;
    int n_acc;             // accumulators in use per CTA: 1 (<= 256 tokens in this CTA) or 2
};

__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    // K-major, 128-byte swizzle: 8-row groups 1024 bytes apart (SBO), LBO unused (1), descriptor version 1
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}

// D format f32, A and B both bf16 (format code 1) or both fp16 (code 0), K-major, N = 256, M = 128
__host__ __device__ constexpr uint32_t pf_idesc(bool f16) {
    return (1u << 4) | ((f16 ? 0u : 1u) << 7) | ((f16 ? 0u : 1u) << 10) | ((uint32_t)(PF_NTILE >> 3) << 17) | ((uint32_t)(PF_ROWS >> 4) << 24);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}

// ---------------------------------------------------------------------------------------------------------------
// Fast dequantization to bf16 pairs for the A operand (K-quants).  An integer n < 128 becomes the bf16 number 128 + n by
// OR-ing it under the bit pattern 0x4300, the bias is subtracted exactly (bf16 holds every integer below 256), and one
// packed bf16 fused multiply-add applies scale and minimum to two weights.  Against the exact dequantizer the scale and
// the minimum are rounded to bf16 before instead of after the multiplication: a relative error of 2^-9 per weight, the
// same size as the rounding of the product to bf16 that the tensor core's operand format imposes anyway.
// p[j] = weights 2j, 2j + 1 of the 32-weight sub-block.
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t bf2_u32(__nv_bfloat162 v) { return *(const uint32_t*)&v; }
__device__ __forceinline__ __nv_bfloat162 u32_bf2(uint32_t v) { return *(const __nv_bfloat162*)&v; }
__device__ __forceinline__ __nv_bfloat162 bf2_splat(float x) { return __float2bfloat162_rn(x); }
// The same for fp16 operands (the reference's prefill path multiplies fp16 weights, src/cuda/prefill.cu:30-85): an integer
// n < 1024 becomes the half 1024 + n under the bit pattern 0x6400.
struct OpBf16 {
    using V2 = __nv_bfloat162;
    static __device__ __forceinline__ V2 splat(float x) { return __float2bfloat162_rn(x); }
    static __device__ __forceinline__ V2 bias(int extra) { const uint32_t h = 0x4300u + (uint32_t)extra; const uint32_t v = h | (h << 16); return *(const V2*)&v; }
    static __device__ __forceinline__ void bytes(uint32_t t, V2 bs, V2& lo, V2& hi) {
        lo = __hsub2(u32_bf2(__byte_perm(t, 0x43434343u, 0x5140)), bs);
        hi = __hsub2(u32_bf2(__byte_perm(t, 0x43434343u, 0x5342)), bs);
    }
    static __device__ __forceinline__ uint32_t bits(V2 v) { return *(const uint32_t*)&v; }
    static __device__ __forceinline__ uint32_t pack(float a, float b) { return bf2_u32(__floats2bfloat162_rn(a, b)); }
};
struct OpF16 {
    using V2 = __half2;
    static __device__ __forceinline__ V2 splat(float x) { return __float2half2_rn(x); }
    static __device__ __forceinline__ V2 bias(int extra) { const uint32_t h = 0x6400u + (uint32_t)extra; const uint32_t v = h | (h << 16); return *(const V2*)&v; }   // 1024 + extra: one ulp = 1 up to 2047
    static __device__ __forceinline__ void bytes(uint32_t t, V2 bs, V2& lo, V2& hi) {
        const uint32_t l = __byte_perm(t, 0x64646464u, 0x5140), h = __byte_perm(t, 0x64646464u, 0x5342);
        lo = __hsub2(*(const V2*)&l, bs);
        hi = __hsub2(*(const V2*)&h, bs);
    }
    static __device__ __forceinline__ uint32_t bits(V2 v) { return *(const uint32_t*)&v; }
    static __device__ __forceinline__ uint32_t pack(float a, float b) { const V2 v = __floats2half2_rn(a, b); return *(const uint32_t*)&v; }
};

template <int FMT, typename OP>
__device__ __forceinline__ bool fast_sub(const uint8_t* b, int s, uint32_t (&p)[16]) {
    using V2 = typename OP::V2;
    if (FMT == T_Q4_K || FMT == T_Q5_K) {
        if (((uintptr_t)b & 3) != 0) return false;   // the 32-bit loads below need it (blocks are multiples of 16 bytes; GGUF tensors are 32-byte aligned)
        const uint32_t dd = *(const uint32_t*)b;
        const float d = __half2float(__ushort_as_half((unsigned short)(dd & 0xFFFFu))), mn = __half2float(__ushort_as_half((unsigned short)(dd >> 16)));
        const uint8_t* sc = b + 4;
        int scv, mv;
        if (s < 4) { scv = sc[s] & 63; mv = sc[s + 4] & 63; }
        else { scv = (sc[s + 4] & 0xF) | ((sc[s - 4] >> 6) << 4); mv = (sc[s + 4] >> 4) | ((sc[s] >> 6) << 4); }
        const V2 a2 = OP::splat(d * (float)scv), c2 = OP::splat(-(mn * (float)mv));
        const V2 bias = OP::bias(0);
        const uint32_t* q = (const uint32_t*)(b + (FMT == T_Q5_K ? 48 : 16) + 32 * (s >> 1));
        const uint32_t* qh = (const uint32_t*)(b + 16);
        const int sh = (s & 1) ? 4 : 0;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            uint32_t t = (q[i] >> sh) & 0x0F0F0F0Fu;
            if (FMT == T_Q5_K) t |= ((qh[i] >> s) & 0x01010101u) << 4;
            V2 lo, hi;
            OP::bytes(t, bias, lo, hi);
            p[2 * i] = OP::bits(__hfma2(lo, a2, c2));
            p[2 * i + 1] = OP::bits(__hfma2(hi, a2, c2));
        }
        return true;
    }
    if (FMT == T_Q6_K) {
        // sub-block s = 4h + j of the super-block: weights 128h + 32j .. + 31; ql nibble (low for j < 2) and two bits of qh
        const float d = __half2float(__ushort_as_half(*(const unsigned short*)(b + 208)));
        const int h = s >> 2, j = s & 3;
        const uint16_t* ql = (const uint16_t*)(b + 64 * h + 32 * (j & 1));   // Q6_K blocks are 210 bytes: 2-byte aligned only
        const uint16_t* qh = (const uint16_t*)(b + 128 + 32 * h);
        const int8_t* sc = (const int8_t*)(b + 192 + 8 * h + 2 * j);
        const V2 bias = OP::bias(32);                                        // the base + 32
        const V2 a0 = OP::splat(d * (float)sc[0]), a1 = OP::splat(d * (float)sc[1]);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t lw = (uint32_t)ql[2 * i] | ((uint32_t)ql[2 * i + 1] << 16);
            const uint32_t hw = (uint32_t)qh[2 * i] | ((uint32_t)qh[2 * i + 1] << 16);
            const uint32_t t = ((lw >> (4 * (j >> 1))) & 0x0F0F0F0Fu) | (((hw >> (2 * j)) & 0x03030303u) << 4);
            V2 lo, hi;
            OP::bytes(t, bias, lo, hi);
            const V2 a2 = i < 4 ? a0 : a1;
            p[2 * i] = OP::bits(__hmul2(lo, a2));
            p[2 * i + 1] = OP::bits(__hmul2(hi, a2));
        }
        return true;
    }
    return false;
}

constexpr int PF_PREFETCH_BLOCKS = 3;   // super-blocks (256 weights) of look-ahead of the L2 prefetch

// F16: operands are fp16 (weights dequantized to fp16, activations fp16) instead of bf16.
template <int FMT, bool F16>
__global__ void __launch_bounds__(PF_THREADS, 1) prefill_kernel(const PrefillArgs a, const __grid_constant__ CUtensorMap xmap) {
    using OP = typename std::conditional<F16, OpF16, OpBf16>::type;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* full_a = (uint64_t*)smem;              // [A stages] the 8 decode warps of the slab's group arrive
    uint64_t* empty_a = full_a + PF_A_STAGES;        // [A stages] tcgen05.commit
    uint64_t* full_b = empty_a + PF_A_STAGES;        // [B stages] TMA bytes
    uint64_t* empty_b = full_b + PF_B_STAGES;        // [B stages] tcgen05.commit
    uint64_t* acc_done = empty_b + PF_B_STAGES;      // [1]
    uint32_t* tmem_slot = (uint32_t*)(acc_done + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    uint8_t* stages = smem + 1024;                                   // ring of weight tiles
    uint8_t* stages_b = stages + PF_A_STAGES * PF_A_BYTES;            // ring of activation tiles
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row0 = blockIdx.x * PF_ROWS;
    const int tok0 = blockIdx.y * a.n_acc * PF_NTILE;
    const int n_slabs = a.K / PF_KSLAB;

    if (tid == 0) {
        *abort_flag = 0;
        for (int s = 0; s < PF_A_STAGES; s++) {
            mbar_init(smem_u32(&full_a[s]), 8);             // one arrival per decode warp of the slab's group
            mbar_init(smem_u32(&empty_a[s]), 1);
        }
        for (int s = 0; s < PF_B_STAGES; s++) {
            mbar_init(smem_u32(&full_b[s]), 1);
            mbar_init(smem_u32(&empty_b[s]), 1);
        }
        mbar_init(smem_u32(acc_done), 1);
        mbar_fence_init();
    }
    if (warp == PF_DECODE_WARPS + 1) {   // this warp owns the tensor memory allocation (512 columns = two 128 x 256 fp32 accumulators)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    if (tid == 0 && (smem_u32(stages) & 1023u)) atomicOr(a.status, ST_TMEM_TIMEOUT);   // swizzled tiles need 1024-byte alignment

    if (warp < PF_DECODE_WARPS) {
        // ---------------- operand A: decode 128 rows x 64 weights per slab ----------------
        const int grp = warp >> 3, t = tid & 255;
        const int r = t >> 1, half = t & 1;                      // row of the tile, which 32-weight half of the slab
        const int grow = min(row0 + r, a.M - 1);                 // rows past the end repeat the last row (never stored)
        const uint8_t* wrow = a.W + (size_t)grow * a.row_bytes;
        for (int slab = grp; slab < n_slabs; slab += PF_DECODE_GROUPS) {
            const int st = slab % PF_A_STAGES;
            const uint32_t use = (uint32_t)(slab / PF_A_STAGES);
            mbar_wait_bounded(smem_u32(&empty_a[st]), (use & 1u) ^ 1u, abort_flag, a.status, ST_WAIT_EMPTY_TIMEOUT);
            const int sub = slab * 2 + half;                     // 32-weight sub-block index within the row
            // the weights come straight from HBM: ask L2 for this row's super-blocks a few slabs ahead (one line each)
            if ((slab & 3) == 0 && half == 0) {
                const size_t ahead = (size_t)((slab >> 2) + PF_PREFETCH_BLOCKS) * Unit<FMT>::BLOCK_BYTES;   // BLOCK_BYTES: bytes per 256 weights for every format
                if (ahead < (size_t)a.row_bytes) {
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(wrow + ahead));
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(wrow + min(ahead + 128, (size_t)a.row_bytes - 2)));
                }
            }
            uint32_t p[16];
            const uint8_t* blk = wrow + (size_t)(sub >> 3) * Unit<FMT>::BLOCK_BYTES;
            if (!fast_sub<FMT, OP>(blk, sub & 7, p)) {
                float y[32];
                dequant_sub<FMT>(blk, sub & 7, y);
#pragma unroll
                for (int j = 0; j < 16; j++) p[j] = OP::pack(y[2 * j], y[2 * j + 1]);
            }
            // row r of the tile: 128 bytes; 16-byte chunk c goes to chunk c ^ (r & 7) (128-byte swizzle)
            uint8_t* arow = stages + (size_t)st * PF_A_BYTES + (size_t)r * 128;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const int chunk = (4 * half + c) ^ (r & 7);
                *(uint4*)(arow + 16 * chunk) = make_uint4(p[4 * c], p[4 * c + 1], p[4 * c + 2], p[4 * c + 3]);
            }
            fence_proxy_async();                                 // generic-proxy stores -> visible to the tensor core
            __syncwarp();                                        // one arrival per warp: 256 arrivals on one barrier word serialise
            if (lane == 0) mbar_arrive(smem_u32(&full_a[st]));
        }
    } else if (warp == PF_DECODE_WARPS) {
        // ---------------- operand B: activation tiles by TMA ----------------
        if (lane == 0) {
            for (int slab = 0; slab < n_slabs; slab++) {
                const int st = slab % PF_B_STAGES;
                const uint32_t use = (uint32_t)(slab / PF_B_STAGES);
                mbar_wait_bounded(smem_u32(&empty_b[st]), (use & 1u) ^ 1u, abort_flag, a.status, ST_WAIT_EMPTY_TIMEOUT);
                const uint32_t fb = smem_u32(&full_b[st]);
                mbar_arrive_expect_tx(fb, (uint32_t)(a.n_acc * PF_B_BYTES));
                uint8_t* b0 = stages_b + (size_t)st * PF_B_STAGE_BYTES;
                for (int n = 0; n < a.n_acc; n++)
                    tma_load_2d(smem_u32(b0 + n * PF_B_BYTES), &xmap, slab * PF_KSLAB, tok0 + n * PF_NTILE, fb);
            }
        }
    } else {
        // ---------------- MMA issue ----------------
        if (lane == 0) {
            for (int slab = 0; slab < n_slabs; slab++) {
                const int sa = slab % PF_A_STAGES, sb = slab % PF_B_STAGES;
                mbar_wait_bounded(smem_u32(&full_a[sa]), (uint32_t)(slab / PF_A_STAGES) & 1u, abort_flag, a.status, ST_WAIT_FULL_TIMEOUT);
                mbar_wait_bounded(smem_u32(&full_b[sb]), (uint32_t)(slab / PF_B_STAGES) & 1u, abort_flag, a.status, ST_WAIT_FULL_TIMEOUT);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t abase = smem_u32(stages + (size_t)sa * PF_A_BYTES);
                const uint32_t bbase = smem_u32(stages_b + (size_t)sb * PF_B_STAGE_BYTES);
#pragma unroll
                for (int k = 0; k < PF_KSLAB / 16; k++) {
                    const uint64_t adesc = umma_desc_sw128(abase + 32 * k);
                    for (int n = 0; n < a.n_acc; n++) {
                        const uint64_t bdesc = umma_desc_sw128(bbase + n * PF_B_BYTES + 32 * k);
                        const uint32_t accum = (slab > 0 || k > 0) ? 1u : 0u;
                        asm volatile(
                            "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
                            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                            ::"r"(tmem_base + (uint32_t)(n * PF_NTILE)), "l"(adesc), "l"(bdesc), "r"(pf_idesc(F16)), "r"(accum)
                            : "memory");
                    }
                }
                // frees the two stages once the tensor core has read them
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&empty_a[sa])) : "memory");
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&empty_b[sb])) : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(acc_done)) : "memory");
        }
    }

    // ---------------- epilogue: warps 0-3 read the accumulators (warp w <-> TMEM lanes 32w..32w+31) ----------------
    if (warp < 4) {
        mbar_wait_bounded(smem_u32(acc_done), 0u, abort_flag, a.status, ST_TMEM_TIMEOUT);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int row = row0 + 32 * warp + lane;
        const int n_tok = min(a.n_acc * PF_NTILE, a.B - tok0);
        for (int c0 = 0; c0 < n_tok; c0 += 32) {
            uint32_t v[32];
            const uint32_t taddr = tmem_base + ((uint32_t)(32 * warp) << 16) + (uint32_t)c0;
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                  "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
                  "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
                  "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                : "r"(taddr)
                : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (row < a.M) {
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    if (c0 + j < n_tok) {
                        float* yo = a.Y + (size_t)(tok0 + c0 + j) * a.ldy + row;
                        const float val = __uint_as_float(v[j]);
                        *yo = a.accumulate ? *yo + val : val;
                    }
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (warp == PF_DECODE_WARPS + 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

template <int FMT, bool F16>
int launch_prefill_op(q38b_ctx* ctx, const PrefillArgs& a, const CUtensorMap& map, dim3 grid, cudaStream_t st) {
    auto kern = prefill_kernel<FMT, F16>;
    bool known = false;   // opt-in shared-memory size: once per context (= device) and kernel
    for (int i = 0; i < ctx->n_configured; i++) known |= ctx->configured[i] == (const void*)kern;
    if (!known) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM);
        if (e != cudaSuccess) { ctx->last_cuda = (int)e; return Q38B_ERR_CUDA; }
        if (ctx->n_configured < (int)(sizeof(ctx->configured) / sizeof(ctx->configured[0]))) ctx->configured[ctx->n_configured++] = (const void*)kern;
    }
    kern<<<grid, PF_THREADS, PF_SMEM, st>>>(a, map);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { ctx->last_cuda = (int)e; return Q38B_ERR_CUDA; }
    return Q38B_OK;
}

template <int FMT>
int launch_prefill(q38b_ctx* ctx, const PrefillArgs& a, const CUtensorMap& map, dim3 grid, cudaStream_t st, bool f16) {
    return f16 ? launch_prefill_op<FMT, true>(ctx, a, map, grid, st) : launch_prefill_op<FMT, false>(ctx, a, map, grid, st);
}

int gemm_prefill_any(q38b_ctx* ctx, uint32_t type, const void* W, size_t row_bytes, int K, int M, const void* X, long long ldx, int B,
                     float* Y, long long ldy, int accumulate, void* stream, bool f16);

}  // namespace

extern "C" int q38b_gemm_prefill(q38b_ctx* ctx, uint32_t type, const void* W, size_t row_bytes, int K, int M, const void* X,
                                 long long ldx, int B, float* Y, long long ldy, int accumulate, void* stream) {
    return gemm_prefill_any(ctx, type, W, row_bytes, K, M, X, ldx, B, Y, ldy, accumulate, stream, false);
}

extern "C" int q38b_gemm_prefill_f16(q38b_ctx* ctx, uint32_t type, const void* W, size_t row_bytes, int K, int M, const void* X,
                                     long long ldx, int B, float* Y, long long ldy, int accumulate, void* stream) {
    return gemm_prefill_any(ctx, type, W, row_bytes, K, M, X, ldx, B, Y, ldy, accumulate, stream, true);
}

namespace {
int gemm_prefill_any(q38b_ctx* ctx, uint32_t type, const void* W, size_t row_bytes, int K, int M, const void* X, long long ldx, int B,
                     float* Y, long long ldy, int accumulate, void* stream, bool f16) {
    if (!ctx || !W || !X || !Y || K <= 0 || K % 256 || M < 1 || B < 1 || ldx < K || ldy < M) return Q38B_ERR_ARG;
    if (!q38b_format_supported(type)) return Q38B_ERR_UNSUPPORTED;
    if (row_bytes < q38b_row_bytes(type, K)) return Q38B_ERR_ARG;
    if (((uintptr_t)W & 1) || (row_bytes & 1) || ((uintptr_t)X & 15) || ((ldx * 2) & 15) || ((uintptr_t)Y & 3)) return Q38B_ERR_ALIGN;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return Q38B_ERR_UNSUPPORTED;
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)B};
    const cuuint64_t strides[1] = {(cuuint64_t)ldx * 2};
    const cuuint32_t box[2] = {PF_KSLAB, PF_NTILE};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)X, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return Q38B_ERR_ARG;
    PrefillArgs a;
    a.W = (const uint8_t*)W;
    a.row_bytes = (long long)row_bytes;
    a.Y = Y;
    a.ldy = ldy;
    a.status = ctx->d_status;
    a.K = K;
    a.M = M;
    a.B = B;
    a.accumulate = accumulate ? 1 : 0;
    const int row_tiles = (M + PF_ROWS - 1) / PF_ROWS;
    a.n_acc = B > PF_NTILE ? 2 : 1;   // 512 tokens per CTA (two accumulators) halve the dequantization work per token
    const int tok_per_cta = a.n_acc * PF_NTILE;
    const dim3 grid((unsigned)row_tiles, (unsigned)((B + tok_per_cta - 1) / tok_per_cta));
    cudaStream_t st = (cudaStream_t)stream;
    switch (type) {
        case T_Q8_0: return launch_prefill<T_Q8_0>(ctx, a, map, grid, st, f16);
        case T_Q4_K: return launch_prefill<T_Q4_K>(ctx, a, map, grid, st, f16);
        case T_Q5_K: return launch_prefill<T_Q5_K>(ctx, a, map, grid, st, f16);
        case T_Q6_K: return launch_prefill<T_Q6_K>(ctx, a, map, grid, st, f16);
        case T_IQ3_XXS: return launch_prefill<T_IQ3_XXS>(ctx, a, map, grid, st, f16);
        case T_IQ3_S: return launch_prefill<T_IQ3_S>(ctx, a, map, grid, st, f16);
        case T_IQ4_XS: return launch_prefill<T_IQ4_XS>(ctx, a, map, grid, st, f16);
        case T_Q2_K: return launch_prefill<T_Q2_K>(ctx, a, map, grid, st, f16);
        case T_IQ2_XXS: return launch_prefill<T_IQ2_XXS>(ctx, a, map, grid, st, f16);
        case T_IQ2_XS: return launch_prefill<T_IQ2_XS>(ctx, a, map, grid, st, f16);
        case T_IQ2_S: return launch_prefill<T_IQ2_S>(ctx, a, map, grid, st, f16);
        case T_IQ1_S: return launch_prefill<T_IQ1_S>(ctx, a, map, grid, st, f16);
        case T_IQ1_M: return launch_prefill<T_IQ1_M>(ctx, a, map, grid, st, f16);
        default: return Q38B_ERR_UNSUPPORTED;
    }
}
}  // namespace
