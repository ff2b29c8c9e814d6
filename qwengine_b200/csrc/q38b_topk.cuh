// q38b_topk.cuh -- the k largest logits of a vector with their positions, sorted (k <= 64).
//
// Replaces topk of the reference's sampling step (src/cuda/ops.cuh:142-144, src/cuda/ops.cu:823-903,1037-1044; called on
// the output head's logits, src/runtime/engine.cpp:1680,1910): the same result -- values descending, equal values by
// ascending position -- from a different construction.  A logit becomes a 32-bit key whose unsigned order is the float
// order (NaN lowest), so that a warp's maximum is one REDUX and the tie-break a second one; no shuffle ladders.
//   stage 1: one warp per 1024 logits (32 per lane, in registers) emits its k best as a descending list;
//   stage 2: the answer's next element is always the head of one of those lists, so one warp walks the heads (a few lists
//            per lane, staged in shared memory by the whole CTA) for k rounds.
#pragma once
#include <cstdint>

namespace q38b {

constexpr int TOPK_MAX_K = 64;
constexpr int TOPK_CHUNK = 1024;
constexpr int TOPK_MAX_CHUNKS = 384;          // stage 2 keeps every list in shared memory: 384 lists x 64 x 8 bytes = 192 KB
constexpr int TOPK_STAGE1_WARPS = 4;
constexpr int TOPK_LISTS_PER_LANE = TOPK_MAX_CHUNKS / 32;

// unsigned order == float order (-0 and +0 are one key, as they compare equal); every NaN maps to 0, below -inf (0x007FFFFF)
__device__ __forceinline__ uint32_t topk_key(float f) {
    uint32_t u = __float_as_uint(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return 0u;
    if (u == 0x80000000u) u = 0u;
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct TopkPair { uint32_t key; int idx; };   // idx = 0x7fffffff: nothing (a list shorter than k)

// The warp's best (key, then lowest idx) among one candidate per lane; every lane gets the result.
__device__ __forceinline__ TopkPair topk_warp_best(uint32_t key, int idx) {
    TopkPair w;
    w.key = __reduce_max_sync(0xffffffffu, key);
    w.idx = (int)__reduce_min_sync(0xffffffffu, key == w.key ? (unsigned)idx : 0x7fffffffu);
    return w;
}

// grid (chunks, columns).  lists: [column][chunk][k] pairs, descending.
static __global__ void __launch_bounds__(TOPK_STAGE1_WARPS * 32) topk_lists_kernel(const float* __restrict__ x, long long x_ld, int n, int k,
                                                                             TopkPair* __restrict__ lists, int n_chunks) {
    const int lane = threadIdx.x & 31;
    const int chunk = blockIdx.x * TOPK_STAGE1_WARPS + (threadIdx.x >> 5);
    if (chunk >= n_chunks) return;
    const float* xc = x + (size_t)blockIdx.y * x_ld;
    const int base = chunk * TOPK_CHUNK;
    uint32_t key[32];
#pragma unroll
    for (int j = 0; j < 32; j++) {
        const int i = base + 32 * j + lane;
        key[j] = i < n ? topk_key(xc[i]) : 0u;
    }
    // This lane's candidate: its largest key, the earliest slot among equals (slots ascend with the position).  Kept
    // per group of eight slots, so that dropping an element rescans eight slots and four group bests, not all 32.
    uint32_t live = 0u;   // bit j: element j of this lane exists and has not been emitted yet
#pragma unroll
    for (int j = 0; j < 32; j++) live |= (base + 32 * j + lane) < n ? 1u << j : 0u;
    uint32_t gbest[4];
    int gslot[4];         // 32: the group has nothing left
    auto scan_group = [&](int g) {
        uint32_t bst = 0u;
        int sl = 32;
#pragma unroll
        for (int j = 7; j >= 0; j--) {
            const int jj = 8 * g + j;
            if (((live >> jj) & 1u) && key[jj] >= bst) { bst = key[jj]; sl = jj; }
        }
        gbest[g] = bst;
        gslot[g] = sl;
    };
#pragma unroll
    for (int g = 0; g < 4; g++) scan_group(g);
    uint32_t best = 0u;
    int slot = 32;        // 32: none left
    auto pick = [&]() {
        best = 0u;
        slot = 32;
#pragma unroll
        for (int g = 3; g >= 0; g--)
            if (gslot[g] < 32 && gbest[g] >= best) { best = gbest[g]; slot = gslot[g]; }
    };
    pick();
    TopkPair* out = lists + ((size_t)blockIdx.y * n_chunks + chunk) * k;
    for (int r = 0; r < k; r++) {
        const int my_idx = slot < 32 ? base + 32 * slot + lane : 0x7fffffff;
        const TopkPair w = topk_warp_best(slot < 32 ? best : 0u, my_idx);
        if (lane == 0) out[r] = w;
        if (my_idx == w.idx && slot < 32) {   // the owner drops the element and looks for its next best
            live &= ~(1u << slot);
#pragma unroll
            for (int g = 0; g < 4; g++)
                if (g == (slot >> 3)) scan_group(g);
            pick();
        }
    }
}

// grid (columns), one CTA of 32 * TOPK_LISTS_PER_LANE threads.  vals / idx: [column][ld] floats and ints.
static __global__ void __launch_bounds__(32 * TOPK_LISTS_PER_LANE) topk_merge_kernel(const TopkPair* __restrict__ lists, int n_chunks, int k,
                                                                               const float* __restrict__ x, long long x_ld, int index_offset,
                                                                               float* __restrict__ vals, int* __restrict__ idx, long long out_ld) {
    extern __shared__ __align__(16) uint8_t topk_smem[];
    TopkPair* sl = (TopkPair*)topk_smem;   // [n_chunks][k]
    const TopkPair* src = lists + (size_t)blockIdx.x * n_chunks * k;
    const int total = n_chunks * k;
    {   // two pairs per 16-byte load where this column's lists start 16-byte aligned (an even number of pairs in front of
        // them in the work area); an odd last pair goes alone
        const bool aligned = (((size_t)blockIdx.x * n_chunks * k) & 1u) == 0;
        const int n2 = aligned ? total >> 1 : 0;
        const uint4* src2 = (const uint4*)src;
        uint4* dst2 = (uint4*)sl;
#pragma unroll 4
        for (int i = threadIdx.x; i < n2; i += blockDim.x) dst2[i] = src2[i];
        for (int i = 2 * n2 + threadIdx.x; i < total; i += blockDim.x) sl[i] = src[i];
    }
    __syncthreads();
    if (threadIdx.x >= 32) return;
    const int lane = threadIdx.x;
    // lane l walks lists l, l + 32, ...: head[t] = how many elements of list l + 32 t are taken, hk / hi = the element at
    // the head (registers: only the list that advanced is read again)
    int head[TOPK_LISTS_PER_LANE];
    uint32_t hk[TOPK_LISTS_PER_LANE];
    int hi[TOPK_LISTS_PER_LANE];
#pragma unroll
    for (int t = 0; t < TOPK_LISTS_PER_LANE; t++) {
        const int list = lane + 32 * t;
        head[t] = 0;
        const TopkPair p = list < n_chunks ? sl[list * k] : TopkPair{0u, 0x7fffffff};
        hk[t] = p.key;
        hi[t] = p.idx;
    }
    uint32_t best = 0u;
    int best_idx = 0x7fffffff, best_t = -1;
    auto pick = [&]() {
        best = 0u;
        best_idx = 0x7fffffff;
        best_t = -1;
#pragma unroll
        for (int t = 0; t < TOPK_LISTS_PER_LANE; t++) {
            if (hi[t] != 0x7fffffff && (best_t < 0 || hk[t] > best || (hk[t] == best && hi[t] < best_idx))) {
                best = hk[t];
                best_idx = hi[t];
                best_t = t;
            }
        }
    };
    pick();
    float* ov = vals + (size_t)blockIdx.x * out_ld;
    int* oi = idx + (size_t)blockIdx.x * out_ld;
    for (int r = 0; r < k; r++) {
        const TopkPair w = topk_warp_best(best_t >= 0 ? best : 0u, best_idx);
        if (lane == 0) {
            const bool none = w.idx == 0x7fffffff;
            ov[r] = none ? __uint_as_float(0x7FC00000u) : x[(size_t)blockIdx.x * x_ld + w.idx];   // the logit itself (the key does not keep -0 or NaN payloads)
            oi[r] = none ? -1 : w.idx + index_offset;
        }
        if (best_t >= 0 && best_idx == w.idx) {
#pragma unroll
            for (int t = 0; t < TOPK_LISTS_PER_LANE; t++) {
                if (t == best_t) {
                    head[t]++;
                    const TopkPair p = head[t] < k ? sl[(lane + 32 * t) * k + head[t]] : TopkPair{0u, 0x7fffffff};
                    hk[t] = p.key;
                    hi[t] = p.idx;
                }
            }
            pick();
        }
    }
}

}  // namespace q38b
