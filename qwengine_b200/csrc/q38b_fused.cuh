// q38b_fused.cuh -- a whole recorded pass (single activation column) as ONE persistent kernel.
//
// One CTA per SM: a producer warp and 16 consumer warps.  The producer walks the pass's matvecs in order and streams
// this CTA's weight tiles (contiguous rows, one bulk copy each) through a ring of shared-memory slots; the matrices of a
// pass are resident and never written, so it runs ahead across matvec boundaries and HBM stays busy while the consumers
// synchronise.  The consumers run the ops in order.  Ops are cut into groups: a group is a run of matvecs that read the
// same activation vector and do not depend on one another, or a single quantize / SwiGLU op.  At a group boundary the
// consumers of a CTA meet at a named barrier, publish "this CTA has finished the previous group" on a global counter,
// wait (bounded) until every CTA has finished the group this one depends on, and stage the new activation vector.
// The kernel is launched cooperatively, so all CTAs are resident and the waits cannot starve.
//
// The per-row arithmetic is that of gemv1_kernel (same granule decoders, same slice sums in the same order), the
// quantizer and SwiGLU are the device functions the stand-alone kernels use: results are bit-identical to the pass
// replayed kernel by kernel.
#pragma once
#include "q38b_act.cuh"
#include "q38b_decode1.cuh"
#include "q38b_gemv.cuh"
#include "q38b_pipe.cuh"

namespace q38b {

constexpr int FU_WARPS = 16;                      // consumer warps
constexpr int FU_THREADS = 32 * (1 + FU_WARPS);
constexpr int FU_MAX_STAGES = 16;                 // stage barriers; stage fill i uses barrier i % 16
constexpr int FU_MAX_INFLIGHT = 12;               // stage fills not yet released by their readers
constexpr int FU_MAX_TILEBUF = 32;
constexpr int FU_RING_SLACK = 1024;               // granules past a ragged row end are read (and discarded)
constexpr int FU_BAR_COUNT = 32;                  // arrivals a stage / tile barrier expects = most slices a row may have
constexpr int FU_HEADER_BYTES = 1024;

enum { FOP_GEMV = 0, FOP_QUANT = 1, FOP_SWIGLU = 2 };

struct FusedOp {
    int kind;
    int fmt;            // ggml type id (matvec)
    int rows_log2;      // rows per tile = 1 << rows_log2 (matvec)
    int group;          // ops of one group run without synchronisation in between
    int wait_group;     // set on the first op of a group: the group that must be complete everywhere first, or -1
    int M;              // matvec: rows
    int nsb;            // super-blocks of 256: per row (matvec) or in total (quantize, SwiGLU)
    int n_tiles;        // matvec: ceil(M / rows per tile)
    int tile_rot;       // matvec: the CTA that owns tile 0 (leftover tiles of consecutive matvecs go to different CTAs)
    unsigned row_bytes; // matvec: bytes per row (rows are packed)
    const void* a;      // matvec: W          quantize: fp32 source     SwiGLU: gate
    const void* b;      // matvec: Q8_K x     quantize: -               SwiGLU: up
    void* out;          // matvec: fp32 y     quantize, SwiGLU: Q8_K blocks
};

struct FusedArgs {
    const FusedOp* ops;
    int n_ops;
    unsigned* done;     // one counter per group: CTAs that have finished it
    int* status;
    const uint32_t* cb_xxs;   // IQ3_XXS grid (256) or nullptr when the pass has no such matrix
    const uint32_t* cb_s;     // IQ3_S grid (512) or nullptr
    int off_actd, off_actq, off_cb_xxs, off_sgn, off_cb_s, off_red, off_stage;
    unsigned long long* prof;   // optional [FU_PROF_N] cycle counters summed over all warps (tracing), or nullptr
    int ring_bytes, n_tilebuf, max_slices;   // the ring holds tiles of any size back to back (128-byte granularity)
};

// tracing counters: cycles consumer warps spent waiting for a stage fill, for the other slices of a tile, at group
// boundaries, and in total; cycles the producer waited for ring space; stage fills; units
enum { FU_PROF_FULL = 0, FU_PROF_TILE, FU_PROF_GROUP, FU_PROF_TOTAL, FU_PROF_SPACE, FU_PROF_FILLS, FU_PROF_UNITS, FU_PROF_PRODUCER, FU_PROF_GROUP_BAR, FU_PROF_GROUP_DEP, FU_PROF_N };
constexpr int ST_FUSED_DEP_TIMEOUT = 32;
constexpr int ST_FUSED_BOUNDS = 64;

template <class T>
__device__ __forceinline__ T* ldg_ptr(T* const* pp) { return (T*)__ldg((const unsigned long long*)pp); }
__device__ __forceinline__ const void* ldg_ptr(const void* const* pp) { return (const void*)__ldg((const unsigned long long*)pp); }

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Bounded wait until `*ctr` has reached `target`.
__device__ __forceinline__ bool wait_done(const unsigned* ctr, unsigned target, volatile int* abort_flag, int* status) {
    if (ld_acquire_gpu(ctr) >= target) return true;
    const long long t0 = clock64();
    for (;;) {
        if (ld_acquire_gpu(ctr) >= target) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_BUDGET_CYCLES) break;
        __nanosleep(32);
    }
    *abort_flag = 1;
    if (status) atomicOr(status, ST_FUSED_DEP_TIMEOUT);
    return false;
}

// ring and tile-buffer position of one consumer warp (warp-uniform)
struct FuWarp {
    int item_base, tile_base, unit_base;   // stage fills / tiles / units of this CTA before the current matvec
    int cur_item, stage;                   // ring slot of stage fill cur_item
    uint32_t stage_par;
    int cur_tile, tslot;                   // tile buffer of tile cur_tile
    uint32_t tile_par;
    int seen_item;                         // last stage fill this warp has waited for
    long long t_full, t_tile;              // tracing
    int n_units;
};

struct FuShared {
    uint8_t* smem;
    uint64_t *full, *empty, *tbar;
    int* issued;
    int* item_off;      // [FU_MAX_STAGES] ring offset of the stage fill that uses each barrier
    volatile int* abort_flag;
};

template <int FMT, int ROWS>
__device__ __forceinline__ void fu_gemv(const FusedArgs& a, const FusedOp* op, FuWarp& w, const FuShared& sh, const Codebook1& cb,
                                        int cw, int lane) {
    constexpr int BB = Unit<FMT>::BLOCK_BYTES;
    constexpr int SLICE_BYTES = 4 * BB;
    constexpr int LPR = Gran<FMT>::LANES_PER_ROW;
    constexpr int PASSES = ROWS * LPR / 32;
    static_assert(PASSES >= 1, "a pass of the warp covers at least one row");
    const int G = (int)gridDim.x;
    const int nsb = __ldg(&op->nsb), n_slices = (nsb + 3) >> 2;
    const int n_tiles = __ldg(&op->n_tiles), M = __ldg(&op->M);
    const uint32_t rb32 = __ldg(&op->row_bytes);
    const uint32_t w_lo = (uint32_t)(uintptr_t)ldg_ptr(&op->a);
    float* y = (float*)ldg_ptr(&op->out);
    int first = (int)blockIdx.x - __ldg(&op->tile_rot);
    if (first < 0) first += G;
    const int my_tiles = first < n_tiles ? (n_tiles - first + G - 1) / G : 0;
    const int n_units = my_tiles * n_slices;

    const SP actq_sp = sp_from(sh.smem + a.off_actq), actd_sp = sp_from(sh.smem + a.off_actd);
    const SP stage0_sp = sp_from(sh.smem + a.off_stage);
    float* red = (float*)(sh.smem + a.off_red);         // [n_tilebuf][max_slices][8]
    const int sub = LPR == 32 ? 0 : (lane >> 4);

    int u = cw - w.unit_base;                           // units (unit_base + u) % FU_WARPS == cw are this warp's
    if (u < 0) u += FU_WARPS;
    int ti = 0, slice = u;
    while (slice >= n_slices) { slice -= n_slices; ti++; }
    for (; u < n_units; u += FU_WARPS) {
        const int item = w.item_base + ti;
        while (w.cur_item < item) { w.cur_item++; if (++w.stage == FU_MAX_STAGES) { w.stage = 0; w.stage_par ^= 1u; } }
        const int gtile = w.tile_base + ti;
        while (w.cur_tile < gtile) { w.cur_tile++; if (++w.tslot == a.n_tilebuf) { w.tslot = 0; w.tile_par ^= 1u; } }
        typename Gran<FMT>::Acts acts;
        Gran<FMT>::load_acts(acts, actq_sp + slice * 1024, actd_sp + slice * 128, lane);
        const int gran_sb = slice * 4 + (LPR == 32 ? (lane >> 3) : ((lane & 15) >> 2));
        const bool live = gran_sb < nsb;
        // the counter of issued fills makes the parity wait unambiguous for a warp that skipped uses of this barrier
        if (item > w.seen_item) {
            const long long t0 = a.prof ? clock64() : 0;
            wait_counter_bounded(smem_u32(sh.issued), item, sh.abort_flag, a.status, ST_WAIT_FULL_TIMEOUT);
            mbar_wait_bounded(smem_u32(&sh.full[w.stage]), w.stage_par, sh.abort_flag, a.status, ST_WAIT_FULL_TIMEOUT);
            if (a.prof) w.t_full += clock64() - t0;
        }
        w.n_units++;
        w.seen_item = item;
        const int tile = first + G * ti;
        const int mis = (int)((w_lo + (uint32_t)(tile * ROWS) * rb32) & 15u);   // the copy kept the low 4 address bits
        // a tile that would not lie inside the ring is skipped and reported (a planner or ring bookkeeping error)
        const int tile_off = (int)sp_ld32(sp_from(sh.item_off), 4 * w.stage);
        const bool in_ring = tile_off >= 0 && (tile_off & 127) == 0 && tile_off + ROWS * (int)rb32 + mis <= a.ring_bytes;
        if (!in_ring && lane == 0) atomicOr(a.status, ST_FUSED_BOUNDS);
        const SP st = stage0_sp + ((in_ring ? tile_off : 0) + slice * SLICE_BYTES);
        float acc[PASSES];
#pragma unroll
        for (int ps = 0; ps < PASSES; ps++) {
            const int r = LPR == 32 ? ps : 2 * ps + sub;
            const float v = Gran<FMT>::dot(st + (r * (int)rb32 + mis), acts, cb, lane);
            acc[ps] = live ? v : 0.0f;
        }
        __syncwarp();
        // barriers expect FU_BAR_COUNT arrivals whatever the number of slices: the last slice makes up the difference
        const int n_arr = slice == n_slices - 1 ? FU_BAR_COUNT - n_slices + 1 : 1;
        if (lane == 0) mbar_arrive_n(smem_u32(&sh.empty[w.stage]), n_arr);

        float rowsum;
        int myrow = 0;
        {
            float v[PASSES];
#pragma unroll
            for (int i = 0; i < PASSES; i++) v[i] = acc[i];
            constexpr int TOP = LPR == 32 ? 16 : 8;
            int n = PASSES, bit = TOP;
#pragma unroll
            for (int step = 0; step < 3; step++) {
                if (n > 1) {
                    const int h = n >> 1;
                    const bool up = (lane & bit) != 0;
#pragma unroll
                    for (int i = 0; i < PASSES / 2; i++) {
                        if (i < h) {
                            const float keep = up ? v[i + h] : v[i], give = up ? v[i] : v[i + h];
                            v[i] = keep + __shfl_xor_sync(0xffffffffu, give, bit);
                        }
                    }
                    if (up) myrow += h;
                    n = h;
                    bit >>= 1;
                }
            }
            rowsum = v[0];
            for (; bit > 0; bit >>= 1) rowsum += __shfl_xor_sync(0xffffffffu, rowsum, bit);
            if (LPR == 16) myrow = 2 * myrow + sub;
        }
        float* rslot = red + ((size_t)w.tslot * a.max_slices + slice) * 8;
        constexpr int LOW_MASK = (LPR == 32 ? 32 : 16) / PASSES - 1;
        if ((lane & LOW_MASK) == 0) rslot[myrow] = rowsum;
        __syncwarp();
        const uint32_t tb = smem_u32(&sh.tbar[w.tslot]);
        if (lane == 0) mbar_arrive_n(tb, n_arr);
        if (slice == n_slices - 1) {
            const long long t0 = a.prof ? clock64() : 0;
            mbar_wait_bounded(tb, w.tile_par, sh.abort_flag, a.status, ST_WAIT_FULL_TIMEOUT);
            if (a.prof) w.t_tile += clock64() - t0;
            const int row = tile * ROWS + lane;
            if (lane < ROWS && row < M) {
                const float* rs = red + (size_t)w.tslot * a.max_slices * 8 + lane;
                float v = 0.0f;
                for (int s = 0; s < n_slices; s++) v += rs[s * 8];
                y[row] = v;
            }
            __syncwarp();
        }
        slice += FU_WARPS;
        while (slice >= n_slices) { slice -= n_slices; ti++; }
    }
    w.item_base += my_tiles;
    w.tile_base += my_tiles;
    w.unit_base = (w.unit_base + n_units) & (FU_WARPS - 1);
}

__global__ void __launch_bounds__(FU_THREADS, 1) fused_pass_kernel(const FusedArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    FuShared sh;
    sh.smem = smem_raw;
    sh.full = (uint64_t*)smem_raw;                          // [FU_MAX_STAGES]
    sh.empty = sh.full + FU_MAX_STAGES;                     // [FU_MAX_STAGES]
    sh.tbar = sh.empty + FU_MAX_STAGES;                     // [FU_MAX_TILEBUF]
    sh.abort_flag = (volatile int*)(sh.tbar + FU_MAX_TILEBUF);
    sh.issued = (int*)sh.abort_flag + 1;
    sh.item_off = sh.issued + 1;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = (int)gridDim.x;

    if (tid == 0) {
        *sh.abort_flag = 0;
        *sh.issued = 0;
        for (int s = 0; s < FU_MAX_STAGES; s++) { mbar_init(smem_u32(&sh.full[s]), 1); mbar_init(smem_u32(&sh.empty[s]), FU_BAR_COUNT); }
        for (int t = 0; t < a.n_tilebuf; t++) mbar_init(smem_u32(&sh.tbar[t]), FU_BAR_COUNT);
        mbar_fence_init();
    }
    __syncthreads();

    if (warp == 0) {
        // ---------------- producer: one lane, one bulk copy per tile ----------------
        if (lane == 0) {
            // The ring is a byte FIFO: tiles of any size lie back to back, space is reclaimed in issue order.
            int item = 0, head = 0, tail_item = 0, n_in = 0;
            long long t_space = 0;
            const long long t_begin = a.prof ? clock64() : 0;
            for (int oi = 0; oi < a.n_ops; oi++) {
                const FusedOp* op = a.ops + oi;
                if (__ldg(&op->kind) != FOP_GEMV) continue;
                const uintptr_t W = (uintptr_t)ldg_ptr(&op->a);
                const uint32_t rb = __ldg(&op->row_bytes);
                const int M = __ldg(&op->M), n_tiles = __ldg(&op->n_tiles), rl = __ldg(&op->rows_log2);
                const uintptr_t w_end = W + (uintptr_t)M * rb;
                const uintptr_t safe_end = w_end & ~(uintptr_t)15;
                int first = (int)blockIdx.x - __ldg(&op->tile_rot);
                if (first < 0) first += G;
                for (int t = first; t < n_tiles; t += G) {
                    const int row0 = t << rl;
                    const uintptr_t src = W + (uintptr_t)row0 * rb;
                    const long long len = (long long)min(1 << rl, M - row0) * rb;
                    const uintptr_t lo = src & ~(uintptr_t)15;
                    uintptr_t hi = (src + len + 15) & ~(uintptr_t)15;
                    // room for a whole tile even when the matrix ends inside it: the consumers read all its rows
                    const int sz = (int)(((src & 15) + ((uintptr_t)rb << rl) + 15 + 127) & ~(uintptr_t)127);
                    int pos = 0;
                    for (;;) {
                        bool ok = false;
                        if (n_in == 0) { pos = 0; ok = true; }
                        else {
                            const int tail = sh.item_off[tail_item & (FU_MAX_STAGES - 1)];
                            if (head > tail) {                       // in use: [tail, head)
                                if (a.ring_bytes - head >= sz) { pos = head; ok = true; }
                                else if (tail >= sz) { pos = 0; ok = true; }
                            } else if (tail - head >= sz) {          // in use: [tail, end) and [0, head)
                                pos = head;
                                ok = true;
                            }
                        }
                        if (ok && n_in < FU_MAX_INFLIGHT) break;
                        // reclaim the oldest fill once all its readers have released it
                        const long long t0 = a.prof ? clock64() : 0;
                        mbar_wait_bounded(smem_u32(&sh.empty[tail_item & (FU_MAX_STAGES - 1)]), (uint32_t)(tail_item >> 4) & 1u, sh.abort_flag,
                                          a.status, ST_WAIT_EMPTY_TIMEOUT);
                        if (a.prof) t_space += clock64() - t0;
                        tail_item++;
                        n_in--;
                    }
                    if (pos < 0 || pos + sz > a.ring_bytes) {   // cannot happen: reported, the copy is skipped
                        atomicOr(a.status, ST_FUSED_BOUNDS);
                        *sh.abort_flag = 1;
                        return;
                    }
                    const int bi = item & (FU_MAX_STAGES - 1);
                    sh.item_off[bi] = pos;
                    head = pos + sz;
                    n_in++;
                    const uint32_t fb = smem_u32(&sh.full[bi]);
                    uint8_t* slot = sh.smem + a.off_stage + pos;
                    if (hi > safe_end) {   // the tensor's last bytes do not fill a 16-byte unit: plain loads
                        hi = safe_end > lo ? safe_end : lo;
                        for (uintptr_t p = hi; p < src + len; p += 2)
                            if (p >= src) *(uint16_t*)(slot + (p - lo)) = *(const uint16_t*)p;
                    }
                    const uint32_t bytes = (uint32_t)(hi - lo);
                    if (bytes) {
                        mbar_arrive_expect_tx(fb, bytes);
                        bulk_copy_g2s(smem_u32(slot), (const void*)lo, bytes, fb);
                    } else {
                        mbar_arrive(fb);
                    }
                    st_release_shared(smem_u32(sh.issued), ++item);
                }
            }
            if (a.prof) {
                atomicAdd(a.prof + FU_PROF_SPACE, (unsigned long long)t_space);
                atomicAdd(a.prof + FU_PROF_FILLS, (unsigned long long)item);
                atomicAdd(a.prof + FU_PROF_PRODUCER, (unsigned long long)(clock64() - t_begin));
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    const int cw = warp - 1, ctid = tid - 32;
    constexpr int NCT = FU_WARPS * 32;
    if (a.cb_xxs) {
        uint32_t* cbw = (uint32_t*)(sh.smem + a.off_cb_xxs);
        for (int i = ctid; i < 256 * 32; i += NCT) cbw[i] = __ldg(a.cb_xxs + (i >> 5));
        uint32_t* sg = (uint32_t*)(sh.smem + a.off_sgn);
        for (int i = ctid; i < 128 * 16; i += NCT) {
            uint32_t lo, hi;
            ksign_entry((uint32_t)i >> 4, lo, hi);
            sg[2 * i] = lo;
            sg[2 * i + 1] = hi;
        }
    }
    if (a.cb_s) {
        uint32_t* cbw = (uint32_t*)(sh.smem + a.off_cb_s);
        for (int i = ctid; i < 512 * 32; i += NCT) cbw[i] = __ldg(a.cb_s + (i >> 5));
    }
    Codebook1 cb_xxs, cb_s;
    cb_xxs.lane_base = sp_from(sh.smem + a.off_cb_xxs) + 4 * lane;
    cb_xxs.sign_base = sp_from(sh.smem + a.off_sgn) + 8 * (lane & 15);
    cb_s.lane_base = sp_from(sh.smem + a.off_cb_s) + 4 * lane;
    cb_s.sign_base = cb_xxs.sign_base;

    FuWarp w;
    w.item_base = w.tile_base = w.unit_base = 0;
    w.cur_item = w.stage = 0;
    w.stage_par = 0;
    w.cur_tile = w.tslot = 0;
    w.tile_par = 0;
    w.seen_item = -1;
    w.t_full = w.t_tile = 0;
    w.n_units = 0;
    long long t_group = 0, t_gbar = 0, t_gdep = 0;
    const long long t_begin = a.prof ? clock64() : 0;
    float* actd = (float*)(sh.smem + a.off_actd);
    uint8_t* actq = sh.smem + a.off_actq;

    int prev_group = -1;
    for (int oi = 0; oi < a.n_ops; oi++) {
        const FusedOp* op = a.ops + oi;
        const int kind = __ldg(&op->kind), group = __ldg(&op->group);
        if (group != prev_group) {
            // everything this CTA did for the previous group is written; the activation area is free
            const long long tg0 = a.prof ? clock64() : 0;
            named_bar_sync(1, NCT);
            const long long tg1 = a.prof ? clock64() : 0;
            if (prev_group >= 0 && ctid == 0) {
                __threadfence();
                atomicAdd(a.done + prev_group, 1u);
            }
            // one thread per CTA polls the counter (thousands of pollers on one address would queue up in L2 in front of
            // the arrivals they wait for); the others wait for it at a second barrier
            const int wg = __ldg(&op->wait_group);
            if (wg >= 0) {
                if (ctid == 0) wait_done(a.done + wg, (unsigned)G, sh.abort_flag, a.status);
                named_bar_sync(3, NCT);
            }
            const long long tg2 = a.prof ? clock64() : 0;
            if (a.prof) { t_gbar += tg1 - tg0; t_gdep += tg2 - tg1; }
            prev_group = group;
            if (kind == FOP_GEMV) {
                // stage the activation vector (written by other SMs during this kernel: read it through L2)
                const uint8_t* xq = (const uint8_t*)ldg_ptr(&op->b);
                const int nsb = __ldg(&op->nsb), n_slices = (nsb + 3) >> 2;
                const bool permute = __ldg(&op->fmt) == T_IQ4_XS;
                for (int i = ctid; i < n_slices * 4; i += NCT)
                    actd[i * 8] = i < nsb ? __ldcg((const float*)(xq + (size_t)i * Q8K_BYTES)) : 0.0f;
                for (int i = ctid; i < n_slices * 256; i += NCT) {
                    const int sb = i >> 6, wi = i & 63;
                    const uint32_t v = sb < nsb ? __ldcg((const uint32_t*)(xq + (size_t)sb * Q8K_BYTES + 4 + 4 * wi)) : 0u;
                    uint8_t* dst = actq + sb * 256;
                    if (permute) {
#pragma unroll
                        for (int b = 0; b < 4; b++) {
                            const int k = 4 * wi + b;
                            dst[(k & ~31) + act_stage_pos(T_IQ4_XS, k & 31)] = (uint8_t)(v >> (8 * b));
                        }
                    } else {
                        *(uint32_t*)(dst + 4 * wi) = v;
                    }
                }
                named_bar_sync(2, NCT);
            }
            if (a.prof) t_group += clock64() - tg0;
        }
        if (kind == FOP_QUANT) {
            const float* src = (const float*)ldg_ptr(&op->a);
            uint8_t* out = (uint8_t*)ldg_ptr(&op->out);
            const int nblk = __ldg(&op->nsb);
            for (int b = (int)blockIdx.x * FU_WARPS + cw; b < nblk; b += G * FU_WARPS)
                quantize_block<true>(src + (size_t)b * 256, out + (size_t)b * Q8K_BYTES);
        } else if (kind == FOP_SWIGLU) {
            const float* g = (const float*)ldg_ptr(&op->a);
            const float* u = (const float*)ldg_ptr(&op->b);
            uint8_t* out = (uint8_t*)ldg_ptr(&op->out);
            const int nblk = __ldg(&op->nsb);
            for (int b = (int)blockIdx.x * FU_WARPS + cw; b < nblk; b += G * FU_WARPS)
                swiglu_block<true>(g + (size_t)b * 256, u + (size_t)b * 256, nullptr, out + (size_t)b * Q8K_BYTES);
        } else {
            const int key = __ldg(&op->fmt) * 8 + __ldg(&op->rows_log2);
#define FU_CASE(F, RL, CB) case (F) * 8 + (RL): fu_gemv<F, (1 << (RL))>(a, op, w, sh, CB, cw, lane); break;
            switch (key) {
                FU_CASE(T_IQ3_XXS, 3, cb_xxs)
                FU_CASE(T_IQ3_XXS, 2, cb_xxs)
                FU_CASE(T_IQ3_XXS, 1, cb_xxs)
                FU_CASE(T_IQ3_S, 3, cb_s)
                FU_CASE(T_IQ3_S, 2, cb_s)
                FU_CASE(T_IQ3_S, 1, cb_s)
                FU_CASE(T_IQ4_XS, 3, cb_xxs)
                FU_CASE(T_IQ4_XS, 2, cb_xxs)
                FU_CASE(T_IQ4_XS, 1, cb_xxs)
                FU_CASE(T_Q4_K, 3, cb_xxs)
                FU_CASE(T_Q4_K, 2, cb_xxs)
                FU_CASE(T_Q4_K, 1, cb_xxs)
                FU_CASE(T_Q5_K, 3, cb_xxs)
                FU_CASE(T_Q5_K, 2, cb_xxs)
                FU_CASE(T_Q5_K, 1, cb_xxs)
                FU_CASE(T_Q6_K, 3, cb_xxs)
                FU_CASE(T_Q6_K, 2, cb_xxs)
                FU_CASE(T_Q6_K, 1, cb_xxs)
                FU_CASE(T_Q8_0, 3, cb_xxs)
                FU_CASE(T_Q8_0, 2, cb_xxs)
                FU_CASE(T_Q8_0, 1, cb_xxs)
                default: break;   // the planner never emits another combination
            }
#undef FU_CASE
        }
    }
    if (a.prof && lane == 0) {
        atomicAdd(a.prof + FU_PROF_FULL, (unsigned long long)w.t_full);
        atomicAdd(a.prof + FU_PROF_TILE, (unsigned long long)w.t_tile);
        atomicAdd(a.prof + FU_PROF_GROUP, (unsigned long long)t_group);
        atomicAdd(a.prof + FU_PROF_GROUP_BAR, (unsigned long long)t_gbar);
        atomicAdd(a.prof + FU_PROF_GROUP_DEP, (unsigned long long)t_gdep);
        atomicAdd(a.prof + FU_PROF_TOTAL, (unsigned long long)(clock64() - t_begin));
        atomicAdd(a.prof + FU_PROF_UNITS, (unsigned long long)w.n_units);
    }
}

// rows-per-tile exponents the kernel is instantiated for (every format), largest first
constexpr int FU_ROWS_LOG2[3] = {3, 2, 1};

}  // namespace q38b
