// q38b_fused.cuh -- a whole recorded pass (single activation column) as ONE persistent kernel.
//
// One CTA per SM, 16 warps.  The weight tiles of this CTA (contiguous rows, one bulk copy each), of all matvecs of the
// pass in order, stream through a ring of equal shared-memory slots: tile i lives in slot i % S.  There is no producer
// warp: the warp that finishes a tile (the last of its readers to arrive on the slot's counter) issues the copy of tile i + S
// into the slot it just freed, walking on into the next matvecs when this one has no more tiles.  The matrices of a pass
// are resident and never written, so the ring stays full across matvec boundaries and HBM stays busy while the warps
// synchronise.
//
// A tile is cut into units of (1024-weight slice, 2 or 4 rows); units go round-robin to the warps, so all warps work on
// one or two tiles at a time and the other slots hold copies in flight (throughput = bytes in flight / latency).  A lane
// owns one granule of the slice, keeps its activations in registers for the rows of the unit, and the row sums of a unit
// go to the slot's (slice, row) table; whichever warp completes the tile's last unit (a counter per slot, nobody waits)
// adds the slices in order and writes y.
//
// Ops are cut into groups: a run of matvecs that read the same activation vector and do not depend on one another, or
// a single quantize / SwiGLU op.  At a group boundary the warps of a CTA meet at a named barrier, publish "this CTA has
// finished the previous group" on a global counter, one thread waits (bounded) until every CTA has finished the group
// this one depends on, and the CTA stages the new activation vector.  The kernel is launched cooperatively, so all CTAs
// are resident and the waits cannot starve.
//
// The per-row arithmetic is that of gemv1_kernel (same granule decoders, same lane butterflies, slice sums added in the
// same order); the quantizer and SwiGLU are the device functions the stand-alone kernels use: results are bit-identical
// to the pass replayed kernel by kernel.
#pragma once
#include "q38b_act.cuh"
#include "q38b_decode1.cuh"
#include "q38b_gemv.cuh"
#include "q38b_pipe.cuh"

namespace q38b {

#ifndef Q38B_FU_WARPS
#define Q38B_FU_WARPS 16
#endif
#ifndef Q38B_FU_CTAS_PER_SM
#define Q38B_FU_CTAS_PER_SM 1
#endif
constexpr int FU_WARPS = Q38B_FU_WARPS;          // warps per CTA
constexpr int FU_CTAS_PER_SM = Q38B_FU_CTAS_PER_SM;
constexpr int FU_THREADS = 32 * FU_WARPS;
constexpr int FU_MAX_SLOTS = 16;
constexpr int FU_BAR_COUNT = 64;                  // most units a tile may have
constexpr int FU_HEADER_BYTES = 1024;
constexpr int FU_RING_SLACK = 1024;               // granules past a ragged row end are read (and discarded)

enum { FOP_GEMV = 0, FOP_QUANT = 1, FOP_SWIGLU = 2 };

struct FusedOp {
    int kind;
    int fmt;            // ggml type id (matvec)
    int rows_log2;      // rows per tile = 1 << rows_log2 (matvec)
    int unit_rows;      // rows per unit: 2 or 4 (matvec)
    int group;          // ops of one group run without synchronisation in between
    int wait_group;     // set on the first op of a group: the group that must be complete everywhere first, or -1
    int M;              // matvec: rows
    int nsb;            // super-blocks of 256: per row (matvec) or in total (quantize, SwiGLU)
    int n_tiles;        // matvec: ceil(M / rows per tile)
    int gemv_index;     // matvec: its number among the matvecs of the pass, else -1
    int tile_rot;       // matvec: the CTA that owns tile 0 (leftover tiles of consecutive matvecs go to different CTAs)
    unsigned row_bytes; // matvec: bytes per row (rows are packed)
    const void* a;      // matvec: W          quantize: fp32 source     SwiGLU: gate
    const void* b;      // matvec: Q8_K x     quantize: -               SwiGLU: up
    void* out;          // matvec: fp32 y     quantize, SwiGLU: Q8_K blocks
};

// tracing counters: cycles the warps waited for a weight tile, for the other units of a tile, at group boundaries (of
// which: for the CTA's own warps, for the other CTAs), in total; tiles copied; units
enum { FU_PROF_FULL = 0, FU_PROF_TILE, FU_PROF_GROUP, FU_PROF_TOTAL, FU_PROF_GROUP_BAR, FU_PROF_GROUP_DEP, FU_PROF_FILLS, FU_PROF_UNITS, FU_PROF_LAT, FU_PROF_LAT_N, FU_PROF_N };

struct FusedArgs {
    const FusedOp* ops;
    int n_ops;
    unsigned* done;     // one counter per group: CTAs that have finished it
    int* status;
    const uint32_t* cb_xxs;   // IQ3_XXS grid (256) or nullptr when the pass has no such matrix
    const uint32_t* cb_s;     // IQ3_S grid (512) or nullptr
    unsigned long long* prof; // optional [FU_PROF_N] cycle counters summed over all warps (tracing), or nullptr
    int off_actd, off_actq, off_cb_xxs, off_sgn, off_cb_s, off_red, off_stage, off_optab, off_gemvtab, off_filltab;
    int slot_bytes, n_slots, max_slices, n_gemv;
};

constexpr int ST_FUSED_DEP_TIMEOUT = 32;

// Per-CTA copies of what the hot paths need of the op list, in shared memory (global loads of the descriptors cost
// hundreds of cycles each: the L1 is small here and every acquire at a group boundary empties it).
struct FuGemvEntry {      // 32 bytes, one per matvec
    unsigned long long W, y;
    uint32_t row_bytes;
    int M;
    uint16_t first;       // this CTA's first tile
    uint16_t my_tiles;    // tiles of this CTA: first, first + G, ...
    uint8_t nsb, rows_log2, unit_rows, fmt;
};
struct FuFillEntry {      // 16 bytes, one per matvec: what a refill needs, precomputed (one lane runs the refill alone,
    unsigned long long src0;   // every instruction of it is on the critical path): address of this CTA's first tile,
    uint32_t step;             // bytes between its consecutive tiles,
    uint32_t tile_bytes;       // bytes of a whole tile
};
struct FuOpEntry {        // 8 bytes, one per op
    int16_t gemv;         // index into the matvec table, or -1
    uint8_t kind;
    uint8_t new_group;    // 1: a group starts here (groups are numbered in order)
    int wait_group;
};
static_assert(sizeof(FuGemvEntry) == 32 && sizeof(FuOpEntry) == 8 && sizeof(FuFillEntry) == 16, "table entries are read with vector loads");

__device__ __forceinline__ const void* ldg_ptr(const void* const* pp) { return (const void*)__ldg((const unsigned long long*)pp); }
__device__ __forceinline__ void* ldg_ptr(void* const* pp) { return (void*)__ldg((const unsigned long long*)pp); }

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

struct FuShared {
    uint8_t* smem;
    uint64_t* full;           // [FU_MAX_SLOTS] "tile landed"
    int* slot_units;          // [FU_MAX_SLOTS] units of the slot's tile that are done
    int* slot_item;           // [FU_MAX_SLOTS] index of the latest tile copied (or being copied) into each slot
    long long* fill_clock;    // [FU_MAX_SLOTS] tracing: when the slot's copy was issued
    const FuGemvEntry* gemvtab;
    const FuFillEntry* filltab;
    const FuOpEntry* optab;
    volatile int* abort_flag;
};

// position of one warp in this CTA's sequence of tiles and units (warp-uniform)
struct FuWarp {
    int item_base, unit_base;    // tiles / units of this CTA before the current matvec
    int cur_item, slot;          // ring slot of tile cur_item
    uint32_t slot_par;           // parity of the number of earlier uses of that slot
    int seen_item;               // last tile this warp has waited for
    long long t_full, t_tile, t_lat;    // tracing
    int n_units, n_fills, n_lat;
};

// Copies this CTA's tile number `ti` (counted from matvec `gi`, running on into the following matvecs) into `slot` as
// tile `item` of the CTA's sequence.  One lane calls it, after every reader of the slot's previous tile has finished.
__device__ __forceinline__ bool fu_fill(const FusedArgs& a, const FuShared& sh, int gi, int ti, int slot, int item) {
    const int G = (int)gridDim.x;
    for (; gi < a.n_gemv; gi++) {
        const int mt = sh.gemvtab[gi].my_tiles;
        if (ti >= mt) { ti -= mt; continue; }
        if (ti < mt - 1) {
            // a whole tile that does not touch the end of the tensor
            const FuFillEntry f = sh.filltab[gi];
            const uintptr_t src = (uintptr_t)f.src0 + (uintptr_t)ti * f.step;
            const uint32_t bytes = (((uint32_t)src & 15u) + f.tile_bytes + 15u) & ~15u;
            const uint32_t fb = smem_u32(&sh.full[slot]);
            mbar_arrive_expect_tx(fb, bytes);
            bulk_copy_g2s(smem_u32(sh.smem + a.off_stage) + (uint32_t)(slot * a.slot_bytes), (const void*)(src & ~(uintptr_t)15), bytes, fb);
            if (a.prof) sh.fill_clock[slot] = clock64();
            st_release_shared(smem_u32(sh.slot_item + slot), item);
            return true;
        }
        const FuGemvEntry e = sh.gemvtab[gi];
        const uintptr_t W = (uintptr_t)e.W;
        const uint32_t rb = e.row_bytes;
        const int M = e.M, rl = e.rows_log2;
        const uintptr_t safe_end = (W + (uintptr_t)M * rb) & ~(uintptr_t)15;
        const int row0 = ((int)e.first + G * ti) << rl;
        const uintptr_t src = W + (uintptr_t)row0 * rb;
        const long long len = (long long)min(1 << rl, M - row0) * rb;
        uint8_t* dst = sh.smem + a.off_stage + (size_t)slot * a.slot_bytes;
        const uintptr_t lo = src & ~(uintptr_t)15;
        uintptr_t hi = (src + len + 15) & ~(uintptr_t)15;
        if (hi > safe_end) {   // the tensor's last bytes do not fill a 16-byte unit: plain loads
            hi = safe_end > lo ? safe_end : lo;
            for (uintptr_t p = hi; p < src + len; p += 2)
                if (p >= src) *(uint16_t*)(dst + (p - lo)) = *(const uint16_t*)p;
        }
        const uint32_t bytes = (uint32_t)(hi - lo);
        const uint32_t fb = smem_u32(&sh.full[slot]);
        if (bytes) {
            mbar_arrive_expect_tx(fb, bytes);
            bulk_copy_g2s(smem_u32(dst), (const void*)lo, bytes, fb);
        } else {
            mbar_arrive(fb);
        }
        if (a.prof) sh.fill_clock[slot] = clock64();
        st_release_shared(smem_u32(sh.slot_item + slot), item);
        return true;
    }
    return false;
}

// RU = rows per unit.  A tile of 2^rows_log2 rows has (slices) x (rows / RU) units, numbered slice-major.
template <int FMT, int RU>
__device__ __forceinline__ void fu_gemv(const FusedArgs& a, const FuGemvEntry& e, int gi, FuWarp& w, const FuShared& sh, const Codebook1& cb,
                                        int cw, int lane) {
    constexpr int BB = Unit<FMT>::BLOCK_BYTES;
    constexpr int SLICE_BYTES = 4 * BB;
    constexpr int LPR = Gran<FMT>::LANES_PER_ROW;
    constexpr int PASSES = RU * LPR / 32;
    static_assert(PASSES >= 1, "a pass of the warp covers at least one row");
    const int G = (int)gridDim.x;
    const int nsb = e.nsb, n_slices = (nsb + 3) >> 2;
    const int M = e.M, rl = e.rows_log2;
    const int rs_log2 = rl - (RU == 4 ? 2 : 1);            // row splits per slice = 2^rs_log2
    const int upt = n_slices << rs_log2;                   // units per tile
    const uint32_t rb32 = e.row_bytes;
    const uint32_t w_lo = (uint32_t)e.W;
    float* y = (float*)e.y;
    const int first = e.first, my_tiles = e.my_tiles;
    const int n_units = my_tiles * upt;

    const SP actq_sp = sp_from(sh.smem + a.off_actq), actd_sp = sp_from(sh.smem + a.off_actd);
    const SP stage0_sp = sp_from(sh.smem + a.off_stage);
    float* red = (float*)(sh.smem + a.off_red);            // [n_slots][max_slices][8]
    const int sub = LPR == 32 ? 0 : (lane >> 4);

    int u = cw - w.unit_base;                              // units (unit_base + u) % FU_WARPS == cw are this warp's
    if (u < 0) u += FU_WARPS;
    int ti = 0, rem = u;
    while (rem >= upt) { rem -= upt; ti++; }
    for (; u < n_units; u += FU_WARPS) {
        const int slice = rem >> rs_log2, rsub = rem & ((1 << rs_log2) - 1);
        const int item = w.item_base + ti;
        while (w.cur_item < item) { w.cur_item++; if (++w.slot == a.n_slots) { w.slot = 0; w.slot_par ^= 1u; } }
        typename Gran<FMT>::Acts acts;
        Gran<FMT>::load_acts(acts, actq_sp + slice * 1024, actd_sp + slice * 128, lane);
        const int gran_sb = slice * 4 + (LPR == 32 ? (lane >> 3) : ((lane & 15) >> 2));
        const bool live = gran_sb < nsb;
        // A tile is copied into its slot only after every reader of the slot's previous tile has finished, so once
        // slot_item says this tile's copy was issued, the parity of the slot's barrier is unambiguous.
        if (item > w.seen_item) {
            const long long t0 = a.prof ? clock64() : 0;
            wait_counter_bounded(smem_u32(sh.slot_item + w.slot), item - 1, sh.abort_flag, a.status, ST_WAIT_FULL_TIMEOUT);
            const bool landed = a.prof && mbar_try_wait(smem_u32(&sh.full[w.slot]), w.slot_par);
            mbar_wait_bounded(smem_u32(&sh.full[w.slot]), w.slot_par, sh.abort_flag, a.status, ST_WAIT_FULL_TIMEOUT);
            if (a.prof) {
                const long long t1 = clock64();
                w.t_full += t1 - t0;
                if (!landed) { w.t_lat += t1 - ((volatile long long*)sh.fill_clock)[w.slot]; w.n_lat++; }   // a copy somebody had to wait for: issue to landing
            }
        }
        w.seen_item = item;
        w.n_units++;
        const int tile = first + G * ti;
        const int row_in_tile = rsub * RU;
        const int mis = (int)((w_lo + (uint32_t)(tile << rl) * rb32) & 15u);   // the copy kept the low 4 address bits
        const SP st = stage0_sp + (w.slot * a.slot_bytes + slice * SLICE_BYTES + row_in_tile * (int)rb32 + mis);
        float acc[PASSES];
#pragma unroll
        for (int ps = 0; ps < PASSES; ps++) {
            const int r = LPR == 32 ? ps : 2 * ps + sub;
            const float v = Gran<FMT>::dot(st + r * (int)rb32, acts, cb, lane);
            acc[ps] = live ? v : 0.0f;
        }

        // sum over the lanes of each row: halving butterflies (each step halves the values a lane holds), then plain ones
        float rowsum;
        int myrow = 0;
        {
            float v[PASSES];
#pragma unroll
            for (int i = 0; i < PASSES; i++) v[i] = acc[i];
            constexpr int TOP = LPR == 32 ? 16 : 8;
            int n = PASSES, bit = TOP;
#pragma unroll
            for (int step = 0; step < 2; step++) {
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
        float* rslot = red + ((size_t)w.slot * a.max_slices + slice) * 8 + row_in_tile;
        constexpr int LOW_MASK = (LPR == 32 ? 32 : 16) / PASSES - 1;
        if ((lane & LOW_MASK) == 0) rslot[myrow] = rowsum;
        __syncwarp();
        // Whichever warp writes the tile's last unit finishes the tile (nobody waits for anybody): a counter per slot.
        int arrived = 0;
        if (lane == 0) {
            __threadfence_block();                                   // this unit's sums before the count
            arrived = atomicAdd(sh.slot_units + w.slot, 1);
        }
        arrived = __shfl_sync(0xffffffffu, arrived, 0);
        if (arrived == upt - 1) {
            // every unit of the tile has been read and summed: add the slices in order, refill the slot, write y
            if (lane == 0) { sh.slot_units[w.slot] = 0; __threadfence_block(); }
            __syncwarp();
            const int row = (tile << rl) + lane;
            const bool mine = lane < (1 << rl) && row < M;
            float v = 0.0f;
            if (mine) {
                const volatile float* rs = red + (size_t)w.slot * a.max_slices * 8 + lane;
                for (int s = 0; s < n_slices; s++) v += rs[s * 8];
            }
            __syncwarp();   // the slot's sums are read: its next tile may come
            const long long tf0 = a.prof ? clock64() : 0;
            if (lane == 0 && !*sh.abort_flag) w.n_fills += fu_fill(a, sh, gi, ti + a.n_slots, w.slot, item + a.n_slots) ? 1 : 0;
            if (a.prof) w.t_tile += clock64() - tf0;
            if (mine) y[row] = v;
            __syncwarp();
        }
        rem += FU_WARPS;
        while (rem >= upt) { rem -= upt; ti++; }
    }
    w.item_base += my_tiles;
    w.unit_base = (w.unit_base + n_units) & (FU_WARPS - 1);
}

__global__ void __launch_bounds__(FU_THREADS, FU_CTAS_PER_SM) fused_pass_kernel(const FusedArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    FuShared sh;
    sh.smem = smem_raw;
    sh.full = (uint64_t*)smem_raw;                          // [FU_MAX_SLOTS]
    sh.slot_units = (int*)(sh.full + FU_MAX_SLOTS);         // [FU_MAX_SLOTS]
    sh.abort_flag = (volatile int*)(sh.slot_units + FU_MAX_SLOTS);
    sh.slot_item = (int*)sh.abort_flag + 1;                 // [FU_MAX_SLOTS]
    sh.fill_clock = (long long*)(smem_raw + 512);           // [FU_MAX_SLOTS]
    const int tid = threadIdx.x, cw = tid >> 5, lane = tid & 31;
    const int G = (int)gridDim.x;
    constexpr int NCT = FU_THREADS;

    if (tid == 0) {
        *sh.abort_flag = 0;
        for (int s = 0; s < a.n_slots; s++) {
            mbar_init(smem_u32(&sh.full[s]), 1);
            sh.slot_units[s] = 0;
            sh.slot_item[s] = -1;
        }
        mbar_fence_init();
    }
    __syncthreads();

    FuWarp w;
    w.item_base = w.unit_base = 0;
    w.cur_item = w.slot = 0;
    w.slot_par = 0;
    w.seen_item = -1;
    w.t_full = w.t_tile = w.t_lat = 0;
    w.n_units = w.n_fills = w.n_lat = 0;
    long long t_group = 0, t_gbar = 0, t_gdep = 0;
    const long long t_begin = a.prof ? clock64() : 0;

    // per-CTA op tables
    {
        FuOpEntry* ot = (FuOpEntry*)(sh.smem + a.off_optab);
        FuGemvEntry* gt = (FuGemvEntry*)(sh.smem + a.off_gemvtab);
        FuFillEntry* ft = (FuFillEntry*)(sh.smem + a.off_filltab);
        for (int oi = tid; oi < a.n_ops; oi += NCT) {
            const FusedOp* op = a.ops + oi;
            FuOpEntry o;
            o.kind = (uint8_t)__ldg(&op->kind);
            o.gemv = (int16_t)__ldg(&op->gemv_index);
            o.new_group = (uint8_t)(oi == 0 || __ldg(&op->group) != __ldg(&(op - 1)->group));
            o.wait_group = __ldg(&op->wait_group);
            ot[oi] = o;
            if (o.kind == FOP_GEMV) {
                FuGemvEntry e;
                e.W = (unsigned long long)ldg_ptr(&op->a);
                e.y = (unsigned long long)ldg_ptr(&op->out);
                e.row_bytes = __ldg(&op->row_bytes);
                e.M = __ldg(&op->M);
                int first = (int)blockIdx.x - __ldg(&op->tile_rot);
                if (first < 0) first += G;
                const int n_tiles = __ldg(&op->n_tiles);
                e.first = (uint16_t)first;
                e.my_tiles = (uint16_t)(first < n_tiles ? (n_tiles - first + G - 1) / G : 0);
                e.nsb = (uint8_t)__ldg(&op->nsb);
                e.rows_log2 = (uint8_t)__ldg(&op->rows_log2);
                e.unit_rows = (uint8_t)__ldg(&op->unit_rows);
                e.fmt = (uint8_t)__ldg(&op->fmt);
                gt[o.gemv] = e;
                FuFillEntry f;
                f.src0 = e.W + (unsigned long long)(first << e.rows_log2) * e.row_bytes;
                f.step = (uint32_t)(G << e.rows_log2) * e.row_bytes;
                f.tile_bytes = e.row_bytes << e.rows_log2;
                ft[o.gemv] = f;
            }
        }
        sh.optab = ot;
        sh.gemvtab = gt;
        sh.filltab = ft;
    }
    __syncthreads();

    // the first tiles: warp s fills slot s
    if (cw < a.n_slots && lane == 0) w.n_fills += fu_fill(a, sh, 0, cw, cw, cw) ? 1 : 0;

    if (a.cb_xxs) {
        uint32_t* cbw = (uint32_t*)(sh.smem + a.off_cb_xxs);
        for (int i = tid; i < 256 * 32; i += NCT) cbw[i] = __ldg(a.cb_xxs + (i >> 5));
        uint32_t* sg = (uint32_t*)(sh.smem + a.off_sgn);
        for (int i = tid; i < 128 * 16; i += NCT) {
            uint32_t lo, hi;
            ksign_entry((uint32_t)i >> 4, lo, hi);
            sg[2 * i] = lo;
            sg[2 * i + 1] = hi;
        }
    }
    if (a.cb_s) {
        uint32_t* cbw = (uint32_t*)(sh.smem + a.off_cb_s);
        for (int i = tid; i < 512 * 16; i += NCT) cbw[i] = __ldg(a.cb_s + (i >> 4));
    }
    Codebook1 cb_xxs, cb_s;
    cb_xxs.lane_base = sp_from(sh.smem + a.off_cb_xxs) + 4 * lane;
    cb_xxs.sign_base = sp_from(sh.smem + a.off_sgn) + 8 * (lane & 15);
    cb_s.lane_base = sp_from(sh.smem + a.off_cb_s) + 4 * (lane & 15);
    cb_s.sign_base = cb_xxs.sign_base;

    float* actd = (float*)(sh.smem + a.off_actd);
    uint8_t* actq = sh.smem + a.off_actq;

    int prev_group = -1;
    for (int oi = 0; oi < a.n_ops; oi++) {
        const FusedOp* op = a.ops + oi;
        const FuOpEntry oe = sh.optab[oi];
        const int kind = oe.kind, group = prev_group + (oe.new_group ? 1 : 0);
        if (oe.new_group) {
            // everything this CTA did for the previous group is written; the activation area is free
            const long long tg0 = a.prof ? clock64() : 0;
            named_bar_sync(1, NCT);
            const long long tg1 = a.prof ? clock64() : 0;
            if (prev_group >= 0 && tid == 0) {
                __threadfence();
                atomicAdd(a.done + prev_group, 1u);
            }
            // one thread per CTA polls the counter (thousands of pollers on one address would queue up in L2 in front of
            // the arrivals they wait for); the others wait for it at a second barrier
            const int wg = oe.wait_group;
            if (wg >= 0) {
                if (tid == 0) wait_done(a.done + wg, (unsigned)G, sh.abort_flag, a.status);
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
                for (int i = tid; i < n_slices * 4; i += NCT)
                    actd[i * 8] = i < nsb ? __ldcg((const float*)(xq + (size_t)i * Q8K_BYTES)) : 0.0f;
                for (int i = tid; i < n_slices * 256; i += NCT) {
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
            const FuGemvEntry e = sh.gemvtab[oe.gemv];
            const int key = (int)e.fmt * 8 + (int)e.unit_rows;
#define FU_CASE(F, CB)                                                              \
    case (F) * 8 + 4: fu_gemv<F, 4>(a, e, oe.gemv, w, sh, CB, cw, lane); break;     \
    case (F) * 8 + 2: fu_gemv<F, 2>(a, e, oe.gemv, w, sh, CB, cw, lane); break;
            switch (key) {
                FU_CASE(T_IQ3_XXS, cb_xxs)
                FU_CASE(T_IQ3_S, cb_s)
                FU_CASE(T_IQ4_XS, cb_xxs)
                FU_CASE(T_Q4_K, cb_xxs)
                FU_CASE(T_Q5_K, cb_xxs)
                FU_CASE(T_Q6_K, cb_xxs)
                FU_CASE(T_Q8_0, cb_xxs)
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
        atomicAdd(a.prof + FU_PROF_FILLS, (unsigned long long)w.n_fills);
        atomicAdd(a.prof + FU_PROF_LAT, (unsigned long long)w.t_lat);
        atomicAdd(a.prof + FU_PROF_LAT_N, (unsigned long long)w.n_lat);
    }
}

}  // namespace q38b
