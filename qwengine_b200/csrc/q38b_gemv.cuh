// q38b_gemv.cuh -- the decode matvec kernel: y[c][r] (+)= W[r,:] . x_c for 1..8 activation columns.
//
// Replaces k_gemv_q8 / gemv_q8n of the reference (src/cuda/gemv.cu:51-125, 215-228).  Shape of the kernel:
//   * persistent CTAs (one per SM): a producer warp plus NGROUPS groups of 8 consumer warps (K-parts: one more warp);
//   * the weight rows stream HBM -> shared memory through 1-D bulk (TMA) copies, one copy per (row, K-chunk) into
//     ONE ring of stages that the groups take tiles from alternately, completion tracked by mbarriers; GGUF blocks of most formats are only 2-byte
//     aligned, so each copy moves the 16-byte aligned superset of its row slice and the consumers index from the
//     remainder;
//   * a stage holds a 16-row tile; the 8 warps of a group split its half super-blocks, decode them into int8 mma
//     fragments (q38b_decode.cuh) and keep float partial sums per (row, column); at the end of a tile the 8
//     partial sums are added in a fixed order through shared memory, so results do not depend on timing;
//   * activations (Q8_K int8 values and block scales of all columns) and the codebook are staged in shared memory
//     once per CTA;
//   * rows longer than 8192 are cut into K-parts of 8 to 16 super-blocks (a rule of K and the format alone).  The work
//     items (part, tile), part-major, are dealt to the CTAs as equal contiguous ranges: a CTA then needs the
//     activations of at most two neighbouring parts, which leaves the shared memory to the weight stages, and 320
//     tiles of 68 super-blocks keep 148 SMs evenly busy instead of 24 of them working a second round.  A part's sums
//     go to a scratch area in global memory and the consumers carry on; a further warp of the CTA counts the tile's
//     parts (a counter per tile) and, where it counted the last one, reads them all back, adds them in part order and
//     stores the row sums -- the result does not depend on who computed what or when.  (Measured on B200, seven
//     columns, 5120 x 17408 IQ4_XS after its SwiGLU: 40.4 us as two launches over the halves of K, 30.8 us this way.
//     The consumers counting and adding themselves, with fences: 33.3 us.  Parts on rows of 5120: in_proj 17 -> 26 us.)
// Every column is computed by the same instructions whatever nb is, so column c of an nb-column call is
// bit-identical to a 1-column call on that column (the reference promises the same: src/cuda/gemv.cuh:31-34).
#pragma once
#include "q38b_act.cuh"
#include "q38b_decode.cuh"
#include "q38b_pipe.cuh"

namespace q38b {

constexpr int TILE_ROWS = 16;
constexpr int GROUP_WARPS = 8;
constexpr int GROUP_THREADS = GROUP_WARPS * 32;
constexpr int MAX_STAGES = 8;
constexpr int Q8K_BYTES = 292;   // float d | int8 qs[256] | int16 bsums[16]  (src/quant/quant_formats.h:95)

constexpr int GEMV_MAX_MATS = 3;
constexpr int GEMV_MAX_PARTS = 32;
constexpr uint32_t PART_EMPTY = 0xFFFFFFFFu;   // a slot of the K-part scratch area that holds no sums (the area rests in this state)

struct GemvArgs {
    // up to three matrices of one format, K and row stride on the same activation columns: their 16-row tiles form one
    // sequence (matrix 0's, then matrix 1's, ...), one launch replaces three
    const uint8_t* W_more[GEMV_MAX_MATS - 1];
    float* y_more[GEMV_MAX_MATS - 1];
    long long y_ld_more[GEMV_MAX_MATS - 1];
    int M_more[GEMV_MAX_MATS - 1];
    int tile_start[GEMV_MAX_MATS];   // first tile of each matrix (unused ones = n_tiles)
    const uint8_t* W;        // [M] rows, row_bytes apart, GGUF blocks
    long long row_bytes;
    const uint8_t* xq;       // Q8_K blocks; column c starts at xq + c * x_stride * 292; or nullptr:
    long long x_stride;      // blocks between columns
    const float* x_f32;      // then the columns as floats (column c at x_f32 + c * x_f32_ld), quantized to Q8_K by every CTA in its prologue
    long long x_f32_ld;
    float* y;                // y[c * y_ld + r]
    long long y_ld;
    float* y_peer[7];        // the same output position in the other GPUs' buffers (peer stores), n_peers used
    float* y_peer_more[GEMV_MAX_MATS - 1][7];   // the same for the further matrices of the launch
    int n_peers;
    int static_weights;     // 1: W was written long before this launch, the producer need not wait for earlier kernels
    int* status;             // device status word (OR of ST_* bits)
    const uint32_t* codebook;   // device copy of the format's codebook (or nullptr)
    int K, M, nb, accumulate;
    int nsb;                 // super-blocks per row
    int n_tiles;
    int chunk_sb;            // super-blocks per K-chunk (last chunk may be shorter)
    int n_chunks;            // K-chunks per work item (1 when the row is cut into parts: a part is one chunk)
    int n_parts;             // K-parts of a row (1: the whole row is one work item per tile)
    int part_sb0[GEMV_MAX_PARTS + 1];   // first super-block of each part (multiples of 4); [n_parts] = nsb
    int act_sb;              // super-blocks of activations a CTA stages per column (nsb, or two parts' worth)
    float* parts;            // n_parts > 1: 128 sums (16 rows x 8 columns) per (tile, part); PART_EMPTY between launches
    int* part_count;         // ... and per tile how many parts are written (zero between launches)
    int n_stages;
    int slot_stride;         // bytes per row slot inside a stage (multiple of 16)
    int cb_rep_log2;         // log2 of codebook replicas
    // shared-memory offsets (bytes from the 128-byte aligned base)
    int off_actd, off_actq, off_cb, off_red, off_stage;
    int stage_bytes;         // TILE_ROWS * slot_stride
};

template <int FMT, int NGROUPS, bool PARTED>
__global__ void __launch_bounds__(32 * (1 + NGROUPS * GROUP_WARPS + (PARTED ? 1 : 0)), 1) gemv_kernel(const GemvArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];   // plain pointer arithmetic from here on keeps loads in the shared space
    uint8_t* smem = smem_raw;
    // One ring of stages for all groups: this CTA's work items k = 0, 1, 2, ... go to group k % NGROUPS; the n_chunks
    // stage fills of item k are fills k * n_chunks .. + n_chunks - 1 of the ring.  Whole rows: item k is tile
    // blockIdx.x + gridDim.x * k.  K-parts: the items (part, tile), part-major, are cut into gridDim.x equal ranges.
    uint64_t* bars = (uint64_t*)smem;                       // full[MAX_STAGES], empty[MAX_STAGES]
    volatile int* abort_flag = (volatile int*)(smem + 8 * 2 * MAX_STAGES);   // the header ends well before off_actd = 256
    int* issued = (int*)abort_flag + 1;                     // stage fills the producer has issued so far
    int* parts_written = (int*)abort_flag + 2;              // [NGROUPS] K-parts: summing warps of the group that have put an item's sums into the scratch area
    constexpr bool parted = PARTED;                         // a.n_parts > 1
    const long long n_items = (long long)a.n_tiles * (parted ? a.n_parts : 1);
    const long long item_lo = parted ? n_items * blockIdx.x / gridDim.x : 0;
    const int my_items = parted ? (int)(n_items * (blockIdx.x + 1) / gridDim.x - item_lo)
                                : (a.n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;   // (the grid is never larger than n_tiles)
    // the activations this CTA stages: super-blocks [win0, win0 + win_sb) of every column
    const int part_first = parted ? (int)(item_lo / a.n_tiles) : 0;
    const int part_last = parted && my_items > 0 ? (int)((item_lo + my_items - 1) / a.n_tiles) : part_first;
    const int win0 = parted ? a.part_sb0[part_first] : 0;
    const int win_sb = parted ? a.part_sb0[part_last + 1] - win0 : a.nsb;
    const int act_ld = a.act_sb * 256;                      // bytes between the staged columns
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        *abort_flag = 0;
        *issued = 0;
        parts_written[0] = parts_written[1] = 0;
        for (int s = 0; s < a.n_stages; s++) {
            mbar_init(smem_u32(&bars[s]), TILE_ROWS);                        // full: one arrival per row copy
            mbar_init(smem_u32(&bars[MAX_STAGES + s]), GROUP_WARPS);         // empty: one per warp of the group that reads the stage
        }
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    const int packed_row = a.nsb * Unit<FMT>::BLOCK_BYTES;

    if (warp == 0) {
        // ---------------- producer: resident weights do not depend on earlier kernels, start at once ----------------
        if (!a.static_weights) pdl_wait_prior();   // otherwise W may be the output of the kernel before this one
        if (lane < TILE_ROWS) {
            int item = 0, stage = 0;
            uint32_t use = 0;
            for (int k = 0; k < my_items; k++) {
                const int part = parted ? (int)((item_lo + k) / a.n_tiles) : 0;
                const int gtile = parted ? (int)(item_lo + k - (long long)part * a.n_tiles) : (int)(blockIdx.x + gridDim.x * k);
                const int mi = (gtile >= a.tile_start[1]) + (gtile >= a.tile_start[2]);
                const int tile = gtile - a.tile_start[mi];
                const uint8_t* Wm = mi == 0 ? a.W : a.W_more[mi - 1];
                const int Mm = mi == 0 ? a.M : a.M_more[mi - 1];
                const uintptr_t safe_end = ((uintptr_t)Wm + (uintptr_t)(Mm - 1) * a.row_bytes + packed_row) & ~(uintptr_t)15;
                const int part_sb = parted ? a.part_sb0[part] : 0, part_end = parted ? a.part_sb0[part + 1] : a.nsb;
                for (int chunk = 0; chunk < a.n_chunks; chunk++) {
                    const uint32_t full = smem_u32(&bars[stage]);
                    const uint32_t empty = smem_u32(&bars[MAX_STAGES + stage]);
                    mbar_wait_bounded(empty, use ^ 1u, abort_flag, a.status, ST_WAIT_EMPTY_TIMEOUT);
                    const int row = tile * TILE_ROWS + lane;
                    if (row >= Mm) {
                        mbar_arrive(full);
                    } else {
                        const int sb0 = part_sb + chunk * a.chunk_sb;
                        const int len = min(a.chunk_sb, part_end - sb0) * Unit<FMT>::BLOCK_BYTES;
                        const uintptr_t src = (uintptr_t)Wm + (uintptr_t)row * a.row_bytes + (uintptr_t)sb0 * Unit<FMT>::BLOCK_BYTES;
                        const uintptr_t lo = src & ~(uintptr_t)15;
                        uintptr_t hi = (src + len + 15) & ~(uintptr_t)15;
                        uint8_t* slot = smem + a.off_stage + (size_t)stage * a.stage_bytes + (size_t)lane * a.slot_stride;
                        if (hi > safe_end) {
                            // the last bytes of the tensor do not fill a 16-byte unit: fetch them with plain loads
                            hi = safe_end > lo ? safe_end : lo;
                            for (uintptr_t p = hi; p < src + len; p += 2)
                                if (p >= src) *(uint16_t*)(slot + (p - lo)) = *(const uint16_t*)p;
                        }
                        const uint32_t bytes = (uint32_t)(hi - lo);
                        if (bytes) {
                            mbar_arrive_expect_tx(full, bytes);
                            bulk_copy_g2s(smem_u32(slot), (const void*)lo, bytes, full);
                        } else {
                            mbar_arrive(full);
                        }
                    }
                    item++;
                    if (++stage == a.n_stages) { stage = 0; use ^= 1u; }
                    __syncwarp((1u << TILE_ROWS) - 1u);
                    if (lane == 0) st_release_shared(smem_u32(issued), item);
                }
            }
        }
        return;
    }

    if (PARTED && warp == 1 + NGROUPS * GROUP_WARPS) {
        // ---------------- K-parts: the warp that counts the parts of a tile and adds them up ----------------
        // The consumers drop an item's 128 sums into the scratch area and carry on.  This warp raises the tile's counter
        // (the count comes back while it waits for the next item); when it drew the last count -- whoever computed the
        // other parts -- it adds the tile's parts up in part order and stores the rows.  No fences: a slot holds
        // PART_EMPTY (a NaN pattern no sum can have) until its sums land, and this warp looks at a slot until it has
        // them -- they are on their way, their writer has already moved on -- then leaves the slot empty and the
        // counter at zero for the next launch.
        pdl_wait_prior();
        auto add_up = [&](int ft) {
            const int mi = (ft >= a.tile_start[1]) + (ft >= a.tile_start[2]);
            const int tile = ft - a.tile_start[mi];
            const int Mm = mi == 0 ? a.M : a.M_more[mi - 1];
            const long long ld = mi == 0 ? a.y_ld : a.y_ld_more[mi - 1];
            float* ym = mi == 0 ? a.y : a.y_more[mi - 1];
            float* sp = a.parts + (size_t)ft * a.n_parts * 128 + lane;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            const long long t0 = clock64();
            for (int p0 = 0; p0 < a.n_parts; p0 += 4) {   // the loads of four parts go out together
                uint32_t u[4][4];
                bool all = false;
                while (!all) {
                    all = true;
#pragma unroll
                    for (int pp = 0; pp < 4; pp++)
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            u[pp][i] = 0u;
                            if (p0 + pp < a.n_parts)
                                asm volatile("ld.relaxed.gpu.global.b32 %0, [%1];" : "=r"(u[pp][i]) : "l"(sp + (p0 + pp) * 128 + 32 * i) : "memory");
                        }
#pragma unroll
                    for (int pp = 0; pp < 4; pp++)
#pragma unroll
                        for (int i = 0; i < 4; i++) all = all && u[pp][i] != PART_EMPTY;
                    all = __all_sync(0xffffffffu, all);
                    if (!all && clock64() - t0 > WAIT_BUDGET_CYCLES) {
                        if (lane == 0) atomicOr(a.status, ST_WAIT_FULL_TIMEOUT);
                        break;
                    }
                }
#pragma unroll
                for (int pp = 0; pp < 4; pp++)
                    if (p0 + pp < a.n_parts) {
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            v[i] = p0 + pp == 0 ? __uint_as_float(u[pp][i]) : v[i] + __uint_as_float(u[pp][i]);
                            __stcg((uint32_t*)(sp + (p0 + pp) * 128 + 32 * i), PART_EMPTY);
                        }
                    }
            }
            if (lane == 0) a.part_count[ft] = 0;
#pragma unroll
            for (int i = 0; i < 4; i++) {   // sum 32 i + lane of the tile: the layout of the consumers' summing threads
                const int row = tile * TILE_ROWS + (lane >> 2) + 8 * (i >> 1);
                const int col = 2 * (lane & 3) + (i & 1);
                if (row < Mm && col < a.nb) {
                    float* yo = ym + (size_t)col * ld + row;
                    const float out = a.accumulate ? *yo + v[i] : v[i];
                    *yo = out;
                    for (int pr = 0; pr < a.n_peers; pr++) (mi == 0 ? a.y_peer[pr] : a.y_peer_more[mi - 1][pr])[(size_t)col * ld + row] = out;
                }
            }
        };
        int pending = -1, pending_tile = 0;
        for (int k = 0; k < my_items; k++) {
            const int grp = k % NGROUPS, nth = k / NGROUPS;
            if (!wait_counter_bounded(smem_u32(parts_written + grp), 4 * (nth + 1) - 1, abort_flag, a.status, ST_WAIT_FULL_TIMEOUT, WAIT_BUDGET_CYCLES, 256)) return;
            const int part = (int)((item_lo + k) / a.n_tiles);
            const int gtile = (int)(item_lo + k - (long long)part * a.n_tiles);
            const int before = pending, before_tile = pending_tile;
            if (lane == 0) pending = atomicAdd(a.part_count + gtile, 1);
            pending_tile = gtile;
            if (k > 0 && __shfl_sync(0xffffffffu, before, 0) == a.n_parts - 1) add_up(before_tile);
        }
        if (my_items > 0 && __shfl_sync(0xffffffffu, pending, 0) == a.n_parts - 1) add_up(pending_tile);
        return;
    }

    // ---------------- consumers ----------------
    const int ctid = tid - 32;                       // 0 .. NGROUPS*256-1
    const int grp = ctid / GROUP_THREADS;
    const int gw = (ctid % GROUP_THREADS) >> 5;      // warp inside the group
    const int gtid = ctid % GROUP_THREADS;
    const int g = lane >> 2, t = lane & 3;

    // stage the codebook (replicated so that lane l reads bank l) and the activations
    float* actd = (float*)(smem + a.off_actd);       // [win_sb][8]
    uint8_t* actq = smem + a.off_actq;               // [nb][act_sb * 256], staged order
    uint32_t* cbw = (uint32_t*)(smem + a.off_cb);
    constexpr int CBN = Unit<FMT>::CODEBOOK_ENTRIES;
    if (CBN > 0) {
        const int rep = 1 << a.cb_rep_log2;
        for (int i = ctid; i < CBN * rep; i += NGROUPS * GROUP_THREADS) cbw[i] = a.codebook[i >> a.cb_rep_log2];
    }
    pdl_wait_prior();   // activations come from the previous kernel of the stream
    if (a.x_f32) {
        // quantize the columns here (every CTA, the arithmetic of quantize_q8k_kernel): one warp per 256 values, the
        // loads of five blocks going out together (seven columns of K = 5120 are 140 blocks for 16 warps: two rounds)
        constexpr int QB = 5, NW = NGROUPS * GROUP_WARPS;
        const int cwarp = ctid >> 5;
        const int n_blocks = a.nb * win_sb;
        for (int i = ctid; i < win_sb * 8; i += NGROUPS * GROUP_THREADS)
            if ((i & 7) >= a.nb) actd[i] = 0.0f;
        for (int b0 = cwarp; b0 < n_blocks; b0 += QB * NW) {
            float4 lo4[QB], hi4[QB];
#pragma unroll
            for (int j = 0; j < QB; j++) {
                const int b = b0 + j * NW;
                lo4[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                hi4[j] = lo4[j];
                if (b < n_blocks) {
                    const int c = b / win_sb, sb = b - c * win_sb;   // sb counts from the window's first super-block
                    const float* src = a.x_f32 + (size_t)c * a.x_f32_ld + (size_t)(win0 + sb) * 256 + 8 * lane;
                    lo4[j] = *(const float4*)src;
                    hi4[j] = *(const float4*)(src + 4);
                }
            }
#pragma unroll
            for (int j = 0; j < QB; j++) {
                const int b = b0 + j * NW;
                if (b >= n_blocks) continue;
                const int c = b / win_sb, sb = b - c * win_sb;
                const float v[8] = {lo4[j].x, lo4[j].y, lo4[j].z, lo4[j].w, hi4[j].x, hi4[j].y, hi4[j].z, hi4[j].w};
                uint32_t w0, w1;
                int s8;
                float d;
                q8k_block_core(v, w0, w1, s8, d);
                if (lane == 0) actd[sb * 8 + c] = d;
                uint8_t* dst = actq + (size_t)c * act_ld + sb * 256;
                if (FMT == T_IQ4_XS) {
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        const int k = 8 * lane + e;
                        dst[(k & ~31) + act_stage_pos(FMT, k & 31)] = (uint8_t)((e < 4 ? w0 : w1) >> (8 * (e & 3)));
                    }
                } else {
                    *(uint2*)(dst + 8 * lane) = make_uint2(w0, w1);
                }
            }
        }
    } else {
        // copy the Q8_K blocks' scales and values: one warp per block (256 values = 64 words: lane l takes words w and
        // w + 4 of the 32-value group l / 4, w = l % 4), the loads of eight blocks going out together
        constexpr int SB = 8, NW = NGROUPS * GROUP_WARPS;
        const int cwarp = ctid >> 5;
        const int n_blocks = a.nb * win_sb;
        for (int i = ctid; i < win_sb * 8; i += NGROUPS * GROUP_THREADS)
            if ((i & 7) >= a.nb) actd[i] = 0.0f;
        const int wofs = 8 * (lane >> 2) + (lane & 3);
        for (int b0 = cwarp; b0 < n_blocks; b0 += SB * NW) {
            uint32_t w0[SB], w1[SB], dw[SB];
#pragma unroll
            for (int jb = 0; jb < SB; jb++) {
                const int b = b0 + jb * NW;
                w0[jb] = w1[jb] = dw[jb] = 0u;
                if (b < n_blocks) {
                    const int c = b / win_sb, sb = b - c * win_sb;
                    const uint32_t* blk = (const uint32_t*)(a.xq + ((size_t)c * a.x_stride + win0 + sb) * Q8K_BYTES);
                    w0[jb] = blk[1 + wofs];
                    w1[jb] = blk[5 + wofs];
                    if (lane == 0) dw[jb] = blk[0];
                }
            }
#pragma unroll
            for (int jb = 0; jb < SB; jb++) {
                const int b = b0 + jb * NW;
                if (b >= n_blocks) continue;
                const int c = b / win_sb, sb = b - c * win_sb;
                if (lane == 0) actd[sb * 8 + c] = __uint_as_float(dw[jb]);
                uint8_t* dst = actq + (size_t)c * act_ld + sb * 256 + 32 * (lane >> 2);
                if (FMT == T_IQ4_XS) {
                    // act_stage_pos: value k of the group goes to 8 (k % 16 / 4) + 2 (k % 4) + k / 16, i.e. the bytes of
                    // words w and w + 4 interleaved
                    *(uint2*)(dst + 8 * (lane & 3)) = make_uint2(prmt(w0[jb], w1[jb], 0x5140u), prmt(w0[jb], w1[jb], 0x7362u));
                } else {
                    *(uint32_t*)(dst + 4 * (lane & 3)) = w0[jb];
                    *(uint32_t*)(dst + 16 + 4 * (lane & 3)) = w1[jb];
                }
            }
        }
    }
    named_bar_sync(15, NGROUPS * GROUP_THREADS);

    Codebook cb;
    cb.words = cbw;
    cb.rep_log2 = a.cb_rep_log2;
    cb.lane_word = (uint32_t)lane & ((1u << a.cb_rep_log2) - 1u);

    float* red = (float*)(smem + a.off_red) + (size_t)grp * 2 * GROUP_THREADS * 4;
    const bool bvalid = g < a.nb;
    const uint8_t* bq_col = actq + (size_t)(bvalid ? g : 0) * act_ld - (size_t)win0 * 256;   // indexed by the super-block's number in the row

    const float* actd_row = actd - win0 * 8;
    // K-parts: (part, tile) of this group's next item, stepped NGROUPS items at a time
    int part_next = parted ? (int)((item_lo + grp) / a.n_tiles) : 0;
    int gtile_next = parted ? (int)(item_lo + grp - (long long)part_next * a.n_tiles) : 0;
    const uint32_t row_bytes_lo = (uint32_t)a.row_bytes;
    int ring_stage = (grp * a.n_chunks) % a.n_stages;   // stage and use count of this group's next fill
    uint32_t ring_use = (uint32_t)((grp * a.n_chunks) / a.n_stages);
    for (int ti = 0;; ti++) {
        const int k = grp + NGROUPS * ti;                // this CTA's work item k
        if (k >= my_items) break;
        const int part = parted ? part_next : 0;
        const int gtile = parted ? gtile_next : (int)(blockIdx.x + gridDim.x * k);
        if (parted) {
            gtile_next += NGROUPS;
            while (gtile_next >= a.n_tiles) { gtile_next -= a.n_tiles; part_next++; }
        }
        const int mi = (gtile >= a.tile_start[1]) + (gtile >= a.tile_start[2]);
        const int tile = gtile - a.tile_start[mi];        // tile of matrix mi
        const uint32_t Wm_lo = (uint32_t)(uintptr_t)(mi == 0 ? a.W : a.W_more[mi - 1]);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        const int rowA = tile * TILE_ROWS + g;
        const int part_sb = parted ? a.part_sb0[part] : 0, part_end = parted ? a.part_sb0[part + 1] : a.nsb;
        for (int chunk = 0; chunk < a.n_chunks; chunk++) {
            const int item = k * a.n_chunks + chunk;      // fill number; its stage and use are stepped, not divided out
            const int stage = ring_stage;
            const uint32_t use = ring_use;
            const int step = chunk + 1 < a.n_chunks ? 1 : 1 + (NGROUPS - 1) * a.n_chunks;   // on to this group's next item
            ring_stage += step;
            while (ring_stage >= a.n_stages) { ring_stage -= a.n_stages; ring_use++; }
            const uint32_t full = smem_u32(&bars[stage]);
            const uint32_t empty = smem_u32(&bars[MAX_STAGES + stage]);
            // a group reads only its own items' fills, so it skips uses of a barrier: once the fill has been issued (the
            // producer issues it after the readers of the stage's previous fill released it) the parity is unambiguous
            wait_counter_bounded(smem_u32(issued), item, abort_flag, a.status, ST_WAIT_FULL_TIMEOUT);
            mbar_wait_bounded(full, use & 1u, abort_flag, a.status, ST_WAIT_FULL_TIMEOUT);
            const int sb0 = part_sb + chunk * a.chunk_sb;
            const int nsb_c = min(a.chunk_sb, part_end - sb0);
            const uint8_t* st = smem + a.off_stage + (size_t)stage * a.stage_bytes;
            // a row slice sits in its slot at the low 4 bits of its global address (32-bit arithmetic is enough for those)
            const uint32_t srcA = Wm_lo + (uint32_t)rowA * row_bytes_lo + (uint32_t)sb0 * Unit<FMT>::BLOCK_BYTES;
            const uint32_t srcB = srcA + 8u * row_bytes_lo;
            const uint8_t* baseA = st + g * a.slot_stride + (srcA & 15u);
            const uint8_t* baseB = st + (g + 8) * a.slot_stride + (srcB & 15u);
            for (int u = gw; u < 2 * nsb_c; u += GROUP_WARPS) {
                const int sbi = u >> 1, h = u & 1;
                const int gsb = sb0 + sbi;
                ActLane al;
                al.q = bq_col + gsb * 256;
                al.valid = bvalid;
                const float2 dx = *(const float2*)(actd_row + gsb * 8 + 2 * t);
                al.dx0 = dx.x;
                al.dx1 = dx.y;
                Unit<FMT>::run(baseA + sbi * Unit<FMT>::BLOCK_BYTES, baseB + sbi * Unit<FMT>::BLOCK_BYTES, h, al, cb, acc);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty);
        }
        // add the 8 warps' partial sums in warp order and store the tile
        float* rbuf = red + (size_t)(ti & 1) * GROUP_THREADS * 4;
        *(float4*)(rbuf + (gw * 32 + lane) * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        named_bar_sync(1 + grp, GROUP_THREADS);
        if (gtid < 128) {
            const int ls = gtid & 31, i = gtid >> 5;
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < GROUP_WARPS; w++) v += rbuf[(w * 32 + ls) * 4 + i];
            if (parted) {   // the tile's other parts are other CTAs' work: hand the sums to the adding warp and carry on
                __stcg(a.parts + ((size_t)gtile * a.n_parts + part) * 128 + gtid, v);
                __syncwarp();
                if (lane == 0) red_release_shared_add(smem_u32(parts_written + grp), 1);
                continue;
            }
            const int row = tile * TILE_ROWS + (ls >> 2) + 8 * (i >> 1);
            const int col = 2 * (ls & 3) + (i & 1);
            const int Mm = mi == 0 ? a.M : a.M_more[mi - 1];
            if (row < Mm && col < a.nb) {
                float* yo = (mi == 0 ? a.y : a.y_more[mi - 1]) + (size_t)col * (mi == 0 ? a.y_ld : a.y_ld_more[mi - 1]) + row;
                const float out = a.accumulate ? *yo + v : v;
                *yo = out;
                for (int pr = 0; pr < a.n_peers; pr++)
                    (mi == 0 ? a.y_peer[pr] : a.y_peer_more[mi - 1][pr])[(size_t)col * (mi == 0 ? a.y_ld : a.y_ld_more[mi - 1]) + row] = out;
            }
        }
    }
}

}  // namespace q38b
