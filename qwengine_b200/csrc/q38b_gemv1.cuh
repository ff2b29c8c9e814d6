// q38b_gemv1.cuh -- single-column decode matvec: y[r] (+)= W[r,:] . x.
//
// Same streaming scheme as gemv_kernel (persistent CTA per SM, producer warp, 1-D bulk copies of each row slice's
// 16-byte aligned superset into a ring of stages guarded by mbarriers).  A stage holds a tile of rows (or a K-chunk of
// it); a (tile, 1024-weight slice) unit belongs to ONE consumer warp: lane l owns granule l of the slice, holds its int8
// activations in registers for all rows of the tile and runs the dp4a decoders of q38b_decode1.cuh (or, for IQ3_XXS,
// the row-group mapping there).  Units go to the warps round-robin, so the warps never synchronise with each other
// except through the per-tile reduction: each (tile, slice) writes its row sums to its own slot and arrives on the
// tile's mbarrier; the warp that took the tile's last slice waits for the others, adds the slices in order
// (deterministic) and stores y.
#pragma once
#include "q38b_act.cuh"
#include "q38b_decode1.cuh"
#include "q38b_pipe.cuh"

namespace q38b {

constexpr int G1_MAX_STAGES = 64;
constexpr int G1_MAX_TILEBUF = 64;

constexpr int G1_MAX_MATS = 3;

struct Gemv1Args {
    // up to three matrices of one format, K and row stride that read the same column: their tiles form one sequence
    // (matrix 0's tiles, then matrix 1's, ...), so one launch replaces three and the CTAs' leftovers even out
    const uint8_t* W;
    const uint8_t* W_more[G1_MAX_MATS - 1];
    float* y_more[G1_MAX_MATS - 1];
    int M_more[G1_MAX_MATS - 1];
    int tile_start[G1_MAX_MATS];   // first tile of each matrix in the sequence (tile_start[0] = 0; unused ones = n_tiles)
    long long row_bytes;
    const float* xd32;      // per-32 activations (kernels instantiated with A32): xq = K int8 values, xd32 = K / 32 scales
    const uint8_t* xq;      // Q8_K blocks of the single column, or nullptr:
    const float* x_f32;     // then the K floats of the column, quantized to Q8_K blocks by every CTA in its prologue
    float* y;
    float* y_peer[7];       // the same output position in the buffers of the other GPUs (peer stores), n_peers used
    float* y_peer_more[G1_MAX_MATS - 1][7];   // the same for matrices 1 and 2
    PeerSync sync;          // cross-GPU barrier before the column is read (the peers pushed parts of it), n = 0: none
    int n_peers;
    int static_weights;     // 1: W was written long before this launch, the producer need not wait for earlier kernels
    int* status;
    const uint32_t* codebook;
    int K, M, accumulate;
    int nsb;                // super-blocks per row
    int n_slices;           // ceil(nsb / 4)
    int n_tiles;            // tiles of all matrices
    int n_stages;
    int chunk_slices;       // slices per stage (K-chunk); n_chunks = ceil(n_slices / chunk_slices)
    int n_chunks;
    int contiguous;         // 1: a stage is 8 whole packed rows, fetched by one bulk copy
    int slot_stride;        // bytes between the rows of a stage (row_bytes when contiguous)
    int stage_bytes;
    int n_tilebuf;
    int cb_rep_log2;
    int off_actd, off_actq, off_cb, off_sgn, off_red, off_stage;   // off_sgn: IQ3_XXS sign-mask table (KSIGN_TABLE_BYTES)
};

// One block of the slice for every row pass of a row-group tile (B is a template argument: the alignment of the block's
// fields follows from it).
template <int FMT, int B, int NPASS>
__device__ __forceinline__ void rowgroup_block(const SP (&rowp)[NPASS], int s, SP act_block, SP actd_block, const TablesR& tabs, float (&acc)[NPASS]) {
    ActsR ar;
    GranR<FMT>::load_acts(ar, act_block, actd_block, s);
#pragma unroll
    for (int ps = 0; ps < NPASS; ps++) acc[ps] += GranR<FMT>::template dot<B>(rowp[ps], s, ar, tabs);
}

// Tile `gtile` of the launch's sequence (matrix 0's tiles, then matrix 1's, ...): the matrix and the first row inside it.
struct TileRef { int mi, row0; };
template <int ROWS>
__device__ __forceinline__ TileRef tile_ref(const Gemv1Args& a, int gtile) {
    TileRef t;
    t.mi = (gtile >= a.tile_start[1]) + (gtile >= a.tile_start[2]);
    t.row0 = (gtile - a.tile_start[t.mi]) * ROWS;
    return t;
}

// shared-memory tables of the row-group decoders (static, so that their addresses are immediates of the loads)
constexpr int RG_CB_WORDS = 256 * 32, RG_SGN_WORDS = 128 * 32;
constexpr int RG_STATIC_BYTES = 4 * (RG_CB_WORDS + RG_SGN_WORDS);

// ROWS = rows per tile and stage (8, 16 for row groups with an SM to themselves, fewer when no such plan fits shared memory).
// RG: the row-group mapping of q38b_decode1.cuh (IQ3_XXS, rows 8 bytes aligned): lane = (row of a group of four,
// sub-block), tables in static shared memory, activations staged in the layout of actr_pos.
// A32: the column is given in the reference GPU path's per-32 format (ActQ8: xq = int8 values, xd32 = one scale per 32).
// OCC: CTAs per SM the kernel is built for: 1 (NWARPS = 24 consumer warps, 20 for row groups, all of the SM's shared
// memory: one set of tables and one quantized column per SM, deeper rings, larger tiles; the default plan) or 2 (eight
// consumer warps and half the shared memory each, for shapes whose one-CTA plan does not fit).
template <int FMT, int NWARPS, int ROWS, bool RG, bool A32, int OCC>
__global__ void __launch_bounds__(32 * (1 + NWARPS), OCC) gemv1_kernel(const Gemv1Args a) {
    constexpr int G1_ROWS = ROWS;
    static_assert(!RG || (FMT == T_IQ3_XXS && ROWS % 4 == 0), "row-group mapping: IQ3_XXS, tiles of 4, 8 or 16 rows");
    static_assert(RG || ROWS <= 8, "the lane-per-granule mapping reduces at most eight rows per unit");
    static_assert(!(RG && A32), "per-32 activations run on the lane-per-granule mapping");
    // tables of the row-group decoders: static shared memory (their addresses become immediates of the loads); kernels
    // without them have no static shared memory at all, so that two CTAs of 113 KB still fit an SM
    uint32_t* rg_cb = nullptr;
    uint32_t* rg_sgn = nullptr;
    if constexpr (RG) {
        __shared__ __align__(128) uint32_t rg_cb_store[RG_CB_WORDS];
        __shared__ __align__(128) uint32_t rg_sgn_store[RG_SGN_WORDS];
        rg_cb = rg_cb_store;
        rg_sgn = rg_sgn_store;
    }
    extern __shared__ __align__(128) uint8_t smem_raw[];   // plain pointer arithmetic from here on keeps loads in the shared space
    uint8_t* smem = smem_raw;
    uint64_t* full = (uint64_t*)smem;                        // [G1_MAX_STAGES]
    uint64_t* empty = full + G1_MAX_STAGES;                  // [G1_MAX_STAGES]
    uint64_t* tbar = empty + G1_MAX_STAGES;                  // [G1_MAX_TILEBUF]
    volatile int* abort_flag = (volatile int*)(tbar + G1_MAX_TILEBUF);
    int* issued = (int*)abort_flag + 1;                      // stage fills the producer has issued so far
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int BB = Unit<FMT>::BLOCK_BYTES;
    constexpr int SLICE_BYTES = 4 * BB;

    if (tid == 0) {
        *abort_flag = 0;
        *issued = 0;
        for (int s = 0; s < a.n_stages; s++) { mbar_init(smem_u32(&full[s]), G1_ROWS); mbar_init(smem_u32(&empty[s]), a.chunk_slices); }
        for (int t = 0; t < a.n_tilebuf; t++) mbar_init(smem_u32(&tbar[t]), a.n_slices);
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    // tiles are dealt round-robin: CTA b takes tiles b, b + grid, b + 2 grid, ...
    const int my_tiles = a.n_tiles > (int)blockIdx.x ? (a.n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int n_items = my_tiles * a.n_chunks;       // stages this CTA streams
    const int packed_row = a.nsb * BB;

    if (warp == 0) {
        // ---------------- producer ----------------
        if (!a.static_weights) pdl_wait_prior();   // W may be the output of the kernel before this one
        if (lane < G1_ROWS) {
            int ti = 0, chunk = 0, stage = 0;
            uint32_t use = 0;                      // parity of the number of earlier fills of this stage
            for (int item = 0; item < n_items; item++) {
                const uint32_t fb = smem_u32(&full[stage]);
                mbar_wait_bounded(smem_u32(&empty[stage]), use ^ 1u, abort_flag, a.status, ST_WAIT_EMPTY_TIMEOUT);
                const TileRef tr = tile_ref<G1_ROWS>(a, (int)blockIdx.x + (int)gridDim.x * ti);
                const int mi = tr.mi, row0 = tr.row0;
                const uint8_t* Wm = mi == 0 ? a.W : a.W_more[mi - 1];
                const int Mm = mi == 0 ? a.M : a.M_more[mi - 1];
                const int rows_here = min(G1_ROWS, Mm - row0);
                const uintptr_t safe_end = ((uintptr_t)Wm + (uintptr_t)(Mm - 1) * a.row_bytes + packed_row) & ~(uintptr_t)15;
                uint8_t* sbase = smem + a.off_stage + (size_t)stage * a.stage_bytes;
                // what this lane copies: the whole tile (lane 0, contiguous rows) or its own row's chunk
                uintptr_t src = 0;
                long long len = 0;
                uint8_t* slot = sbase;
                if (a.contiguous) {
                    if (lane == 0) {
                        src = (uintptr_t)Wm + (uintptr_t)row0 * a.row_bytes;
                        len = (long long)rows_here * a.row_bytes;
                    }
                } else if (lane < rows_here) {
                    const int off = chunk * a.chunk_slices * SLICE_BYTES;
                    src = (uintptr_t)Wm + (uintptr_t)(row0 + lane) * a.row_bytes + (uintptr_t)off;
                    len = min(a.chunk_slices * SLICE_BYTES, packed_row - off);
                    slot = sbase + (size_t)lane * a.slot_stride;
                }
                if (len <= 0) {
                    mbar_arrive(fb);
                } else {
                    const uintptr_t lo = src & ~(uintptr_t)15;
                    uintptr_t hi = (src + len + 15) & ~(uintptr_t)15;
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
                }
                if (++chunk == a.n_chunks) { chunk = 0; ti++; }
                if (++stage == a.n_stages) { stage = 0; use ^= 1u; }
                __syncwarp((1u << G1_ROWS) - 1u);
                if (lane == 0) st_release_shared(smem_u32(issued), item + 1);
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    const int cw = warp - 1;
    const int ctid = tid - 32;
    float* actd = (float*)(smem + a.off_actd);       // [nsb][8], column 0 used
    uint8_t* actq = smem + a.off_actq;               // [n_slices * 1024] staged order
    uint32_t* cbw = (uint32_t*)(smem + a.off_cb);
    constexpr int CBN = Unit<FMT>::CODEBOOK_ENTRIES;
    if (a.sync.n > 0 && blockIdx.x == 0 && ctid < a.sync.n) {   // tell the peers first: the flags travel while the tables are filled
        pdl_wait_prior();
        peer_sync_signal(a.sync, ctid);
    }
    if (RG) {
        // the 32 replicas of an entry are 128 bytes: thread t writes 16 of them, so that a warp's store covers 512
        // consecutive bytes (entries by the thread would put all 32 lanes on the same four banks)
        constexpr int NT = NWARPS * 32, CB_ROUNDS = (256 * 8 + NT - 1) / NT;
        uint32_t cbv[CB_ROUNDS];
#pragma unroll
        for (int i = 0; i < CB_ROUNDS; i++) cbv[i] = a.codebook[min(ctid + i * NT, 256 * 8 - 1) >> 3];   // the loads go out together
#pragma unroll
        for (int i = 0; i < CB_ROUNDS; i++)
            if (ctid + i * NT < 256 * 8) ((uint4*)rg_cb)[ctid + i * NT] = make_uint4(cbv[i], cbv[i], cbv[i], cbv[i]);
        for (int t = ctid; t < 128 * 8; t += NWARPS * 32) {
            const uint32_t v = ksign_selectors((uint32_t)t >> 3);
            ((uint4*)rg_sgn)[t] = make_uint4(v, v, v, v);
        }
    } else if (CBN > 0) {
        const int rep = 1 << a.cb_rep_log2;
        for (int i = ctid; i < CBN * rep; i += NWARPS * 32) cbw[i] = a.codebook[i >> a.cb_rep_log2];
    } else if (code16_entries(FMT) > 0) {   // the grid as 16-bit codes, one copy (two entries per word)
        for (int i = ctid; i < code16_entries(FMT) / 2; i += NWARPS * 32) cbw[i] = a.codebook[i];
    }
    if (FMT == T_IQ3_XXS && !RG) {
        uint32_t* sg = (uint32_t*)(smem + a.off_sgn);
        for (int i = ctid; i < 128 * 16; i += NWARPS * 32) {   // code i / 16, replica i % 16
            uint32_t lo, hi;
            ksign_entry((uint32_t)i >> 4, lo, hi);
            sg[2 * i] = lo;
            sg[2 * i + 1] = hi;
        }
    }
    pdl_wait_prior();
    if (a.sync.n > 0) {
        peer_sync_poll(a.sync, ctid, a.status);
        named_bar_sync(14, NWARPS * 32);
    }
    if (a.x_f32) {
        // quantize the column here (every CTA, the same arithmetic as quantize_q8k_kernel): one warp per 256 values.  The
        // loads of three blocks go out together, so the warp pays the round trip to L2 once per three blocks.
        constexpr int QB = 3;
        for (int sb0 = cw; sb0 < a.n_slices * 4; sb0 += QB * NWARPS) {
            float4 lo4[QB], hi4[QB];
#pragma unroll
            for (int j = 0; j < QB; j++) {
                const int sb = sb0 + j * NWARPS;
                lo4[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                hi4[j] = lo4[j];
                if (sb < a.nsb) {
                    lo4[j] = *(const float4*)(a.x_f32 + (size_t)sb * 256 + 8 * lane);
                    hi4[j] = *(const float4*)(a.x_f32 + (size_t)sb * 256 + 8 * lane + 4);
                }
            }
#pragma unroll
            for (int j = 0; j < QB; j++) {
                const int sb = sb0 + j * NWARPS;
                if (sb >= a.n_slices * 4) continue;
                uint32_t w0 = 0, w1 = 0;
                float d = 0.0f;
                if (sb < a.nsb) {
                    const float v[8] = {lo4[j].x, lo4[j].y, lo4[j].z, lo4[j].w, hi4[j].x, hi4[j].y, hi4[j].z, hi4[j].w};
                    int s8;
                    q8k_block_core(v, w0, w1, s8, d);
                }
                if (lane == 0) actd[sb * 8] = d;
                uint8_t* dst = actq + (sb >> 2) * 1024;   // the block's slice
                const int k0 = (sb & 3) * 256 + 8 * lane;    // this lane's eight values in the slice
                if (RG) {
                    uint8_t* blk = actq + sb * ACTR_BLOCK_BYTES;
                    *(uint2*)(blk + actr_pos(8 * lane, 0)) = make_uint2(w0, w1);
                    *(uint2*)(blk + actr_pos(8 * lane, 1)) = make_uint2(neg_bytes4(w0), neg_bytes4(w1));
                } else if (FMT == T_IQ4_XS) {
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        const int k = k0 + e;
                        dst[act_slice_pos(FMT, (k & ~31) + act_stage_pos(FMT, k & 31))] = (uint8_t)((e < 4 ? w0 : w1) >> (8 * (e & 3)));
                    }
                } else {
                    *(uint2*)(dst + act_slice_pos(FMT, k0)) = make_uint2(w0, w1);
                }
            }
        }
    } else {
    if (A32) {
        for (int i = ctid; i < a.n_slices * 32; i += NWARPS * 32) actd[i] = i < a.nsb * 8 ? a.xd32[i] : 0.0f;
    } else {
        for (int i = ctid; i < a.n_slices * 4; i += NWARPS * 32)
            actd[i * 8] = i < a.nsb ? *(const float*)(a.xq + (size_t)i * Q8K_BYTES) : 0.0f;
    }
    for (int i = ctid; i < a.n_slices * 256; i += NWARPS * 32) {   // word i of the (zero padded) activation vector
        const int sb = i >> 6, wi = i & 63;
        const uint32_t v = sb >= a.nsb ? 0u : A32 ? *(const uint32_t*)(a.xq + 4 * (size_t)i) : *(const uint32_t*)(a.xq + (size_t)sb * Q8K_BYTES + 4 + 4 * wi);
        uint8_t* dst = actq + (sb >> 2) * 1024;   // the block's slice
        const int k0 = (sb & 3) * 256 + 4 * wi;      // this word's four values in the slice
        if (RG) {
            uint8_t* blk = actq + sb * ACTR_BLOCK_BYTES;
            *(uint32_t*)(blk + actr_pos(4 * wi, 0)) = v;
            *(uint32_t*)(blk + actr_pos(4 * wi, 1)) = neg_bytes4(v);
        } else if (FMT == T_IQ4_XS) {
#pragma unroll
            for (int b = 0; b < 4; b++) {
                const int k = k0 + b;
                dst[act_slice_pos(FMT, (k & ~31) + act_stage_pos(FMT, k & 31))] = (uint8_t)(v >> (8 * b));
            }
        } else {
            *(uint32_t*)(dst + act_slice_pos(FMT, k0)) = v;
        }
    }
    }
    named_bar_sync(15, NWARPS * 32);

    Codebook1 cb;                                    // 32 replicas: lane l reads bank l
    cb.lane_base = sp_from(cbw) + 4 * (lane & ((1 << cb1_rep_log2(FMT)) - 1));
    cb.sign_base = sp_from(smem + a.off_sgn) + 8 * (lane & 15);
    const TablesR tabs{sp_from(rg_cb), sp_from(rg_sgn), 4u * (uint32_t)lane};
    const SP actq_sp = sp_from(actq), actd_sp = sp_from(actd);
    const SP stage0_sp = sp_from(smem + a.off_stage);
    float* red = (float*)(smem + a.off_red);         // [n_tilebuf][n_slices][8]

    constexpr int LPR = RG ? 8 : Gran<FMT>::LANES_PER_ROW;   // 32, or 16 when two rows share a warp pass; 8: row groups
    constexpr int PASSES = G1_ROWS * LPR / 32;       // row passes per stage
    const int sub = LPR == 32 ? 0 : LPR == 16 ? (lane >> 4) : (lane >> 3);   // which of the rows of a pass this lane works on

    const int n_units = my_tiles * a.n_slices;       // (tile, slice) units, dealt round-robin to the warps
    // The unit's (tile, slice, chunk) and the ring positions of its stage and tile buffer are stepped, never divided.
    int ti = 0, slice = cw;
    while (slice >= a.n_slices) { slice -= a.n_slices; ti++; }
    int chunk = 0, cslice = slice;
    while (cslice >= a.chunk_slices) { cslice -= a.chunk_slices; chunk++; }
    int cur_item = 0, stage = 0, cur_ti = 0, tslot = 0;
    uint32_t stage_par = 0, tile_par = 0;            // parities of the earlier uses of `stage` / `tslot`
    int seen_item = -1;                              // last stage fill this warp has waited for
    const uint32_t rb32 = (uint32_t)a.row_bytes;
    const uint32_t rb_step = a.contiguous ? 0u : rb32;   // rows of a contiguous stage share the copy's low address bits
    for (int unit = cw; unit < n_units; unit += NWARPS) {
        const int item = ti * a.n_chunks + chunk;
        while (cur_item < item) { cur_item++; if (++stage == a.n_stages) { stage = 0; stage_par ^= 1u; } }
        while (cur_ti < ti) { cur_ti++; if (++tslot == a.n_tilebuf) { tslot = 0; tile_par ^= 1u; } }
        // A warp reads only some of the stages, so it can reach stage fill `item` while the fill before it of the same
        // barrier is still in flight (bulk copies complete in any order); a parity wait alone would take that older
        // phase for this one.  The producer issues a fill only after the readers of the previous use of the barrier have
        // released it, i.e. after that phase completed: once `issued` has passed `item` the parity is unambiguous.
        if (item > seen_item) {
            wait_counter_bounded(smem_u32(issued), item, abort_flag, a.status, ST_WAIT_FULL_TIMEOUT);
            mbar_wait_bounded(smem_u32(&full[stage]), stage_par, abort_flag, a.status, ST_WAIT_FULL_TIMEOUT);
        }
        seen_item = item;
        const TileRef tr = tile_ref<G1_ROWS>(a, (int)blockIdx.x + (int)gridDim.x * ti);
        const int mi = tr.mi;
        const uint32_t w_lo = (uint32_t)(uintptr_t)(mi == 0 ? a.W : a.W_more[mi - 1]);
        const SP st = stage0_sp + (stage * a.stage_bytes + cslice * SLICE_BYTES);
        // low address bits of row 0 of the tile at this stage's first byte (the copy kept its low 4 address bits)
        const uint32_t src_lo = w_lo + (uint32_t)tr.row0 * rb32 + (a.contiguous ? 0u : (uint32_t)(chunk * a.chunk_slices * SLICE_BYTES));
        float* rslot = red + ((size_t)tslot * a.n_slices + slice) * G1_ROWS;
        // a short last chunk holds fewer slices than the barrier expects: its last slice makes up the difference
        const int in_chunk = min(a.chunk_slices, a.n_slices - chunk * a.chunk_slices);
        const int n_arr = (cslice == in_chunk - 1) ? a.chunk_slices - in_chunk + 1 : 1;
        if constexpr (RG) {
            // row groups: lane / 8 picks one of the four rows of a pass, the four blocks of the slice in turn.  A 16-row
            // tile deals rows ps, ps + 8, ps + 4, ps + 12 to pass ps: with packed rows of 1960 bytes (K = 5120; 6664 for
            // K = 17408) rows 8 apart sit 64 bytes apart modulo a 128-byte line and rows 4 apart 32 bytes, so the two rows
            // of a half warp's 64-bit loads and the four rows of a warp's 32-bit loads fall on disjoint banks.
            const int s = lane & 7;
            const int row_of_sub = G1_ROWS == 16 ? (sub & 1) * 8 + (sub >> 1) * 4 : sub;
            SP rowp[PASSES];
            float acc[PASSES];
#pragma unroll
            for (int ps = 0; ps < PASSES; ps++) {
                const int r = G1_ROWS == 16 ? ps + row_of_sub : 4 * ps + sub;
                rowp[ps] = st + (r * a.slot_stride + (int)((src_lo + (uint32_t)r * rb_step) & 15u));
                acc[ps] = 0.0f;
            }
            const int sb0 = slice * 4;
            if (sb0 + 0 < a.nsb) rowgroup_block<FMT, 0, PASSES>(rowp, s, actq_sp + (sb0 + 0) * ACTR_BLOCK_BYTES, actd_sp + (sb0 + 0) * 32, tabs, acc);
            if (sb0 + 1 < a.nsb) rowgroup_block<FMT, 1, PASSES>(rowp, s, actq_sp + (sb0 + 1) * ACTR_BLOCK_BYTES, actd_sp + (sb0 + 1) * 32, tabs, acc);
            if (sb0 + 2 < a.nsb) rowgroup_block<FMT, 2, PASSES>(rowp, s, actq_sp + (sb0 + 2) * ACTR_BLOCK_BYTES, actd_sp + (sb0 + 2) * 32, tabs, acc);
            if (sb0 + 3 < a.nsb) rowgroup_block<FMT, 3, PASSES>(rowp, s, actq_sp + (sb0 + 3) * ACTR_BLOCK_BYTES, actd_sp + (sb0 + 3) * 32, tabs, acc);
            __syncwarp();
            if (lane == 0) mbar_arrive_n(smem_u32(&empty[stage]), n_arr);
#pragma unroll
            for (int ps = 0; ps < PASSES; ps++) {
                float v = acc[ps];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                if (s == 0) rslot[G1_ROWS == 16 ? ps + row_of_sub : 4 * ps + sub] = v;
            }
        } else {
        typename Gran<FMT>::Acts acts;
        Gran<FMT>::template load_acts<A32>(acts, actq_sp + slice * 1024, actd_sp + slice * 128, lane);
        // granules past the end of the row (K not a multiple of 1024) contribute nothing
        const int gran_sb = slice * 4 + (LPR == 32 ? (lane >> 3) : ((lane & 15) >> 2));
        const bool live = gran_sb < a.nsb;
        float acc[PASSES];
#pragma unroll
        for (int ps = 0; ps < PASSES; ps++) {
            const int r = LPR == 32 ? ps : 2 * ps + sub;
            const SP rowp = st + (r * a.slot_stride + (int)((src_lo + (uint32_t)r * rb_step) & 15u));
            const float v = Gran<FMT>::template dot<A32>(rowp, acts, cb, lane);
            acc[ps] = live ? v : 0.0f;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive_n(smem_u32(&empty[stage]), n_arr);

        // sum over the lanes of each row: halving butterflies (each step halves the values a lane holds), then plain ones
        float rowsum;
        int myrow = 0;      // the row whose sum this lane ends up with
        {
            float v[PASSES];
#pragma unroll
            for (int i = 0; i < PASSES; i++) v[i] = acc[i];
            constexpr int TOP = LPR == 32 ? 16 : 8;    // highest lane bit inside one row's lane set
            int n = PASSES, bit = TOP;
#pragma unroll
            for (int step = 0; step < 3; step++) {
                if (n > 1) {
                    const int h = n >> 1;
                    const bool up = (lane & bit) != 0;
#pragma unroll
                    for (int i = 0; i < (PASSES > 1 ? PASSES / 2 : 1); i++) {
                        if (i < h && i + h < PASSES) {
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
        // one lane per row writes: the lanes whose low bits (those folded by the plain butterflies) are zero
        constexpr int LOW_MASK = (LPR == 32 ? 32 : 16) / PASSES - 1;
        if ((lane & LOW_MASK) == 0) rslot[myrow] = rowsum;
        }
        __syncwarp();
        const uint32_t tb = smem_u32(&tbar[tslot]);
        if (lane == 0) mbar_arrive(tb);
        if (slice == a.n_slices - 1) {
            // this warp finishes the tile: wait for the other slices, add them in slice order
            mbar_wait_bounded(tb, tile_par, abort_flag, a.status, ST_WAIT_FULL_TIMEOUT);
            const int row = tr.row0 + lane;
            float* ym = mi == 0 ? a.y : a.y_more[mi - 1];
            const int Mm = mi == 0 ? a.M : a.M_more[mi - 1];
            if (lane < G1_ROWS && row < Mm) {
                const float* rs = red + (size_t)tslot * a.n_slices * G1_ROWS + lane;
                float v = 0.0f;
                for (int s = 0; s < a.n_slices; s++) v += rs[s * G1_ROWS];
                const float out = a.accumulate ? ym[row] + v : v;
                ym[row] = out;
                for (int pr = 0; pr < a.n_peers; pr++) (mi == 0 ? a.y_peer[pr] : a.y_peer_more[mi - 1][pr])[row] = out;   // fused all-gather: push to every peer
            }
        }
        slice += NWARPS;
        while (slice >= a.n_slices) { slice -= a.n_slices; ti++; }
        chunk = 0;
        cslice = slice;
        while (cslice >= a.chunk_slices) { cslice -= a.chunk_slices; chunk++; }
    }
}

}  // namespace q38b
