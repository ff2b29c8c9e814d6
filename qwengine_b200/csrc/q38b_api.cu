// q38b_api.cu -- host side of libq38b200.so: context, launch planning, C ABI (include/q38b200.h).
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>

#include "../../include/q38b200.h"
#include "q38b_act.cuh"
#include "q38b_internal.h"
#include "q38b_gemv.cuh"
#include "q38b_topk.cuh"
#include "q38b_gemv1.cuh"

using namespace q38b;

namespace {

constexpr int NGROUPS = 2;
constexpr int GEMV_WHOLE_ROW_K = 8192;          // longer rows run as K-parts (measured on B200: parts on K = 5120 / 6144 cost more per item than they even out)
constexpr long long GEMV_PART_ITEMS = 131072;   // (tile, K-part) sums the scratch area of the multi-column kernel holds: 64 MB
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

// Opt-in shared-memory size of a kernel, set once per context (= per device) and kernel; the record lives in the
// context, so two contexts on two devices never disturb each other.
int ensure_kernel_smem(q38b_ctx* ctx, const void* kern, int dyn_smem_bytes, bool max_carveout) {
    for (int i = 0; i < ctx->n_configured; i++)
        if (ctx->configured[i] == kern) return Q38B_OK;
    Q38B_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn_smem_bytes));
    if (max_carveout) Q38B_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
    if (ctx->n_configured < (int)(sizeof(ctx->configured) / sizeof(ctx->configured[0]))) ctx->configured[ctx->n_configured++] = kern;
    return Q38B_OK;
}

bool known_format(uint32_t t) {
    switch (t) {
        case T_Q8_0: case T_Q4_K: case T_Q5_K: case T_Q6_K: case T_IQ3_XXS: case T_IQ3_S: case T_IQ4_XS: return true;
        case T_Q2_K: case T_IQ2_XXS: case T_IQ2_XS: case T_IQ2_S: case T_IQ1_S: case T_IQ1_M: return true;   // one-column kernel, dequantizer, prefill
        default: return false;
    }
}

// alignment (bytes) the shared-memory loads of a format need from W and row_bytes
int format_alignment(uint32_t t) {
    switch (t) {
        case T_Q4_K: case T_Q5_K: return 16;
        case T_IQ4_XS: return 8;
        case T_Q2_K: return 4;
        default: return 2;
    }
}

// 4-super-block units per K-part: as long as two parts of activations for 8 columns and three stages of 16 rows fit
static int gemv_units_per_part(uint32_t type) { return type == T_Q8_0 ? 2 : (type == T_Q6_K || type == T_Q5_K) ? 3 : 4; }

struct Plan {
    GemvArgs a;
    int grid;
    int smem;
};

// Carves the 227 KB of shared memory of one CTA: barriers | activation scales | activations | codebook |
// reduction buffers | NGROUPS rings of n_stages stages of 16 row slots.
int plan_gemv(const q38b_ctx* ctx, uint32_t type, int K, const int* Ms, int n_mats, int nb, Plan* p) {
    if (one_column_only((int)type)) return Q38B_ERR_UNSUPPORTED;   // no fragment builders for these formats
    const int bb = block_bytes((int)type);
    const int nsb = K / 256;
    int cb_entries = type == T_IQ3_XXS ? 256 : type == T_IQ3_S ? 512 : 0;
    const int budget = ctx->smem_optin - 128;   // base is aligned up to 128 inside the kernel
    GemvArgs& a = p->a;
    a.nsb = nsb;
    a.n_tiles = 0;
    for (int i = 0; i < GEMV_MAX_MATS; i++) {
        a.tile_start[i] = a.n_tiles;
        if (i < n_mats) a.n_tiles += (Ms[i] + TILE_ROWS - 1) / TILE_ROWS;
    }
    for (int i = n_mats; i < GEMV_MAX_MATS; i++) a.tile_start[i] = a.n_tiles;
    // K-parts for rows longer than 8192: up to 16 super-blocks each (12 for Q5_K / Q6_K, 8 for Q8_0: larger blocks),
    // boundaries at multiples of 4 super-blocks.  A rule of K and the format alone, so that a sum is built from the same pieces whatever the
    // column count, the row count or the GPU count.
    const int n_units = (nsb + 3) / 4;
    const int units_per_part = gemv_units_per_part(type);
    a.n_parts = K <= GEMV_WHOLE_ROW_K ? 1 : (n_units + units_per_part - 1) / units_per_part;
    if (a.n_parts > GEMV_MAX_PARTS) a.n_parts = GEMV_MAX_PARTS;   // longer parts; the plan fails below if they do not fit
    int max_part = 0;
    for (int q = 0; q <= a.n_parts; q++) a.part_sb0[q] = std::min(nsb, 4 * (int)((long long)n_units * q / a.n_parts));
    for (int q = 0; q < a.n_parts; q++) max_part = std::max(max_part, a.part_sb0[q + 1] - a.part_sb0[q]);
    if (a.n_parts > 1 && (long long)a.n_tiles * a.n_parts > ctx->part_items) return Q38B_ERR_NOMEM;   // the scratch area's size
    // a CTA's range of (part, tile) items touches at most two neighbouring parts: it stages their activations only
    a.act_sb = a.n_parts == 1 ? nsb : std::min(nsb, 2 * max_part);
    a.off_actd = 256;
    a.off_actq = a.off_actd + align_up(a.act_sb * 32, 16);
    a.off_cb = a.off_actq + align_up(nb * a.act_sb * 256, 128);
    // rows of a group land 16 bytes (32 for the formats read with 64-bit loads) further round the 32 banks
    const int bank_skew = (type == T_Q4_K || type == T_Q5_K) ? 32 : 16;
    for (int rep_log2 = cb_entries ? 5 : 0; rep_log2 >= 0; rep_log2 -= (rep_log2 == 5 ? 2 : 3)) {
        a.cb_rep_log2 = rep_log2;
        a.off_red = a.off_cb + align_up(cb_entries * 4 << rep_log2, 128);
        a.off_stage = a.off_red + NGROUPS * 2 * GROUP_THREADS * 16;
        const int avail = budget - a.off_stage;
        // K-chunk sizes to try: the whole row (or part), then -- whole rows only -- fewer super-blocks, multiples of 4
        // first (8 half super-blocks per 4 keep the 8 warps of a group evenly loaded)
        for (int pass = 0; pass < 2; pass++)
            for (int cs = max_part; cs >= (a.n_parts == 1 ? 1 : max_part); cs--) {
                const bool even = cs == max_part || cs % 4 == 0;
                if (even != (pass == 0)) continue;
                int slot = align_up(cs * bb + 32, 16);
                while (slot % 128 != bank_skew) slot += 16;
                const int stage = TILE_ROWS * slot;
                // one ring for both groups: each reads one stage while at least one more is being filled
                const int stages = avail / stage;
                if (stages < 3 && !(stages == 2 && cs == 1)) continue;
                a.chunk_sb = cs;
                a.n_chunks = (max_part + cs - 1) / cs;
                a.n_stages = std::min(stages, MAX_STAGES);
                a.slot_stride = slot;
                a.stage_bytes = stage;
                p->smem = a.off_stage + a.n_stages * stage + 128;
                const long long items = (long long)a.n_tiles * a.n_parts;
                p->grid = (int)std::max<long long>(1, std::min<long long>(ctx->sm_count, (items + NGROUPS - 1) / NGROUPS));
                return Q38B_OK;
            }
        if (!cb_entries) break;
    }
    return Q38B_ERR_NOMEM;
}

template <int FMT>
int launch_gemv(q38b_ctx* ctx, const Plan& p, cudaStream_t st) {
    auto kern = p.a.n_parts > 1 ? gemv_kernel<FMT, NGROUPS, true> : gemv_kernel<FMT, NGROUPS, false>;
    const int rc = ensure_kernel_smem(ctx, (const void*)kern, ctx->smem_optin, false);
    if (rc != Q38B_OK) return rc;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)p.grid);
    cfg.blockDim = dim3(GEMV_THREADS + (p.a.n_parts > 1 ? 32 : 0));   // K-parts: one more warp, which adds the parts up
    cfg.dynamicSmemBytes = (size_t)p.smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->pdl ? 1 : 0;
    GemvArgs a = p.a;
    a.parts = ctx->d_parts;
    a.part_count = ctx->d_part_count;
    Q38B_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, a));
    return Q38B_OK;
}

constexpr int G1_WARPS = 8;                  // consumer warps of a CTA when two CTAs share an SM
// ... when a CTA has the SM to itself (measured on B200: the row-group decoder wants its 80 registers, which 20 warps
// leave it; the others gain from more warps in flight, 5120 x 17408 IQ4_XS 15.7 -> 12.5 us)
constexpr int G1_WARPS_ONE = 24, G1_WARPS_ONE_RG = 20;
constexpr int G1_SMEM_BUDGET = 113 * 1024;   // two CTAs per SM (228 KB of shared memory per SM, 1 KB reserved per CTA)


struct Plan1 {
    Gemv1Args a;
    int grid;
    int smem;
    int rows;   // rows per tile: 8, 4 or 2
    int rg;     // 1: row-group mapping (tables in static shared memory, activations staged twice)
    int occ;    // CTAs per SM: 2 (8 consumer warps) or 1 (16 consumer warps, the whole shared memory)
};

// The row-group decoders want every row to start 8 bytes aligned: W is 16-byte aligned, so the row stride decides.
bool rowgroup_eligible(uint32_t type, size_t row_bytes, int rows) { return type == T_IQ3_XXS && row_bytes % 8 == 0 && rows % 4 == 0; }

// Shared-memory carve-up of the single-column kernel: barriers | activation scales | activations | codebook |
// per-tile slice sums | ring of stages (8 row slots of one 1024-weight slice each).
int plan_gemv1_rows(const q38b_ctx* ctx, uint32_t type, int K, const int* Ms, int n_mats, size_t row_bytes, int G1_ROWS, int occ, Plan1* p) {
    const int bb = block_bytes((int)type);
    p->occ = occ;
    const int nsb = K / 256;
    const int rg = ctx->rowgroup && rowgroup_eligible(type, row_bytes, G1_ROWS) ? 1 : 0;
    const int warps = occ == 1 ? (rg ? G1_WARPS_ONE_RG : G1_WARPS_ONE) : G1_WARPS;
    const int cb_entries = rg ? 0 : type == T_IQ3_XXS ? 256 : type == T_IQ3_S ? 512 : 0;   // row groups keep their tables in static shared memory
    const int budget = (occ == 1 ? ctx->smem_optin : std::min(ctx->smem_optin, G1_SMEM_BUDGET)) - 128 - (rg ? RG_STATIC_BYTES : 0);
    Gemv1Args& a = p->a;
    p->rows = G1_ROWS;
    p->rg = rg;
    a.nsb = nsb;
    a.n_slices = (nsb + 3) / 4;
    a.n_tiles = 0;
    for (int i = 0; i < G1_MAX_MATS; i++) {
        a.tile_start[i] = a.n_tiles;
        if (i < n_mats) a.n_tiles += (Ms[i] + G1_ROWS - 1) / G1_ROWS;
    }
    for (int i = n_mats; i < G1_MAX_MATS; i++) a.tile_start[i] = a.n_tiles;
    a.off_actd = 1664;   // barriers (1536 bytes), flags
    a.off_actq = a.off_actd + a.n_slices * 4 * 32;
    a.off_cb = a.off_actq + a.n_slices * (rg ? 4 * ACTR_BLOCK_BYTES : 1024);
    const int packed = nsb * bb;
    // stage shape: 8 whole rows in one bulk copy when the rows are packed and small enough, else 8 per-row copies of a
    // K-chunk of `chunk_slices` slices (bulk copies are issue-rate limited: keep each above ~2 KB)
    const int target = occ == 1 ? 40 * 1024 : 28 * 1024;
    if ((long long)row_bytes == packed && G1_ROWS * packed <= target) {
        a.contiguous = 1;
        a.chunk_slices = a.n_slices;
        a.slot_stride = packed;
        a.stage_bytes = align_up(G1_ROWS * packed + 64, 128);
    } else {
        a.contiguous = 0;
        int cs = std::max(1, std::min(a.n_slices, (target / G1_ROWS - 32) / (4 * bb)));
        const int nch = (a.n_slices + cs - 1) / cs;
        cs = (a.n_slices + nch - 1) / nch;          // even chunks
        a.chunk_slices = cs;
        a.slot_stride = align_up(cs * 4 * bb + 32, 16);
        a.stage_bytes = align_up(G1_ROWS * a.slot_stride + 64, 128);
    }
    a.n_chunks = (a.n_slices + a.chunk_slices - 1) / a.chunk_slices;
    const int min_stages = (warps + a.chunk_slices - 1) / a.chunk_slices + 1;
    for (int rep_log2 = cb_entries ? cb1_rep_log2((int)type) : 0; rep_log2 >= (cb_entries ? cb1_rep_log2((int)type) : 0); rep_log2--) {   // the replica count is part of the format's decoder
        a.cb_rep_log2 = rep_log2;
        a.off_sgn = a.off_cb + align_up((cb_entries * 4 << rep_log2) + 2 * code16_entries((int)type), 128);
        a.off_red = a.off_sgn + (type == T_IQ3_XXS && !rg ? KSIGN_TABLE_BYTES : 0);
        for (int stages = G1_MAX_STAGES; stages >= min_stages; stages--) {
            // tile buffers: a warp can run at most (stages + warps) units ahead of a tile that is still being finished
            const int tb = (warps + stages * a.chunk_slices + 2 * a.n_slices - 1) / a.n_slices + 1;
            if (tb > G1_MAX_TILEBUF) continue;
            a.off_stage = align_up(a.off_red + tb * a.n_slices * G1_ROWS * 4, 128);
            if (a.off_stage + stages * a.stage_bytes + align_up(3 * bb, 128) > budget) continue;
            a.n_stages = stages;
            a.n_tilebuf = tb;
            p->smem = a.off_stage + stages * a.stage_bytes + 128 + align_up(3 * bb, 128);   // granules past a ragged row end are read (and discarded)
            p->grid = std::max(1, std::min(occ * ctx->sm_count, a.n_tiles));
            return Q38B_OK;
        }
        if (!cb_entries) break;
    }
    return Q38B_ERR_NOMEM;
}

// Rows per tile: the largest of 8, 4, 2 that can be planned.  Measured on B200 for every shape of the benchmark pass,
// eight rows win even where fewer rows would balance the CTAs better or let a tile be fetched by one copy: the cost per
// (tile, slice) unit (activation loads, waits, lane reduction) outweighs both.
// One CTA per SM with three times the consumer warps (ctx->one_cta, on by default) is tried first: one set of tables and
// one quantized column per SM, deeper rings, 16-row tiles for the row groups.  Measured on B200 it is faster than two
// CTAs per SM for every shape of the benchmark pass (4.23 ms against 4.30 ms with only long rows and row groups on it,
// 5.2 ms with none); the two-CTA plans remain for shapes whose one-CTA plan does not fit.
int plan_gemv1(const q38b_ctx* ctx, uint32_t type, int K, const int* Ms, int n_mats, size_t row_bytes, Plan1* best) {
    if (ctx->one_cta) {
        const int cands1[4] = {16, 8, 4, 2};
        for (int rows : cands1) {
            if (rows == 16 && !(ctx->rowgroup && rowgroup_eligible(type, row_bytes, 16))) continue;
            memset(best, 0, sizeof(*best));
            if (plan_gemv1_rows(ctx, type, K, Ms, n_mats, row_bytes, rows, 1, best) == Q38B_OK) return Q38B_OK;
        }
    }
    const int cands[3] = {8, 4, 2};
    for (int rows : cands) {
        memset(best, 0, sizeof(*best));
        if (plan_gemv1_rows(ctx, type, K, Ms, n_mats, row_bytes, rows, 2, best) == Q38B_OK) return Q38B_OK;
    }
    return Q38B_ERR_NOMEM;
}

template <int FMT, int ROWS, bool RG, bool A32 = false, int OCC = 2>
int launch_gemv1_rows(q38b_ctx* ctx, const Plan1& p, cudaStream_t st) {
    constexpr int WARPS = OCC == 1 ? (RG ? G1_WARPS_ONE_RG : G1_WARPS_ONE) : G1_WARPS;
    auto kern = gemv1_kernel<FMT, WARPS, ROWS, RG, A32, OCC>;
    const int rc = ensure_kernel_smem(ctx, (const void*)kern, (OCC == 1 ? ctx->smem_optin : G1_SMEM_BUDGET) - (RG ? RG_STATIC_BYTES : 0), true);
    if (rc != Q38B_OK) return rc;
    if (ctx->check_occupancy) {   // test hook: count launches whose CTAs would not be resident as often as planned
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, 32 * (1 + WARPS), (size_t)p.smem) != cudaSuccess || per_sm < OCC)
            ctx->occupancy_shortfalls++;
    }
    const Gemv1Args& args = p.a;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)p.grid);
    cfg.blockDim = dim3(32 * (1 + WARPS));
    cfg.dynamicSmemBytes = (size_t)p.smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->pdl ? 1 : 0;
    Q38B_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, args));
    return Q38B_OK;
}

template <int FMT>
int launch_gemv1(q38b_ctx* ctx, const Plan1& p, cudaStream_t st) {
    if (p.a.xd32) {   // per-32 activations: lane-per-granule mapping only
        if (p.rg) return Q38B_ERR_ARG;
        switch (p.rows) {
            case 8: return launch_gemv1_rows<FMT, 8, false, true>(ctx, p, st);
            case 4: return launch_gemv1_rows<FMT, 4, false, true>(ctx, p, st);
            case 2: return launch_gemv1_rows<FMT, 2, false, true>(ctx, p, st);
            default: return Q38B_ERR_ARG;
        }
    }
    if constexpr (FMT == T_IQ3_XXS) {
        if (p.rg && p.occ == 1 && p.rows == 16) return launch_gemv1_rows<FMT, 16, true, false, 1>(ctx, p, st);
        if (p.rg && p.occ == 1 && p.rows == 8) return launch_gemv1_rows<FMT, 8, true, false, 1>(ctx, p, st);
        if (p.rg && p.occ == 1 && p.rows == 4) return launch_gemv1_rows<FMT, 4, true, false, 1>(ctx, p, st);
        if (p.rg && p.rows == 8) return launch_gemv1_rows<FMT, 8, true>(ctx, p, st);
        if (p.rg && p.rows == 4) return launch_gemv1_rows<FMT, 4, true>(ctx, p, st);
    }
    if (p.occ == 1) {
        switch (p.rows) {
            case 8: return launch_gemv1_rows<FMT, 8, false, false, 1>(ctx, p, st);
            case 4: return launch_gemv1_rows<FMT, 4, false, false, 1>(ctx, p, st);
            case 2: return launch_gemv1_rows<FMT, 2, false, false, 1>(ctx, p, st);
            default: return Q38B_ERR_ARG;
        }
    }
    switch (p.rows) {
        case 8: return launch_gemv1_rows<FMT, 8, false>(ctx, p, st);
        case 4: return launch_gemv1_rows<FMT, 4, false>(ctx, p, st);
        case 2: return launch_gemv1_rows<FMT, 2, false>(ctx, p, st);
        default: return Q38B_ERR_ARG;
    }
}

// device table a format's decoders stage into shared memory (32-bit codebook words or 16-bit grid codes), or nullptr
const uint32_t* codebook_of(const q38b_ctx* ctx, uint32_t type) {
    switch (type) {
        case T_IQ3_XXS: return ctx->d_cb_iq3xxs;
        case T_IQ3_S: return ctx->d_cb_iq3s;
        case T_IQ2_XXS: return ctx->d_code16[0];
        case T_IQ2_XS: return ctx->d_code16[1];
        case T_IQ2_S: return ctx->d_code16[2];
        case T_IQ1_S: case T_IQ1_M: return ctx->d_code16[3];
        default: return nullptr;
    }
}

int dispatch_gemv1(q38b_ctx* ctx, uint32_t type, const Plan1& p1, cudaStream_t st) {
    switch (type) {
        case T_Q8_0: return launch_gemv1<T_Q8_0>(ctx, p1, st);
        case T_Q4_K: return launch_gemv1<T_Q4_K>(ctx, p1, st);
        case T_Q5_K: return launch_gemv1<T_Q5_K>(ctx, p1, st);
        case T_Q6_K: return launch_gemv1<T_Q6_K>(ctx, p1, st);
        case T_IQ3_XXS: return launch_gemv1<T_IQ3_XXS>(ctx, p1, st);
        case T_IQ3_S: return launch_gemv1<T_IQ3_S>(ctx, p1, st);
        case T_IQ4_XS: return launch_gemv1<T_IQ4_XS>(ctx, p1, st);
        case T_Q2_K: return launch_gemv1<T_Q2_K>(ctx, p1, st);
        case T_IQ2_XXS: return launch_gemv1<T_IQ2_XXS>(ctx, p1, st);
        case T_IQ2_XS: return launch_gemv1<T_IQ2_XS>(ctx, p1, st);
        case T_IQ2_S: return launch_gemv1<T_IQ2_S>(ctx, p1, st);
        case T_IQ1_S: return launch_gemv1<T_IQ1_S>(ctx, p1, st);
        case T_IQ1_M: return launch_gemv1<T_IQ1_M>(ctx, p1, st);
        default: return Q38B_ERR_UNSUPPORTED;
    }
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
        case T_Q2_K: dequant_rows_kernel<T_Q2_K, KIND><<<blocks, 128, 0, st>>>(W, rb, K, rows, out); break;
        case T_IQ2_XXS: dequant_rows_kernel<T_IQ2_XXS, KIND><<<blocks, 128, 0, st>>>(W, rb, K, rows, out); break;
        case T_IQ2_XS: dequant_rows_kernel<T_IQ2_XS, KIND><<<blocks, 128, 0, st>>>(W, rb, K, rows, out); break;
        case T_IQ2_S: dequant_rows_kernel<T_IQ2_S, KIND><<<blocks, 128, 0, st>>>(W, rb, K, rows, out); break;
        case T_IQ1_S: dequant_rows_kernel<T_IQ1_S, KIND><<<blocks, 128, 0, st>>>(W, rb, K, rows, out); break;
        case T_IQ1_M: dequant_rows_kernel<T_IQ1_M, KIND><<<blocks, 128, 0, st>>>(W, rb, K, rows, out); break;
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
        const void* t16[4] = {nullptr, nullptr, nullptr, nullptr};
        if (cudaGetSymbolAddress((void**)&t16[0], q38b_iq2xxs_codes) != cudaSuccess || cudaGetSymbolAddress((void**)&t16[1], q38b_iq2xs_codes) != cudaSuccess ||
            cudaGetSymbolAddress((void**)&t16[2], q38b_iq2s_codes) != cudaSuccess || cudaGetSymbolAddress((void**)&t16[3], q38b_iq1s_codes) != cudaSuccess) { rc = Q38B_ERR_CUDA; break; }
        for (int i = 0; i < 4; i++) c->d_code16[i] = (const uint32_t*)t16[i];
        // candidate lists of q38b_topk: 8 columns x TOPK_MAX_CHUNKS lists x TOPK_MAX_K pairs (1.5 MB), so that the decode path never allocates
        c->part_items = GEMV_PART_ITEMS;
        if (cudaMalloc(&c->d_parts, (size_t)GEMV_PART_ITEMS * 128 * sizeof(float)) != cudaSuccess) { rc = Q38B_ERR_CUDA; break; }
        if (cudaMemset(c->d_parts, 0xFF, (size_t)GEMV_PART_ITEMS * 128 * sizeof(float)) != cudaSuccess) { rc = Q38B_ERR_CUDA; break; }   // PART_EMPTY
        if (cudaMalloc(&c->d_part_count, (size_t)GEMV_PART_ITEMS * sizeof(int)) != cudaSuccess) { rc = Q38B_ERR_CUDA; break; }
        if (cudaMemset(c->d_part_count, 0, (size_t)GEMV_PART_ITEMS * sizeof(int)) != cudaSuccess) { rc = Q38B_ERR_CUDA; break; }
        if (cudaMalloc(&c->d_topk, (size_t)8 * TOPK_MAX_CHUNKS * TOPK_MAX_K * sizeof(TopkPair)) != cudaSuccess) { rc = Q38B_ERR_CUDA; break; }
    } while (0);
    if (rc != Q38B_OK) {
        c->last_cuda = (int)cudaGetLastError();
        if (c->d_status) cudaFree(c->d_status);
        if (c->d_topk) cudaFree(c->d_topk);
        if (c->d_parts) cudaFree(c->d_parts);
        if (c->d_part_count) cudaFree(c->d_part_count);
        delete c;
        return rc;
    }
    *out = c;
    return Q38B_OK;
}

void q38b_ctx_destroy(q38b_ctx* ctx) {
    if (!ctx) return;
    if (ctx->d_status) cudaFree(ctx->d_status);
    if (ctx->d_topk) cudaFree(ctx->d_topk);
    if (ctx->d_parts) cudaFree(ctx->d_parts);
    if (ctx->d_part_count) cudaFree(ctx->d_part_count);
    if (ctx->d_flags) cudaFree(ctx->d_flags);
    delete ctx;
}

int q38b_ctx_check(q38b_ctx* ctx, void* stream) {
    if (!ctx) return Q38B_ERR_ARG;
    int bits = 0;
    Q38B_CUDA(ctx, cudaMemcpyAsync(&bits, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    Q38B_CUDA(ctx, cudaStreamSynchronize((cudaStream_t)stream));
    if (bits) {
        Q38B_CUDA(ctx, cudaMemsetAsync(ctx->d_status, 0, sizeof(int), (cudaStream_t)stream));
        // a multi-column matvec that gave up may have left K-part sums and counts behind: back to the resting state
        Q38B_CUDA(ctx, cudaMemsetAsync(ctx->d_parts, 0xFF, (size_t)GEMV_PART_ITEMS * 128 * sizeof(float), (cudaStream_t)stream));
        Q38B_CUDA(ctx, cudaMemsetAsync(ctx->d_part_count, 0, (size_t)GEMV_PART_ITEMS * sizeof(int), (cudaStream_t)stream));
        return Q38B_ERR_DEVICE_WAIT;
    }
    return Q38B_OK;
}

int q38b_last_cuda_error(const q38b_ctx* ctx) { return ctx ? ctx->last_cuda : 0; }

int q38b_ctx_set_static_weights(q38b_ctx* ctx, int enabled) {
    if (!ctx) return Q38B_ERR_ARG;
    ctx->static_weights = enabled ? 1 : 0;
    return Q38B_OK;
}

int q38b_ctx_set_uniform_columns(q38b_ctx* ctx, int enabled) {
    if (!ctx) return Q38B_ERR_ARG;
    ctx->uniform_columns = enabled ? 1 : 0;
    return Q38B_OK;
}

// Test hook (not in the public header): 0 keeps the one-column kernel on its lane-per-granule mapping for every format,
// so that tests and timings can compare the two mappings on the same inputs.
int q38b_debug_set_rowgroup(q38b_ctx* ctx, int enabled) {
    if (!ctx) return Q38B_ERR_ARG;
    ctx->rowgroup = enabled ? 1 : 0;
    return Q38B_OK;
}
// Test hook: one CTA per SM for the one-column kernel: 0 never, otherwise wherever such a plan fits (the default).
int q38b_debug_set_one_cta(q38b_ctx* ctx, int mode) {
    if (!ctx || mode < 0 || mode > 2) return Q38B_ERR_ARG;
    ctx->one_cta = mode ? 1 : 0;
    return Q38B_OK;
}
// Test hook: the multi-column kernel's K-part scratch area counts as `items` (tile, part) sums (0: its real size), so that
// the launch per block of rows that very tall matrices take can be reached with a small one.
int q38b_debug_set_gemv_part_items(q38b_ctx* ctx, long long items) {
    if (!ctx || items < 0 || items > GEMV_PART_ITEMS) return Q38B_ERR_ARG;
    ctx->part_items = items ? items : GEMV_PART_ITEMS;
    return Q38B_OK;
}
// Test hook: enabled = 1 starts counting one-column launches whose CTAs fit an SM less often than their plan assumes;
// returns the count so far.
int q38b_debug_occupancy_shortfalls(q38b_ctx* ctx, int enabled) {
    if (!ctx) return -1;
    ctx->check_occupancy = enabled ? 1 : 0;
    return ctx->occupancy_shortfalls;
}

int q38b_ctx_set_wait_budget_cycles(q38b_ctx* ctx, long long cycles) {
    if (!ctx || cycles < 1000) return Q38B_ERR_ARG;
    ctx->wait_budget_cycles = cycles;
    return Q38B_OK;
}

// Test hook: makes this context believe it is rank 0 of 2 whose peer's flag block is its own arena, which nobody
// signals, so that a cross-GPU barrier runs into its bounded wait on one GPU (enabled = 0 undoes it).
int q38b_debug_fake_silent_peer(q38b_ctx* ctx, int enabled) {
    if (!ctx) return Q38B_ERR_ARG;
    if (enabled) {
        if (!ctx->d_flags) {
            unsigned char handle[64];
            const int rc = q38b_peer_arena_create(ctx, 1 << 20, handle);
            if (rc != Q38B_OK) return rc;
        }
        ctx->peer_flags[0] = ctx->d_flags;
        ctx->peer_flags[1] = ctx->d_flags + 64;   // rank 1 "writes" into words nobody reads; its own word [1] of the local block stays 0
        ctx->n_ranks = 2;
        ctx->rank = 0;
        ctx->peers_connected = 1;
    } else {
        ctx->n_ranks = 1;
        ctx->rank = 0;
        ctx->peers_connected = 0;
    }
    return Q38B_OK;
}

int q38b_ctx_set_pdl(q38b_ctx* ctx, int enabled) {
    if (!ctx) return Q38B_ERR_ARG;
    ctx->pdl = enabled ? 1 : 0;
    ctx->pass_pdl = enabled ? 1 : 0;
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

// takes the cross-GPU barrier the planner left for the next launch, if any
static PeerSync take_pending_sync(q38b_ctx* ctx) {
    PeerSync ps;
    memset(&ps, 0, sizeof(ps));
    if (ctx->pending_sync_seq >= 0 && ctx->n_ranks > 1 && ctx->peers_connected) {
        ps.local = ctx->d_flags;
        for (int r = 0; r < 8; r++) ps.peer[r] = ctx->peer_flags[r];
        ps.n = ctx->n_ranks;
        ps.rank = ctx->rank;
        ps.seq = ctx->pending_sync_seq;
        ps.budget = ctx->wait_budget_cycles;
    }
    ctx->pending_sync_seq = -1;
    return ps;
}

int q38b_swiglu_q8k(q38b_ctx* ctx, const float* g, const float* u, long long ld, int n, int n_rows, float* h, void* q8k,
                    long long q8k_stride, void* stream) {
    if (!ctx || !g || !u || n <= 0 || n % 256 || n_rows < 1 || ld < n || (q8k && q8k_stride < n / 256)) return Q38B_ERR_ARG;
    if (((uintptr_t)g | (uintptr_t)u | (uintptr_t)h | (uintptr_t)q8k) & 3) return Q38B_ERR_ALIGN;
    const long long blocks = (long long)n_rows * (n / 256);
    swiglu_q8k_kernel<<<(unsigned)((blocks + ACT_WARPS - 1) / ACT_WARPS), ACT_WARPS * 32, 0, (cudaStream_t)stream>>>(
        g, u, ld, n, n_rows, h, (uint8_t*)q8k, q8k_stride, take_pending_sync(ctx), ctx->d_status);
    Q38B_CUDA(ctx, cudaGetLastError());
    return Q38B_OK;
}

int q38b_add_rmsnorm_q8k(q38b_ctx* ctx, float* x, const float* a, const float* b, const float* w, int n, long long ld, int n_rows, float eps,
                         float* xn, void* q8k, long long q8k_stride, void* stream) {
    if (!ctx || !x || !w || n <= 0 || n % 256 || n > 32 * 256 || ld < n || ld % 4 || n_rows < 1 || (q8k && q8k_stride < n / 256)) return Q38B_ERR_ARG;
    if (((uintptr_t)x | (uintptr_t)a | (uintptr_t)b | (uintptr_t)w | (uintptr_t)xn) & 15) return Q38B_ERR_ALIGN;
    if ((uintptr_t)q8k & 3) return Q38B_ERR_ALIGN;
    add_rmsnorm_q8k_kernel<<<(unsigned)n_rows, (unsigned)(n / 256) * 32, 0, (cudaStream_t)stream>>>(x, a, b, w, n, ld, eps, xn, (uint8_t*)q8k,
                                                                                                  q8k_stride);
    Q38B_CUDA(ctx, cudaGetLastError());
    return Q38B_OK;
}

int q38b_gemv_bf16(q38b_ctx* ctx, const void* W_bf16, int K, int N, const float* x, float* y, void* stream) {
    if (!ctx || !W_bf16 || !x || !y || K <= 0 || K % 8 || N < 1) return Q38B_ERR_ARG;
    if (((uintptr_t)W_bf16 & 15) || ((uintptr_t)x & 15) || ((uintptr_t)y & 3)) return Q38B_ERR_ALIGN;
    gemv_bf16_kernel<<<(unsigned)N, BF16_THREADS, 0, (cudaStream_t)stream>>>((const uint16_t*)W_bf16, K, N, x, y);
    Q38B_CUDA(ctx, cudaGetLastError());
    return Q38B_OK;
}

int q38b_topk(q38b_ctx* ctx, const float* logits, long long ld, int n, int n_rows, int k, int index_offset, float* vals, int* idx, int out_ld,
              void* stream) {
    if (!ctx || !logits || !vals || !idx || n < 1 || n_rows < 1 || n_rows > 8 || k < 1 || k > TOPK_MAX_K || out_ld < k) return Q38B_ERR_ARG;
    if (n_rows > 1 && ld < n) return Q38B_ERR_ARG;
    const int n_chunks = (n + TOPK_CHUNK - 1) / TOPK_CHUNK;
    if (n_chunks > TOPK_MAX_CHUNKS) return Q38B_ERR_UNSUPPORTED;
    if (((uintptr_t)logits & 3) || ((uintptr_t)vals & 3) || ((uintptr_t)idx & 3)) return Q38B_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t smem = (size_t)n_chunks * k * sizeof(TopkPair);
    const int rc = ensure_kernel_smem(ctx, (const void*)topk_merge_kernel, ctx->smem_optin, false);
    if (rc != Q38B_OK) return rc;
    TopkPair* lists = (TopkPair*)ctx->d_topk;
    topk_lists_kernel<<<dim3((unsigned)((n_chunks + TOPK_STAGE1_WARPS - 1) / TOPK_STAGE1_WARPS), (unsigned)n_rows), TOPK_STAGE1_WARPS * 32, 0, st>>>(
        logits, ld, n, k, lists, n_chunks);
    topk_merge_kernel<<<(unsigned)n_rows, 32 * TOPK_LISTS_PER_LANE, smem, st>>>(lists, n_chunks, k, logits, ld, index_offset, vals, idx, (long long)out_ld);
    Q38B_CUDA(ctx, cudaGetLastError());
    return Q38B_OK;
}

int q38b_swiglu_rows_inplace(q38b_ctx* ctx, float* G, const float* U, int B, int n, long long ld, int out_kind, void* stream) {
    if (!ctx || !G || !U || B < 1 || n <= 0 || n % 8 || ld < n || ld % 4) return Q38B_ERR_ARG;
    if (out_kind != Q38B_OUT_F16 && out_kind != Q38B_OUT_BF16) return Q38B_ERR_ARG;
    if (((uintptr_t)G & 15) || ((uintptr_t)U & 15)) return Q38B_ERR_ALIGN;
    const int smem = 2 * n;
    if (smem > ctx->smem_optin) return Q38B_ERR_NOMEM;
    cudaStream_t st = (cudaStream_t)stream;
    if (out_kind == Q38B_OUT_BF16) {
        const int rc = ensure_kernel_smem(ctx, (const void*)swiglu_rows_inplace_kernel<true>, ctx->smem_optin, false);
        if (rc != Q38B_OK) return rc;
        swiglu_rows_inplace_kernel<true><<<(unsigned)B, 256, smem, st>>>(G, U, n, ld);
    } else {
        const int rc = ensure_kernel_smem(ctx, (const void*)swiglu_rows_inplace_kernel<false>, ctx->smem_optin, false);
        if (rc != Q38B_OK) return rc;
        swiglu_rows_inplace_kernel<false><<<(unsigned)B, 256, smem, st>>>(G, U, n, ld);
    }
    Q38B_CUDA(ctx, cudaGetLastError());
    return Q38B_OK;
}

int q38b_gemv_q8k(q38b_ctx* ctx, uint32_t type, const void* W, size_t row_bytes, int K, int M, const void* q8k,
                  long long q8k_stride, int nb, float* y, long long y_ld, int accumulate, void* stream) {
    return q38b_gemv_q8k_scatter(ctx, type, W, row_bytes, K, M, q8k, q8k_stride, nb, y, y_ld, accumulate, nullptr, 0, stream);
}

int q38b_gemv_q8k_scatter(q38b_ctx* ctx, uint32_t type, const void* W, size_t row_bytes, int K, int M, const void* q8k,
                          long long q8k_stride, int nb, float* y, long long y_ld, int accumulate, float* const* y_peers,
                          int n_peers, void* stream) {
    if (!ctx || !W || !q8k || !y) return Q38B_ERR_ARG;
    if (n_peers < 0 || n_peers > 7 || (n_peers > 0 && !y_peers)) return Q38B_ERR_ARG;
    for (int i = 0; i < n_peers; i++) if (!y_peers[i] || ((uintptr_t)y_peers[i] & 3)) return Q38B_ERR_ARG;
    if (!known_format(type)) return Q38B_ERR_UNSUPPORTED;
    if (K <= 0 || K % 256 || M < 1 || nb < 1 || nb > 8 || y_ld < M || q8k_stride < K / 256) return Q38B_ERR_ARG;
    if (row_bytes < q38b_row_bytes(type, K)) return Q38B_ERR_ARG;
    const int al = format_alignment(type);
    if (((uintptr_t)W & 15) || (row_bytes % al) || ((uintptr_t)q8k & 3) || ((uintptr_t)y & 3)) return Q38B_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    if (one_column_only((int)type) && nb > 1) {
        // formats that only the one-column kernel decodes: one launch per column (every column is the nb = 1 result)
        for (int c = 0; c < nb; c++) {
            float* peers_c[7];
            for (int i = 0; i < n_peers; i++) peers_c[i] = y_peers[i] + (size_t)c * y_ld;
            const int rc = q38b_gemv_q8k_scatter(ctx, type, W, row_bytes, K, M, (const uint8_t*)q8k + (size_t)c * q8k_stride * Q8K_BYTES, q8k_stride, 1,
                                                 y + (size_t)c * y_ld, y_ld, accumulate, peers_c, n_peers, stream);
            if (rc != Q38B_OK) return rc;
        }
        return Q38B_OK;
    }
    if (nb == 1 && (!ctx->uniform_columns || one_column_only((int)type))) {
        // single column: the dp4a kernel (one lane per 32- or 64-weight granule)
        Plan1 p1;
        memset(&p1, 0, sizeof(p1));
        const int rc1 = plan_gemv1(ctx, type, K, &M, 1, row_bytes, &p1);
        if (rc1 == Q38B_OK) {
            Gemv1Args& g = p1.a;
            g.W = (const uint8_t*)W;
            g.row_bytes = (long long)row_bytes;
            g.xq = (const uint8_t*)q8k;
            g.x_f32 = nullptr;
            g.y = y;
            g.n_peers = n_peers;
            g.static_weights = ctx->static_weights;
            for (int i = 0; i < n_peers; i++) g.y_peer[i] = y_peers[i];
            g.status = ctx->d_status;
            g.codebook = codebook_of(ctx, type);
            g.K = K;
            g.M = M;
            g.accumulate = accumulate ? 1 : 0;
            return dispatch_gemv1(ctx, type, p1, st);
        }
    }
    {   // more (tile, K-part) sums than the scratch area holds: one launch per block of rows
        const int n_units = (K / 256 + 3) / 4, upp = gemv_units_per_part(type);
        const int n_parts = K <= GEMV_WHOLE_ROW_K ? 1 : std::min(GEMV_MAX_PARTS, (n_units + upp - 1) / upp);
        const long long rows_per_launch = ctx->part_items / n_parts * TILE_ROWS;
        if (n_parts > 1 && M > rows_per_launch) {
            for (long long m0 = 0; m0 < M; m0 += rows_per_launch) {
                const int m = (int)std::min<long long>(rows_per_launch, M - m0);
                float* peers_at[7];
                for (int i = 0; i < n_peers; i++) peers_at[i] = y_peers[i] + m0;
                const int rc = q38b_gemv_q8k_scatter(ctx, type, (const uint8_t*)W + (size_t)m0 * row_bytes, row_bytes, K, m, q8k, q8k_stride, nb, y + m0,
                                                     y_ld, accumulate, n_peers ? peers_at : nullptr, n_peers, stream);
                if (rc != Q38B_OK) return rc;
            }
            return Q38B_OK;
        }
    }
    Plan p;
    memset(&p, 0, sizeof(p));
    int rc = plan_gemv(ctx, type, K, &M, 1, nb, &p);
    if (rc != Q38B_OK) return rc;
    GemvArgs& a = p.a;
    a.W = (const uint8_t*)W;
    a.row_bytes = (long long)row_bytes;
    a.xq = (const uint8_t*)q8k;
    a.x_stride = q8k_stride;
    a.y = y;
    a.y_ld = y_ld;
    a.n_peers = n_peers;
    a.static_weights = ctx->static_weights;
    for (int i = 0; i < n_peers; i++) a.y_peer[i] = y_peers[i];
    a.status = ctx->d_status;
    a.codebook = codebook_of(ctx, type);
    a.K = K;
    a.M = M;
    a.nb = nb;
    a.accumulate = accumulate ? 1 : 0;
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

int q38b_gemvn_group_plannable(const q38b_ctx* ctx, uint32_t type, int n_mats, size_t row_bytes, int K, const int* M, int nb) {
    if (!ctx || n_mats < 1 || n_mats > GEMV_MAX_MATS || !known_format(type) || K <= 0 || K % 256 || nb < 1 || nb > 8) return 0;
    if (row_bytes < q38b_row_bytes(type, K)) return 0;
    Plan p;
    memset(&p, 0, sizeof(p));
    return plan_gemv(ctx, type, K, M, n_mats, nb, &p) == Q38B_OK;
}

int q38b_gemvn_group(q38b_ctx* ctx, uint32_t type, int n_mats, const void* const* W, size_t row_bytes, int K, const int* M,
                     const void* q8k, long long q8k_stride, int nb, float* const* y, const long long* y_ld, void* stream) {
    return q38b_gemvn_group_x(ctx, type, n_mats, W, row_bytes, K, M, q8k, q8k_stride, nullptr, 0, nb, y, y_ld, nullptr, 0, stream);
}

int q38b_gemvn_group_x(q38b_ctx* ctx, uint32_t type, int n_mats, const void* const* W, size_t row_bytes, int K, const int* M,
                       const void* q8k, long long q8k_stride, const float* x_f32, long long x_f32_ld, int nb, float* const* y,
                       const long long* y_ld, float* const* y_peers, int n_peers, void* stream) {
    if (!ctx || !W || !M || !y || !y_ld || (!q8k == !x_f32) || n_mats < 1 || n_mats > GEMV_MAX_MATS) return Q38B_ERR_ARG;
    if (n_peers < 0 || n_peers > 7 || (n_peers > 0 && !y_peers)) return Q38B_ERR_ARG;   // y_peers[i * n_peers + r]: peer r's copy of matrix i's output
    if (!q38b_gemvn_group_plannable(ctx, type, n_mats, row_bytes, K, M, nb)) return Q38B_ERR_UNSUPPORTED;
    const int al = format_alignment(type);
    if (row_bytes % al) return Q38B_ERR_ALIGN;
    if (q8k && (((uintptr_t)q8k & 3) || q8k_stride < K / 256)) return Q38B_ERR_ALIGN;
    if (x_f32 && (((uintptr_t)x_f32 & 15) || x_f32_ld < K || x_f32_ld % 4)) return Q38B_ERR_ALIGN;
    for (int i = 0; i < n_mats; i++) {
        if (!W[i] || !y[i] || M[i] < 1 || y_ld[i] < M[i]) return Q38B_ERR_ARG;
        if (((uintptr_t)W[i] & 15) || ((uintptr_t)y[i] & 3)) return Q38B_ERR_ALIGN;
    }
    Plan p;
    memset(&p, 0, sizeof(p));
    const int rc = plan_gemv(ctx, type, K, M, n_mats, nb, &p);
    if (rc != Q38B_OK) return rc;
    GemvArgs& a = p.a;
    a.W = (const uint8_t*)W[0];
    a.y = y[0];
    a.y_ld = y_ld[0];
    a.M = M[0];
    for (int i = 1; i < n_mats; i++) {
        a.W_more[i - 1] = (const uint8_t*)W[i];
        a.y_more[i - 1] = y[i];
        a.y_ld_more[i - 1] = y_ld[i];
        a.M_more[i - 1] = M[i];
    }
    a.row_bytes = (long long)row_bytes;
    a.xq = (const uint8_t*)q8k;
    a.x_stride = q8k_stride;
    a.x_f32 = x_f32;
    a.x_f32_ld = x_f32_ld;
    a.n_peers = n_peers;
    for (int i = 0; i < n_peers; i++) a.y_peer[i] = y_peers[i];
    for (int m = 1; m < n_mats; m++)
        for (int i = 0; i < n_peers; i++) a.y_peer_more[m - 1][i] = y_peers[m * n_peers + i];
    a.static_weights = ctx->static_weights;
    a.status = ctx->d_status;
    a.codebook = codebook_of(ctx, type);
    a.K = K;
    a.nb = nb;
    a.accumulate = 0;
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

int q38b_gemv_group_plannable(const q38b_ctx* ctx, uint32_t type, int n_mats, size_t row_bytes, int K, const int* M) {
    if (!ctx || ctx->uniform_columns || n_mats < 1 || n_mats > G1_MAX_MATS || !known_format(type) || K <= 0 || K % 256) return 0;
    Plan1 p1;
    return plan_gemv1(ctx, type, K, M, n_mats, row_bytes, &p1) == Q38B_OK;
}

// Test hook: the one-column kernel's plan on a 148-SM device as CTAs per SM * 100000 + one-copy tiles * 10000 + rows per
// tile * 100 + stages (0: the shape does not fit it).
int q38b_debug_gemv1_rows(uint32_t type, int K, int M, size_t row_bytes, int rowgroup, int one_cta) {
    q38b_ctx ctx;
    ctx.sm_count = 148;
    ctx.smem_optin = 232448;
    ctx.rowgroup = rowgroup;
    ctx.one_cta = one_cta;
    Plan1 p1;
    if (!known_format(type) || K <= 0 || K % 256 || plan_gemv1(&ctx, type, K, &M, 1, row_bytes, &p1) != Q38B_OK) return 0;
    return p1.occ * 100000 + p1.a.contiguous * 10000 + p1.rows * 100 + p1.a.n_stages;
}

int q38b_gemv_group(q38b_ctx* ctx, uint32_t type, int n_mats, const void* const* W, size_t row_bytes, int K, const int* M,
                    const void* q8k, const float* x_f32, float* const* y, void* stream) {
    return q38b_gemv_group_peers(ctx, type, n_mats, W, row_bytes, K, M, q8k, x_f32, y, nullptr, 0, stream);
}

int q38b_gemv_group_peers(q38b_ctx* ctx, uint32_t type, int n_mats, const void* const* W, size_t row_bytes, int K, const int* M,
                          const void* q8k, const float* x_f32, float* const* y, float* const* y_peers, int n_peers, void* stream) {
    if (!ctx || !W || !M || !y || n_mats < 1 || n_mats > G1_MAX_MATS || (!q8k == !x_f32)) return Q38B_ERR_ARG;
    if (n_peers < 0 || n_peers > 7 || (n_peers > 0 && !y_peers)) return Q38B_ERR_ARG;
    for (int i = 0; i < n_mats * n_peers; i++) if (!y_peers[i] || ((uintptr_t)y_peers[i] & 3)) return Q38B_ERR_ARG;
    if (!known_format(type)) return Q38B_ERR_UNSUPPORTED;
    if (K <= 0 || K % 256 || row_bytes < q38b_row_bytes(type, K)) return Q38B_ERR_ARG;
    const int al = format_alignment(type);
    if ((row_bytes % al) || (q8k && ((uintptr_t)q8k & 3)) || (x_f32 && ((uintptr_t)x_f32 & 15))) return Q38B_ERR_ALIGN;
    for (int i = 0; i < n_mats; i++) {
        if (!W[i] || !y[i] || M[i] < 1) return Q38B_ERR_ARG;
        if (((uintptr_t)W[i] & 15) || ((uintptr_t)y[i] & 3)) return Q38B_ERR_ALIGN;
    }
    if (ctx->uniform_columns) return Q38B_ERR_UNSUPPORTED;
    Plan1 p1;
    memset(&p1, 0, sizeof(p1));
    if (plan_gemv1(ctx, type, K, M, n_mats, row_bytes, &p1) != Q38B_OK) return Q38B_ERR_UNSUPPORTED;   // shapes only the tensor-core kernel takes
    Gemv1Args& g = p1.a;
    g.W = (const uint8_t*)W[0];
    g.y = y[0];
    g.M = M[0];
    for (int i = 1; i < n_mats; i++) {
        g.W_more[i - 1] = (const uint8_t*)W[i];
        g.y_more[i - 1] = y[i];
        g.M_more[i - 1] = M[i];
    }
    g.row_bytes = (long long)row_bytes;
    g.xq = (const uint8_t*)q8k;
    g.x_f32 = x_f32;
    g.sync = take_pending_sync(ctx);
    g.n_peers = n_peers;
    for (int i = 0; i < n_mats; i++)
        for (int pr = 0; pr < n_peers; pr++) (i == 0 ? g.y_peer[pr] : g.y_peer_more[i - 1][pr]) = y_peers[i * n_peers + pr];
    g.static_weights = ctx->static_weights;
    g.status = ctx->d_status;
    g.codebook = codebook_of(ctx, type);
    g.K = K;
    g.accumulate = 0;
    cudaStream_t st = (cudaStream_t)stream;
    return dispatch_gemv1(ctx, type, p1, st);
}

int q38b_quantize_act_q8(q38b_ctx* ctx, const float* x, int K, int n_rows, int8_t* q, float* d, float* s, void* stream) {
    if (!ctx || !x || !q || !d || !s || K <= 0 || K % 32 || n_rows < 1) return Q38B_ERR_ARG;
    if (((uintptr_t)x | (uintptr_t)d | (uintptr_t)s) & 3) return Q38B_ERR_ALIGN;
    const long long blocks = (long long)n_rows * (K / 32);
    quantize_act_q8_kernel<<<(unsigned)((blocks + ACT_WARPS - 1) / ACT_WARPS), ACT_WARPS * 32, 0, (cudaStream_t)stream>>>(x, blocks, q, d, s);
    Q38B_CUDA(ctx, cudaGetLastError());
    return Q38B_OK;
}

int q38b_gemv_act_q8(q38b_ctx* ctx, uint32_t type, const void* W, size_t row_bytes, int K, int M, const int8_t* q, const float* d,
                     int nb, int act_ld, float* y, int y_ld, int accumulate, void* stream) {
    if (!ctx || !W || !q || !d || !y) return Q38B_ERR_ARG;
    if (!known_format(type)) return Q38B_ERR_UNSUPPORTED;
    if (K <= 0 || K % 256 || M < 1 || nb < 1 || nb > 8 || y_ld < M || act_ld < K || act_ld % 32) return Q38B_ERR_ARG;
    if (row_bytes < q38b_row_bytes(type, K)) return Q38B_ERR_ARG;
    const int al = format_alignment(type);
    if (((uintptr_t)W & 15) || (row_bytes % al) || ((uintptr_t)q & 3) || (act_ld & 3) || ((uintptr_t)d & 3) || ((uintptr_t)y & 3)) return Q38B_ERR_ALIGN;
    // One launch of the one-column kernel per column: every column is the single-column result by construction (the
    // promise of src/cuda/gemv.cuh:31-34 of the reference), at nb times the cost of one column.
    const int saved_rg = ctx->rowgroup, saved_one = ctx->one_cta;
    ctx->rowgroup = 0;
    ctx->one_cta = 0;
    int rc = Q38B_OK;
    for (int c = 0; c < nb && rc == Q38B_OK; c++) {
        Plan1 p1;
        memset(&p1, 0, sizeof(p1));
        if (plan_gemv1(ctx, type, K, &M, 1, row_bytes, &p1) != Q38B_OK) { rc = Q38B_ERR_NOMEM; break; }
        Gemv1Args& g = p1.a;
        g.W = (const uint8_t*)W;
        g.row_bytes = (long long)row_bytes;
        g.xq = (const uint8_t*)(q + (size_t)c * act_ld);
        g.xd32 = d + (size_t)c * (act_ld / 32);
        g.x_f32 = nullptr;
        g.y = y + (size_t)c * y_ld;
        g.n_peers = 0;
        g.static_weights = ctx->static_weights;
        g.status = ctx->d_status;
        g.codebook = codebook_of(ctx, type);
        g.K = K;
        g.M = M;
        g.accumulate = accumulate ? 1 : 0;
        cudaStream_t st = (cudaStream_t)stream;
        rc = dispatch_gemv1(ctx, type, p1, st);
    }
    ctx->rowgroup = saved_rg;
    ctx->one_cta = saved_one;
    return rc;
}

int q38b_gemv_f32(q38b_ctx* ctx, uint32_t type, const void* W, size_t row_bytes, int K, int M, const float* x, long long x_ld,
                  int nb, float* y, long long y_ld, int accumulate, void* q8k_scratch, size_t scratch_bytes, void* stream) {
    if (!ctx || !x || !q8k_scratch || nb < 1 || nb > 8 || K <= 0 || K % 256) return Q38B_ERR_ARG;
    if (scratch_bytes < (size_t)nb * q38b_q8k_bytes(K)) return Q38B_ERR_NOMEM;
    int rc = q38b_quantize_q8k(ctx, x, x_ld, K, nb, q8k_scratch, K / 256, stream);
    if (rc != Q38B_OK) return rc;
    return q38b_gemv_q8k(ctx, type, W, row_bytes, K, M, q8k_scratch, K / 256, nb, y, y_ld, accumulate, stream);
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
