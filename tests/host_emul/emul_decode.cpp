// CPU emulation of one consumer warp of the matvec kernel, for the GPU-free unit test of the
// fragment builders in qwengine_b200/csrc/q38b_decode.cuh.  32 host threads play the 32 lanes;
// mma.sync and shuffles are rendezvous points that apply the PTX fragment layouts.  The test
// lays a 16-row tile out in memory exactly as the kernel's stage holds it (each row at its own
// slot, shifted by the low 4 bits of its global address) and runs every half super-block.
#include <pthread.h>

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../../qwengine_b200/csrc/q38b_decode.cuh"

namespace {
thread_local int tl_lane = 0;
pthread_barrier_t g_bar;
uint32_t g_a[32][4], g_b[32][2], g_sh[32];
}  // namespace

namespace q38b {
int emul_lane() { return tl_lane; }

void emul_mma(int (&c)[4], const uint32_t* a, int n_a, const uint32_t* b, int n_b) {
    const int lane = tl_lane;
    for (int i = 0; i < n_a; i++) g_a[lane][i] = a[i];
    for (int i = 0; i < n_b; i++) g_b[lane][i] = b[i];
    pthread_barrier_wait(&g_bar);
    const int kdim = n_b * 16;
    const int g = lane >> 2, t = lane & 3;
    for (int ci = 0; ci < 4; ci++) {
        const int m = g + 8 * (ci >> 1), n = 2 * t + (ci & 1);
        int sum = 0;
        for (int k = 0; k < kdim; k++) {
            // A[m][k]: held by lane (m % 8) * 4 + (k % 16) / 4, register (m / 8) + 2 * (k / 16), byte k % 4
            const int la = (m & 7) * 4 + ((k & 15) >> 2), ra = (m >> 3) + 2 * (k >> 4);
            const int lb = n * 4 + ((k & 15) >> 2), rb = k >> 4;
            const int av = (int8_t)(g_a[la][ra] >> (8 * (k & 3)));
            const int bv = (int8_t)(g_b[lb][rb] >> (8 * (k & 3)));
            sum += av * bv;
        }
        c[ci] += sum;
    }
    pthread_barrier_wait(&g_bar);
}

uint32_t emul_shfl(uint32_t v, int src) {
    g_sh[tl_lane] = v;
    pthread_barrier_wait(&g_bar);
    const uint32_t r = g_sh[src & 31];
    pthread_barrier_wait(&g_bar);
    return r;
}
}  // namespace q38b

using namespace q38b;

namespace {
struct Job {
    int fmt, K, nb, rep_log2;
    const uint8_t* stage;       // 16 slots
    int slot_stride;
    const int* row_shift;       // per row: low 4 address bits
    const uint8_t* actq;        // [nb][K] staged order
    const float* actd;          // [nsb][8]
    const uint32_t* cb;         // replicated codebook
    float* y;                   // [16][8]
};
struct LaneArg { const Job* job; int lane; };

template <int FMT>
void run_lane(const Job& j, int lane) {
    const int g = lane >> 2, t = lane & 3;
    Codebook cb{j.cb, j.rep_log2, (uint32_t)lane & ((1u << j.rep_log2) - 1u)};
    float acc[4] = {0, 0, 0, 0};
    const uint8_t* baseA = j.stage + (size_t)g * j.slot_stride + j.row_shift[g];
    const uint8_t* baseB = j.stage + (size_t)(g + 8) * j.slot_stride + j.row_shift[g + 8];
    const bool valid = g < j.nb;
    const int nsb = j.K / 256;
    for (int u = 0; u < 2 * nsb; u++) {
        const int sb = u >> 1, h = u & 1;
        ActLane al;
        al.q = j.actq + (size_t)(valid ? g : 0) * j.K + sb * 256;
        al.valid = valid;
        al.dx0 = j.actd[sb * 8 + 2 * t];
        al.dx1 = j.actd[sb * 8 + 2 * t + 1];
        Unit<FMT>::run(baseA + sb * Unit<FMT>::BLOCK_BYTES, baseB + sb * Unit<FMT>::BLOCK_BYTES, h, al, cb, acc);
    }
    for (int i = 0; i < 4; i++) j.y[(g + 8 * (i >> 1)) * 8 + 2 * t + (i & 1)] = acc[i];
}

void* lane_main(void* v) {
    const LaneArg* la = (const LaneArg*)v;
    tl_lane = la->lane;
    const Job& j = *la->job;
    switch (j.fmt) {
        case T_Q8_0: run_lane<T_Q8_0>(j, la->lane); break;
        case T_Q4_K: run_lane<T_Q4_K>(j, la->lane); break;
        case T_Q5_K: run_lane<T_Q5_K>(j, la->lane); break;
        case T_Q6_K: run_lane<T_Q6_K>(j, la->lane); break;
        case T_IQ3_XXS: run_lane<T_IQ3_XXS>(j, la->lane); break;
        case T_IQ3_S: run_lane<T_IQ3_S>(j, la->lane); break;
        case T_IQ4_XS: run_lane<T_IQ4_XS>(j, la->lane); break;
    }
    return nullptr;
}
}  // namespace

#define Q38B_CODEBOOK_QUALIFIER static const
#include "../../qwengine_b200/csrc/codebooks.inc"

// W: 16 packed rows of GGUF blocks; xq: Q8_K blocks [nb][K/256]; addr_lo: pretend low address bits of row 0
// (row r then sits at (addr_lo + r * row_bytes) & 15 inside its slot); y: [16][8].
extern "C" int emul_tile(int fmt, int K, const uint8_t* W, const uint8_t* xq, int nb, int addr_lo, int rep_log2, float* y) {
    const int bb = block_bytes(fmt), nsb = K / 256, row_bytes = nsb * bb;
    if (!bb) return -1;
    const int slot = (row_bytes + 32 + 15) / 16 * 16 + 16;
    std::vector<uint8_t> stage((size_t)16 * slot + 64, 0xA5);
    uint8_t* st = (uint8_t*)(((uintptr_t)stage.data() + 15) & ~(uintptr_t)15);
    int shift[16];
    for (int r = 0; r < 16; r++) {
        shift[r] = (addr_lo + r * row_bytes) & 15;
        memcpy(st + (size_t)r * slot + shift[r], W + (size_t)r * row_bytes, row_bytes);
    }
    std::vector<uint8_t> actq((size_t)8 * K, 0);
    std::vector<float> actd((size_t)nsb * 8, 0.f);
    for (int c = 0; c < nb; c++)
        for (int sb = 0; sb < nsb; sb++) {
            const uint8_t* blk = xq + ((size_t)c * nsb + sb) * 292;
            memcpy(&actd[sb * 8 + c], blk, 4);
            for (int k = 0; k < 256; k++) actq[(size_t)c * K + sb * 256 + (k & ~31) + act_stage_pos(fmt, k & 31)] = blk[4 + k];
        }
    const int entries = fmt == T_IQ3_XXS ? 256 : fmt == T_IQ3_S ? 512 : 0;
    std::vector<uint32_t> cb((size_t)(entries ? entries : 1) << rep_log2);
    for (size_t i = 0; i < ((size_t)entries << rep_log2); i++)
        cb[i] = fmt == T_IQ3_XXS ? q38b_iq3xxs_grid[i >> rep_log2] : q38b_iq3s_grid[i >> rep_log2];
    Job job{fmt, K, nb, rep_log2, st, slot, shift, actq.data(), actd.data(), cb.data(), y};
    pthread_barrier_init(&g_bar, nullptr, 32);
    pthread_t th[32];
    LaneArg la[32];
    for (int l = 0; l < 32; l++) { la[l] = {&job, l}; pthread_create(&th[l], nullptr, lane_main, &la[l]); }
    for (int l = 0; l < 32; l++) pthread_join(th[l], nullptr);
    pthread_barrier_destroy(&g_bar);
    return 0;
}

// ---------------------------------------------------------------------------------------------------------------
// Single-column path (q38b_decode1.cuh): the lanes run one after the other, there is no warp-collective step.
// ---------------------------------------------------------------------------------------------------------------
#include "../../qwengine_b200/csrc/q38b_decode1.cuh"

namespace {
template <int FMT, bool A32>
void run_slices(int K, const uint8_t* const* rowp, int n_rows, const uint8_t* actq, const float* actd, const Codebook1* cbs, float* y) {
    constexpr int LPR = Gran<FMT>::LANES_PER_ROW;
    const int nsb = K / 256, n_slices = (nsb + 3) / 4;
    for (int r = 0; r < n_rows; r++) {
        float sum = 0;
        for (int s = 0; s < n_slices; s++) {
            float ssum = 0;
            for (int lane = 0; lane < LPR; lane++) {
                tl_lane = lane;
                const int gran_sb = s * 4 + (LPR == 32 ? (lane >> 3) : (lane >> 2));
                if (gran_sb >= nsb) continue;
                typename Gran<FMT>::Acts acts;
                Gran<FMT>::template load_acts<A32>(acts, sp_from(actq + s * 1024), sp_from(actd + s * 32), lane);
                ssum += Gran<FMT>::template dot<A32>(sp_from(rowp[r] + (size_t)s * 4 * Unit<FMT>::BLOCK_BYTES), acts, cbs[lane], lane);
            }
            sum += ssum;
        }
        y[r] = sum;
    }
}
}  // namespace

// W: n_rows packed rows; xq: Q8_K blocks of one column; y[n_rows].
static int emul_gemv1_any(int fmt, int K, const uint8_t* W, int n_rows, const uint8_t* xq, const float* d32, int addr_lo, int rep_log2, float* y);
extern "C" int emul_gemv1(int fmt, int K, const uint8_t* W, int n_rows, const uint8_t* xq, int addr_lo, int rep_log2, float* y) {
    return emul_gemv1_any(fmt, K, W, n_rows, xq, nullptr, addr_lo, rep_log2, y);
}
// the same with the column in the per-32 format: q = K int8 values, d32 = K / 32 scales
extern "C" int emul_gemv1_act32(int fmt, int K, const uint8_t* W, int n_rows, const int8_t* q, const float* d32, int addr_lo, float* y) {
    return emul_gemv1_any(fmt, K, W, n_rows, (const uint8_t*)q, d32, addr_lo, 0, y);
}
static int emul_gemv1_any(int fmt, int K, const uint8_t* W, int n_rows, const uint8_t* xq, const float* d32, int addr_lo, int rep_log2, float* y) {
    const int bb = block_bytes(fmt), nsb = K / 256, row_bytes = nsb * bb, n_slices = (nsb + 3) / 4;
    if (!bb) return -1;
    const int slot = (row_bytes + 64 + 15) / 16 * 16;
    std::vector<uint8_t> stage((size_t)n_rows * slot + 64, 0x5A);
    uint8_t* st = (uint8_t*)(((uintptr_t)stage.data() + 15) & ~(uintptr_t)15);
    std::vector<const uint8_t*> rowp(n_rows);
    for (int r = 0; r < n_rows; r++) {
        uint8_t* p = st + (size_t)r * slot + ((addr_lo + r * row_bytes) & 15);
        memcpy(p, W + (size_t)r * row_bytes, row_bytes);
        rowp[r] = p;
    }
    std::vector<uint8_t> actq((size_t)n_slices * 1024 + 64, 0);
    uint8_t* aq = (uint8_t*)(((uintptr_t)actq.data() + 15) & ~(uintptr_t)15);
    std::vector<float> actd((size_t)n_slices * 32, 0.f);
    for (int sb = 0; sb < nsb; sb++) {
        const uint8_t* blk = xq + (size_t)sb * 292;
        if (d32) {
            for (int j = 0; j < 8; j++) actd[sb * 8 + j] = d32[sb * 8 + j];
            for (int k = 0; k < 256; k++) aq[(sb >> 2) * 1024 + act_slice_pos(fmt, (sb & 3) * 256 + (k & ~31) + act_stage_pos(fmt, k & 31))] = xq[sb * 256 + k];
            continue;
        }
        memcpy(&actd[sb * 8], blk, 4);
        for (int k = 0; k < 256; k++) aq[(sb >> 2) * 1024 + act_slice_pos(fmt, (sb & 3) * 256 + (k & ~31) + act_stage_pos(fmt, k & 31))] = blk[4 + k];
    }
    const int entries = fmt == T_IQ3_XXS ? 256 : fmt == T_IQ3_S ? 512 : 0;
    (void)rep_log2;                                        // the single-column decoders fix their replica counts
    const int rl = cb1_rep_log2(fmt), reps = 1 << rl;
    std::vector<uint32_t> cb((size_t)(entries ? entries : 1) * reps);
    for (size_t i = 0; i < (size_t)entries * reps; i++) cb[i] = fmt == T_IQ3_XXS ? q38b_iq3xxs_grid[i >> rl] : q38b_iq3s_grid[i >> rl];
    std::vector<uint32_t> sgn(KSIGN_TABLE_BYTES / 4);
    for (int i = 0; i < 128 * 16; i++) ksign_entry((uint32_t)i >> 4, sgn[2 * i], sgn[2 * i + 1]);
    Codebook1 cbs[32];
    for (int l = 0; l < 32; l++) cbs[l] = Codebook1{sp_from(cb.data()) + 4 * (l & (reps - 1)), sp_from(sgn.data()) + 8 * (l & 15)};
    // the formats whose grids are 16-bit codes read one shared copy of the table
    const unsigned short* codes = fmt == T_IQ2_XXS ? q38b_iq2xxs_codes : fmt == T_IQ2_XS ? q38b_iq2xs_codes : fmt == T_IQ2_S ? q38b_iq2s_codes
                                  : (fmt == T_IQ1_S || fmt == T_IQ1_M) ? q38b_iq1s_codes : nullptr;
    if (codes)
        for (int l = 0; l < 32; l++) cbs[l].lane_base = sp_from(codes);
    switch (fmt) {
        case T_Q8_0: if (d32) run_slices<T_Q8_0, true>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); else run_slices<T_Q8_0, false>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); break;
        case T_Q4_K: if (d32) run_slices<T_Q4_K, true>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); else run_slices<T_Q4_K, false>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); break;
        case T_Q5_K: if (d32) run_slices<T_Q5_K, true>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); else run_slices<T_Q5_K, false>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); break;
        case T_Q6_K: if (d32) run_slices<T_Q6_K, true>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); else run_slices<T_Q6_K, false>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); break;
        case T_IQ3_XXS: if (d32) run_slices<T_IQ3_XXS, true>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); else run_slices<T_IQ3_XXS, false>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); break;
        case T_IQ3_S: if (d32) run_slices<T_IQ3_S, true>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); else run_slices<T_IQ3_S, false>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); break;
        case T_IQ4_XS: if (d32) run_slices<T_IQ4_XS, true>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); else run_slices<T_IQ4_XS, false>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); break;
        case T_Q2_K: if (d32) run_slices<T_Q2_K, true>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); else run_slices<T_Q2_K, false>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); break;
        case T_IQ2_XXS: if (d32) run_slices<T_IQ2_XXS, true>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); else run_slices<T_IQ2_XXS, false>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); break;
        case T_IQ2_XS: if (d32) run_slices<T_IQ2_XS, true>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); else run_slices<T_IQ2_XS, false>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); break;
        case T_IQ2_S: if (d32) run_slices<T_IQ2_S, true>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); else run_slices<T_IQ2_S, false>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); break;
        case T_IQ1_S: if (d32) run_slices<T_IQ1_S, true>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); else run_slices<T_IQ1_S, false>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); break;
        case T_IQ1_M: if (d32) run_slices<T_IQ1_M, true>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); else run_slices<T_IQ1_M, false>(K, rowp.data(), n_rows, aq, actd.data(), cbs, y); break;
        default: return -1;
    }
    return 0;
}

// ---------------------------------------------------------------------------------------------------------------
// Row-group mapping of the single-column path (GranR): rows 8 bytes aligned, a pass = one super-block of four rows.
// ---------------------------------------------------------------------------------------------------------------
namespace {
template <int FMT, int B>
float block_r(const uint8_t* row, int s, const ActsR& a, const TablesR& t) { return GranR<FMT>::template dot<B>(sp_from(row), s, a, t); }

template <int FMT>
void run_rowgroup(int K, const uint8_t* const* rowp, int n_rows, const uint8_t* act, const float* actd, const uint32_t* cb, const uint32_t* sgn, float* y) {
    const int nsb = K / 256, n_slices = (nsb + 3) / 4;
    for (int r = 0; r < n_rows; r++) {
        float lane_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int sl = 0; sl < n_slices; sl++)
            for (int b = 0; b < 4; b++) {
                const int sb = sl * 4 + b;
                if (sb >= nsb) continue;
                for (int s = 0; s < 8; s++) {
                    const int lane = 8 * (r & 3) + s;
                    tl_lane = lane;
                    ActsR a;
                    GranR<FMT>::load_acts(a, sp_from(act + (size_t)sb * ACTR_BLOCK_BYTES), sp_from(actd + sb * 8), s);
                    const TablesR t{sp_from(cb), sp_from(sgn), 4u * (uint32_t)lane};
                    const uint8_t* row = rowp[r] + (size_t)sl * 4 * GranR<FMT>::BB;
                    float v = 0;
                    switch (b) {
                        case 0: v = block_r<FMT, 0>(row, s, a, t); break;
                        case 1: v = block_r<FMT, 1>(row, s, a, t); break;
                        case 2: v = block_r<FMT, 2>(row, s, a, t); break;
                        default: v = block_r<FMT, 3>(row, s, a, t); break;
                    }
                    lane_acc[s] += v;
                }
            }
        // the butterfly over the row's eight lanes: xor 1, 2, 4
        for (int bit = 1; bit < 8; bit <<= 1) {
            float nxt[8];
            for (int s = 0; s < 8; s++) nxt[s] = lane_acc[s] + lane_acc[s ^ bit];
            for (int s = 0; s < 8; s++) lane_acc[s] = nxt[s];
        }
        y[r] = lane_acc[0];
    }
}
}  // namespace

// W: n_rows rows `row_bytes` apart (a multiple of 8); xq: Q8_K blocks of one column; addr_lo: 0 or 8, the pretended low
// address bits of row 0; y[n_rows].
extern "C" int emul_gemv1_rowgroup(int fmt, int K, const uint8_t* W, int row_bytes, int n_rows, const uint8_t* xq, int addr_lo, float* y) {
    const int bb = block_bytes(fmt), nsb = K / 256, n_slices = (nsb + 3) / 4;
    if (fmt != T_IQ3_XXS || row_bytes % 8 || (addr_lo & 7) || row_bytes < nsb * bb) return -1;
    const int slot = (row_bytes + 4 * bb + 15) / 16 * 16 + 16;
    std::vector<uint8_t> stage((size_t)n_rows * slot + 64, 0x5A);
    uint8_t* st = (uint8_t*)(((uintptr_t)stage.data() + 15) & ~(uintptr_t)15);
    std::vector<const uint8_t*> rowp(n_rows);
    for (int r = 0; r < n_rows; r++) {
        uint8_t* p = st + (size_t)r * slot + ((addr_lo + r * row_bytes) & 15);
        memcpy(p, W + (size_t)r * row_bytes, nsb * bb);
        rowp[r] = p;
    }
    std::vector<uint8_t> actbuf((size_t)n_slices * 4 * ACTR_BLOCK_BYTES + 64, 0);
    uint8_t* act = (uint8_t*)(((uintptr_t)actbuf.data() + 15) & ~(uintptr_t)15);
    std::vector<float> actd((size_t)n_slices * 32, 0.f);
    for (int sb = 0; sb < nsb; sb++) {
        const uint8_t* blk = xq + (size_t)sb * 292;
        memcpy(&actd[sb * 8], blk, 4);
        for (int w = 0; w < 64; w++) {
            uint32_t v;
            memcpy(&v, blk + 4 + 4 * w, 4);
            const uint32_t n = neg_bytes4(v);
            memcpy(act + (size_t)sb * ACTR_BLOCK_BYTES + actr_pos(4 * w, 0), &v, 4);
            memcpy(act + (size_t)sb * ACTR_BLOCK_BYTES + actr_pos(4 * w, 1), &n, 4);
        }
    }
    std::vector<uint32_t> cb(256 * 32 + 4), sgn(128 * 32 + 4);
    uint32_t* cba = (uint32_t*)(((uintptr_t)cb.data() + 15) & ~(uintptr_t)15);
    uint32_t* sga = (uint32_t*)(((uintptr_t)sgn.data() + 15) & ~(uintptr_t)15);
    for (int i = 0; i < 256 * 32; i++) cba[i] = q38b_iq3xxs_grid[i >> 5];
    for (int i = 0; i < 128 * 32; i++) sga[i] = ksign_selectors((uint32_t)i >> 5);
    run_rowgroup<T_IQ3_XXS>(K, rowp.data(), n_rows, act, actd.data(), cba, sga, y);
    return 0;
}
