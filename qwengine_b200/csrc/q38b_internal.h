// q38b_internal.h -- host-side state shared by the translation units of libq38b200.so.
#pragma once
#include <cstddef>
#include <cstdint>

struct q38b_ctx {
    int device = 0;
    int sm_count = 0;
    int smem_optin = 0;
    int last_cuda = 0;
    int pdl = 0;               // programmatic dependent launch for direct calls (passes use pass_pdl)
    int pass_pdl = 1;          // programmatic dependent launch between the kernels of a recorded pass
    int static_weights = 0;    // 1: matvec producers start streaming W before the previous kernel of the stream has finished
    int rowgroup = 1;          // 0: the row-group mapping of the one-column kernel is not used (test hook q38b_debug_set_rowgroup)
    int one_cta = 1;           // one-column kernel with one CTA per SM where such a plan fits; 0: never (test hook q38b_debug_set_one_cta)
    int check_occupancy = 0, occupancy_shortfalls = 0;   // test hook q38b_debug_occupancy_shortfalls
    int uniform_columns = 0;   // 1: single-column calls also run the tensor-core kernel (bit-identical to columns of wider calls)
    long long wait_budget_cycles = 4000000000LL;   // bounded waits on other GPUs (q38b_ctx_set_wait_budget_cycles)
    int* d_status = nullptr;
    long long part_items = 0;      // (tile, K-part) sums one multi-column launch may use of d_parts (test hook: fewer)
    float* d_parts = nullptr;      // multi-column matvec: (tile, K-part) sums of tiles that two groups share; one stream at a time
    int* d_part_count = nullptr;   // ... and how many parts of each tile are written (zero between launches)
    void* d_topk = nullptr;    // work area of q38b_topk (candidate lists)
    uint32_t* d_cb_iq3xxs = nullptr;
    uint32_t* d_cb_iq3s = nullptr;
    const uint32_t* d_code16[4] = {};   // 16-bit grid codes of IQ2_XXS, IQ2_XS, IQ2_S, IQ1_S / IQ1_M (two per word)
    void* comm = nullptr;   // ncclComm_t when q38b_comm_init was called
    int n_ranks = 1, rank = 0;
    // peer-store gather: flags[0..7] written by the peers, [8] = this rank's barrier count
    // One arena per rank holds the flags (first 256 bytes) and every peer-visible activation buffer, so that a single
    // IPC handle per rank is exchanged and a buffer sits at the same offset on every rank.
    uint32_t* d_flags = nullptr;      // = arena base
    uint32_t* peer_flags[8] = {};     // arena bases of all ranks
    size_t arena_bytes = 0, arena_used = 0;
    int peers_connected = 0;
    const void* configured[96] = {};  // kernels whose opt-in shared-memory size has been set on this context's device
    int n_configured = 0;
    int pending_sync_seq = -1;        // >= 0: the next merged matvec or SwiGLU launch starts with cross-GPU barrier number seq of the run
};

// 1 when q38b_gemv_group would run these matrices (single column) on the one-column kernel
extern "C" int q38b_gemv_group_plannable(const q38b_ctx* ctx, uint32_t type, int n_mats, size_t row_bytes, int K, const int* M);
// q38b_gemv_group with peer stores: y_peers[i * n_peers + r] is where peer r keeps the output of matrix i
extern "C" int q38b_gemv_group_peers(q38b_ctx* ctx, uint32_t type, int n_mats, const void* const* W, size_t row_bytes, int K, const int* M,
                                     const void* q8k, const float* x_f32, float* const* y, float* const* y_peers, int n_peers, void* stream);
// the same for the multi-column kernel (nb columns of Q8_K blocks, q8k_stride blocks apart; y[i][c * y_ld[i] + r]); no peers
extern "C" int q38b_gemvn_group_plannable(const q38b_ctx* ctx, uint32_t type, int n_mats, size_t row_bytes, int K, const int* M, int nb);
// the same with the columns given as floats (x_f32, x_f32_ld floats apart; quantized inside the kernel) instead of Q8_K
// blocks, and with peer stores (y_peers[i * n_peers + r]: peer r's copy of matrix i's output)
extern "C" int q38b_gemvn_group_x(q38b_ctx* ctx, uint32_t type, int n_mats, const void* const* W, size_t row_bytes, int K, const int* M,
                                  const void* q8k, long long q8k_stride, const float* x_f32, long long x_f32_ld, int nb, float* const* y,
                                  const long long* y_ld, float* const* y_peers, int n_peers, void* stream);
extern "C" int q38b_gemvn_group(q38b_ctx* ctx, uint32_t type, int n_mats, const void* const* W, size_t row_bytes, int K, const int* M,
                                const void* q8k, long long q8k_stride, int nb, float* const* y, const long long* y_ld, void* stream);
