// q38b_plan.cu -- the all-HBM planner: resident row-sharded matrices, pass recording, CUDA-graph replay,
// NCCL all-gather of output slices (NCCL is bound at run time with dlopen so that single-GPU users need no NCCL).
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <algorithm>
#include <cstring>
#include <new>
#include <vector>

#include "../../include/q38b200.h"
#include "q38b_act.cuh"
#include "q38b_pipe.cuh"
#include "q38b_internal.h"

using namespace q38b;

namespace {

// ---- minimal NCCL binding -------------------------------------------------------------------------------------
typedef struct { char internal[128]; } NcclId;
typedef int (*FnGetUniqueId)(NcclId*);
typedef int (*FnCommInitRank)(void**, int, NcclId, int);
typedef int (*FnAllGather)(const void*, void*, size_t, int, void*, cudaStream_t);
typedef int (*FnGroup)();
typedef int (*FnCommDestroy)(void*);
struct Nccl {
    void* lib = nullptr;
    FnGetUniqueId get_id = nullptr;
    FnCommInitRank init_rank = nullptr;
    FnAllGather all_gather = nullptr;
    FnGroup group_start = nullptr, group_end = nullptr;
    FnCommDestroy destroy = nullptr;
    bool ok() const { return lib && get_id && init_rank && all_gather && group_start && group_end; }
};
Nccl& nccl() {
    static Nccl n;
    if (!n.lib) {
        n.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!n.lib) n.lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (n.lib) {
            n.get_id = (FnGetUniqueId)dlsym(n.lib, "ncclGetUniqueId");
            n.init_rank = (FnCommInitRank)dlsym(n.lib, "ncclCommInitRank");
            n.all_gather = (FnAllGather)dlsym(n.lib, "ncclAllGather");
            n.group_start = (FnGroup)dlsym(n.lib, "ncclGroupStart");
            n.group_end = (FnGroup)dlsym(n.lib, "ncclGroupEnd");
            n.destroy = (FnCommDestroy)dlsym(n.lib, "ncclCommDestroy");
        }
    }
    return n;
}
constexpr int NCCL_FLOAT = 7;

enum OpKind { OP_QUANT, OP_GEMV, OP_SWIGLU, OP_GATHER, OP_BARRIER, OP_TOPK };
struct Op { int kind, a, b, c, d, n, off; };
struct Buf { void* ptr; int n; bool q8k; void* peer[8]; int n_peer_ranks; bool in_arena; };
struct Mat { uint32_t type; const void* W; size_t row_bytes; int K, M; bool owned; };

struct PeerPtrs { uint32_t* p[8]; };

// Cross-GPU barrier of the peer-store gather as a kernel of its own (barriers that no matvec or SwiGLU launch follows;
// q38b_peer_barrier).  Runs after the matvecs whose outputs were pushed to the peers: the kernel boundary plus the system
// fence make those stores visible before the flag.  n_new > 0: first claim n_new epochs for a new run (see PeerSync).
__global__ void peer_barrier_kernel(PeerSync ps, int n_new, int do_barrier, int* status) {
    if (n_new > 0) {
        if (threadIdx.x == 0) {
            const uint32_t base = ps.local[9];
            ps.local[10] = base;
            ps.local[9] = base + (uint32_t)n_new;
        }
        __syncwarp();
    }
    if (do_barrier) peer_sync_wait(ps, true, (int)threadIdx.x, status);
}

}  // namespace

struct q38b_pass {
    q38b_ctx* ctx = nullptr;
    int max_nb = 1;
    std::vector<Buf> bufs;
    std::vector<Mat> mats;
    std::vector<Op> ops;
    cudaGraphExec_t graphs[9] = {};
    size_t arena_mark = (size_t)-1;
    int peer_store = 1;
    cudaStream_t cap_stream = nullptr;   // capture happens here: the caller's stream may be the legacy default stream
    float* pin_in = nullptr;
    float* pin_out = nullptr;
    size_t pin_in_n = 0, pin_out_n = 0;
    int merge_steps = 1;         // replays: one launch for matvecs that share a column, quantize steps folded into single-column launches
    // What each recorded graph was captured with: a graph is recorded again when any of it has changed since (steps
    // appended, merging or peer stores switched, a context option that picks kernels or launch attributes).
    struct Captured {
        size_t n_ops; int peer_store, merge_steps, uniform_columns, pdl, n_ranks, peers_connected, rowgroup, one_cta; long long part_items;
        bool operator==(const Captured& o) const {
            return n_ops == o.n_ops && peer_store == o.peer_store && merge_steps == o.merge_steps && uniform_columns == o.uniform_columns &&
                   pdl == o.pdl && n_ranks == o.n_ranks && peers_connected == o.peers_connected && rowgroup == o.rowgroup && one_cta == o.one_cta && part_items == o.part_items;
        }
    };
    Captured captured[9] = {};
};

#define PASS_CUDA(p, call)                                \
    do {                                                  \
        cudaError_t e_ = (call);                          \
        if (e_ != cudaSuccess) {                          \
            (p)->ctx->last_cuda = (int)e_;                \
            return Q38B_ERR_CUDA;                         \
        }                                                 \
    } while (0)

namespace {
bool is_f32(const q38b_pass* p, int id) { return id >= 0 && id < (int)p->bufs.size() && !p->bufs[id].q8k; }
bool is_q8k(const q38b_pass* p, int id) { return id >= 0 && id < (int)p->bufs.size() && p->bufs[id].q8k; }

PeerSync make_sync(const q38b_ctx* ctx, int seq) {
    PeerSync ps;
    memset(&ps, 0, sizeof(ps));
    ps.local = ctx->d_flags;
    for (int r = 0; r < 8; r++) ps.peer[r] = ctx->peer_flags[r];
    ps.n = ctx->n_ranks;
    ps.rank = ctx->rank;
    ps.seq = seq;
    ps.budget = ctx->wait_budget_cycles;
    return ps;
}
int launch_barrier(q38b_ctx* ctx, int n_new, int do_barrier, int seq, cudaStream_t st) {
    peer_barrier_kernel<<<1, 32, 0, st>>>(make_sync(ctx, seq), n_new, do_barrier, ctx->d_status);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { ctx->last_cuda = (int)e; return Q38B_ERR_CUDA; }
    return Q38B_OK;
}

int enqueue_ops(q38b_pass* p, int nb, cudaStream_t st);

// matrices of a pass are resident: their producers may run ahead of the previous kernel
int enqueue(q38b_pass* p, int nb, cudaStream_t st) {
    const int saved = p->ctx->static_weights, saved_pdl = p->ctx->pdl;
    p->ctx->static_weights = 1;
    p->ctx->pdl = p->ctx->pass_pdl;   // inside a pass every matvec follows one of this library's kernels
    const int rc = enqueue_ops(p, nb, st);
    p->ctx->static_weights = saved;
    p->ctx->pdl = saved_pdl;
    return rc;
}

// One launch of the merged single-column replay: `n` matvec ops (indices into p->ops) that read one column, which comes
// as the Q8_K buffer of the ops or, when `quant` >= 0, as the fp32 source of that quantize op (folded into the launch:
// the kernel forms the Q8_K blocks in its prologue).
struct Merged { int first_op; int n; int ops[3]; int quant; };

// number of ranks a matvec step's output is pushed to (0 for steps recorded with q38b_pass_op_gemv_local)
int pushes(const q38b_pass* p, const Op& o) { return o.d ? 0 : p->bufs[o.c].n_peer_ranks; }

// Which steps of a replay can share launches.  A quantize step is folded into the
// matvecs that read its output when they follow it directly, nothing else reads that output before it is rewritten, and
// all of them run on the one-column kernel.  Consecutive matvecs of one format, K and row stride on one column share a launch.
void merge_plan(const q38b_pass* p, int nb, std::vector<Merged>& out, std::vector<char>& skip) {
    const q38b_ctx* ctx = p->ctx;
    const std::vector<Op>& ops = p->ops;
    const size_t n = ops.size();
    out.clear();
    skip.assign(n, 0);
    const bool ranks = ctx->n_ranks > 1;
    auto next_real = [&](size_t i) { while (i < n && (ops[i].kind == OP_GATHER || ops[i].kind == OP_BARRIER)) i++; return i; };
    auto on_column = [&](size_t k, int col) { return k < n && ops[k].kind == OP_GEMV && ops[k].b == col; };
    // The step after matvec k that may still join k's launch, which is emitted at the position of the run's first matvec:
    // on several ranks a cross-GPU barrier is a hard cut, and an all-gather may only be stepped over by a matvec whose
    // output does not lie in the gathered range (the recorded order of those two must be kept).  n when there is none.
    auto next_in_run = [&](size_t k) {
        size_t j = k + 1;
        if (!ranks) return next_real(j);
        const size_t first_skipped = j;
        while (j < n && ops[j].kind == OP_GATHER) j++;
        if (j >= n || ops[j].kind != OP_GEMV) return j < n && ops[j].kind == OP_BARRIER ? n : j;
        const long long lo = ops[j].off, hi = lo + p->mats[ops[j].a].M;
        for (size_t g = first_skipped; g < j; g++) {
            const long long glo = ops[g].off, ghi = glo + (long long)ops[g].n * ctx->n_ranks;
            if (ops[g].a == ops[j].c && lo < ghi && glo < hi) return n;
        }
        return j;
    };
    size_t i = next_real(0);
    while (i < n) {
        int quant = -1;
        size_t g0 = i;
        if (ops[i].kind == OP_QUANT) {
            const int col = ops[i].b;
            const size_t j = ranks ? i + 1 : next_real(i + 1);   // several ranks: only a matvec right after the quantize step
            std::vector<size_t> run;                              // the matvecs the quantize step would be folded into
            for (size_t k = j; on_column(k, col); k = next_in_run(k)) run.push_back(k);
            const size_t run_end = run.empty() ? j : next_real(run.back() + 1);
            bool ok = !run.empty() && ops[i].off % 4 == 0;
            for (size_t k = run_end; ok && k < n; k++) {   // nobody else reads the Q8_K buffer before it is written again
                const Op& o = ops[k];
                if ((o.kind == OP_QUANT && o.b == col) || (o.kind == OP_SWIGLU && o.c == col)) break;
                if (o.kind == OP_GEMV && o.b == col) ok = false;
            }
            for (size_t k : run) {
                if (!ok) break;
                const Mat& m = p->mats[ops[k].a];
                if (m.K != ops[i].n) ok = false;
                else if (nb == 1 ? !q38b_gemv_group_plannable(ctx, m.type, 1, m.row_bytes, m.K, &m.M)
                                 : !q38b_gemvn_group_plannable(ctx, m.type, 1, m.row_bytes, m.K, &m.M, nb)) ok = false;
            }
            if (!ok) { i = next_real(i + 1); continue; }   // the quantize step runs as a kernel of its own
            quant = (int)i;
            skip[i] = 1;
            g0 = j;
        } else if (ops[i].kind != OP_GEMV) {
            i = next_real(i + 1);
            continue;
        }
        // cut the run of matvecs on this column into launches of up to three
        const int col = ops[g0].b;
        size_t k = g0, resume = g0 + 1;   // resume: the step after the last matvec this run has taken
        while (on_column(k, col)) {
            Merged mg = {(int)k, 0, {0, 0, 0}, quant};
            const Mat& m0 = p->mats[ops[k].a];
            int Ms[3];
            while (on_column(k, col) && mg.n < 3) {
                const Mat& m = p->mats[ops[k].a];
                if (m.type != m0.type || m.K != m0.K || m.row_bytes != m0.row_bytes) break;
                if (pushes(p, ops[k]) != pushes(p, ops[mg.first_op])) break;   // outputs pushed to the peers or not: one kind per launch
                Ms[mg.n] = m.M;
                if (nb == 1 ? !q38b_gemv_group_plannable(ctx, m0.type, mg.n + 1, m0.row_bytes, m0.K, Ms)
                            : !q38b_gemvn_group_plannable(ctx, m0.type, mg.n + 1, m0.row_bytes, m0.K, Ms, nb)) break;
                mg.ops[mg.n++] = (int)k;
                resume = k + 1;
                k = next_in_run(k);
            }
            if (mg.n == 0) {   // runs on the multi-column kernel only (never after a folded quantize): left alone
                resume = k + 1;
                k = next_in_run(k);
                continue;
            }
            if (mg.n > 1 || quant >= 0) {
                for (int t = 0; t < mg.n; t++) skip[mg.ops[t]] = 1;
                out.push_back(mg);
            }
        }
        i = next_real(resume);
    }
}

bool merging(const q38b_pass* p, int nb) { return p->merge_steps && (nb > 1 || !p->ctx->uniform_columns); }

int enqueue_ops(q38b_pass* p, int nb, cudaStream_t st) {
    q38b_ctx* ctx = p->ctx;
    std::vector<Merged> merged;
    std::vector<char> skip(p->ops.size(), 0);
    if (merging(p, nb)) merge_plan(p, nb, merged, skip);
    size_t next_merged = 0;
    // Cross-GPU barriers of this run: numbered in order; a barrier that a merged matvec launch or a SwiGLU kernel
    // follows is folded into that launch's prologue, the others run as a kernel of their own.
    int n_barriers = 0, barrier_seq = 0;
    if (ctx->n_ranks > 1 && ctx->peers_connected)
        for (const Op& o : p->ops) n_barriers += o.kind == OP_BARRIER;
    if (n_barriers > 0) {
        const int rc = launch_barrier(ctx, n_barriers, 0, 0, st);   // claims the run's epochs
        if (rc != Q38B_OK) return rc;
    }
    ctx->pending_sync_seq = -1;
    for (size_t oi = 0; oi < p->ops.size(); oi++) {
        while (next_merged < merged.size() && merged[next_merged].first_op == (int)oi) {
            const Merged& mg = merged[next_merged++];
            const void* W[3];
            float* y[3];
            int M[3];
            for (int t = 0; t < mg.n; t++) {
                const Op& g = p->ops[mg.ops[t]];
                const Mat& m = p->mats[g.a];
                W[t] = m.W;
                M[t] = m.M;
                y[t] = (float*)p->bufs[g.c].ptr + g.off;
            }
            const Op& g0 = p->ops[mg.ops[0]];
            const Mat& m0 = p->mats[g0.a];
            if (nb > 1) {
                long long ylds[3];
                for (int t = 0; t < mg.n; t++) ylds[t] = p->bufs[p->ops[mg.ops[t]].c].n;
                const Buf& sb = p->bufs[g0.b];
                const float* xf = nullptr;
                long long xf_ld = 0;
                if (mg.quant >= 0) {   // the quantize step is folded: the kernel reads the fp32 columns
                    const Buf& src = p->bufs[p->ops[mg.quant].a];
                    xf = (const float*)src.ptr + p->ops[mg.quant].off;
                    xf_ld = src.n;
                }
                float* peers[3 * 7];
                int np = 0;
                if (p->peer_store && ctx->n_ranks > 1 && !g0.d) {
                    const Buf& d0 = p->bufs[g0.c];
                    for (int r = 0; r < d0.n_peer_ranks; r++) np += r != ctx->rank && d0.peer[r];
                    for (int t = 0; t < mg.n; t++) {
                        const Op& g = p->ops[mg.ops[t]];
                        const Buf& d = p->bufs[g.c];
                        int k = 0;
                        for (int r = 0; r < d.n_peer_ranks; r++)
                            if (r != ctx->rank && d.peer[r]) peers[t * np + k++] = (float*)d.peer[r] + g.off;
                        if (k != np) return Q38B_ERR_ARG;   // all outputs of one launch live in peer-visible buffers, or none
                    }
                }
                const int rc = q38b_gemvn_group_x(ctx, m0.type, mg.n, W, m0.row_bytes, m0.K, M, xf ? nullptr : sb.ptr, sb.n / 256, xf, xf_ld, nb, y,
                                                  ylds, peers, np, st);
                if (rc != Q38B_OK) return rc;
                continue;
            }
            const void* q8k = mg.quant >= 0 ? nullptr : p->bufs[g0.b].ptr;
            const float* xf = mg.quant >= 0 ? (const float*)p->bufs[p->ops[mg.quant].a].ptr + p->ops[mg.quant].off : nullptr;
            float* peers[3 * 7];
            int np = 0;
            if (p->peer_store && ctx->n_ranks > 1 && !g0.d) {
                const Buf& d0 = p->bufs[g0.c];
                for (int r = 0; r < d0.n_peer_ranks; r++) np += r != ctx->rank && d0.peer[r];
                for (int t = 0; t < mg.n; t++) {
                    const Op& g = p->ops[mg.ops[t]];
                    const Buf& d = p->bufs[g.c];
                    int k = 0;
                    for (int r = 0; r < d.n_peer_ranks; r++)
                        if (r != ctx->rank && d.peer[r]) peers[t * np + k++] = (float*)d.peer[r] + g.off;
                    if (k != np) return Q38B_ERR_ARG;   // all outputs of one launch live in peer-visible buffers, or none
                }
            }
            const int rc = q38b_gemv_group_peers(ctx, m0.type, mg.n, W, m0.row_bytes, m0.K, M, q8k, xf, y, peers, np, st);
            if (rc != Q38B_OK) return rc;
        }
        if (skip[oi]) continue;
        const Op& o = p->ops[oi];
        int rc = Q38B_OK;
        switch (o.kind) {
            case OP_QUANT: {
                const Buf& s = p->bufs[o.a];
                const Buf& d = p->bufs[o.b];
                rc = q38b_quantize_q8k(ctx, (const float*)s.ptr + o.off, s.n, o.n, nb, d.ptr, d.n / 256, st);
                break;
            }
            case OP_GEMV: {
                const Mat& m = p->mats[o.a];
                const Buf& s = p->bufs[o.b];
                const Buf& d = p->bufs[o.c];
                float* peers[7];
                int np = 0;
                for (int r = 0; p->peer_store && !o.d && r < d.n_peer_ranks; r++)
                    if (r != ctx->rank && d.peer[r]) peers[np++] = (float*)d.peer[r] + o.off;
                rc = q38b_gemv_q8k_scatter(ctx, m.type, m.W, m.row_bytes, m.K, m.M, s.ptr, s.n / 256, nb, (float*)d.ptr + o.off, d.n, 0,
                                           peers, np, st);
                break;
            }
            case OP_SWIGLU: {
                const Buf& g = p->bufs[o.a];
                const Buf& u = p->bufs[o.b];
                const Buf& d = p->bufs[o.c];
                if (g.n != u.n) return Q38B_ERR_ARG;
                rc = q38b_swiglu_q8k(ctx, (const float*)g.ptr + o.off, (const float*)u.ptr + o.d, g.n, o.n, nb, nullptr, d.ptr,
                                     d.n / 256, st);
                break;
            }
            case OP_TOPK: {   // a: logits buffer, off: first logit, n: how many, d: k, b: destination (k values, then k positions as int bits)
                const Buf& s = p->bufs[o.a];
                const Buf& d = p->bufs[o.b];
                rc = q38b_topk(ctx, (const float*)s.ptr + o.off, s.n, o.n, nb, o.d, 0, (float*)d.ptr, (int*)d.ptr + o.d, d.n, st);
                break;
            }
            case OP_BARRIER: {
                if (n_barriers == 0) break;
                if (ctx->pending_sync_seq >= 0) {   // two barriers in a row: the earlier one runs by itself
                    rc = launch_barrier(ctx, 0, 1, ctx->pending_sync_seq, st);
                    ctx->pending_sync_seq = -1;
                    if (rc != Q38B_OK) return rc;
                }
                size_t j = oi + 1;
                while (j < p->ops.size() && (p->ops[j].kind == OP_GATHER || p->ops[j].kind == OP_BARRIER)) j++;
                bool next_is_merged = false;   // op j opens a merged launch: its folded quantize step or its first matvec
                for (const Merged& mg : merged) next_is_merged |= (mg.quant >= 0 ? mg.quant : mg.first_op) == (int)j;
                const bool next_is_swiglu = j < p->ops.size() && !skip[j] && p->ops[j].kind == OP_SWIGLU;
                const bool adjacent = j == oi + 1;   // nothing (not even a gather) between the barrier and that launch
                // (the multi-column kernel has no barrier in its prologue: in front of it the barrier is a kernel of its own)
                if (adjacent && ((next_is_merged && nb == 1) || next_is_swiglu)) ctx->pending_sync_seq = barrier_seq++;
                else rc = launch_barrier(ctx, 0, 1, barrier_seq++, st);
                break;
            }
            case OP_GATHER: {
                if (ctx->n_ranks <= 1) break;
                Nccl& n = nccl();
                if (!n.ok() || !ctx->comm) return Q38B_ERR_ARG;
                const Buf& b = p->bufs[o.a];
                if (n.group_start()) return Q38B_ERR_CUDA;
                for (int c = 0; c < nb; c++) {
                    float* base = (float*)b.ptr + (size_t)c * b.n + o.off;
                    if (n.all_gather(base + (size_t)ctx->rank * o.n, base, (size_t)o.n, NCCL_FLOAT, ctx->comm, st)) return Q38B_ERR_CUDA;
                }
                if (n.group_end()) return Q38B_ERR_CUDA;
                break;
            }
        }
        if (rc != Q38B_OK) return rc;
    }
    return Q38B_OK;
}
}  // namespace

extern "C" {

int q38b_comm_unique_id(void* id128) {
    if (!id128) return Q38B_ERR_ARG;
    Nccl& n = nccl();
    if (!n.ok()) return Q38B_ERR_UNSUPPORTED;
    NcclId id;
    if (n.get_id(&id)) return Q38B_ERR_CUDA;
    memcpy(id128, &id, 128);
    return Q38B_OK;
}

int q38b_comm_init(q38b_ctx* ctx, int n_ranks, int rank, const void* id128) {
    if (!ctx || !id128 || n_ranks < 1 || rank < 0 || rank >= n_ranks) return Q38B_ERR_ARG;
    Nccl& n = nccl();
    if (!n.ok()) return Q38B_ERR_UNSUPPORTED;
    NcclId id;
    memcpy(&id, id128, 128);
    void* comm = nullptr;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return Q38B_ERR_CUDA;
    if (n.init_rank(&comm, n_ranks, id, rank)) return Q38B_ERR_CUDA;
    ctx->comm = comm;
    ctx->n_ranks = n_ranks;
    ctx->rank = rank;
    return Q38B_OK;
}

int q38b_peer_export(q38b_ctx* ctx, const void* dev_ptr, void* handle64) {
    if (!ctx || !dev_ptr || !handle64) return Q38B_ERR_ARG;
    cudaIpcMemHandle_t h;
    static_assert(sizeof(h) == 64, "IPC handle size");
    cudaError_t e = cudaIpcGetMemHandle(&h, (void*)dev_ptr);
    if (e != cudaSuccess) { ctx->last_cuda = (int)e; return Q38B_ERR_CUDA; }
    memcpy(handle64, &h, 64);
    return Q38B_OK;
}

int q38b_peer_import(q38b_ctx* ctx, const void* handle64, void** dev_ptr) {
    if (!ctx || !handle64 || !dev_ptr) return Q38B_ERR_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    cudaError_t e = cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) { ctx->last_cuda = (int)e; return Q38B_ERR_CUDA; }
    return Q38B_OK;
}

int q38b_peer_arena_create(q38b_ctx* ctx, size_t bytes, void* handle64) {
    if (!ctx || !handle64 || bytes < 4096) return Q38B_ERR_ARG;
    if (!ctx->d_flags) {
        bytes = (bytes + ((size_t)2 << 20) - 1) & ~(((size_t)2 << 20) - 1);   // whole 2 MB units: an allocation of its own
        cudaError_t e = cudaMalloc(&ctx->d_flags, bytes);
        if (e == cudaSuccess) e = cudaMemset(ctx->d_flags, 0, bytes);
        if (e != cudaSuccess) { ctx->last_cuda = (int)e; return Q38B_ERR_CUDA; }
        ctx->arena_bytes = bytes;
        ctx->arena_used = 256;
    }
    return q38b_peer_export(ctx, ctx->d_flags, handle64);
}

int q38b_peer_connect(q38b_ctx* ctx, int n_ranks, int rank, const void* handles) {
    if (!ctx || !handles || n_ranks < 2 || n_ranks > 8 || rank < 0 || rank >= n_ranks || !ctx->d_flags) return Q38B_ERR_ARG;
    for (int r = 0; r < n_ranks; r++) {
        if (r == rank) { ctx->peer_flags[r] = ctx->d_flags; continue; }
        void* ptr = nullptr;
        const int rc = q38b_peer_import(ctx, (const char*)handles + 64 * r, &ptr);
        if (rc != Q38B_OK) return rc;
        ctx->peer_flags[r] = (uint32_t*)ptr;
    }
    ctx->n_ranks = n_ranks;
    ctx->rank = rank;
    ctx->peers_connected = 1;
    return Q38B_OK;
}

int q38b_peer_barrier(q38b_ctx* ctx, void* stream) {
    if (!ctx) return Q38B_ERR_ARG;
    if (ctx->n_ranks <= 1) return Q38B_OK;
    if (!ctx->peers_connected) return Q38B_ERR_ARG;
    return launch_barrier(ctx, 1, 1, 0, (cudaStream_t)stream);   // a run of one barrier
}

int q38b_pass_set_peer_store(q38b_pass* p, int enabled) {
    if (!p) return Q38B_ERR_ARG;
    p->peer_store = enabled ? 1 : 0;
    return Q38B_OK;
}

int q38b_pass_op_barrier(q38b_pass* p) {
    if (!p) return Q38B_ERR_ARG;
    p->ops.push_back({OP_BARRIER, 0, 0, 0, 0, 0, 0});
    return Q38B_OK;
}

int q38b_pass_create(q38b_ctx* ctx, int max_nb, q38b_pass** out) {
    if (!ctx || !out || max_nb < 1 || max_nb > 8) return Q38B_ERR_ARG;
    q38b_pass* p = new (std::nothrow) q38b_pass;
    if (!p) return Q38B_ERR_NOMEM;
    p->ctx = ctx;
    p->max_nb = max_nb;
    if (ctx->peers_connected) p->arena_mark = ctx->arena_used;
    *out = p;
    return Q38B_OK;
}

void q38b_pass_destroy(q38b_pass* p) {
    if (!p) return;
    for (auto& g : p->graphs) if (g) cudaGraphExecDestroy(g);
    for (auto& b : p->bufs) if (b.ptr && !b.in_arena) cudaFree(b.ptr);
    if (p->arena_mark != (size_t)-1) p->ctx->arena_used = p->arena_mark;   // passes release arena space in LIFO order
    for (auto& m : p->mats) if (m.owned && m.W) cudaFree((void*)m.W);
    if (p->cap_stream) cudaStreamDestroy(p->cap_stream);
    if (p->pin_in) cudaFreeHost(p->pin_in);
    if (p->pin_out) cudaFreeHost(p->pin_out);
    delete p;
}

int q38b_pass_buffer_f32(q38b_pass* p, int n) {
    if (!p || n < 1) return Q38B_ERR_ARG;
    const size_t bytes = (size_t)p->max_nb * n * sizeof(float);
    q38b_ctx* ctx = p->ctx;
    Buf b = {nullptr, n, false, {}, 0, false};
    if (ctx->peers_connected) {
        // peer-visible: carve from the arena; every rank allocates in the same order, so offsets agree
        const size_t off = (ctx->arena_used + 255) & ~(size_t)255;
        if (off + bytes > ctx->arena_bytes) return Q38B_ERR_NOMEM;
        ctx->arena_used = off + bytes;
        b.ptr = (char*)ctx->d_flags + off;
        b.in_arena = true;
        b.n_peer_ranks = ctx->n_ranks;
        for (int r = 0; r < ctx->n_ranks; r++) b.peer[r] = (char*)ctx->peer_flags[r] + off;
    } else {
        PASS_CUDA(p, cudaMalloc(&b.ptr, bytes));
    }
    PASS_CUDA(p, cudaMemset(b.ptr, 0, bytes));
    p->bufs.push_back(b);
    return (int)p->bufs.size() - 1;
}

int q38b_pass_buffer_q8k(q38b_pass* p, int K) {
    if (!p || K < 256 || K % 256) return Q38B_ERR_ARG;
    void* ptr = nullptr;
    PASS_CUDA(p, cudaMalloc(&ptr, (size_t)p->max_nb * (K / 256) * 292));
    PASS_CUDA(p, cudaMemset(ptr, 0, (size_t)p->max_nb * (K / 256) * 292));
    p->bufs.push_back({ptr, K, true, {}, 0, false});
    return (int)p->bufs.size() - 1;
}

void* q38b_pass_buffer_ptr(q38b_pass* p, int id) { return p && id >= 0 && id < (int)p->bufs.size() ? p->bufs[id].ptr : nullptr; }

int q38b_pass_matrix_device(q38b_pass* p, uint32_t type, const void* W, size_t row_bytes, int K, int M) {
    if (!p || !W || M < 1) return Q38B_ERR_ARG;
    if (!q38b_format_supported(type)) return Q38B_ERR_UNSUPPORTED;
    if (row_bytes < q38b_row_bytes(type, K) || !q38b_row_bytes(type, K)) return Q38B_ERR_ARG;
    if ((uintptr_t)W & 15) return Q38B_ERR_ALIGN;
    p->mats.push_back({type, W, row_bytes, K, M, false});
    return (int)p->mats.size() - 1;
}

int q38b_pass_matrix_upload(q38b_pass* p, uint32_t type, const void* W_host, size_t row_bytes, int K, int M, int shard,
                            int n_shards) {
    if (!p || !W_host || M < 1 || n_shards < 1 || shard < 0 || shard >= n_shards || M % n_shards) return Q38B_ERR_ARG;
    if (!q38b_format_supported(type)) return Q38B_ERR_UNSUPPORTED;
    const size_t packed = q38b_row_bytes(type, K);
    if (!packed || row_bytes < packed) return Q38B_ERR_ARG;
    const int rows = M / n_shards;
    // the shard starts on a 16-byte boundary of a packed copy: rows are packed on upload
    void* dev = nullptr;
    PASS_CUDA(p, cudaMalloc(&dev, (size_t)rows * packed + 16));
    const uint8_t* src = (const uint8_t*)W_host + (size_t)shard * rows * row_bytes;
    PASS_CUDA(p, cudaMemcpy2D(dev, packed, src, row_bytes, packed, rows, cudaMemcpyHostToDevice));
    p->mats.push_back({type, dev, packed, K, rows, true});
    return (int)p->mats.size() - 1;
}

int q38b_pass_op_quantize(q38b_pass* p, int src, int off, int K, int dst) {
    if (!p || !is_f32(p, src) || !is_q8k(p, dst) || K % 256 || off < 0 || off + K > p->bufs[src].n || p->bufs[dst].n < K) return Q38B_ERR_ARG;
    p->ops.push_back({OP_QUANT, src, dst, 0, 0, K, off});
    return Q38B_OK;
}

int q38b_pass_op_gemv(q38b_pass* p, int mat, int src, int dst, int off) {
    if (!p || mat < 0 || mat >= (int)p->mats.size() || !is_q8k(p, src) || !is_f32(p, dst)) return Q38B_ERR_ARG;
    const Mat& m = p->mats[mat];
    if (p->bufs[src].n < m.K || off < 0 || off + m.M > p->bufs[dst].n) return Q38B_ERR_ARG;
    p->ops.push_back({OP_GEMV, mat, src, dst, 0, 0, off});
    return Q38B_OK;
}

int q38b_pass_op_gemv_local(q38b_pass* p, int mat, int src, int dst, int off) {
    const int rc = q38b_pass_op_gemv(p, mat, src, dst, off);
    if (rc == Q38B_OK) p->ops.back().d = 1;   // d = 1: the output is not pushed to the peers
    return rc;
}

int q38b_pass_op_topk(q38b_pass* p, int src, int off, int n, int k, int dst) {
    if (!p || !is_f32(p, src) || !is_f32(p, dst) || src == dst || off < 0 || n < 1 || off + n > p->bufs[src].n || k < 1 || k > 64 ||
        p->bufs[dst].n < 2 * k)
        return Q38B_ERR_ARG;
    if ((n + 1023) / 1024 > 384) return Q38B_ERR_UNSUPPORTED;
    p->ops.push_back({OP_TOPK, src, dst, 0, k, n, off});
    return Q38B_OK;
}

int q38b_pass_op_swiglu(q38b_pass* p, int g, int g_off, int u, int u_off, int n, int dst) {
    if (!p || !is_f32(p, g) || !is_f32(p, u) || !is_q8k(p, dst) || n % 256 || g_off < 0 || u_off < 0) return Q38B_ERR_ARG;
    if (g_off + n > p->bufs[g].n || u_off + n > p->bufs[u].n || p->bufs[dst].n < n || p->bufs[g].n != p->bufs[u].n) return Q38B_ERR_ARG;
    p->ops.push_back({OP_SWIGLU, g, u, dst, u_off, n, g_off});
    return Q38B_OK;
}

int q38b_pass_op_allgather(q38b_pass* p, int buf, int off, int count) {
    if (!p || !is_f32(p, buf) || off < 0 || count < 1) return Q38B_ERR_ARG;
    const int ranks = p->ctx->n_ranks > 1 ? p->ctx->n_ranks : 1;
    if (off + (long long)count * ranks > p->bufs[buf].n) return Q38B_ERR_ARG;
    p->ops.push_back({OP_GATHER, buf, 0, 0, 0, count, off});
    return Q38B_OK;
}

int q38b_pass_run(q38b_pass* p, int nb, void* stream) {
    if (!p || nb < 1 || nb > p->max_nb) return Q38B_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const q38b_pass::Captured now = {p->ops.size(), p->peer_store, p->merge_steps, p->ctx->uniform_columns, p->ctx->pass_pdl,
                                     p->ctx->n_ranks, p->ctx->peers_connected, p->ctx->rowgroup, p->ctx->one_cta, p->ctx->part_items};
    if (p->graphs[nb] && !(now == p->captured[nb])) {
        cudaGraphExecDestroy(p->graphs[nb]);
        p->graphs[nb] = nullptr;
    }
    if (!p->graphs[nb]) {
        cudaGraph_t g = nullptr;
        if (!p->cap_stream) PASS_CUDA(p, cudaStreamCreateWithFlags(&p->cap_stream, cudaStreamNonBlocking));
        PASS_CUDA(p, cudaStreamBeginCapture(p->cap_stream, cudaStreamCaptureModeThreadLocal));
        const int rc = enqueue(p, nb, p->cap_stream);
        const cudaError_t e = cudaStreamEndCapture(p->cap_stream, &g);
        if (rc != Q38B_OK) { if (g) cudaGraphDestroy(g); return rc; }
        if (e != cudaSuccess) { p->ctx->last_cuda = (int)e; return Q38B_ERR_CUDA; }
        const cudaError_t ei = cudaGraphInstantiate(&p->graphs[nb], g, 0);
        cudaGraphDestroy(g);
        if (ei != cudaSuccess) { p->ctx->last_cuda = (int)ei; p->graphs[nb] = nullptr; return Q38B_ERR_CUDA; }
        p->captured[nb] = now;
    }
    PASS_CUDA(p, cudaGraphLaunch(p->graphs[nb], st));
    return Q38B_OK;
}

int q38b_pass_run_host(q38b_pass* p, int nb, int in_buf, const float* x_host, int x_len, int out_buf, int out_off,
                       float* y_host, int y_len, void* stream) {
    if (!p || !x_host || !y_host || nb < 1 || nb > p->max_nb || !is_f32(p, in_buf) || !is_f32(p, out_buf)) return Q38B_ERR_ARG;
    if (x_len < 1 || x_len > p->bufs[in_buf].n || out_off < 0 || y_len < 1 || out_off + y_len > p->bufs[out_buf].n) return Q38B_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t need_in = (size_t)p->max_nb * x_len, need_out = (size_t)p->max_nb * y_len;
    if (p->pin_in_n < need_in) {
        if (p->pin_in) cudaFreeHost(p->pin_in);
        PASS_CUDA(p, cudaMallocHost(&p->pin_in, need_in * sizeof(float)));
        p->pin_in_n = need_in;
    }
    if (p->pin_out_n < need_out) {
        if (p->pin_out) cudaFreeHost(p->pin_out);
        PASS_CUDA(p, cudaMallocHost(&p->pin_out, need_out * sizeof(float)));
        p->pin_out_n = need_out;
    }
    memcpy(p->pin_in, x_host, (size_t)nb * x_len * sizeof(float));
    const Buf& bi = p->bufs[in_buf];
    const Buf& bo = p->bufs[out_buf];
    PASS_CUDA(p, cudaMemcpy2DAsync(bi.ptr, (size_t)bi.n * 4, p->pin_in, (size_t)x_len * 4, (size_t)x_len * 4, nb, cudaMemcpyHostToDevice, st));
    const int rc = q38b_pass_run(p, nb, stream);
    if (rc != Q38B_OK) return rc;
    PASS_CUDA(p, cudaMemcpy2DAsync(p->pin_out, (size_t)y_len * 4, (const float*)bo.ptr + out_off, (size_t)bo.n * 4, (size_t)y_len * 4, nb,
                                   cudaMemcpyDeviceToHost, st));
    PASS_CUDA(p, cudaStreamSynchronize(st));
    memcpy(y_host, p->pin_out, (size_t)nb * y_len * sizeof(float));
    return Q38B_OK;
}

long long q38b_pass_weight_bytes(const q38b_pass* p) {
    if (!p) return 0;
    long long b = 0;
    for (const Op& o : p->ops)
        if (o.kind == OP_GEMV) b += (long long)p->mats[o.a].M * (long long)q38b_row_bytes(p->mats[o.a].type, p->mats[o.a].K);
    return b;
}

int q38b_pass_set_merge(q38b_pass* p, int enabled) {
    if (!p) return Q38B_ERR_ARG;
    p->merge_steps = enabled ? 1 : 0;   // graphs captured with the other setting are recorded again at their next run
    return Q38B_OK;
}

// Test hook (not in the public header): runs the launch planner on a list of steps without touching a device.
// steps[3 i ..] = {kind (0 quantize, 1 matvec, 2 SwiGLU, 3 all-gather, 4 barrier), column buffer, output offset}; every
// matvec is a 512 x 1024 Q4_K matrix writing 512 floats at its offset.  launch_of[i] receives the position in the step
// list at which step i is launched (its own index unless it joined an earlier launch), -1 for folded quantize steps.
int q38b_debug_merge_plan(int n_ranks, int nb, int n_steps, const int* steps, int* launch_of) {
    if (n_ranks < 1 || nb < 1 || n_steps < 0 || !steps || !launch_of) return Q38B_ERR_ARG;
    q38b_ctx ctx;
    ctx.sm_count = 148;
    ctx.smem_optin = 232448;
    ctx.n_ranks = n_ranks;
    q38b_pass p;
    p.ctx = &ctx;
    p.mats.push_back({(uint32_t)T_Q4_K, nullptr, 576, 1024, 512, false});
    for (int b = 0; b < 8; b++) p.bufs.push_back({nullptr, 1 << 20, b >= 4, {}, 0, false});   // 0..3 fp32, 4..7 Q8_K columns
    for (int i = 0; i < n_steps; i++) {
        const int kind = steps[3 * i], col = steps[3 * i + 1], off = steps[3 * i + 2];
        switch (kind) {
            case 0: p.ops.push_back({OP_QUANT, 0, col, 0, 0, 1024, off}); break;
            case 1: p.ops.push_back({OP_GEMV, 0, col, 1, 0, 0, off}); break;
            case 2: p.ops.push_back({OP_SWIGLU, 1, 1, col, 0, 1024, off}); break;
            case 3: p.ops.push_back({OP_GATHER, 1, 0, 0, 0, 512, off}); break;
            case 4: p.ops.push_back({OP_BARRIER, 0, 0, 0, 0, 0, 0}); break;
            default: return Q38B_ERR_ARG;
        }
    }
    std::vector<Merged> merged;
    std::vector<char> skip;
    merge_plan(&p, nb, merged, skip);
    for (int i = 0; i < n_steps; i++) launch_of[i] = i;
    for (const Merged& mg : merged) {
        if (mg.quant >= 0) launch_of[mg.quant] = -1;
        for (int t = 0; t < mg.n; t++) launch_of[mg.ops[t]] = mg.first_op;
    }
    return (int)merged.size();
}

int q38b_pass_kernel_count(const q38b_pass* p) {
    if (!p) return 0;
    int n = 0;
    std::vector<Merged> merged;
    std::vector<char> skip(p->ops.size(), 0);
    if (merging(p, 1)) merge_plan(p, 1, merged, skip);
    for (size_t i = 0; i < p->ops.size(); i++) {
        const Op& o = p->ops[i];
        n += !skip[i] && (o.kind != OP_GATHER) && (o.kind != OP_BARRIER || p->ctx->n_ranks > 1);
        n += o.kind == OP_TOPK;   // two kernels
    }
    return n + (int)merged.size();
}

}  // extern "C"
