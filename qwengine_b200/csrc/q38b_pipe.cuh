// q38b_pipe.cuh -- sm_100a plumbing shared by the kernels: mbarrier, 1-D bulk (TMA) copies,
// named barriers, programmatic dependent launch.  Every wait is bounded: when a barrier does not
// complete within the budget the waiter records an error and returns false, and the kernel runs
// to its end without waiting again (results are then invalid and the host sees the status).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace q38b {

// device-side status bits (OR-ed into the status word of the context)
enum : int { ST_OK = 0, ST_WAIT_FULL_TIMEOUT = 1, ST_WAIT_EMPTY_TIMEOUT = 2, ST_DRAIN_TIMEOUT = 4, ST_TMEM_TIMEOUT = 8 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_n(uint32_t bar, int count) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait on phase `parity` of an mbarrier: gives up after WAIT_BUDGET_CYCLES SM clocks (about a second).
// `abort_flag` (shared memory) is set by whoever times out first; everybody else stops waiting as soon as they
// see it, so a kernel that lost a barrier still runs to its end.
constexpr long long WAIT_BUDGET_CYCLES = 1500000000LL;
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                                  int code, long long budget = WAIT_BUDGET_CYCLES) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > budget) break;
    }
    *abort_flag = 1;
    if (status) atomicOr(status, code);
    return false;
}

// A counter in shared memory that one thread advances (release) and others poll (acquire) until it exceeds `than`.
__device__ __forceinline__ void st_release_shared(uint32_t addr, int v) {
    asm volatile("st.release.cta.shared::cta.s32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_shared(uint32_t addr) {
    int v;
    asm volatile("ld.acquire.cta.shared::cta.s32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_shared_add(uint32_t addr, int v) {
    asm volatile("red.release.cta.shared::cta.add.s32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
// (pause_ns: a background warp's poll leaves the issue slots to the working warps between looks)
__device__ __forceinline__ bool wait_counter_bounded(uint32_t addr, int than, volatile int* abort_flag, int* status, int code,
                                                     long long budget = WAIT_BUDGET_CYCLES, unsigned pause_ns = 0) {
    if (ld_acquire_shared(addr) > than) return true;
    const long long t0 = clock64();
    for (;;) {
        if (ld_acquire_shared(addr) > than) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > budget) break;
        if (pause_ns) __nanosleep(pause_ns);
    }
    *abort_flag = 1;
    if (status) atomicOr(status, code);
    return false;
}

// global -> shared bulk copy of `bytes` (multiple of 16; both addresses 16-byte aligned), completion counted on `bar`.
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Cross-GPU barrier folded into the prologue of a kernel (one process per GPU, peer-mapped flag blocks).  A flag block
// holds [r] = the latest epoch rank r has signalled, [9] = the next free epoch, [10] = the first epoch of the pass run in
// progress (written by a one-thread kernel at the start of every run, so epochs only grow whatever passes alternate).
// Barrier number `seq` of a run has epoch [10] + seq + 1 on every rank.  n = 0: no barrier.
struct PeerSync {
    uint32_t* local;
    uint32_t* peer[8];
    int n, rank, seq;
    long long budget;   // SM clocks a rank waits for a peer before it gives up (q38b_ctx_set_wait_budget_cycles)
};
constexpr long long PEER_WAIT_BUDGET_CYCLES = 4000000000LL;   // default: about two seconds
constexpr int ST_PEER_TIMEOUT = 16;
// The two halves of the barrier, for threads t = 0 .. n - 1.  peer_sync_signal: thread t of ONE CTA tells rank t, once the
// stream's earlier kernels are complete (their stores into the peers' buffers are done).  peer_sync_poll: thread t of
// every CTA waits (bounded) for rank t.  A kernel may do other set-up between the two while the flags travel.
__device__ __forceinline__ void peer_sync_signal(const PeerSync& ps, int t) {
    if (t >= ps.n || t == ps.rank) return;
    const uint32_t e = *(volatile uint32_t*)(ps.local + 10) + (uint32_t)ps.seq + 1u;
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(ps.peer[t] + ps.rank), "r"(e) : "memory");
}
__device__ __forceinline__ void peer_sync_poll(const PeerSync& ps, int t, int* status) {
    if (t >= ps.n || t == ps.rank) return;
    const uint32_t e = *(volatile uint32_t*)(ps.local + 10) + (uint32_t)ps.seq + 1u;
    const long long t0 = clock64();
    for (;;) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ps.local + t) : "memory");
        if ((int)(v - e) >= 0) break;
        if (clock64() - t0 > ps.budget) { if (status) atomicOr(status, ST_PEER_TIMEOUT); break; }
    }
}
// both at once
__device__ __forceinline__ void peer_sync_wait(const PeerSync& ps, bool signaller, int t, int* status) {
    if (signaller) peer_sync_signal(ps, t);
    peer_sync_poll(ps, t, status);
}

// Programmatic dependent launch: let the next kernel of the stream start its prologue now; wait until the
// kernels this one depends on have finished and their writes are visible (no-ops without the launch attribute).
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait_prior() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

}  // namespace q38b
