// Ordering between the launches of the ranks of a data-parallel job (one process per GPU) by flags in memory
// that all ranks have mapped, used by the kernels that exchange data over NVLink inside the launch.
#pragma once

#include "common.cuh"

namespace d3gs {

// ---- ordering between the ranks' launches without a host-side collective ------------------------------------
// Every rank owns a block of D3GS_PEER_FLAG_WORDS words that all ranks have mapped.  Word q: rank q's gradient
// buffer is complete for launch `epoch`; word 8 + q: rank q has finished launch `epoch` (its parameter stores have
// been performed and it no longer reads anybody's gradients); word 16 + q: rank q's status bits of that launch;
// word 24: count of this rank's CTAs that have finished.  Epochs only grow, so nothing is ever reset.  One such
// kernel runs per GPU at a time and the ranks are different GPUs, so the waits below spin on a flag that a kernel
// on ANOTHER device sets; they are bounded and report D3GS_STATUS_PEER_TIMEOUT instead of hanging.
constexpr int kFlagReady = 0, kFlagDone = 8, kFlagErr = 16, kFlagCount = 24;
constexpr uint32_t kDefaultFlagPolls = 1u << 24;   // with the back-off below: on the order of seconds

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// true when every rank's word base + q of MY block has reached `epoch`; gives up after `limit` polls
__device__ __forceinline__ bool wait_flags(const D3gsPeerSet& ps, int base) {
    const uint32_t limit = ps.wait_limit != 0 ? ps.wait_limit : kDefaultFlagPolls;
    const uint32_t* mine = ps.flags[ps.rank] + base;
    for (int q = 0; q < ps.world; ++q) {
        uint32_t it = 0;
        while ((int32_t)(ld_acquire_sys(mine + q) - ps.epoch) < 0) {
            if (++it > limit) return false;
            if (it > 32) __nanosleep(it > 4096 ? 256 : 32);
        }
    }
    return true;
}

// Start of a launch: CTA 0 announces that this rank's gradients are complete (they were written by earlier work
// of this stream), and every CTA waits until all ranks have announced.  Returns false (to all threads of the CTA)
// when the wait ran out; the status bit is set then.
__device__ __forceinline__ bool exchange_begin(const D3gsPeerSet& ps) {
    if (ps.flags[0] == nullptr) return true;      // the caller orders the launches with a collective
    __shared__ int s_ok;
    if (threadIdx.x == 0) {
        if (blockIdx.x == 0) {
            __threadfence_system();
            for (int q = 0; q < ps.world; ++q) st_release_sys(ps.flags[q] + kFlagReady + ps.rank, ps.epoch);
        }
        const bool ok = wait_flags(ps, kFlagReady);
        if (!ok && ps.status != nullptr) atomicOr(ps.status, D3GS_STATUS_PEER_TIMEOUT);
        s_ok = ok ? 1 : 0;
    }
    __syncthreads();
    return s_ok != 0;
}

// End of a launch, called by every thread of every CTA: the last CTA to finish tells all ranks that this rank is
// done (with its status bits) and waits until all ranks are done, so that when the kernel ends every slice of the
// parameters has arrived in this rank's buffer and nobody reads this rank's gradients any more.  A failure on
// any rank reaches every rank's status word here: all ranks raise at the same step.
__device__ __forceinline__ void exchange_end(const D3gsPeerSet& ps) {
    if (ps.flags[0] == nullptr) return;
    __threadfence_system();                      // this thread's parameter stores are performed for every GPU
    __syncthreads();
    if (threadIdx.x != 0) return;
    uint32_t* mine = ps.flags[ps.rank];
    const uint32_t ticket = atomicAdd(mine + kFlagCount, 1u);
    if (ticket != gridDim.x - 1) return;
    mine[kFlagCount] = 0;                        // the next launch counts from zero
    __threadfence_system();
    const uint32_t bits = ps.status != nullptr ? *reinterpret_cast<volatile uint32_t*>(ps.status) : 0u;
    for (int q = 0; q < ps.world; ++q) {
        *reinterpret_cast<volatile uint32_t*>(ps.flags[q] + kFlagErr + ps.rank) = bits;
        st_release_sys(ps.flags[q] + kFlagDone + ps.rank, ps.epoch);
    }
    const bool ok = wait_flags(ps, kFlagDone);
    uint32_t all = ok ? 0u : D3GS_STATUS_PEER_TIMEOUT;
    for (int q = 0; q < ps.world; ++q) all |= *reinterpret_cast<volatile uint32_t*>(mine + kFlagErr + q);
    if (all != 0 && ps.status != nullptr) atomicOr(ps.status, all);
}


}  // namespace d3gs
