// Bounded device-side waits shared by every kernel that spins on an mbarrier.
//
// A wait polls mbarrier.try_wait; after a burst of polls without success it reads the global nanosecond
// timer and gives up once `limit_ns` have passed since its first failed poll (default 2 s: far beyond any
// legitimate copy or MMA latency, short enough that a lost completion does not look like a hang).  Giving up
// is reported through a status word in host-mapped memory that the host reads without synchronising
// (runtime.cu): the kernel then leaves through its normal exit, releasing what it holds.
#pragma once
#include <stdint.h>

namespace xn {

constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

struct WaitCtx {
    unsigned *status;             // host-mapped word: number of waits that ran out on this device (may be null)
    unsigned long long limit_ns;  // how long one wait may last
};

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ bool mbar_try(unsigned bar_smem_addr, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(bar_smem_addr), "r"(parity)
        : "memory");
    return ok != 0;
}

// One running-out is one increment, visible to the host as soon as the store lands in host memory.
__device__ __forceinline__ void report_wait_timeout(const WaitCtx &w) {
    if (w.status) {
        atomicAdd_system(w.status, 1u);
        __threadfence_system();
    }
}

__device__ __forceinline__ bool mbar_wait_bounded(unsigned bar_smem_addr, unsigned parity, const WaitCtx &w) {
    if (mbar_try(bar_smem_addr, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i)
            if (mbar_try(bar_smem_addr, parity)) return true;
        if (global_ns() - t0 > w.limit_ns) break;
    }
    report_wait_timeout(w);
    return false;
}

}  // namespace xn
