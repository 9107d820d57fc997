// mbarrier / bulk-async-copy (TMA) helpers shared by the decode and prefill kernels.
// Every wait is bounded in wall-clock time: when it runs out it records a code in the device status word,
// raises the CTA's abort flag (which every other wait polls) and returns false.
#pragma once

#include "w4a16_common.cuh"

namespace kiln {

// A wait gives up after this much wall-clock time (nanoseconds of %globaltimer) unless the launch says otherwise.
// Legitimate waits in these kernels last microseconds to a few milliseconds.
constexpr unsigned long long kWaitLimitNs = 400ull * 1000 * 1000;

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// One poll; the hardware may park the thread for at most `hint_ns` before answering.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity, uint32_t hint_ns = 2000) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait.  Returns false if the CTA is aborting (this wait or another one ran out).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                          uint32_t *status, uint32_t code, unsigned long long limit_ns = kWaitLimitNs) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (uint32_t i = 0;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 15) == 15) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > limit_ns) break;
        }
    }
    *abort_flag = 1;
    atomicCAS(status, 0u, code);
    return false;
}

// Drain helper for abort paths: bounded (about 20 ms), ignores the abort flag.
__device__ __forceinline__ void mbar_wait_quiet(uint32_t bar, uint32_t parity) {
    const unsigned long long t0 = global_ns();
    while (!mbar_try_wait(bar, parity) && global_ns() - t0 < 20ull * 1000 * 1000) {
    }
}

// 1-D bulk copy global -> shared; dst, src and bytes are multiples of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}

}  // namespace kiln
