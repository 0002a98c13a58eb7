// Shared-memory ring plumbing of the decode kernels: mbarriers, 1-D bulk copies global -> shared, the bounded wait.
#pragma once
#include "common.cuh"

namespace q4fc {

constexpr unsigned long long kWaitLimitNs = 1000000000ull;  // every wait of a kernel gives up after one second

// ---- PTX wrappers -------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// 1-D bulk copy global -> this CTA's shared memory; bytes % 16 == 0, both addresses 16-byte aligned
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait on an mbarrier phase.  Once one wait of the CTA has run out (*fail != 0) all others end at once.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile int* fail, int* status, int code) {
    if (mbar_try_wait(bar, parity)) return;
    const unsigned long long t0 = globaltimer_ns();
    for (unsigned it = 1;; it++) {
        if (mbar_try_wait(bar, parity)) return;
        if ((it & 255) == 0) {
            if (*fail != 0) return;
            if (globaltimer_ns() - t0 > kWaitLimitNs) {
                *fail = 1;
                atomicCAS(status, 0, code);
                return;
            }
        }
    }
}

}  // namespace q4fc
