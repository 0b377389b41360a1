// Bulk asynchronous copies (the TMA engine's untiled form) and mbarrier completion, as inline PTX for sm_100a.
//
// Used by the persistent kernels to stage the gathered input rows of the NEXT work item into shared memory while
// the current one is being computed, so that a warp never waits on a global load it has just issued.
// Rules kept here: source and destination 16-byte aligned, size a multiple of 16 bytes; every wait on an mbarrier
// is bounded -- on expiry the caller records a fault code in the device's fault word (fault_word(), read back by
// bbcu_b200_device_fault()) and leaves the kernel.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace bb200 {

constexpr int kFaultBarrierTimeout = 1;
constexpr int kWaitSpins = 1 << 22;    // try_wait suspends in hardware for a while per attempt; this bounds a wait to seconds

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t arrivals)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
}

// makes the initialised barriers visible to the async proxy that will complete transactions on them
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void bulk_copy_g2s(void *smem_dst, const void *gmem_src, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_addr(smem_dst)), "l"(__cvta_generic_to_global(gmem_src)), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}

// Bounded wait: false when the phase did not complete within kWaitSpins attempts.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity)
{
    for (int i = 0; i < kWaitSpins; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// orders this thread's earlier generic-proxy accesses of shared memory before later async-proxy (bulk copy) accesses
__device__ __forceinline__ void proxy_fence_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

}   // namespace bb200
