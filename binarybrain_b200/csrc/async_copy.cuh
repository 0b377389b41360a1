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

// Bounded wait, called by all 32 lanes of a warp together: false when the phase did not complete within kWaitSpins attempts.
// The outcome is made warp-uniform (a lane that saw the phase complete on its last attempt does not carry on alone while its
// neighbours give up).
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity)
{
    bool ok = false;
    for (int i = 0; i < kWaitSpins && !ok; ++i) ok = mbar_try_wait(bar, parity);
    return __all_sync(0xffffffffu, ok);
}

// orders this thread's earlier generic-proxy accesses of shared memory before later async-proxy (bulk copy) accesses
__device__ __forceinline__ void proxy_fence_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

}   // namespace bb200

// ---------------------------------------------------------------------------------------------------
// Per-thread 16-byte asynchronous copies (global -> shared, bypassing L1) with commit / wait groups.  A lane that copies only
// bytes it will read back itself needs no barrier: cp_async_wait<N>() makes its own groups (all but the N newest) visible to it.
// `valid` false writes 16 zero bytes without reading the source.
// ---------------------------------------------------------------------------------------------------
namespace bb200 {

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gmem_src, bool valid)
{
    const uint32_t src_bytes = valid ? 16u : 0u;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(smem_dst)), "l"(__cvta_generic_to_global(gmem_src)), "r"(src_bytes)
                 : "memory");
}

// The same copy with both addresses given as a base register plus a compile-time byte offset, so that a run of copies off one
// base costs no address arithmetic.  `smem_base` is a shared-window address (smem_addr), `gmem_base` a global-space address.
template <int SMEM_OFF, int GMEM_OFF>
__device__ __forceinline__ void cp_async16_at(uint32_t smem_base, uint64_t gmem_base)
{
    asm volatile("cp.async.cg.shared.global [%0+%2], [%1+%3], 16;" ::"r"(smem_base), "l"(gmem_base), "n"(SMEM_OFF), "n"(GMEM_OFF) : "memory");
}

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }

template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Vector reductions into global memory (resolved in L2): 16 / 8 bytes per lane, address aligned to the vector size.
__device__ __forceinline__ void red_add_v4(float *addr, float a, float b, float c, float d)
{
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(__cvta_generic_to_global(addr)), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__device__ __forceinline__ void red_add_v2(float *addr, float a, float b)
{
    asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(__cvta_generic_to_global(addr)), "f"(a), "f"(b) : "memory");
}

}   // namespace bb200
