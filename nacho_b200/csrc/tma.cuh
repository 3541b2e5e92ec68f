// Thin wrappers over the sm_90+/sm_100a asynchronous-copy PTX used by the tile kernels:
// one-dimensional bulk copies between global and shared memory (the TMA engine's untiled
// form, cp.async.bulk), the shared-memory mbarrier they complete on, and the proxy fence that
// orders ordinary shared-memory writes before an engine read. No multicast form is used
// anywhere: every copy has exactly one destination CTA, the one that issued it.
//
// Both addresses of a bulk copy must be 16-byte aligned and the size a multiple of 16 bytes.
#pragma once

#include <stdint.h>

namespace nb200 {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, int arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(arrivals) : "memory");
}

// Makes a freshly initialised mbarrier visible to the asynchronous proxy (the copy engine).
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// One arrival that also announces `bytes` of copy traffic the barrier must see before the
// current phase completes.
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// Waits for phase `parity` of `bar`, giving up after `limit` polls. Returns false on give-up.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, int limit) {
    for (int i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    return false;
}

// global -> shared, completion counted in bytes on `bar`.
__device__ __forceinline__ void bulk_load(void *smem_dst, const void *gmem_src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// shared -> global, tracked by the issuing thread's bulk group.
__device__ __forceinline__ void bulk_store(void *gmem_dst, const void *smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_u32(smem_src)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

// Blocks the issuing thread until the engine has finished READING shared memory for all of
// its committed bulk stores (the data may still be on its way to global memory).
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

// Orders this thread's earlier ordinary shared-memory writes before later copy-engine reads.
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

}  // namespace nb200
