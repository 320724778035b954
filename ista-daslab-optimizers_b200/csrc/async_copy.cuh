// Asynchronous global -> shared copies for sm_100a: the 1-D bulk copy engine (TMA) completing
// on an mbarrier, and 4-byte cp.async for small ragged pieces.  Every wait is bounded.
#pragma once
#include "common.cuh"

namespace mab {

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// One arrival that also announces `bytes` of bulk-copy traffic.
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}

// Bulk copy of `bytes` (multiple of 16; both addresses 16-byte aligned) global -> shared, completing on `bar`.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_addr(dst_smem)), "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}

// Waits for the phase with the given parity; gives up after `limit` probes (each probe itself waits
// up to a hardware time limit) and returns false, so that no launch can spin for ever.
constexpr int MBAR_WAIT_PROBES = 1 << 20;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int limit = MBAR_WAIT_PROBES) {
    const uint32_t a = smem_addr(bar);
    for (int it = 0; it < limit; ++it) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(a), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}

// Bulk copy shared -> global (`bytes` a multiple of 16, both addresses 16-byte aligned) as one
// bulk group of the calling thread.  Shared memory written by ordinary stores must be made visible
// to the copy engine first (fence_async_smem by the writers, then a barrier).
__device__ __forceinline__ void bulk_s2g(void* dst_gmem, const void* src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst_gmem), "r"(smem_addr(src_smem)), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// The calling thread's bulk stores have finished reading shared memory / have completed.
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Orders this thread's ordinary shared-memory accesses before later copy-engine accesses.
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Asks L2 for the 128-byte lines of [base, base + bytes), the block's NT threads sharing the lines.
template <int NT>
__device__ __forceinline__ void prefetch_l2(uintptr_t base, int64_t bytes) {
    const uintptr_t first = base & ~(uintptr_t)127;
    const int lines = (int)((base + bytes - first + 127) >> 7);
    for (int i = threadIdx.x; i < lines; i += NT)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(first + ((uintptr_t)i << 7)));
}

__device__ __forceinline__ void cp_async_4(void* dst_smem, const void* src_gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_addr(dst_smem)), "l"(src_gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

}  // namespace mab
