// Bulk-copy (TMA) staging ring: one producer thread streams fixed-size slots of global memory into
// shared memory with cp.async.bulk; consumer warps wait on a slot's "full" mbarrier, read it with
// ordinary shared loads and hand it back through its "empty" mbarrier.  The bytes in flight are then
// set by the ring depth instead of by registers and occupancy, and memory latency never sits in a
// consumer warp's dependency chain.
//
// Rules kept here:
//  * plain one-destination bulk copies of this GPU's own memory into this CTA's shared memory, no
//    cluster launch;
//  * source address, destination address and size are multiples of 16 bytes;
//  * every wait is bounded: after kSpinLimit failed polls the waiter records an error in the
//    library's per-device error word (passed to the kernel) and gives up; kernels that synchronise
//    their consumers make the give-up a CTA-wide decision behind their row barrier, so nobody is left
//    waiting at a barrier for threads that have gone.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace rh {

namespace host {
// Device address of the sticky per-device error word (0 = none; otherwise (line << 8) | code of the
// first failure), resolved once per device.  rh_device_error() reads it.
int* device_error_word();
}  // namespace host

namespace pipe {

// A failed poll does not come back at once: try_wait suspends the thread in hardware until the phase
// completes or kSuspendNs have passed, so a waiting warp issues next to nothing while it waits and is
// woken the moment the copy lands.  kSpinLimit polls of up to kSuspendNs each bound a wait to ~1.3 s.
constexpr int kSpinLimit = 1 << 16;
constexpr uint32_t kSuspendNs = 20000;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(kSuspendNs)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (after recording the error) when the barrier never completed.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int where, int* error_word,
                                          int limit = kSpinLimit) {
    for (int i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    if (error_word != nullptr) atomicCAS(error_word, 0, (where << 8) | 1);
    return false;
}
// global -> shared bulk copy that reports its bytes to `bar`.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// Barrier among the first `count` threads of the CTA only (the producer warp does not take part).
__device__ __forceinline__ void consumer_sync(int count) {
    asm volatile("bar.sync 1, %0;" ::"r"(count) : "memory");
}

}  // namespace pipe
}  // namespace rh
