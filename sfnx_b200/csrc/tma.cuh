// Bulk asynchronous copies (the TMA unit's untiled form, cp.async.bulk) into shared memory with mbarrier completion,
// for kernels that stream contiguous weight panels.  Both addresses must be 16-byte aligned and the size a multiple of
// 16 bytes.  Every wait is bounded: after the limit the kernel records a fault bit and carries on, it never spins for
// ever.
#pragma once

#include <stdint.h>

namespace fnxk {

// device-side fault word of the translation unit that includes this header: bit 1 = a bulk copy never completed
// (read and cleared through fnx_device_fault)
static __device__ unsigned g_fault = 0;

__device__ __forceinline__ unsigned sm_addr(const void* p) { return (unsigned) __cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(sm_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
// one arrival that also announces `bytes` of copies to come
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(sm_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, unsigned bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(sm_addr(dst)), "l"(src),
                 "r"(bytes), "r"(sm_addr(bar))
                 : "memory");
}
// waits for the phase of the given parity to complete; false after the limit
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity) {
    for (int spin = 0; spin < (1 << 22); ++spin) {
        unsigned ok;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(ok)
            : "r"(sm_addr(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    atomicOr(&g_fault, 1u);
    return false;
}

}  // namespace fnxk
