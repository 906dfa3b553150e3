// tcgen05 (fifth-generation tensor cores) plumbing shared by the kernels that issue tcgen05.mma: shared-memory operand
// descriptors, the kind::f16 MMA with operands in shared memory and the accumulator in tensor memory, and a bounded
// mbarrier wait.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

namespace fnxk {

__device__ __forceinline__ unsigned um_s32(const void* p) { return (unsigned) __cvta_generic_to_shared(p); }

// A shared-memory operand descriptor: start address, leading and stride byte offsets (all in 16-byte units), version 1,
// swizzle (2: 128 bytes, 4: 64 bytes).
__device__ __forceinline__ unsigned long long um_desc_x(unsigned addr, unsigned lbo, unsigned sbo, unsigned layout) {
    return (unsigned long long) ((addr & 0x3FFFF) >> 4) | ((unsigned long long) (lbo >> 4) << 16) | ((unsigned long long) (sbo >> 4) << 32) | (1ull << 46) |
           ((unsigned long long) layout << 61);
}
// K-major operand tile with the 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart
__device__ __forceinline__ unsigned long long um_desc(unsigned addr) { return um_desc_x(addr, 16, 1024, 2); }

// D[tmem] (+)= A B, M x N x 16, f16 operands through descriptors da / db, fp32 accumulator; issued by one thread
__device__ __forceinline__ void um_mma(unsigned tmem, unsigned long long da, unsigned long long db, unsigned idesc, unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem), "l"(da),
                 "l"(db), "r"(idesc), "r"(accumulate)
                 : "memory");
}

// Waits for the phase of `bar` with this parity; gives up after 2^22 polls, sets bit 8 of *fault and returns false (the
// caller goes on with what it has: no wait in these kernels is unbounded).
__device__ __forceinline__ bool um_wait(unsigned long long* bar, unsigned parity, unsigned* fault) {
    unsigned ok = 0;
    for (int spin = 0; spin < (1 << 22) && !ok; ++spin)
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok)
                     : "r"(um_s32(bar)), "r"(parity)
                     : "memory");
    if (!ok) atomicOr(fault, 8u);
    return ok != 0;
}

// ---- the TMA unit: plain loads of this GPU's own memory (no multicast), completion as bytes on an mbarrier
__device__ __forceinline__ void um_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(um_s32(bar)), "r"(bytes) : "memory");
}
// a box of a 2-D tensor map at element x (x times the element size a multiple of 16 bytes), row y
__device__ __forceinline__ void um_tma2d(unsigned dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst), "l"(map),
                 "r"(x), "r"(y), "r"(um_s32(bar))
                 : "memory");
}
// a contiguous run of bytes (both addresses and the size multiples of 16)
__device__ __forceinline__ void um_bulk(unsigned dst, const void* src, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes),
                 "r"(um_s32(bar))
                 : "memory");
}

// the driver's tensor-map encoder, looked up once (no link against the driver library); null when it is not there
typedef CUresult (*UmEncode)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                             CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline UmEncode um_encoder() {
    static UmEncode fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess && qr == cudaDriverEntryPointSuccess) fn = (UmEncode) p;
    }
    return fn;
}

}  // namespace fnxk
