// Launchers shared between the expert kernels' translation units.
#pragma once

#include <cuda_runtime.h>

#include "../../include/sfnx_b200.h"
#include "common.cuh"

namespace fnxk {

// attn_umma.cu: the tcgen05 scan of fnx_attn_partial (head dimension 256); -1 when it does not apply
int attn_umma_launch(const float* qg, const uint16_t* kc, const uint16_t* vc, FnxKvPages g, float* scratch, int card, int ncard, int T,
                     const int* pos0, int nq, int nkv, int nsplit, cudaStream_t st);

// dense_umma.cu: the tcgen05 dense kernel (sums in block order) over 1..3 split-Q8_0 matrices; -1 when the shape is not its
int q8s_umma_launch(const FnxQ8S* w, const int* rows, float* const* out, const int* out_stride, int nseg, int cols, const void* yq, int T, cudaStream_t st,
                    const char* what);

// where a kernel with bounded on-chip waits reports a wait that ran out (bit 8): the window's error word while a window
// stage is being enqueued (fault_sink), else the library's own word, which fnx_device_fault() reads and clears
unsigned* device_fault_word();
void fault_sink(unsigned* err);

// shared memory past the default 48 KB has to be asked for, once per kernel
template <typename K> int smem_optin(K kernel, size_t bytes, const char* what) {
    if (bytes > 227 * 1024) return fail("%s: %zu bytes of shared memory exceed an SM's 227 KB", what, bytes);
    if (bytes > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) bytes);
        if (e != cudaSuccess) return fail("%s: shared memory opt-in: %s", what, cudaGetErrorString(e));
    }
    return 0;
}

#ifdef __CUDACC__
// The 6-bit scales and mins of sub-blocks 2 jg and 2 jg + 1 out of the 12 packed bytes (h.y, h.z, h.w), both at once
// as byte pairs: sub-blocks 0..3 have their scale in bytes 0..3 and their min in bytes 4..7 (low 6 bits); sub-blocks
// 4..7 have the low 4 bits in bytes 8..11 (scale: low nibble, min: high nibble) and the high 2 bits in the top of
// bytes 0..3 (scale) and 4..7 (min).
__device__ __forceinline__ void q4k_scale_min_pair(const uint4& h, int jg, float& sc0, float& m0, float& sc1, float& m1) {
    const int sh = 16 * (jg & 1);
    const unsigned y = h.y >> sh, z = h.z >> sh, w = h.w >> sh;
    const unsigned sc_lo = y & 0x3F3Fu, m_lo = z & 0x3F3Fu;
    const unsigned sc_hi = (w & 0x0F0Fu) | ((y >> 2) & 0x3030u), m_hi = ((w >> 4) & 0x0F0Fu) | ((z >> 2) & 0x3030u);
    const unsigned sc = jg & 2 ? sc_hi : sc_lo, m = jg & 2 ? m_hi : m_lo;
    sc0 = (float) (sc & 0xFFu), sc1 = (float) (sc >> 8);
    m0 = (float) (m & 0xFFu), m1 = (float) (m >> 8);
}
#endif

}  // namespace fnxk
