// Launchers shared between the expert kernels' translation units.
#pragma once

#include <cuda_runtime.h>

#include "../../include/sfnx_b200.h"

namespace fnxk {

// TMA-staged persistent Q4_K gate|up (moe_tma.cu): shared memory it needs for n columns, and the launch
size_t gu_q4k_tma_smem(int n);
int gu_q4k_tma_launch(const uint8_t* A, size_t sa, int nrows, int n, const FnxJob* jobs, const int* njobs, const uint8_t* xq, float* gu,
                      cudaStream_t st);

// attn_umma.cu: the tcgen05 scan of fnx_attn_partial (head dimension 256); -1 when it does not apply
int attn_umma_launch(const float* qg, const uint16_t* kc, const uint16_t* vc, FnxKvPages g, float* scratch, int card, int ncard, int T,
                     const int* pos0, int nq, int nkv, int nsplit, cudaStream_t st);

// the device word fnx_device_fault() reads (bit 1: a bounded wait ran out), for kernels of other translation units
unsigned* device_fault_word();

}  // namespace fnxk
