// Launchers shared between the expert kernels' translation units.
#pragma once

#include <cuda_runtime.h>

#include "../../include/sfnx_b200.h"

namespace fnxk {

// TMA-staged persistent Q4_K gate|up (moe_tma.cu): shared memory it needs for n columns, and the launch
size_t gu_q4k_tma_smem(int n);
int gu_q4k_tma_launch(const uint8_t* A, size_t sa, int nrows, int n, const FnxJob* jobs, const int* njobs, const uint8_t* xq, float* gu,
                      cudaStream_t st);

}  // namespace fnxk
