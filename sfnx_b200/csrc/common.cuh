// Shared host-side helpers of the C-ABI launchers: error reporting and launch checks.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/sfnx_b200.h"

namespace fnxk {

// the calling thread's last error text (fnx_last_error)
char* err_buf();
int fail(const char* fmt, ...);
// cudaGetLastError after a launch: 0, or the failure recorded under `what`
int launch_ok(const char* what);
// kernels launched by this library so far (every launch is checked by one launch_ok()); reset: read and zero
long launch_count(bool reset);

inline cudaStream_t strm(void* st) { return (cudaStream_t) st; }

// ---- programmatic dependent launch.  A kernel launched through launch() may be scheduled while the kernel before
// it in the stream still runs: its blocks do what does not depend on that kernel (index arithmetic, the first loads
// of weights) and then call pdl_wait(), which returns once the kernel before has finished and its writes are visible.
// Rules every such kernel keeps: before pdl_wait() it reads nothing the kernel directly before it writes and writes
// no global memory; it calls pdl_go() only after pdl_wait(), so the kernel after it overlaps with this one and with
// nothing older.  Off (plain stream order) while a window is traced, since the trace times single kernels, and with
// FNX_NO_PDL set.
bool pdl_on(int kind);   // kind: a launch site's class, for FNX_PDL_MASK (a tuning knob: bit k switches class k)
void pdl_hold(bool hold);   // the trace's switch

template <typename... KArgs, typename... Args>
inline void launch(int kind, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at, cfg.numAttrs = pdl_on(kind) ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);   // a failure shows in launch_ok()
}

#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_go() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

#define FNX_REQUIRE(cond, ...) \
    do {                       \
        if (!(cond)) return fnxk::fail(__VA_ARGS__); \
    } while (0)

}  // namespace fnxk
