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

inline cudaStream_t strm(void* st) { return (cudaStream_t) st; }

#define FNX_REQUIRE(cond, ...) \
    do {                       \
        if (!(cond)) return fnxk::fail(__VA_ARGS__); \
    } while (0)

}  // namespace fnxk
