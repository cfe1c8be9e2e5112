// Device-side error reporting.  Every kernel takes `int* status`, a device int32[4]:
//   [0] error code (0 = none; the first error wins), [1] site (kernel id << 8 | site id),
//   [2], [3] two detail words (e.g. the offending index and its limit).
// Kernels never trap or assert: they record the error, skip the offending access and return.
#pragma once

#include <cuda_runtime.h>

enum MskStatus : int {
    MSK_OK = 0,
    MSK_ERR_TIMEOUT = 1,     // a bounded wait (mbarrier, cluster flag) expired
    MSK_ERR_BOUNDS = 2,      // a page id / cache row / expert id / token index was out of range
    MSK_ERR_CAPACITY = 3,    // a work list exceeded the capacity the kernel was built for
    // host-side return codes (negative) of the C ABI
    MSK_ERR_INVALID = -1,    // bad argument (shape, alignment, null pointer)
    MSK_ERR_CUDA = -2,       // a CUDA runtime / driver call failed
    MSK_ERR_UNSUPPORTED = -3 // shape outside what the kernels are built for
};

// kernel ids used in status[1]
enum MskKernelId : int {
    MSK_K_SELFTEST = 1,
    MSK_K_PROJ = 2,
    MSK_K_ATTN = 3,
    MSK_K_MOE1 = 4,
    MSK_K_MOE2 = 5,
    MSK_K_COMBINE = 6,
    MSK_K_GLUE = 7,
    MSK_K_EP = 8
};

namespace msk {

__device__ __forceinline__ void report(int* status, int code, int where, int a = 0, int b = 0) {
    if (status != nullptr && atomicCAS(status, 0, code) == 0) {
        status[1] = where;
        status[2] = a;
        status[3] = b;
    }
}

}  // namespace msk
