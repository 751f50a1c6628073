// Shared helpers of the library's translation units: status codes, the per-thread error message
// and the CUDA-call check.  Nothing here crosses the C ABI.
#pragma once
#include <cstdarg>
#include <cstdio>
#include <cstdint>
#include "../../include/mggb200.h"

namespace mggb {

// Stores a printf-style message for mggb_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);
void clear_error();

}  // namespace mggb

#define MGGB_REQUIRE(cond, ...)                                            \
    do {                                                                   \
        if (!(cond)) return mggb::fail(MGGB_ERR_INVALID_ARG, __VA_ARGS__); \
    } while (0)

#ifdef __CUDACC__
#include <cuda_runtime.h>
#define MGGB_CUDA(call)                                                                   \
    do {                                                                                  \
        cudaError_t e__ = (call);                                                         \
        if (e__ != cudaSuccess)                                                           \
            return mggb::fail(MGGB_ERR_CUDA, "%s failed: %s (%s:%d)", #call,              \
                              cudaGetErrorString(e__), __FILE__, __LINE__);               \
    } while (0)

namespace mggb {
// Internal flag of dense_tc() (never part of the public MGGB_DENSE_* set): the epilogue stores the softmax of every
// output row instead of the row.  Used by mggb_dense_softmax_forward for shapes the tensor-core kernel takes.
constexpr int DENSE_TC_SOFTMAX = 1 << 20;

// Multiprocessors of the current device (asked once per device; 1 if the query fails, which only
// makes a grid smaller).  Grids are sized from this, never from a typed-in count.
inline int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) return 1;
        cached[dev] = n;
    }
    return cached[dev];
}
}  // namespace mggb
#endif
