/* Parse-only stand-in for <nvshmemx.h>; see nvshmem.h beside it.  Never executed. */
#ifndef MGGB_ORACLE_NVSHMEMX_STUB_H
#define MGGB_ORACLE_NVSHMEMX_STUB_H
#include <cstddef>
__device__ inline void nvshmemx_float_get_warp(float*, const float*, size_t, int) {}
__device__ inline void nvshmemx_float_get_block(float*, const float*, size_t, int) {}
__device__ inline void nvshmemx_float_get_nbi_warp(float*, const float*, size_t, int) {}
__device__ inline void nvshmemx_getmem_nbi_warp(void*, const void*, size_t, int) {}
#endif
