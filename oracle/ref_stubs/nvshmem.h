/* Parse-only stand-in for <nvshmem.h>.
 *
 * The reference's headers include NVSHMEM because their GPU kernels fetch remote rows with it.
 * The oracle build links none of those kernels' callers: it only calls the reference's HOST
 * functions (SAG_ref, split_CSR, build_part).  These empty declarations let the unmodified
 * reference headers compile without the NVSHMEM runtime; nothing here is ever executed.
 * Test infrastructure only. */
#ifndef MGGB_ORACLE_NVSHMEM_STUB_H
#define MGGB_ORACLE_NVSHMEM_STUB_H
#include <cstddef>
static inline void* nvshmem_malloc(size_t) { return nullptr; }
static inline void nvshmem_free(void*) {}
__device__ inline void nvshmem_float_get(float*, const float*, size_t, int) {}
__device__ inline void nvshmem_quiet() {}
#endif
