// Symmetric (peer-readable) embedding buffers without NVSHMEM.
//
// The reference allocates them from the NVSHMEM symmetric heap (nvshmem_malloc,
// src/mgg_np_div_mem.cu:139) and lets nvshmemx_float_get_warp translate (local address, pe) into a
// peer address.  Here a symmetric buffer is a plain device allocation; peers reach it either through
// CUDA peer access (one process driving several devices) or through a CUDA IPC mapping (one process
// per device), and the aggregation kernel receives the table of base pointers explicitly.
#include <cstring>
#include "common.h"

static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is exchanged as 64 opaque bytes");

extern "C" {

int mggb_sym_alloc(size_t bytes, void** dev_ptr) {
    MGGB_REQUIRE(dev_ptr, "sym_alloc: NULL output");
    MGGB_REQUIRE(bytes > 0, "sym_alloc: zero-size allocation");
    void* p = nullptr;
    MGGB_CUDA(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    if (e != cudaSuccess) {
        cudaFree(p);
        return mggb::fail(MGGB_ERR_CUDA, "sym_alloc: cudaMemset failed: %s", cudaGetErrorString(e));
    }
    *dev_ptr = p;
    return MGGB_OK;
}

int mggb_sym_free(void* dev_ptr) {
    if (!dev_ptr) return MGGB_OK;
    MGGB_CUDA(cudaFree(dev_ptr));
    return MGGB_OK;
}

int mggb_sym_export(void* dev_ptr, unsigned char handle_out[64]) {
    MGGB_REQUIRE(dev_ptr && handle_out, "sym_export: NULL argument");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, dev_ptr);
    if (e != cudaSuccess)
        return mggb::fail(MGGB_ERR_PEER, "sym_export: cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
    std::memcpy(handle_out, &h, 64);
    return MGGB_OK;
}

int mggb_sym_import(const unsigned char handle[64], void** peer_ptr) {
    MGGB_REQUIRE(handle && peer_ptr, "sym_import: NULL argument");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, 64);
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return mggb::fail(MGGB_ERR_PEER, "sym_import: cudaIpcOpenMemHandle failed: %s", cudaGetErrorString(e));
    }
    *peer_ptr = p;
    return MGGB_OK;
}

int mggb_sym_close(void* peer_ptr) {
    if (!peer_ptr) return MGGB_OK;
    cudaError_t e = cudaIpcCloseMemHandle(peer_ptr);
    if (e != cudaSuccess)
        return mggb::fail(MGGB_ERR_PEER, "sym_close: cudaIpcCloseMemHandle failed: %s", cudaGetErrorString(e));
    return MGGB_OK;
}

int mggb_enable_peer_access(int device, int peer_device) {
    if (device == peer_device) return MGGB_OK;
    int can = 0;
    MGGB_CUDA(cudaDeviceCanAccessPeer(&can, device, peer_device));
    if (!can)
        return mggb::fail(MGGB_ERR_PEER, "enable_peer_access: device %d cannot map device %d", device, peer_device);
    int prev = 0;
    MGGB_CUDA(cudaGetDevice(&prev));
    MGGB_CUDA(cudaSetDevice(device));
    cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    cudaSetDevice(prev);
    if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return MGGB_OK; }
    if (e != cudaSuccess)
        return mggb::fail(MGGB_ERR_PEER, "enable_peer_access(%d,%d): %s", device, peer_device, cudaGetErrorString(e));
    return MGGB_OK;
}

}  // extern "C"
