// mgg_compat.hpp - the reference's C++ names on top of the C ABI (header-only).
//
// A driver written against the reference's headers calls free functions and pokes public struct
// fields; this header restores those names, parameter lists and side effects so that such a
// `main()` can switch over by changing its includes:
//
//   split_CSR<T>, build_part<T>            include/neighbor_utils.cuh:381-460
//   mgg_SAG_np_div, mgg_GIN_np_div         include/neighbor_utils.cuh:787-841, :902-958
//   dense_param_new_beg / _hidden          include/layer_new.cuh:272-393
//   softmax_new_param                      include/layer_new.cuh:59-103
//   dense_beg_new_forward, dense_hidden_new_forward, softmax_new_forward   include/gnn_layer.cuh:36-52
//   dense_param_beg / dense_param_hidden / softmax_param (the older structs, which OWN their output
//       buffer; the dense ones own a SYMMETRIC one)                        include/layer_new.cuh:13-55, 210-269, 396-451
//   dense_beg_forward, dense_hidden_forward, softmax_forward               include/gnn_layer.cuh:15-32
//   mgg_symmetric_malloc                   stands in for nvshmem_malloc (src/mgg_np_div_mem.cu:139)
//
// Behaviour kept from the reference: the aggregation ADDS into `output`; both launchers synchronise
// the device and exit(-1) with a message on a CUDA error (include/neighbor_utils.cuh:835-840);
// build_part prints its one summary line (:457-458); dense weights are filled with 1.0
// (include/layer_new.cuh:307).  Behaviour changed on purpose: the dense forward multiplies d_in by d_W
// (the reference's call multiplies d_out in place and never reads d_in).
//
// Symmetric memory: the reference passes a local symmetric-heap address and NVSHMEM finds the peer's
// copy.  Here the process registers, per device, the table of all PEs' base pointers for a symmetric
// buffer (mgg_register_symmetric); mgg_SAG_np_div looks its `input` argument up in that registry and
// falls back to a one-PE table when it is not registered.
// nvshmem_malloc is a collective: every PE calls it in the same order and the k-th call of each PE
// names one symmetric buffer.  A program that drives several PEs from one process gets the same rule
// from mgg_set_pe(pe, num_pes) + mgg_symmetric_malloc: the k-th allocation made while PE p is current
// is PE p's part of symmetric buffer k, and as soon as all num_pes parts of a buffer exist their table
// is registered for every one of them.  The older dense structs allocate their d_out this way, so a
// driver that builds `new dense_param_beg(...)` once per PE needs no further call.
#pragma once

#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "mggb200.h"

using nidType = int;

#define MGG_COMPAT_CHECK(call)                                                         \
    do {                                                                               \
        int st__ = (call);                                                             \
        if (st__ != MGGB_OK) {                                                         \
            printf("MGG error @%s: %s\n", #call, mggb_last_error());                   \
            exit(-1);                                                                  \
        }                                                                              \
    } while (0)

// ---- partitioner -------------------------------------------------------------------------------

template <typename T>
std::vector<std::vector<T>> split_CSR(std::vector<T>& origin_ptr, std::vector<T>& origin_col_idx, T lb, T ub) {
    static_assert(sizeof(T) == 4, "split_CSR is provided for 32-bit ids (the reference's nidType)");
    int64_t nl = 0, nr = 0;
    const int32_t* ptr = reinterpret_cast<const int32_t*>(origin_ptr.data());
    const int32_t* col = reinterpret_cast<const int32_t*>(origin_col_idx.data());
    MGG_COMPAT_CHECK(mggb_split_csr_count(ptr, col, (int32_t)lb, (int32_t)ub, &nl, &nr));
    std::vector<T> local_ptr(ub - lb + 1), remote_ptr(ub - lb + 1), local_col(nl), remote_col(nr);
    MGG_COMPAT_CHECK(mggb_split_csr_fill(ptr, col, (int32_t)lb, (int32_t)ub,
                                         reinterpret_cast<int32_t*>(local_ptr.data()), reinterpret_cast<int32_t*>(remote_ptr.data()),
                                         reinterpret_cast<int32_t*>(local_col.data()), reinterpret_cast<int32_t*>(remote_col.data())));
    return {local_ptr, remote_ptr, local_col, remote_col};
}

template <typename T>
std::vector<std::vector<T>> build_part(std::string name, std::vector<T>& indptr, T num_nodes, T partSize) {
    static_assert(sizeof(T) == 4, "build_part is provided for 32-bit ids (the reference's nidType)");
    int64_t parts = 0;
    const int32_t* ptr = reinterpret_cast<const int32_t*>(indptr.data());
    MGG_COMPAT_CHECK(mggb_build_part_count(ptr, (int32_t)num_nodes, (int32_t)partSize, &parts));
    std::vector<T> partPtr(parts + 1), part2Node(parts), node2Part(num_nodes + 2);
    MGG_COMPAT_CHECK(mggb_build_part_fill(ptr, (int32_t)num_nodes, (int32_t)partSize, /*exact_sentinel=*/0,
                                          reinterpret_cast<int32_t*>(partPtr.data()), reinterpret_cast<int32_t*>(part2Node.data()),
                                          reinterpret_cast<int32_t*>(node2Part.data())));
    printf("%s, num_nodes: %d, part_size, %d, num_parts, %d\n", name.c_str(), (int)num_nodes, (int)partSize, (int)parts);
    return {partPtr, part2Node, node2Part};
}

// ---- symmetric buffers ----------------------------------------------------------------------------

namespace mgg_compat {

struct SymEntry { std::vector<const float*> table; };

inline std::map<const void*, SymEntry>& registry() { static std::map<const void*, SymEntry> r; return r; }
inline std::mutex& registry_mutex() { static std::mutex m; return m; }

inline bool lookup(const float* local, std::vector<const float*>& table) {
    std::lock_guard<std::mutex> g(registry_mutex());
    auto it = registry().find(local);
    if (it == registry().end()) return false;
    table = it->second.table;
    return true;
}

}  // namespace mgg_compat

// Declares that `local` (this PE's buffer) is the entry `pe` of the given table of all PEs' buffers.
inline void mgg_register_symmetric(const float* local, const float* const* table, int num_pes) {
    std::lock_guard<std::mutex> g(mgg_compat::registry_mutex());
    mgg_compat::registry()[local] = mgg_compat::SymEntry{std::vector<const float*>(table, table + num_pes)};
}

namespace mgg_compat {
// The emulated symmetric heap of a one-process, several-PE program (see the header comment).
struct Heap {
    int pe = 0, num_pes = 1;
    std::vector<std::vector<float*>> parts;   // parts[k][p] = PE p's part of symmetric buffer k (nullptr until allocated)
    std::vector<int> next;                    // next[p] = index of PE p's next allocation
};
inline Heap& heap() { static Heap h; return h; }
}  // namespace mgg_compat

// Makes `pe` (of `num_pes`) the PE on whose behalf the following mgg_symmetric_malloc calls are made.
// The caller selects the PE's device itself (cudaSetDevice), as the reference's drivers do.
inline void mgg_set_pe(int pe, int num_pes) {
    auto& h = mgg_compat::heap();
    if (num_pes < 1 || num_pes > MGGB_MAX_PES || pe < 0 || pe >= num_pes) { printf("mgg_set_pe: bad pe %d of %d\n", pe, num_pes); exit(-1); }
    if (h.num_pes != num_pes) { h.parts.clear(); h.next.assign(num_pes, 0); }
    if ((int)h.next.size() != num_pes) h.next.assign(num_pes, 0);
    h.pe = pe; h.num_pes = num_pes;
}

// Allocates a zero-filled symmetric buffer on the current device for the current PE (mgg_set_pe; one
// PE by default).  Stands in for nvshmem_malloc.
inline void* mgg_symmetric_malloc(size_t bytes) {
    void* p = nullptr;
    MGG_COMPAT_CHECK(mggb_sym_alloc(bytes, &p));
    auto& h = mgg_compat::heap();
    if ((int)h.next.size() != h.num_pes) h.next.assign(h.num_pes, 0);
    const int k = h.next[h.pe]++;
    if ((int)h.parts.size() <= k) h.parts.resize(k + 1, std::vector<float*>(h.num_pes, nullptr));
    h.parts[k][h.pe] = (float*)p;
    bool complete = true;
    for (float* q : h.parts[k]) complete = complete && q != nullptr;
    if (complete) {
        std::vector<const float*> table(h.parts[k].begin(), h.parts[k].end());
        for (float* q : h.parts[k]) mgg_register_symmetric(q, table.data(), h.num_pes);
    }
    return p;
}

// ---- aggregation ----------------------------------------------------------------------------------

inline void mgg_SAG_np_div(float* output, const float* input, const nidType* row_pointers_l,
                           const nidType* column_index_l, const nidType* row_pointers_r,
                           const nidType* column_index_r, const nidType lb, const nidType ub, const int dim,
                           const int nodePerPE, const int peid, const int np_size, const int warpPerBlock,
                           const int interleaved_dist) {
    std::vector<const float*> table;
    int pe = peid;
    if (!mgg_compat::lookup(input, table)) { table = {input}; pe = 0; }
    int st = mggb_sag_np_div(output, table.data(), (int)table.size(), row_pointers_l, column_index_l, row_pointers_r,
                             column_index_r, lb, ub, dim, nodePerPE, pe, np_size, warpPerBlock, interleaved_dist,
                             nullptr, MGGB_AGG_ACCUMULATE, nullptr, 0, nullptr);
    cudaError_t error = (st == MGGB_OK) ? cudaDeviceSynchronize() : cudaSuccess;
    if (st != MGGB_OK || error != cudaSuccess) {
        printf("CUDA error @mgg_SAG_np_div_cuda: %s\n", st != MGGB_OK ? mggb_last_error() : cudaGetErrorString(error));
        exit(-1);
    }
}

inline void mgg_GIN_np_div(float* output, const float* input, const nidType* row_pointers_l,
                           const nidType* column_index_l, const nidType* row_pointers_r,
                           const nidType* column_index_r, const nidType lb, const nidType ub, const int dim,
                           const int nodePerPE, const int peid, const int np_size, const int warpPerBlock,
                           const int interleaved_dist, const float eps) {
    std::vector<const float*> table;
    int pe = peid;
    if (!mgg_compat::lookup(input, table)) { table = {input}; pe = 0; }
    int st = mggb_gin_np_div(output, table.data(), (int)table.size(), row_pointers_l, column_index_l, row_pointers_r,
                             column_index_r, lb, ub, dim, nodePerPE, pe, np_size, warpPerBlock, interleaved_dist, eps,
                             0, nullptr);
    cudaError_t error = (st == MGGB_OK) ? cudaDeviceSynchronize() : cudaSuccess;
    if (st != MGGB_OK || error != cudaSuccess) {
        printf("CUDA error @mgg_GIN_np_div_cuda: %s\n", st != MGGB_OK ? mggb_last_error() : cudaGetErrorString(error));
        exit(-1);
    }
}

// ---- dense / softmax parameter structs --------------------------------------------------------------

class mgg_dense_param_base {
public:
    mgg_dense_param_base(const char* name_in, float* d_in_ext, float* d_out_ext, int numNodes_in, int dim1_in, int dim2_in) {
        strncpy(name, name_in, 7);
        name[7] = '\0';
        numNodes = numNodes_in; dim1 = dim1_in; dim2 = dim2_in;
        m = dim2; n = numNodes; k = dim1;
        ldx = dim1; ldw = dim2; ldout = dim2;
        alpha = 1.0f; beta = 0.0f;
        d_in = d_in_ext; d_out = d_out_ext;
        h_W = (float*)malloc(sizeof(float) * dim1 * dim2);
        for (int i = 0; i < dim1 * dim2; i++) h_W[i] = 1.0f;
        if (cudaMalloc((void**)&d_W, sizeof(float) * dim1 * dim2) != cudaSuccess ||
            cudaMemcpy(d_W, h_W, sizeof(float) * dim1 * dim2, cudaMemcpyHostToDevice) != cudaSuccess) {
            printf("CUDA error @dense_param: cannot allocate the %dx%d weight\n", dim1, dim2);
            exit(-1);
        }
    }
    ~mgg_dense_param_base() { free(h_W); cudaFree(d_W); }
    mgg_dense_param_base(const mgg_dense_param_base&) = delete;
    mgg_dense_param_base& operator=(const mgg_dense_param_base&) = delete;

    // Uploads dim1*dim2 row-major weights (the reference only ever uses the all-ones fill).
    void set_weight(const float* host_w) {
        memcpy(h_W, host_w, sizeof(float) * dim1 * dim2);
        cudaMemcpy(d_W, h_W, sizeof(float) * dim1 * dim2, cudaMemcpyHostToDevice);
    }

    int m, n, k, ldx, ldw, ldout;
    int numNodes, dim1, dim2;
    float *h_W = nullptr, *d_W = nullptr, *d_out = nullptr, *d_in = nullptr;
    float alpha, beta;
    char name[8];
};

class dense_param_new_beg : public mgg_dense_param_base { public: using mgg_dense_param_base::mgg_dense_param_base; };
class dense_param_new_hidden : public mgg_dense_param_base { public: using mgg_dense_param_base::mgg_dense_param_base; };

class softmax_new_param {
public:
    softmax_new_param(const char* name_in, float* d_in_input, float* d_out_ext, int numNodes_in, int dim_in) {
        strncpy(name, name_in, 7);
        name[7] = '\0';
        numNodes = numNodes_in; dim = dim_in; d_in = d_in_input; d_out = d_out_ext;
        alpha = 1.0f; beta = 0.0f;
    }
    int numNodes, dim;
    float *d_out, *d_in;
    float alpha, beta;
    char name[8];
};

inline void dense_beg_new_forward(dense_param_new_beg* dp, cudaStream_t stream = nullptr) {
    MGG_COMPAT_CHECK(mggb_dense_forward(dp->d_out, dp->d_in, dp->d_W, dp->numNodes, dp->dim1, dp->dim2, nullptr, 0, nullptr, 0, stream));
}
inline void dense_hidden_new_forward(dense_param_new_hidden* dp, cudaStream_t stream = nullptr) {
    MGG_COMPAT_CHECK(mggb_dense_forward(dp->d_out, dp->d_in, dp->d_W, dp->numNodes, dp->dim1, dp->dim2, nullptr, 0, nullptr, 0, stream));
}
inline void softmax_new_forward(softmax_new_param* smx, cudaStream_t stream = nullptr) {
    MGG_COMPAT_CHECK(mggb_softmax_forward(smx->d_out, smx->d_in, smx->numNodes, smx->dim, stream));
}
// dense_hidden_new_forward(dp); softmax_new_forward(smx); (src/mgg_np_div_mem.cu:220-226) as one kernel that
// also stores the logits in dp->d_out; falls back to the two calls for shapes the fused kernel refuses.
inline void dense_hidden_softmax_new_forward(dense_param_new_hidden* dp, softmax_new_param* smx, cudaStream_t stream = nullptr) {
    if (smx->d_in == dp->d_out && smx->numNodes == dp->numNodes && smx->dim == dp->dim2 &&
        mggb_dense_softmax_forward(smx->d_out, dp->d_out, dp->d_in, dp->d_W, dp->numNodes, dp->dim1, dp->dim2, stream) == MGGB_OK)
        return;
    dense_hidden_new_forward(dp, stream);
    softmax_new_forward(smx, stream);
}

// ---- the older structs and forwards (src/mgg_np_div_kernel.cu:127, src/mgg_np_div.cu:130-132) -------------
// They differ from the _new ones in who owns the output: dense_param_beg / dense_param_hidden take only
// their input and allocate d_out themselves, in symmetric memory (include/layer_new.cuh:250-252, :436),
// zero-filled; softmax_param allocates a private d_out (:40-43).

class dense_param_beg : public mgg_dense_param_base {
public:
    dense_param_beg(const char* name_in, float* d_in_ext, int numNodes_in, int dim1_in, int dim2_in)
        : mgg_dense_param_base(name_in, d_in_ext, (float*)mgg_symmetric_malloc(sizeof(float) * (size_t)numNodes_in * dim2_in),
                               numNodes_in, dim1_in, dim2_in) {}
};

class dense_param_hidden : public mgg_dense_param_base {
public:
    dense_param_hidden(const char* name_in, float* d_in_input, int numNodes_in, int dim1_in, int dim2_in)
        : mgg_dense_param_base(name_in, d_in_input, (float*)mgg_symmetric_malloc(sizeof(float) * (size_t)numNodes_in * dim2_in),
                               numNodes_in, dim1_in, dim2_in) {}
};

class softmax_param {
public:
    softmax_param(const char* name_in, float* d_in_input, int numNodes_in, int dim_in) {
        strncpy(name, name_in, 7);
        name[7] = '\0';
        numNodes = numNodes_in; dim = dim_in; d_in = d_in_input;
        alpha = 1.0f; beta = 0.0f;
        if (cudaMalloc((void**)&d_out, sizeof(float) * (size_t)numNodes * dim) != cudaSuccess ||
            cudaMemset(d_out, 0, sizeof(float) * (size_t)numNodes * dim) != cudaSuccess) {
            printf("CUDA error @softmax_param: cannot allocate the %dx%d output\n", numNodes, dim);
            exit(-1);
        }
    }
    ~softmax_param() { cudaFree(d_out); }
    softmax_param(const softmax_param&) = delete;
    softmax_param& operator=(const softmax_param&) = delete;
    int numNodes, dim;
    float *d_out = nullptr, *d_in = nullptr;
    float alpha, beta;
    char name[8];
};

// d_out = d_in * d_W (the reference's calls, include/gnn_layer.cuh:22-32, multiply d_out in place and
// never read d_in).  softmax_forward synchronises the device like the reference's (:19).
inline void dense_beg_forward(dense_param_beg* dp, cudaStream_t stream = nullptr) {
    MGG_COMPAT_CHECK(mggb_dense_forward(dp->d_out, dp->d_in, dp->d_W, dp->numNodes, dp->dim1, dp->dim2, nullptr, 0, nullptr, 0, stream));
}
inline void dense_hidden_forward(dense_param_hidden* dp, cudaStream_t stream = nullptr) {
    MGG_COMPAT_CHECK(mggb_dense_forward(dp->d_out, dp->d_in, dp->d_W, dp->numNodes, dp->dim1, dp->dim2, nullptr, 0, nullptr, 0, stream));
}
inline void softmax_forward(softmax_param* smx, cudaStream_t stream = nullptr) {
    MGG_COMPAT_CHECK(mggb_softmax_forward(smx->d_out, smx->d_in, smx->numNodes, smx->dim, stream));
    cudaDeviceSynchronize();
}
