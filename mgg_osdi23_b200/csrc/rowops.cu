// Row-wise helpers around the aggregation: softmax over classes, row scaling, 1/sqrt(degree).
#include <algorithm>
#include <cfloat>
#include <cstdint>
#include "common.h"

namespace {

// One warp per row.  Stands in for cudnnSoftmaxForward(ACCURATE, MODE_CHANNEL) on an [N, C, 1, 1]
// tensor (include/gnn_layer.cuh:36-38, include/layer_new.cuh:80-85): max-subtracted exp / sum.
__global__ void softmax_rows_kernel(float* __restrict__ out, const float* __restrict__ in, long long n, int dim) {
    const int lane = threadIdx.x & 31;
    const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < n; row += warps) {
        const float* r = in + row * dim;
        float m = -FLT_MAX;
        for (int c = lane; c < dim; c += 32) m = fmaxf(m, r[c]);
        for (int off = 16; off; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
        float s = 0.f;
        for (int c = lane; c < dim; c += 32) s += expf(r[c] - m);
        for (int off = 16; off; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        const float inv = 1.f / s;
        for (int c = lane; c < dim; c += 32) out[row * dim + c] = expf(r[c] - m) * inv;
    }
}

__global__ void row_scale_kernel(float* __restrict__ out, const float* __restrict__ in,
                                 const float* __restrict__ scale, long long total, int dim) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride)
        out[i] = in[i] * scale[i / dim];
}

__global__ void inv_sqrt_degree_kernel(float* __restrict__ scale, const int32_t* __restrict__ rp_l,
                                       const int32_t* __restrict__ rp_r, long long n) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        int deg = rp_l[i + 1] - rp_l[i];
        if (rp_r) deg += rp_r[i + 1] - rp_r[i];
        scale[i] = deg > 0 ? rsqrtf((float)deg) : 0.f;
    }
}

// Destinations of a publishing copy (the peers' replicas).
struct PublishTable {
    float* dst[MGGB_MAX_PES];
    int n;
};

// in[0, count) -> every destination, 16 bytes per thread per step, consecutive threads on consecutive
// addresses: a peer receives whole 512-byte runs per warp instead of one row per store.
template <typename T>
__global__ void __launch_bounds__(256) publish_copy_kernel(const T* __restrict__ in, long long count, const PublishTable pub) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        const T v = in[i];
        for (int q = 0; q < pub.n; q++) reinterpret_cast<T*>(pub.dst[q])[i] = v;
    }
}

int grid_for(long long work_items, int block) {
    long long g = (work_items + block - 1) / block;
    const long long cap = 16LL * mggb::sm_count();
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

extern "C" {

int mggb_publish_rows(const float* in, int64_t count, float* const* publish_out, int num_publish, void* stream) {
    MGGB_REQUIRE(num_publish >= 0 && num_publish <= MGGB_MAX_PES && (num_publish == 0 || publish_out),
                 "publish_rows: num_publish must be in [0,%d] with a non-NULL table (got %d)", MGGB_MAX_PES, num_publish);
    MGGB_REQUIRE(count >= 0 && (count == 0 || in), "publish_rows: need count >= 0 and a non-NULL source");
    if (count == 0 || num_publish == 0) return MGGB_OK;
    PublishTable pub{};
    pub.n = num_publish;
    bool wide = ((uintptr_t)in % 16 == 0) && (count % 4 == 0);
    for (int q = 0; q < num_publish; q++) {
        MGGB_REQUIRE(publish_out[q] != nullptr && publish_out[q] != in, "publish_rows: publish_out[%d] is NULL or the source itself", q);
        pub.dst[q] = publish_out[q];
        wide = wide && ((uintptr_t)publish_out[q] % 16 == 0);
    }
    // One block per SM at most: enough stores in flight for the links, and room left on every SM for a
    // kernel that runs beside this one on another stream.
    const int sms = mggb::sm_count();
    if (wide)
        publish_copy_kernel<float4><<<std::min(grid_for(count / 4, 256), sms), 256, 0, (cudaStream_t)stream>>>(
            reinterpret_cast<const float4*>(in), count / 4, pub);
    else
        publish_copy_kernel<float><<<std::min(grid_for(count, 256), sms), 256, 0, (cudaStream_t)stream>>>(in, count, pub);
    MGGB_CUDA(cudaGetLastError());
    return MGGB_OK;
}

int mggb_softmax_forward(float* out, const float* in, int64_t n, int dim, void* stream) {
    MGGB_REQUIRE(out && in, "softmax_forward: NULL argument");
    MGGB_REQUIRE(n >= 0 && dim >= 1, "softmax_forward: need n >= 0 and dim >= 1 (n=%lld dim=%d)", (long long)n, dim);
    if (n == 0) return MGGB_OK;
    softmax_rows_kernel<<<grid_for(n * 32, 256), 256, 0, (cudaStream_t)stream>>>(out, in, n, dim);
    MGGB_CUDA(cudaGetLastError());
    return MGGB_OK;
}

int mggb_row_scale(float* out, const float* in, const float* scale, int64_t n, int dim, void* stream) {
    MGGB_REQUIRE(out && in && scale, "row_scale: NULL argument");
    MGGB_REQUIRE(n >= 0 && dim >= 1, "row_scale: need n >= 0 and dim >= 1");
    if (n == 0) return MGGB_OK;
    row_scale_kernel<<<grid_for(n * dim, 256), 256, 0, (cudaStream_t)stream>>>(out, in, scale, n * dim, dim);
    MGGB_CUDA(cudaGetLastError());
    return MGGB_OK;
}

int mggb_inv_sqrt_degree(float* scale, const int32_t* row_ptr_l, const int32_t* row_ptr_r, int64_t n, void* stream) {
    MGGB_REQUIRE(scale && row_ptr_l, "inv_sqrt_degree: NULL argument");
    MGGB_REQUIRE(n >= 0, "inv_sqrt_degree: need n >= 0");
    if (n == 0) return MGGB_OK;
    inv_sqrt_degree_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(scale, row_ptr_l, row_ptr_r, n);
    MGGB_CUDA(cudaGetLastError());
    return MGGB_OK;
}

}  // extern "C"
