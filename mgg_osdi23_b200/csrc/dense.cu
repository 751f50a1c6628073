// Dense node update out[n, dim2] = x[n, dim1] * w[dim1, dim2] (row-major, alpha 1, beta 0, no bias)
// with an optional per-row scale and ReLU epilogue.
//
// Stands in for dense_beg_new_forward / dense_hidden_new_forward (include/gnn_layer.cuh:42-52), which
// hand the product to cublasSgemm with m=dim2, n=numNodes, k=dim1 (include/layer_new.cuh:285-286).
// The matrices are tall and skinny (n up to millions, dim2 16..172), so the product is bound by
// streaming x once from HBM.
//
// This file holds the fp32 CUDA-core kernel: a block keeps a [BM x 32] slab of x and the matching
// [32 x dim2] slab of w in shared memory and each thread owns a 4x4 output micro-tile.
#include "common.h"

namespace {

// Extra destinations of every output row (the peers' replicas of the embedding matrix).
struct Publish {
    float* dst[MGGB_MAX_PES];
    int n;
};

constexpr int BK = 32;
constexpr int TM = 4;
constexpr int TN = 4;
constexpr int THREADS = 256;

__global__ void __launch_bounds__(THREADS)
dense_simt_kernel(float* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w,
                  long long n, int K, int M, const float* __restrict__ row_scale, int relu, int CT, int RT,
                  const Publish pub) {
    extern __shared__ __align__(16) float smem[];
    const int BM = RT * TM;
    const int Mpad = CT * TN;
    float* Xs = smem;                       // [BM][BK+1]
    float* Ws = smem + (size_t)BM * (BK + 1);  // [BK][Mpad]
    const int t = threadIdx.x;
    const int ct = t % CT, rt = t / CT;
    const bool active = rt < RT;
    const long long tiles = (n + BM - 1) / BM;

    for (long long tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const long long row0 = tile * BM;
        float acc[TM][TN];
#pragma unroll
        for (int i = 0; i < TM; i++)
#pragma unroll
            for (int j = 0; j < TN; j++) acc[i][j] = 0.f;

        for (int k0 = 0; k0 < K; k0 += BK) {
            for (int idx = t; idx < BM * BK; idx += THREADS) {
                const int r = idx / BK, k = idx % BK;
                const long long gr = row0 + r;
                Xs[r * (BK + 1) + k] = (gr < n && k0 + k < K) ? __ldcs(x + gr * K + k0 + k) : 0.f;
            }
            for (int idx = t; idx < BK * Mpad; idx += THREADS) {
                const int k = idx / Mpad, c = idx % Mpad;
                Ws[idx] = (k0 + k < K && c < M) ? __ldg(w + (long long)(k0 + k) * M + c) : 0.f;
            }
            __syncthreads();
            if (active) {
#pragma unroll 8
                for (int k = 0; k < BK; k++) {
                    const float4 b = *reinterpret_cast<const float4*>(Ws + k * Mpad + ct * TN);
#pragma unroll
                    for (int i = 0; i < TM; i++) {
                        const float a = Xs[(rt * TM + i) * (BK + 1) + k];
                        acc[i][0] = fmaf(a, b.x, acc[i][0]);
                        acc[i][1] = fmaf(a, b.y, acc[i][1]);
                        acc[i][2] = fmaf(a, b.z, acc[i][2]);
                        acc[i][3] = fmaf(a, b.w, acc[i][3]);
                    }
                }
            }
            __syncthreads();
        }
        if (active) {
#pragma unroll
            for (int i = 0; i < TM; i++) {
                const long long gr = row0 + rt * TM + i;
                if (gr >= n) continue;
                const float s = row_scale ? row_scale[gr] : 1.f;
#pragma unroll
                for (int j = 0; j < TN; j++) {
                    const int c = ct * TN + j;
                    if (c < M) {
                        float v = acc[i][j] * s;
                        if (relu) v = fmaxf(v, 0.f);
                        out[gr * M + c] = v;
                        for (int q = 0; q < pub.n; q++) pub.dst[q][gr * M + c] = v;
                    }
                }
            }
        }
    }
}

}  // namespace

namespace mggb {

int dense_simt(float* out, const float* x, const float* w, int64_t n, int dim1, int dim2,
               const float* row_scale, int flags, float* const* publish_out, int num_publish, cudaStream_t st) {
    Publish pub{};
    pub.n = num_publish;
    for (int q = 0; q < num_publish; q++) pub.dst[q] = publish_out[q];
    const int CT = (dim2 + TN - 1) / TN;
    if (CT > THREADS)
        return fail(MGGB_ERR_UNSUPPORTED, "dense_forward: dim2=%d exceeds %d", dim2, THREADS * TN);
    const int RT = THREADS / CT;
    const int BM = RT * TM;
    const size_t smem = ((size_t)BM * (BK + 1) + (size_t)BK * CT * TN) * sizeof(float);
    if (smem > 48 * 1024)
        MGGB_CUDA(cudaFuncSetAttribute(dense_simt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int sms = mggb::sm_count();
    const long long tiles = (n + BM - 1) / BM;
    const int grid = (int)(tiles < (long long)sms * 4 ? tiles : (long long)sms * 4);
    dense_simt_kernel<<<grid, THREADS, smem, st>>>(out, x, w, n, dim1, dim2, row_scale,
                                                   (flags & MGGB_DENSE_RELU) ? 1 : 0, CT, RT, pub);
    MGGB_CUDA(cudaGetLastError());
    return MGGB_OK;
}

// Row-streaming CUDA-core kernel for outputs of at most 16 columns (dense_rowstream.cu) and the
// tensor-core kernel (dense_tc.cu); each sets *launched = false when the shape does not fit it.
int dense_rowstream(float* out, const float* x, const float* w, int64_t n, int dim1, int dim2, const float* row_scale,
                    int flags, float* const* publish_out, int num_publish, cudaStream_t st, bool even_if_aligned, bool* launched);
int dense_tc(float* out, const float* x, const float* w, int64_t n, int dim1, int dim2, const float* row_scale,
             int flags, float* const* publish_out, int num_publish, cudaStream_t st, bool* launched);

}  // namespace mggb

extern "C" int mggb_dense_forward(float* out, const float* x, const float* w, int64_t n, int dim1,
                                  int dim2, const float* row_scale, int flags, float* const* publish_out,
                                  int num_publish, void* stream) {
    MGGB_REQUIRE(num_publish >= 0 && num_publish <= MGGB_MAX_PES && (num_publish == 0 || publish_out),
                 "dense_forward: num_publish must be in [0,%d] with a non-NULL table (got %d)", MGGB_MAX_PES, num_publish);
    for (int q = 0; q < num_publish; q++) MGGB_REQUIRE(publish_out[q] != nullptr, "dense_forward: publish_out[%d] is NULL", q);
    MGGB_REQUIRE(out && x && w, "dense_forward: NULL argument");
    MGGB_REQUIRE(n >= 0 && dim1 >= 1 && dim2 >= 1, "dense_forward: need n >= 0, dim1 >= 1, dim2 >= 1 (n=%lld dim1=%d dim2=%d)", (long long)n, dim1, dim2);
    MGGB_REQUIRE(out != x, "dense_forward: out must not alias x");
    if (n == 0) return MGGB_OK;
    // Narrow outputs from rows that no tensor map takes (stride not a multiple of 16 bytes): the row-streaming
    // kernel (fp32 FMA), unless the caller asked for tensor cores.  With MGGB_DENSE_SIMT it also takes aligned rows.
    if (!(flags & (MGGB_DENSE_TENSOR | MGGB_DENSE_TF32))) {
        bool launched = false;
        const int st = mggb::dense_rowstream(out, x, w, n, dim1, dim2, row_scale, flags, publish_out, num_publish,
                                             (cudaStream_t)stream, (flags & MGGB_DENSE_SIMT) != 0, &launched);
        if (st != MGGB_OK || launched) return st;
    }
    if (!(flags & MGGB_DENSE_SIMT)) {
        bool launched = false;
        const int st = mggb::dense_tc(out, x, w, n, dim1, dim2, row_scale, flags, publish_out, num_publish,
                                      (cudaStream_t)stream, &launched);
        if (st != MGGB_OK || launched) return st;
    }
    return mggb::dense_simt(out, x, w, n, dim1, dim2, row_scale, flags, publish_out, num_publish, (cudaStream_t)stream);
}
