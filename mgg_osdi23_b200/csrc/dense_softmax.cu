// Last layer in one pass: out[n, M] = softmax_rows(x[n, K] * w[K, M]), optionally keeping the logits.
//
// Stands in for dense_hidden_new_forward followed by softmax_new_forward
// (src/mgg_np_div_mem.cu:220-226, src/mgg_np_div_gin_mem.cu:220-222; include/gnn_layer.cuh:36-52).
// Done as two kernels the [n, M] logits are written, read back and the probabilities written
// (3 * n * M * 4 bytes); fused, only the probabilities leave the chip.  With a wide class count
// and a narrow hidden width (172 classes from 16 features) the pass is bound by that traffic.
//
// A warp owns 8 rows at a time.  Lane l holds output columns l, l+32, ... (J of them) of each of
// its rows in registers, as PAIRS (columns 64p + l and 64p + 32 + l in one 64-bit register) updated with
// fma.rn.f32x2: two multiply-adds per instruction, each rounding like fmaf (sm_100).  The kernel is bound
// by instruction issue, so both operands are laid out in shared memory as ready-made pairs: w once per
// block as {w[k][64p+l], w[k][64p+32+l]}, zero-padded to 64*JP columns, and the warp's 8 rows of x with
// every element stored twice ({x, x}), read back as broadcasts.  Softmax is the max-subtracted exp / sum
// of the separate kernel, reduced over the warp with shuffles, the 8 rows side by side.
#include <algorithm>
#include <cfloat>
#include <cstdint>
#include "common.h"

namespace {

constexpr int FS_WARPS = 8;
constexpr int FS_ROWS = 8;     // rows per warp step

// e^d for d <= 0 as 2^(d * log2 e) on the special-function unit: relative error below 1e-6 * max(1, |d|/10)
// down to d = -87, flushed to 0 below (the exact value is under 1e-37 there).  The kernel issues one
// of these per output element, and it is bound by its instruction count.
__device__ __forceinline__ float exp_neg(float d) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d * 1.4426950408889634f));
    return r;
}

__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

// J = ceil(M / 32) column slots per lane, JP = ceil(J / 2) pairs of them.
template <int J>
__global__ void __launch_bounds__(FS_WARPS * 32, 2)
dense_softmax_kernel(float* __restrict__ out, float* __restrict__ logits, const float* __restrict__ x,
                     const float* __restrict__ w, long long n, int K, int M, int vec_ok) {
    extern __shared__ __align__(16) float fs_smem[];
    constexpr int JP = (J + 1) / 2;
    float2* Ws = reinterpret_cast<float2*>(fs_smem);       // [K][JP][32 lanes] of {column 64p + l, column 64p + 32 + l}
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float2* Xs = Ws + (size_t)K * JP * 32 + (size_t)warp * FS_ROWS * K;   // [FS_ROWS][K] of {x, x}
    for (int idx = threadIdx.x; idx < K * JP * 32; idx += FS_WARPS * 32) {
        const int l = idx & 31, p = (idx >> 5) % JP, k = idx / (32 * JP);
        const int c0 = 64 * p + l, c1 = c0 + 32;
        Ws[idx] = make_float2(c0 < M ? __ldg(w + (long long)k * M + c0) : 0.f, c1 < M ? __ldg(w + (long long)k * M + c1) : 0.f);
    }
    __syncthreads();

    const long long groups = (n + FS_ROWS - 1) / FS_ROWS;
    const long long stride = (long long)gridDim.x * FS_WARPS;
    for (long long g = (long long)blockIdx.x * FS_WARPS + warp; g < groups; g += stride) {
        const long long row0 = g * FS_ROWS;
        const int rows = (int)min((long long)FS_ROWS, n - row0);
        const int count = rows * K;
        const float* src = x + row0 * K;
        __syncwarp();                                      // the previous step's reads of Xs are done
        if (vec_ok) {
            for (int i = lane * 4; i < FS_ROWS * K; i += 128) {
                const float4 v = i < count ? __ldcs(reinterpret_cast<const float4*>(src + i)) : make_float4(0.f, 0.f, 0.f, 0.f);
                *reinterpret_cast<float4*>(Xs + i) = make_float4(v.x, v.x, v.y, v.y);
                *reinterpret_cast<float4*>(Xs + i + 2) = make_float4(v.z, v.z, v.w, v.w);
            }
        } else {
            for (int i = lane; i < FS_ROWS * K; i += 32) {
                const float v = i < count ? __ldcs(src + i) : 0.f;
                Xs[i] = make_float2(v, v);
            }
        }
        __syncwarp();

        unsigned long long acc2[FS_ROWS][JP];
#pragma unroll
        for (int r = 0; r < FS_ROWS; r++)
#pragma unroll
            for (int p = 0; p < JP; p++) acc2[r][p] = 0ull;

        const unsigned long long* Wp = reinterpret_cast<const unsigned long long*>(Ws);
        if (vec_ok) {
            for (int k = 0; k < K; k += 2) {
                ulonglong2 xv[FS_ROWS];                    // {x[k], x[k]} and {x[k+1], x[k+1]} of every row
#pragma unroll
                for (int r = 0; r < FS_ROWS; r++) xv[r] = *reinterpret_cast<const ulonglong2*>(Xs + r * K + k);
#pragma unroll
                for (int kk = 0; kk < 2; kk++) {
                    unsigned long long wv[JP];
#pragma unroll
                    for (int p = 0; p < JP; p++) wv[p] = Wp[((k + kk) * JP + p) * 32 + lane];
#pragma unroll
                    for (int r = 0; r < FS_ROWS; r++) {
                        const unsigned long long a = kk == 0 ? xv[r].x : xv[r].y;
#pragma unroll
                        for (int p = 0; p < JP; p++) acc2[r][p] = fma2(a, wv[p], acc2[r][p]);
                    }
                }
            }
        } else {
            const unsigned long long* Xp = reinterpret_cast<const unsigned long long*>(Xs);
            for (int k = 0; k < K; k++) {
                unsigned long long wv[JP];
#pragma unroll
                for (int p = 0; p < JP; p++) wv[p] = Wp[(k * JP + p) * 32 + lane];
#pragma unroll
                for (int r = 0; r < FS_ROWS; r++) {
                    const unsigned long long a = Xp[r * K + k];
#pragma unroll
                    for (int p = 0; p < JP; p++) acc2[r][p] = fma2(a, wv[p], acc2[r][p]);
                }
            }
        }
        // column slot j = 2p (+1) of lane l is column 32j + l, as the softmax and the stores below expect
        float acc[FS_ROWS][2 * JP];
#pragma unroll
        for (int r = 0; r < FS_ROWS; r++)
#pragma unroll
            for (int p = 0; p < JP; p++) unpack2(acc2[r][p], acc[r][2 * p], acc[r][2 * p + 1]);

        // Softmax of the 8 rows side by side: the shuffle chains of different rows overlap.
        const bool last_ok = lane < M - 32 * (J - 1);      // only the last column slot can run past M
        if (logits) {
#pragma unroll
            for (int r = 0; r < FS_ROWS; r++)
#pragma unroll
                for (int j = 0; j < J; j++)
                    if (r < rows && (j < J - 1 || last_ok)) __stcs(logits + (row0 + r) * M + j * 32 + lane, acc[r][j]);
        }
        float m[FS_ROWS], sum[FS_ROWS];
#pragma unroll
        for (int r = 0; r < FS_ROWS; r++) {
            m[r] = -FLT_MAX;
#pragma unroll
            for (int j = 0; j < J; j++)
                if (j < J - 1 || last_ok) m[r] = fmaxf(m[r], acc[r][j]);
        }
#pragma unroll
        for (int off = 16; off; off >>= 1)
#pragma unroll
            for (int r = 0; r < FS_ROWS; r++) m[r] = fmaxf(m[r], __shfl_xor_sync(0xffffffffu, m[r], off));
#pragma unroll
        for (int r = 0; r < FS_ROWS; r++) {
            sum[r] = 0.f;
#pragma unroll
            for (int j = 0; j < J; j++) {
                acc[r][j] = (j < J - 1 || last_ok) ? exp_neg(acc[r][j] - m[r]) : 0.f;
                sum[r] += acc[r][j];
            }
        }
#pragma unroll
        for (int off = 16; off; off >>= 1)
#pragma unroll
            for (int r = 0; r < FS_ROWS; r++) sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], off);
#pragma unroll
        for (int r = 0; r < FS_ROWS; r++) {
            const float inv = 1.f / sum[r];
            float* dst = out + (row0 + r) * M + lane;
#pragma unroll
            for (int j = 0; j < J; j++)
                if (r < rows && (j < J - 1 || last_ok)) __stcs(dst + j * 32, acc[r][j] * inv);
        }
    }
}

template <int J>
int launch_fused(float* out, float* logits, const float* x, const float* w, long long n, int K, int M,
                 int vec_ok, size_t smem, int grid, cudaStream_t st) {
    if (smem > 48 * 1024)
        MGGB_CUDA(cudaFuncSetAttribute(dense_softmax_kernel<J>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dense_softmax_kernel<J><<<grid, FS_WARPS * 32, smem, st>>>(out, logits, x, w, n, K, M, vec_ok);
    MGGB_CUDA(cudaGetLastError());
    return MGGB_OK;
}

}  // namespace

namespace mggb {
int dense_tc(float* out, const float* x, const float* w, int64_t n, int dim1, int dim2, const float* row_scale,
             int flags, float* const* publish_out, int num_publish, cudaStream_t st, bool* launched);
}

extern "C" int mggb_dense_softmax_forward(float* out, float* logits, const float* x, const float* w, int64_t n,
                                          int dim1, int dim2, void* stream) {
    MGGB_REQUIRE(out && x && w, "dense_softmax_forward: NULL argument");
    MGGB_REQUIRE(n >= 0 && dim1 >= 1 && dim2 >= 1, "dense_softmax_forward: need n >= 0, dim1 >= 1, dim2 >= 1 (n=%lld dim1=%d dim2=%d)",
                 (long long)n, dim1, dim2);
    MGGB_REQUIRE(out != x && logits != x, "dense_softmax_forward: outputs must not alias x");
    // Wide inputs (dim1 a multiple of 4 above 32, at most 128 classes, logits not wanted): the tcgen05 kernel with the
    // softmax in its epilogue, where every thread owns a whole accumulator row.  The multiply-adds of such a shape
    // (2,449,029 x 64 -> 47: 10 G) keep the fp32 pipes busy for 0.95 ms in the kernel below; on the tensor cores the
    // pass is bound by streaming x and the probabilities.
    if (n > 0 && logits == nullptr && dim1 % 4 == 0 && ((uintptr_t)x % 16) == 0 && dim2 <= 128) {
        bool launched = false;
        const int rc = mggb::dense_tc(out, x, w, n, dim1, dim2, nullptr, mggb::DENSE_TC_SOFTMAX, nullptr, 0, (cudaStream_t)stream, &launched);
        if (rc != MGGB_OK || launched) return rc;
    }
    const int J = (dim2 + 31) / 32;
    const int JP = (J + 1) / 2;
    const size_t smem = ((size_t)dim1 * 32 * JP + (size_t)FS_WARPS * FS_ROWS * dim1) * sizeof(float2);
    if (J > 8 || smem > 160 * 1024)
        return mggb::fail(MGGB_ERR_UNSUPPORTED, "dense_softmax_forward: dim1=%d dim2=%d does not fit the fused kernel "
                          "(dim2 <= 256 and %zu bytes of shared memory <= 160 KiB); call mggb_dense_forward then mggb_softmax_forward",
                          dim1, dim2, smem);
    if (n == 0) return MGGB_OK;
    const int sms = mggb::sm_count();
    const long long groups = (n + FS_ROWS - 1) / FS_ROWS;
    const long long blocks = (groups + FS_WARPS - 1) / FS_WARPS;
    const int per_sm = smem > 64 * 1024 ? 1 : 2;
    const int grid = (int)std::min<long long>(blocks, (long long)sms * per_sm);
    const int vec_ok = (dim1 % 4 == 0 && ((uintptr_t)x % 16) == 0) ? 1 : 0;
    cudaStream_t st = (cudaStream_t)stream;
    switch (J) {
        case 1: return launch_fused<1>(out, logits, x, w, n, dim1, dim2, vec_ok, smem, grid, st);
        case 2: return launch_fused<2>(out, logits, x, w, n, dim1, dim2, vec_ok, smem, grid, st);
        case 3: return launch_fused<3>(out, logits, x, w, n, dim1, dim2, vec_ok, smem, grid, st);
        case 4: return launch_fused<4>(out, logits, x, w, n, dim1, dim2, vec_ok, smem, grid, st);
        case 5: return launch_fused<5>(out, logits, x, w, n, dim1, dim2, vec_ok, smem, grid, st);
        case 6: return launch_fused<6>(out, logits, x, w, n, dim1, dim2, vec_ok, smem, grid, st);
        case 7: return launch_fused<7>(out, logits, x, w, n, dim1, dim2, vec_ok, smem, grid, st);
        default: return launch_fused<8>(out, logits, x, w, n, dim1, dim2, vec_ok, smem, grid, st);
    }
}
