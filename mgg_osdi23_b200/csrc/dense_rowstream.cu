// Dense node update for NARROW outputs (dim2 <= 16): out[n, dim2] = x[n, dim1] * w[dim1, dim2], with x
// streamed row by row (sm_100a, CUDA cores, fp32 FMA).
//
// Stands in for the same cublasSgemm as dense_tc.cu (include/gnn_layer.cuh:42-52; operands
// include/layer_new.cuh:285-286) on the shapes where the output is 16 columns or fewer: the first GCN
// layer of the benchmark (602 -> 16) and 128 -> 16.  There the product needs only 2*dim2 = 32 flops
// per loaded float, which the fp32 pipes sustain at HBM speed, and the K-slab organisation a tensor
// core tile imposes (128 bytes of each of 128 rows per step) is what hurts: a 602-float row is
// visited 19 times, 128 bytes at a time, and HBM serves that strided walk at under a third of its
// streaming rate (measured: 0.30 ms for 561 MB with every slab-wise kernel, tensor core or not).
//
// Here a warp owns R consecutive rows and reads them front to back, every lane VEC consecutive floats
// of each row per step (8-byte loads for rows that are only 8-byte aligned, 16-byte loads otherwise):
// one contiguous stream per warp.  Each lane multiplies its floats by the matching rows of w (kept in
// shared memory in the order the lanes read them: conflict-free 128-bit reads, each reused for the R
// rows) into R x 16 private sums.  The 32 lanes' sums are then folded with a halving butterfly: at
// every step a lane sends the half of its sums that its partner keeps, so 16*R*(1 - 1/32) shuffles
// finish the job (not 5 per sum) and lane L ends up with outputs 2L and 2L+1 of the R x 16 block, which
// it stores as one 8-byte piece: the warp's store is one contiguous run of R rows.
//
// With 8-byte loads the sums are kept as PAIRS (columns 2j, 2j+1 in one 64-bit register) and updated with
// fma.rn.f32x2, two multiply-adds per instruction, each rounding like fmaf (sm_100); w is read from shared
// memory as ready-made pairs.
//
// The lanes load their floats into registers two steps ahead (three buffers in rotation).  What was measured
// on 232,965 x 602 -> 16 (561 MB of x; 86 us at the measured HBM copy rate), and dropped:
//   * four or five register buffers instead of three: 231 and 238 us against 206 us;
//   * x staged in a per-warp shared-memory ring by cp.async (8 bytes per lane and row, 7 KB in flight per
//     warp): the waits on loads disappear from the profile (long-scoreboard stall 3.2 -> 0.5 cycles per issued
//     instruction) but the warps then queue for the FMA pipe (math-pipe throttle) with a third more
//     instructions to issue: 215 us;
//   * a ninth warp staging the block's next 32 rows with bulk copies (77 KiB in flight per SM): 270 us, one
//     block of eight computing warps per SM does not keep the FMA pipes as busy as sixteen warps.
// With sixteen resident warps per SM (128 registers each) the kernel sits between the two limits: issue slots
// 49 % busy, FMA pipe 24 % (paired instructions), DRAM 34 %.
#include <algorithm>
#include "common.h"

namespace {

struct Publish {
    float* dst[MGGB_MAX_PES];
    int n;
};

constexpr int RS_THREADS = 256;
constexpr int RS_COLS = 16;      // padded output width
// Register buffers per row that a lane rotates through (loads in flight = buffers - 1 steps).  Measured on
// 232,965 x 602 -> 16: 3 buffers 206 us, 4 buffers 231 us, 5 buffers 238 us: issue slots, not latency, are
// what this kernel runs out of.
constexpr int RS_BUFFERS = 3;

template <int VEC> struct XVec;
template <> struct XVec<2> { using T = float2; };
template <> struct XVec<4> { using T = float4; };

// Two fp32 multiply-adds per instruction (sm_100: fma.rn.f32x2; each half rounds like fmaf).  A pair lives
// in one 64-bit register: low half = first element.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

// Halves the number of live sums: lanes whose `mask` bit is clear keep a[0 .. N/2), the others keep
// a[N/2 .. N); what a lane does not keep goes to its partner.  On return a[0 .. N/2) holds the kept sums.
template <int N>
__device__ __forceinline__ void fold(float (&a)[RS_COLS * 8], int lane, int mask) {
    const bool up = (lane & mask) != 0;
#pragma unroll
    for (int j = 0; j < N / 2; j++) {
        const float keep = up ? a[j + N / 2] : a[j];
        const float send = up ? a[j] : a[j + N / 2];
        a[j] = keep + __shfl_xor_sync(0xffffffffu, send, mask);
    }
}

// w into shared memory in lane order: slot ((i*VEC + e)*4 + g)*32 + l holds w[k][4g .. 4g+3] for
// k = (i*32 + l)*VEC + e (zeros past K or M).  Ends with a block barrier.
template <int VEC>
__device__ __forceinline__ void stage_w(float4* Wt, const float* __restrict__ w, int K, int M, int steps) {
    const bool vec_w = (M == RS_COLS) && ((uintptr_t)w % 16 == 0);
    for (int idx = threadIdx.x; idx < steps * VEC * 4 * 32; idx += RS_THREADS) {
        const int l = idx & 31, g = (idx >> 5) & 3, ie = idx >> 7;
        const int i = ie / VEC, e = ie - i * VEC;
        const int k = (i * 32 + l) * VEC + e;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (k < K && vec_w) {
            v = __ldg(reinterpret_cast<const float4*>(w + (long long)k * RS_COLS) + g);   // full-width w, 16-byte aligned
        } else if (k < K) {
            const float* src = w + (long long)k * M + 4 * g;
            if (4 * g + 0 < M) v.x = __ldg(src + 0);
            if (4 * g + 1 < M) v.y = __ldg(src + 1);
            if (4 * g + 2 < M) v.z = __ldg(src + 2);
            if (4 * g + 3 < M) v.w = __ldg(src + 3);
        }
        Wt[idx] = v;
    }
    __syncthreads();
}

// Folds the 32 lanes' R x 16 sums (16*R -> 2 per lane; lane L is left with flat elements 2L, 2L+1, +64 per
// further block of 64) and stores rows row0 .. row0+R-1 with the epilogue, also to every publish destination.
template <int R>
__device__ __forceinline__ void fold_and_store(float (&acc)[RS_COLS * 8], int lane, long long row0, long long n, int M,
                                               float* __restrict__ out, const float* __restrict__ row_scale, int relu,
                                               const Publish& pub, bool pair_ok) {
    constexpr int BLOCKS = RS_COLS * R / 64;
    float res[2 * BLOCKS];
#pragma unroll
    for (int b = 0; b < BLOCKS; b++) {
        float a[RS_COLS * 8];
#pragma unroll
        for (int j = 0; j < 64; j++) a[j] = acc[b * 64 + j];
        fold<64>(a, lane, 16);
        fold<32>(a, lane, 8);
        fold<16>(a, lane, 4);
        fold<8>(a, lane, 2);
        fold<4>(a, lane, 1);
        res[2 * b] = a[0];
        res[2 * b + 1] = a[1];
    }
#pragma unroll
    for (int b = 0; b < BLOCKS; b++) {
        // flat element f = b*64 + 2*lane (+1) of the R x 16 block: row f / 16, column f % 16
        const int f = b * 64 + 2 * lane;
        const long long row = row0 + f / RS_COLS;
        const int c = f % RS_COLS;
        if (row >= n) continue;
        const float s = row_scale ? row_scale[row] : 1.f;
        float v0 = res[2 * b] * s, v1 = res[2 * b + 1] * s;
        if (relu) { v0 = fmaxf(v0, 0.f); v1 = fmaxf(v1, 0.f); }
        const long long o = row * M + c;
        if (pair_ok) {
            // full-width rows and 8-byte aligned destinations: one 8-byte store per lane, so the warp writes
            // its R rows as one contiguous run (what a peer's replica wants to receive over NVLink)
            const float2 v = make_float2(v0, v1);
            *reinterpret_cast<float2*>(out + o) = v;
            for (int q = 0; q < pub.n; q++) *reinterpret_cast<float2*>(pub.dst[q] + o) = v;
        } else {
            if (c < M) { out[o] = v0; for (int q = 0; q < pub.n; q++) pub.dst[q][o] = v0; }
            if (c + 1 < M) { out[o + 1] = v1; for (int q = 0; q < pub.n; q++) pub.dst[q][o + 1] = v1; }
        }
    }
}

// R rows per warp (R * 16 must be a multiple of 64: R = 4 or 8), VEC floats per lane and step.
template <int VEC, int R, bool PACKED>
__global__ void __launch_bounds__(RS_THREADS, 2)
dense_rowstream_kernel(float* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w, long long n, int K, int M,
                       const float* __restrict__ row_scale, int relu, int steps, const Publish pub) {
    using V = typename XVec<VEC>::T;
    extern __shared__ __align__(16) float4 Wt[];     // [steps][VEC][4 column groups][32 lanes] of float4
    const int lane = threadIdx.x & 31;
    stage_w<VEC>(Wt, w, K, M, steps);

    bool pair_ok = (M == RS_COLS) && ((uintptr_t)out % 8 == 0);
    for (int q = 0; q < pub.n; q++) pair_ok = pair_ok && ((uintptr_t)pub.dst[q] % 8 == 0);
    const long long warps = ((long long)gridDim.x * RS_THREADS) >> 5;
    const long long groups = (n + R - 1) / R;
    for (long long grp = (((long long)blockIdx.x * RS_THREADS + threadIdx.x) >> 5); grp < groups; grp += warps) {
        const long long row0 = grp * R;
        float acc[RS_COLS * 8];
        unsigned long long acc2[RS_COLS * 4];   // PACKED: the same sums as pairs (columns 2j, 2j+1)
#pragma unroll
        for (int j = 0; j < RS_COLS * R; j++) acc[j] = 0.f;
#pragma unroll
        for (int j = 0; j < RS_COLS * R / 2; j++) acc2[j] = 0ull;

        auto load_step = [&](int i, V* xv) {
            const int k0 = (i * 32 + lane) * VEC;
#pragma unroll
            for (int r = 0; r < R; r++) {
                V v = V{};
                if (i < steps && k0 < K && row0 + r < n) v = __ldcs(reinterpret_cast<const V*>(x + (row0 + r) * K + k0));
                xv[r] = v;
            }
        };
        auto fma_step = [&](int i, const V* xv) {
            if (PACKED) {
#pragma unroll
                for (int e = 0; e < VEC; e++) {
                    unsigned long long aa[R];
#pragma unroll
                    for (int r = 0; r < R; r++) {
                        const float a = reinterpret_cast<const float*>(&xv[r])[e];
                        aa[r] = pack2(a, a);
                    }
#pragma unroll
                    for (int g = 0; g < 4; g++) {
                        // a float4 of w read as two ready-made pairs
                        const ulonglong2 wv = reinterpret_cast<const ulonglong2*>(Wt)[((i * VEC + e) * 4 + g) * 32 + lane];
#pragma unroll
                        for (int r = 0; r < R; r++) {
                            acc2[r * 8 + 2 * g + 0] = fma2(aa[r], wv.x, acc2[r * 8 + 2 * g + 0]);
                            acc2[r * 8 + 2 * g + 1] = fma2(aa[r], wv.y, acc2[r * 8 + 2 * g + 1]);
                        }
                    }
                }
            } else {
#pragma unroll
                for (int e = 0; e < VEC; e++) {
#pragma unroll
                    for (int g = 0; g < 4; g++) {
                        const float4 wv = Wt[((i * VEC + e) * 4 + g) * 32 + lane];
#pragma unroll
                        for (int r = 0; r < R; r++) {
                            const float a = reinterpret_cast<const float*>(&xv[r])[e];
                            acc[r * RS_COLS + 4 * g + 0] = fmaf(a, wv.x, acc[r * RS_COLS + 4 * g + 0]);
                            acc[r * RS_COLS + 4 * g + 1] = fmaf(a, wv.y, acc[r * RS_COLS + 4 * g + 1]);
                            acc[r * RS_COLS + 4 * g + 2] = fmaf(a, wv.z, acc[r * RS_COLS + 4 * g + 2]);
                            acc[r * RS_COLS + 4 * g + 3] = fmaf(a, wv.w, acc[r * RS_COLS + 4 * g + 3]);
                        }
                    }
                }
            }
        };
        // RS_BUFFERS register buffers in rotation: RS_BUFFERS - 1 steps of loads in flight while one is multiplied
        V buf[RS_BUFFERS][R];
#pragma unroll
        for (int b = 0; b < RS_BUFFERS - 1; b++) load_step(b, buf[b]);
        for (int i = 0; i < steps; i += RS_BUFFERS) {
#pragma unroll
            for (int b = 0; b < RS_BUFFERS; b++) {
                if (i + b < steps) {
                    load_step(i + b + RS_BUFFERS - 1, buf[(b + RS_BUFFERS - 1) % RS_BUFFERS]);
                    fma_step(i + b, buf[b]);
                }
            }
        }

        if (PACKED) {
#pragma unroll
            for (int j = 0; j < RS_COLS * R / 2; j++) unpack2(acc2[j], acc[2 * j], acc[2 * j + 1]);
        }
        fold_and_store<R>(acc, lane, row0, n, M, out, row_scale, relu, pub, pair_ok);
    }
}


}  // namespace

namespace mggb {

// *launched = false (and MGGB_OK) when the shape is not served: dim2 > 16, odd dim1, x not 8-byte
// aligned, or w too large for shared memory.  `even_if_aligned`: also take rows whose stride is a
// multiple of 16 bytes; by default those are left to the tensor-core kernel, whose TMA loads stream them
// faster (measured: 4,206,785 x 128 -> 16 in 0.64 ms against 1.28 ms here; 232,965 x 602 -> 16, which no
// tensor map takes, in 0.22 ms here against 0.34 ms there).
int dense_rowstream(float* out, const float* x, const float* w, int64_t n, int dim1, int dim2,
                    const float* row_scale, int flags, float* const* publish_out, int num_publish, cudaStream_t st,
                    bool even_if_aligned, bool* launched) {
    *launched = false;
    if (dim2 > RS_COLS || dim1 % 2 != 0 || ((uintptr_t)x % 8) != 0) return MGGB_OK;
    const bool wide = (dim1 % 4 == 0) && ((uintptr_t)x % 16 == 0);
    if (wide && !even_if_aligned) return MGGB_OK;
    const int vec = wide ? 4 : 2;
    const int steps = (dim1 + 32 * vec - 1) / (32 * vec);
    const size_t smem = (size_t)steps * vec * 4 * 32 * sizeof(float4);
    if (smem > 160 * 1024) return MGGB_OK;
    Publish pub{};
    pub.n = num_publish;
    for (int q = 0; q < num_publish; q++) pub.dst[q] = publish_out[q];
    constexpr int R = 4;
    const long long groups = (n + R - 1) / R;
    const long long blocks = (groups + RS_THREADS / 32 - 1) / (RS_THREADS / 32);
    const int grid = (int)std::min<long long>(blocks, 2LL * mggb::sm_count());
    const int relu = (flags & MGGB_DENSE_RELU) ? 1 : 0;
    auto go = [&](auto kernel) -> int {
        if (smem > 48 * 1024) MGGB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kernel<<<grid, RS_THREADS, smem, st>>>(out, x, w, n, dim1, dim2, row_scale, relu, steps, pub);
        return MGGB_OK;
    };
    // 8-byte loads: two multiply-adds per instruction (measured 235 -> 206 us on 232,965 x 602 -> 16);
    // 16-byte loads leave no registers for the paired accumulators
    const int rc = wide ? go(dense_rowstream_kernel<4, R, false>) : go(dense_rowstream_kernel<2, R, true>);
    if (rc != MGGB_OK) return rc;
    MGGB_CUDA(cudaGetLastError());
    *launched = true;
    return MGGB_OK;
}

}  // namespace mggb
