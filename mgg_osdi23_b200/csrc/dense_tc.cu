// Dense node update on the 5th-generation tensor cores (tcgen05, sm_100a):
//     out[n, M] = x[n, K] * w[K, M]      (row-major, fp32 in / fp32 out)
//
// Stands in for the cublasSgemm behind dense_beg_new_forward / dense_hidden_new_forward
// (include/gnn_layer.cuh:42-52; m=dim2, n=numNodes, k=dim1, include/layer_new.cuh:285-286).
// n is huge and M small (16..64), so the product is bound by streaming x from HBM once; the tensor
// cores are used because 2*M flops per loaded float is more than the CUDA cores sustain at HBM speed.
//
// Precision.  The tensor core multiplies TF32 (10-bit mantissa) values.  Each fp32 operand is split
// exactly into hi + lo with both parts representable in TF32 (hi = top bits, lo = next bits; what is
// dropped is below 2^-21 of the value) and all four partial products hi*hi, hi*lo, lo*hi, lo*lo are
// accumulated in fp32 in tensor memory, so the result matches an fp32 GEMM to about 1e-6 relative.
//
// One persistent CTA per SM, 9 warps, no clusters:
//   warps 0-3  loaders: cp.async a [128 rows x 32 floats] slab of x into a 4-stage ring in the
//              128-byte-swizzled K-major layout the tensor core reads, then split what landed into
//              hi and lo slabs.  Plain cp.async rather than TMA because Reddit-shaped rows
//              (602 floats = 2408 bytes) break TMA's 16-byte stride rule; 8- or 16-byte pieces.
//   warp 8     allocates tensor memory; one lane issues tcgen05.mma (M=128, N=pad16(M), K=8 per
//              instruction, 4 k-steps x 4 partial products per slab) and commits to mbarriers.
//   warps 4-7  epilogue: tcgen05.ld the 128 x N accumulator (double-buffered in tensor memory), apply
//              row scale / ReLU, store the rows (and publish them to peers' replicas).
// w is split and laid out in shared memory once per CTA.  Every wait on an mbarrier is bounded: on
// expiry the CTA raises a status word the host can read (mggb_dense_device_status), drains its
// copies, frees its tensor memory and returns.
#include <algorithm>
#include "common.h"

namespace mggb {
int dense_simt(float* out, const float* x, const float* w, int64_t n, int dim1, int dim2,
               const float* row_scale, int flags, float* const* publish_out, int num_publish, cudaStream_t st);
}

namespace {

constexpr int TILE_M = 128;              // rows of x per tile (UMMA M)
constexpr int CHUNK_K = 32;              // floats of K per slab = one 128-byte swizzle row
constexpr int SLAB_BYTES = TILE_M * 128; // 16 KiB
constexpr int STAGE_BYTES = 2 * SLAB_BYTES;  // hi + lo
constexpr int LOADERS = 128;
constexpr int THREADS = 288;
constexpr int MAX_STAGES = 4;
constexpr unsigned SPIN_LIMIT = 1u << 22;
constexpr unsigned TF32_MASK = 0xFFFFE000u;

__device__ int g_dense_status = 0;   // 0 ok; otherwise which wait expired (1 full, 2 empty, 3 tmem_full, 4 tmem_empty)

struct Publish {
    float* dst[MGGB_MAX_PES];
    int n;
};

struct TcParams {
    float* out;
    const float* x;
    const float* w;
    const float* row_scale;
    long long n;
    int K, M, Npad, nchunks, stages, relu;
    unsigned tmem_cols;
    Publish pub;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false when the limit ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, unsigned parity, volatile int* abort_flag, int code) {
    for (unsigned i = 0; i < SPIN_LIMIT; i++) {
        if (mbar_try(bar, parity)) return true;
        if (*abort_flag) return false;
        if (i > 32) __nanosleep(64);
    }
    *abort_flag = code;
    atomicCAS(&g_dense_status, 0, code);
    return false;
}

// Byte offset of (row, byte b of its 128-byte K slab) in the 128B-swizzled K-major layout:
// 8-row groups of 1024 bytes, 16-byte pieces XOR-ed with the row index inside the group.
__device__ __forceinline__ uint32_t swz(int row, int b) {
    return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((((b >> 4) ^ (row & 7)) << 4) | (b & 15)));
}

// Shared-memory matrix descriptor: K-major, SWIZZLE_128B, 8-row group stride 1024 bytes.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);   // start address, bits [0,14)
    d |= (uint64_t)1 << 16;                     // leading byte offset (unused for swizzled K-major), bits [16,30)
    d |= (uint64_t)(1024 >> 4) << 32;           // stride byte offset, bits [32,46)
    d |= (uint64_t)1 << 46;                     // descriptor version (Blackwell), bits [46,48)
    d |= (uint64_t)2 << 61;                     // layout type SWIZZLE_128B, bits [61,64)
    return d;
}

__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        :: "r"(d_tmem), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

template <int G>
__device__ __forceinline__ void cp_async_zfill(uint32_t dst, const void* src, int src_bytes) {
    if (G == 16)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
    else
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

// ---- roles ---------------------------------------------------------------------------------------

// Splits the pieces this thread copied for one slab into TF32-exact hi (in place) and lo parts.
template <int G>
__device__ __forceinline__ void split_slab(unsigned char* stage, int p) {
    constexpr int PPR = 128 / G;
#pragma unroll
    for (int i = 0; i < PPR; i++) {
        const int q = i * LOADERS + p;
        const uint32_t off = swz(q / PPR, (q % PPR) * G);
        float* hi = reinterpret_cast<float*>(stage + off);
        float* lo = reinterpret_cast<float*>(stage + SLAB_BYTES + off);
#pragma unroll
        for (int e = 0; e < G / 4; e++) {
            const float v = hi[e];
            const float h = __uint_as_float(__float_as_uint(v) & TF32_MASK);
            hi[e] = h;
            lo[e] = __uint_as_float(__float_as_uint(v - h) & TF32_MASK);
        }
    }
}

// Waits until at most `pending` of this thread's cp.async groups are still in flight.
__device__ __forceinline__ void cp_async_wait_pending(int pending) {
    switch (pending) {
        case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
        case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
        case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
        default: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    }
}

template <int G>
__device__ __forceinline__ void hand_over_slab(unsigned char* ring, int stage_idx, uint32_t full0, int p) {
    split_slab<G>(ring + (size_t)stage_idx * STAGE_BYTES, p);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the tensor core
    mbar_arrive(full0 + 8 * stage_idx);
}

// Each slab is one cp.async group per thread.  A thread keeps stages-1 slabs in flight: after
// committing slab c it waits for slab c-(stages-1), splits its own pieces of it and arrives on that
// slab's "full" barrier (128 arrivals complete it).
template <int G>
__device__ void loader_role(const TcParams& P, unsigned char* ring, uint32_t full0, uint32_t empty0,
                            volatile int* abort_flag, long long first_tile, long long tile_step, long long tiles) {
    constexpr int PPR = 128 / G;
    const int p = threadIdx.x;           // 0..127
    const int S = P.stages;
    const int lookahead = S - 1;
    long long issued = 0, finished = 0;  // slab counters of this CTA
    bool ok = true;
    for (long long tile = first_tile; tile < tiles && ok; tile += tile_step) {
        const long long row0 = tile * TILE_M;
        for (int kc = 0; kc < P.nchunks; kc++) {
            const int s = (int)(issued % S);
            const long long use = issued / S;
            if (use >= 1) ok = mbar_wait(empty0 + 8 * s, (unsigned)((use - 1) & 1), abort_flag, 2);
            if (!ok) break;
            const uint32_t sbase = smem_u32(ring + (size_t)s * STAGE_BYTES);
#pragma unroll
            for (int i = 0; i < PPR; i++) {
                const int q = i * LOADERS + p;
                const int r = q / PPR, piece = q % PPR;
                const long long gr = row0 + r;
                const int k = kc * CHUNK_K + piece * (G / 4);
                const bool valid = gr < P.n && k < P.K;
                const float* src = valid ? P.x + gr * P.K + k : P.x;
                cp_async_zfill<G>(sbase + swz(r, piece * G), src, valid ? G : 0);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            issued++;
            if (issued - finished > lookahead) {
                cp_async_wait_pending(lookahead);
                hand_over_slab<G>(ring, (int)(finished % S), full0, p);
                finished++;
            }
        }
    }
    // drain: whatever is still in flight lands; unless the CTA gave up it is split and handed over too
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    while (ok && finished < issued) {
        hand_over_slab<G>(ring, (int)(finished % S), full0, p);
        finished++;
    }
}

__device__ void mma_role(const TcParams& P, uint32_t ring_base, uint32_t w_hi, uint32_t w_lo, uint32_t full0,
                         uint32_t empty0, uint32_t tfull0, uint32_t tempty0, uint32_t tmem_base,
                         volatile int* abort_flag, long long first_tile, long long tile_step, long long tiles) {
    const int S = P.stages;
    const uint32_t panel = (uint32_t)P.Npad * 128u;
    // instruction descriptor: D fp32, A/B TF32, both K-major, N = Npad, M = 128
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(P.Npad >> 3) << 17) | ((uint32_t)(TILE_M >> 4) << 24);
    long long consumed = 0, t = 0;
    for (long long tile = first_tile; tile < tiles; tile += tile_step, t++) {
        const int buf = (int)(t & 1);
        const long long use_t = t >> 1;
        if (use_t >= 1 && !mbar_wait(tempty0 + 8 * buf, (unsigned)((use_t - 1) & 1), abort_flag, 4)) return;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * P.Npad);
        for (int kc = 0; kc < P.nchunks; kc++, consumed++) {
            const int s = (int)(consumed % S);
            if (!mbar_wait(full0 + 8 * s, (unsigned)((consumed / S) & 1), abort_flag, 1)) return;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_hi = ring_base + (uint32_t)s * STAGE_BYTES, a_lo = a_hi + SLAB_BYTES;
            const uint32_t b_hi = w_hi + (uint32_t)kc * panel, b_lo = w_lo + (uint32_t)kc * panel;
#pragma unroll
            for (int ks = 0; ks < CHUNK_K / 8; ks++) {
                const uint32_t koff = (uint32_t)ks * 32u;   // 8 TF32 = 32 bytes along K inside the swizzled row
                const uint64_t dah = umma_desc(a_hi + koff), dal = umma_desc(a_lo + koff);
                const uint64_t dbh = umma_desc(b_hi + koff), dbl = umma_desc(b_lo + koff);
                umma_tf32(d_tmem, dah, dbh, idesc, (kc > 0 || ks > 0) ? 1u : 0u);
                umma_tf32(d_tmem, dah, dbl, idesc, 1u);
                umma_tf32(d_tmem, dal, dbh, idesc, 1u);
                umma_tf32(d_tmem, dal, dbl, idesc, 1u);
            }
            umma_commit(empty0 + 8 * s);            // the slab may be overwritten once these MMAs are done
        }
        umma_commit(tfull0 + 8 * buf);              // the accumulator of this tile is complete
    }
}

__device__ void epilogue_role(const TcParams& P, uint32_t tfull0, uint32_t tempty0, uint32_t tmem_base,
                              volatile int* abort_flag, long long first_tile, long long tile_step, long long tiles) {
    const int quarter = (threadIdx.x >> 5) & 3;   // warps 4..7 own tensor-memory lanes 32*quarter ..
    const int lane = threadIdx.x & 31;
    long long t = 0;
    for (long long tile = first_tile; tile < tiles; tile += tile_step, t++) {
        const int buf = (int)(t & 1);
        // all lanes leave together: tcgen05.ld below needs the whole warp
        if (!__all_sync(0xffffffffu, mbar_wait(tfull0 + 8 * buf, (unsigned)((t >> 1) & 1), abort_flag, 3))) return;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const long long row = tile * TILE_M + quarter * 32 + lane;
        const float scale = (P.row_scale && row < P.n) ? P.row_scale[row] : 1.f;
        for (int c0 = 0; c0 < P.Npad; c0 += 16) {
            uint32_t r[16];
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * P.Npad + c0);
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                  "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                : "r"(taddr));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (row < P.n) {
                float v[16];
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    v[j] = __uint_as_float(r[j]) * scale;
                    if (P.relu) v[j] = fmaxf(v[j], 0.f);
                }
                const long long o = row * P.M + c0;
                if ((P.M & 3) == 0 && c0 + 16 <= P.M) {
#pragma unroll
                    for (int j = 0; j < 16; j += 4) {
                        const float4 f = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                        *reinterpret_cast<float4*>(P.out + o + j) = f;
                        for (int q = 0; q < P.pub.n; q++) *reinterpret_cast<float4*>(P.pub.dst[q] + o + j) = f;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j++)
                        if (c0 + j < P.M) {
                            P.out[o + j] = v[j];
                            for (int q = 0; q < P.pub.n; q++) P.pub.dst[q][o + j] = v[j];
                        }
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        mbar_arrive(tempty0 + 8 * buf);
    }
}

template <int G>
__global__ void __launch_bounds__(THREADS, 1) dense_tc_kernel(const TcParams P) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // carve: [w_hi][w_lo][ring][barriers][tmem ptr]; every region a multiple of 1024 bytes
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const size_t w_bytes = (size_t)P.nchunks * P.Npad * 128;
    unsigned char* w_hi = base;
    unsigned char* w_lo = base + w_bytes;
    unsigned char* ring = base + 2 * w_bytes;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(ring + (size_t)P.stages * STAGE_BYTES);
    // bars: full[MAX_STAGES], empty[MAX_STAGES], tmem_full[2], tmem_empty[2]
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;

    const int warp = threadIdx.x >> 5;
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * MAX_STAGES;
    const uint32_t tfull0 = empty0 + 8 * MAX_STAGES, tempty0 = tfull0 + 16;

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < MAX_STAGES; s++) { mbar_init(full0 + 8 * s, LOADERS); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; b++) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, 128); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)), "r"(P.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // w, split into hi/lo, transposed into K-major swizzled panels of [Npad rows x 32 floats]
    for (int idx = threadIdx.x; idx < P.nchunks * CHUNK_K * P.Npad; idx += THREADS) {
        const int nn = idx % P.Npad, kk = (idx / P.Npad) % CHUNK_K, kc = idx / (P.Npad * CHUNK_K);
        const int k = kc * CHUNK_K + kk;
        const float v = (k < P.K && nn < P.M) ? __ldg(P.w + (long long)k * P.M + nn) : 0.f;
        const float h = __uint_as_float(__float_as_uint(v) & TF32_MASK);
        const uint32_t off = (uint32_t)kc * P.Npad * 128u + swz(nn, kk * 4);
        *reinterpret_cast<float*>(w_hi + off) = h;
        *reinterpret_cast<float*>(w_lo + off) = __uint_as_float(__float_as_uint(v - h) & TF32_MASK);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = s_tmem_base;

    const long long tiles = (P.n + TILE_M - 1) / TILE_M;
    if (warp < 4) {
        loader_role<G>(P, ring, full0, empty0, &s_abort, blockIdx.x, gridDim.x, tiles);
    } else if (warp < 8) {
        epilogue_role(P, tfull0, tempty0, tmem_base, &s_abort, blockIdx.x, gridDim.x, tiles);
    } else if ((threadIdx.x & 31) == 0) {
        mma_role(P, smem_u32(ring), smem_u32(w_hi), smem_u32(w_lo), full0, empty0, tfull0, tempty0, tmem_base,
                 &s_abort, blockIdx.x, gridDim.x, tiles);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 8) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(P.tmem_cols) : "memory");
    }
}

}  // namespace

namespace mggb {

// Returns MGGB_ERR_UNSUPPORTED (without touching the error text) when the shape does not fit this
// kernel; the caller then uses the CUDA-core kernel.
int dense_tc(float* out, const float* x, const float* w, int64_t n, int dim1, int dim2,
             const float* row_scale, int flags, float* const* publish_out, int num_publish, cudaStream_t st,
             bool* launched) {
    *launched = false;
    if (dim1 % 2 != 0 || ((uintptr_t)x % 8) != 0) return MGGB_OK;         // cp.async pieces are 8 or 16 bytes
    const int Npad = (dim2 + 15) / 16 * 16;
    if (Npad > 256) return MGGB_OK;
    const int nchunks = (dim1 + CHUNK_K - 1) / CHUNK_K;
    const size_t w_bytes = 2 * (size_t)nchunks * Npad * 128;
    const size_t budget = 225 * 1024;                                      // of the 227 KiB a CTA may use
    const size_t fixed = w_bytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
    if (fixed + 2 * STAGE_BYTES > budget) return MGGB_OK;                  // needs at least a 2-stage ring
    const int stages = (int)std::min<size_t>(MAX_STAGES, (budget - fixed) / STAGE_BYTES);
    unsigned tmem_cols = 32;
    while (tmem_cols < 2u * Npad) tmem_cols <<= 1;
    if (tmem_cols > 512) return MGGB_OK;

    TcParams P{};
    P.out = out; P.x = x; P.w = w; P.row_scale = row_scale; P.n = n;
    P.K = dim1; P.M = dim2; P.Npad = Npad; P.nchunks = nchunks; P.stages = stages;
    P.relu = (flags & MGGB_DENSE_RELU) ? 1 : 0;
    P.tmem_cols = tmem_cols;
    P.pub.n = num_publish;
    for (int q = 0; q < num_publish; q++) P.pub.dst[q] = publish_out[q];

    const size_t smem = fixed + (size_t)stages * STAGE_BYTES;
    int dev = 0, sms = 148;
    MGGB_CUDA(cudaGetDevice(&dev));
    MGGB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const long long tiles = (n + TILE_M - 1) / TILE_M;
    const int grid = (int)std::min<long long>(tiles, sms);
    const bool wide = (dim1 % 4 == 0) && ((uintptr_t)x % 16 == 0);
    if (wide) {
        MGGB_CUDA(cudaFuncSetAttribute(dense_tc_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        dense_tc_kernel<16><<<grid, THREADS, smem, st>>>(P);
    } else {
        MGGB_CUDA(cudaFuncSetAttribute(dense_tc_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        dense_tc_kernel<8><<<grid, THREADS, smem, st>>>(P);
    }
    MGGB_CUDA(cudaGetLastError());
    *launched = true;
    return MGGB_OK;
}

}  // namespace mggb

extern "C" int mggb_dense_device_status(int* status, int reset) {
    MGGB_REQUIRE(status, "dense_device_status: NULL output");
    MGGB_CUDA(cudaMemcpyFromSymbol(status, g_dense_status, sizeof(int)));
    if (reset) {
        const int zero = 0;
        MGGB_CUDA(cudaMemcpyToSymbol(g_dense_status, &zero, sizeof(int)));
    }
    return MGGB_OK;
}
