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
// MGGB_DENSE_TF32 keeps only hi * hi: one pass, operands truncated to 10 mantissa bits (about 1e-3).
//
// One persistent CTA per SM, 13 warps, no clusters:
//   bringing x in, a [128 rows x 32 floats] slab at a time, into a ring in the 128-byte-swizzled
//   K-major layout the tensor core reads, split into hi and lo slabs:
//     rows whose stride is a multiple of 16 bytes (dim1 % 4 == 0): TMA.  One thread (warp 13) issues
//              one cp.async.bulk.tensor.2d per slab (SWIZZLE_128B tensor map over x, no multicast,
//              this GPU's memory only; rows and columns past the matrix are zero-filled by the copy
//              engine); warps 0-7 split the landed slab in place.
//     other even dim1 (Reddit-shaped rows: 602 floats = 2408 bytes, which no tensor map takes):
//              warps 0-7 load 8-byte pieces into registers, several slabs ahead, and write hi/lo.
//     (aligned rows on a driver that cannot encode a tensor map: warps 0-3 cp.async 16-byte pieces, warps
//     4-7 split what landed.)
//   warp 12    allocates tensor memory; one lane issues tcgen05.mma (M=128, N=pad16(M), K=8 per
//              instruction, 4 k-steps x 4 partial products per slab) and commits to mbarriers.
//   warps 8-11 epilogue: tcgen05.ld the 128 x N accumulator (double-buffered in tensor memory), apply
//              row scale / ReLU, store the rows (and publish them to peers' replicas).
// w is split and laid out in shared memory once per CTA.  Every wait on an mbarrier is bounded: on
// expiry the CTA raises a status word the host can read (mggb_dense_device_status), drains its
// copies, frees its tensor memory and returns.
#include <cuda.h>
#include <algorithm>
#include <cstring>
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
constexpr int LOADERS = 128;              // warps 0-3 copy slabs, warps 4-7 split them (same piece mapping)
constexpr int LOADER_WARPS = LOADERS / 32;
constexpr int THREADS = 2 * LOADERS + 128 + 32;  // + 4 epilogue warps + the MMA warp
constexpr int MAX_STAGES = 4;               // ring depth (fewer when w leaves less room)
// Which warps bring x in: register-staged producers for 8-byte pieces, the cp.async loader/splitter
// pair for 16-byte pieces (each measured faster on its shapes, see producer_role).
template <int G> struct UseProducer { static constexpr bool value = (G == 8); };
constexpr int TMA_THREADS = 2 * LOADERS + 128 + 32 + 32;   // the TMA path adds warp 13, the copy issuer
// Consecutive K slabs a loader fetches per row visit: 2 for 8-byte pieces (a warp's copy instruction
// then covers 256 contiguous bytes of a row pair), 1 for 16-byte pieces.  Measured on B200; the copy
// rate is bound by the number of cp.async instructions an SM keeps in flight (about 40).
template <int G> struct Run { static constexpr int value = (G == 8) ? 2 : 1; };
constexpr unsigned SPIN_LIMIT = 1u << 22;
constexpr unsigned TF32_MASK = 0xFFFFE000u;

__device__ int g_dense_status = 0;   // 0 ok; otherwise which wait expired (1 full, 2 empty, 3 tmem_full, 4 tmem_empty, 5 landed)

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
    int K, M, Npad, nchunks, stages, relu, stage_out;
    int tf32;        // 1: one TF32 pass (hi * hi only); the lo halves are neither written nor multiplied
    int vec_store;   // 1: dim2 % 4 == 0 and out and every publish destination are 16-byte aligned (128-bit stores)
    int softmax;     // 1: the epilogue stores softmax(row) instead of the row (needs stage_out; no row scale, no ReLU)
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

// Which pieces of a slab a loader thread owns.  Piece q = i*LOADERS + p of the slab is row q / PPR,
// 16- or 8-byte piece q % PPR of that row.  LOADERS is a multiple of 8*PPR, so for a given thread the
// piece index and the row's position inside its 8-row swizzle group never change with i: the thread's
// pieces sit at a fixed stride in shared memory (whole swizzle groups) and in global memory (whole rows).
template <int G>
struct Pieces {
    static constexpr int PPR = 128 / G;                 // pieces per 128-byte slab row
    static constexpr int COUNT = TILE_M * PPR / LOADERS; // pieces per thread and slab
    static constexpr int ROW_STEP = LOADERS / PPR;      // rows between a thread's consecutive pieces
    static constexpr uint32_t SMEM_STEP = (ROW_STEP / 8) * 1024;
    static_assert(ROW_STEP % 8 == 0, "a thread's pieces must keep their place inside the swizzle group");
};

// Splits the pieces this thread copied for one slab into TF32-exact hi (in place) and lo parts.
template <int G>
__device__ __forceinline__ void split_slab(unsigned char* stage, uint32_t off0) {
    using PC = Pieces<G>;
#pragma unroll
    for (int i = 0; i < PC::COUNT; i++) {
        float* hi = reinterpret_cast<float*>(stage + off0 + i * PC::SMEM_STEP);
        float* lo = reinterpret_cast<float*>(stage + SLAB_BYTES + off0 + i * PC::SMEM_STEP);
        float v[G / 4];
        if (G == 16) *reinterpret_cast<float4*>(v) = *reinterpret_cast<const float4*>(hi);
        else         *reinterpret_cast<float2*>(v) = *reinterpret_cast<const float2*>(hi);
        float h[G / 4], l[G / 4];
#pragma unroll
        for (int e = 0; e < G / 4; e++) {
            h[e] = __uint_as_float(__float_as_uint(v[e]) & TF32_MASK);
            l[e] = __uint_as_float(__float_as_uint(v[e] - h[e]) & TF32_MASK);
        }
        if (G == 16) { *reinterpret_cast<float4*>(hi) = *reinterpret_cast<float4*>(h); *reinterpret_cast<float4*>(lo) = *reinterpret_cast<float4*>(l); }
        else         { *reinterpret_cast<float2*>(hi) = *reinterpret_cast<float2*>(h); *reinterpret_cast<float2*>(lo) = *reinterpret_cast<float2*>(l); }
    }
}

// Loaders only copy.  For slab c a loader waits until the ring stage is free, issues its cp.async
// pieces and lets the copy engine arrive on the stage's "landed" barrier when they complete
// (cp.async.mbarrier.arrive.noinc), so it never waits for data and every stage can be in flight.
template <int G>
__device__ void loader_role(const TcParams& P, unsigned char* ring, uint32_t landed0, uint32_t empty0,
                            volatile int* abort_flag, long long first_tile, long long tile_step, long long tiles) {
    using PC = Pieces<G>;
    const int p = threadIdx.x;                       // 0..LOADERS-1
    const int piece = p % PC::PPR, r0 = p / PC::PPR; // this thread's piece of the row, and its first row
    const uint32_t off0 = swz(r0, piece * G);        // byte offset of its first piece in a slab
    const int kpiece = piece * (G / 4);              // float offset of the piece inside the 32-float slab row
    const int S = P.stages;
    long long issued = 0;                            // slab counter of this CTA
    bool ok = true;
    for (long long tile = first_tile; tile < tiles && ok; tile += tile_step) {
        const long long row0 = tile * TILE_M + r0;
        const bool rows_full = tile * TILE_M + TILE_M <= P.n;
        // Slabs are fetched in groups of up to RUN consecutive K slabs of the same rows, piece by piece,
        // so that each row visit asks HBM for RUN*128 contiguous bytes instead of 128.
        constexpr int RUN = Run<G>::value;
        for (int kc0 = 0; kc0 < P.nchunks && ok; kc0 += RUN) {
            const int run = min(RUN, P.nchunks - kc0);
            uint32_t dst0[RUN];
            for (int j = 0; j < run; j++) {
                const long long c = issued + j;
                const int s = (int)(c % S);
                if (c / S >= 1) ok = ok && mbar_wait(empty0 + 8 * s, (unsigned)((c / S - 1) & 1), abort_flag, 2);
                dst0[j] = smem_u32(ring + (size_t)s * STAGE_BYTES) + off0;
            }
            if (!ok) break;
            const size_t src_step = (size_t)PC::ROW_STEP * P.K;
            const float* src0 = P.x + row0 * P.K + kc0 * CHUNK_K + kpiece;
            const bool all_valid = rows_full && (kc0 + run) * CHUNK_K <= P.K;
#pragma unroll
            for (int i = 0; i < PC::COUNT; i++) {
                const bool row_ok = all_valid || (row0 + i * PC::ROW_STEP < P.n);
#pragma unroll
                for (int j = 0; j < RUN; j++) {
                    if (j < run) {
                        const bool valid = row_ok && (all_valid || (kc0 + j) * CHUNK_K + kpiece < P.K);
                        cp_async_zfill<G>(dst0[j] + i * PC::SMEM_STEP, valid ? src0 + i * src_step + j * CHUNK_K : P.x, valid ? G : 0);
                    }
                }
            }
            for (int j = 0; j < run; j++)
                asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(landed0 + 8 * (int)((issued + j) % S)) : "memory");
            issued += run;
        }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");   // nothing of this thread's is in flight when it leaves
}

// Splitters turn a landed slab into its TF32-exact hi (in place) and lo halves and hand it to the
// tensor core.  Same piece mapping as the loaders, but a splitter reads pieces other threads copied:
// the "landed" barrier makes them visible.
template <int G>
__device__ void splitter_role(const TcParams& P, unsigned char* ring, uint32_t landed0, uint32_t full0,
                              volatile int* abort_flag, long long first_tile, long long tile_step, long long tiles) {
    using PC = Pieces<G>;
    const int p = threadIdx.x - LOADERS;
    const uint32_t off0 = swz(p / PC::PPR, (p % PC::PPR) * G);
    const int S = P.stages;
    long long done = 0;
    for (long long tile = first_tile; tile < tiles; tile += tile_step) {
        for (int kc = 0; kc < P.nchunks; kc++, done++) {
            const int s = (int)(done % S);
            if (!mbar_wait(landed0 + 8 * s, (unsigned)((done / S) & 1), abort_flag, 5)) return;
            split_slab<G>(ring + (size_t)s * STAGE_BYTES, off0);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the tensor core
            mbar_arrive(full0 + 8 * s);
        }
    }
}

// Register-staged producers, used for 8-byte pieces (rows that are only 8-byte aligned, e.g. 602
// floats); 16-byte pieces use the cp.async loader/splitter pair above.  All eight producer warps load
// their pieces of the next slabs into registers with streaming loads, then split the oldest slab
// (already in registers) into hi/lo straight into its ring stage and hand it to the tensor core.
// The slabs rotate through PIPE register buffers with the loop unrolled PIPE times, so no buffer is
// ever copied into another: a register move would wait for its load, and with it every later load
// would be issued only after the earlier one had returned.  PIPE - 1 slabs (16 KiB each) are in
// flight per SM while one is being split.
constexpr int PRODUCERS = 2 * LOADERS;
constexpr int PIPE = 4;

template <int G> struct PVec;
template <> struct PVec<16> { using T = float4; };
template <> struct PVec<8> { using T = float2; };

template <int G>
__device__ void producer_role(const TcParams& P, unsigned char* ring, uint32_t full0, uint32_t empty0,
                              volatile int* abort_flag, long long first_tile, long long tile_step, long long tiles) {
    using V = typename PVec<G>::T;
    constexpr int PPR = 128 / G;                       // pieces per 128-byte slab row
    constexpr int COUNT = TILE_M * PPR / PRODUCERS;    // pieces per thread and slab
    constexpr int ROW_STEP = PRODUCERS / PPR;          // rows between a thread's consecutive pieces
    constexpr uint32_t SMEM_STEP = (ROW_STEP / 8) * 1024;
    static_assert(ROW_STEP % 8 == 0 && COUNT >= 1, "piece mapping");
    const int p = threadIdx.x;                         // 0..PRODUCERS-1
    const int piece = p % PPR, r0 = p / PPR;
    const uint32_t off0 = swz(r0, piece * G);
    const int kpiece = piece * (G / 4);
    const int S = P.stages;
    const long long my_tiles = first_tile < tiles ? (tiles - first_tile + tile_step - 1) / tile_step : 0;
    const long long slabs = my_tiles * P.nchunks;
    const size_t src_step = (size_t)ROW_STEP * P.K;

    auto load_slab = [&](long long c, V* buf) {
        if (c >= slabs) return;
        const long long tile = first_tile + (c / P.nchunks) * tile_step;
        const int kc = (int)(c % P.nchunks);
        const long long row0 = tile * TILE_M + r0;
        const int k = kc * CHUNK_K + kpiece;
        const float* src0 = P.x + row0 * P.K + k;
        const bool k_ok = k < P.K;
        const bool rows_full = tile * TILE_M + TILE_M <= P.n;
#pragma unroll
        for (int i = 0; i < COUNT; i++) {
            V v = V{};
            if (k_ok && (rows_full || row0 + i * ROW_STEP < P.n)) v = __ldcs(reinterpret_cast<const V*>(src0 + i * src_step));
            buf[i] = v;
        }
    };
    // splits the slab held in buf into hi/lo in its ring stage and hands it to the tensor core
    auto store_slab = [&](long long c, const V* buf) -> bool {
        const int s = (int)(c % S);
        const long long use = c / S;
        if (use >= 1 && !mbar_wait(empty0 + 8 * s, (unsigned)((use - 1) & 1), abort_flag, 2)) return false;
        unsigned char* stage = ring + (size_t)s * STAGE_BYTES;
#pragma unroll
        for (int i = 0; i < COUNT; i++) {
            const float* v = reinterpret_cast<const float*>(&buf[i]);
            float h[G / 4], l[G / 4];
#pragma unroll
            for (int e = 0; e < G / 4; e++) {
                h[e] = __uint_as_float(__float_as_uint(v[e]) & TF32_MASK);
                l[e] = __uint_as_float(__float_as_uint(v[e] - h[e]) & TF32_MASK);
            }
            *reinterpret_cast<V*>(stage + off0 + i * SMEM_STEP) = *reinterpret_cast<V*>(h);
            if (!P.tf32) *reinterpret_cast<V*>(stage + SLAB_BYTES + off0 + i * SMEM_STEP) = *reinterpret_cast<V*>(l);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the tensor core
        mbar_arrive(full0 + 8 * s);
        return true;
    };

    // A slab is 128 bytes of each of 128 rows: on its own that is a strided walk through DRAM (one short
    // read per row, 19 passes over a 602-float row), which HBM serves at a fraction of its streaming rate.
    // So the CTA's NEXT tile - one contiguous range of 128 rows - is requested into L2 as a whole
    // (cp.async.bulk.prefetch.L2, a few threads, 8 KiB each) while the current tile is consumed: DRAM sees
    // a sequential stream and the strided slab reads hit L2.  The streaming loads above evict what they
    // have read first, so the working set in L2 stays near one tile per SM.
    const bool can_prefetch = ((uintptr_t)P.x % 16) == 0;
    auto prefetch_tile = [&](long long t) {       // t-th tile of this CTA
        if (!can_prefetch || t >= my_tiles) return;
        const long long tile = first_tile + t * tile_step;
        const long long rows = min((long long)TILE_M, P.n - tile * TILE_M);
        const long long bytes = (rows * P.K * 4) & ~15LL;
        const long long off = (long long)p * 8192;
        if (off < bytes) {
            const char* src = reinterpret_cast<const char*>(P.x + tile * TILE_M * P.K) + off;
            const unsigned sz = (unsigned)min(8192LL, bytes - off);
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(sz) : "memory");
        }
    };
    prefetch_tile(0);
    prefetch_tile(1);

    V buf[PIPE][COUNT];
#pragma unroll
    for (int j = 0; j < PIPE - 1; j++) load_slab(j, buf[j]);
    for (long long c0 = 0; c0 < slabs; c0 += PIPE) {
#pragma unroll
        for (int j = 0; j < PIPE; j++) {
            const long long c = c0 + j;
            if (c < slabs) {
                if (c % P.nchunks == 0 && c > 0) prefetch_tile(c / P.nchunks + 1);   // entering tile c/nchunks: ask for the one after
                load_slab(c + PIPE - 1, buf[(j + PIPE - 1) % PIPE]);   // the buffer split in the previous step is free again
                if (!store_slab(c, buf[j])) return;
            }
        }
    }
}

// TMA path (row stride a multiple of 16 bytes).  The issuer: one thread, one tensor copy per slab.
__device__ void tma_issuer_role(const TcParams& P, const CUtensorMap* tmap, uint32_t ring_base, uint32_t landed0, uint32_t empty0,
                                volatile int* abort_flag, long long first_tile, long long tile_step, long long tiles) {
    const int S = P.stages;
    long long c = 0;
    for (long long tile = first_tile; tile < tiles; tile += tile_step) {
        for (int kc = 0; kc < P.nchunks; kc++, c++) {
            const int s = (int)(c % S);
            if (c / S >= 1 && !mbar_wait(empty0 + 8 * s, (unsigned)((c / S - 1) & 1), abort_flag, 2)) return;
            const uint32_t bar = landed0 + 8 * s;
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((unsigned)SLAB_BYTES) : "memory");
            // coordinates: x = first float of the K slab (a multiple of 32 floats = 128 bytes), y = first row of the tile
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                         ::"r"(ring_base + (uint32_t)s * STAGE_BYTES), "l"(tmap), "r"(kc * CHUNK_K), "r"((int)(tile * TILE_M)), "r"(bar) : "memory");
        }
    }
}

// The splitters of the TMA path: eight warps turn the landed raw slab into hi (in place) and lo.
__device__ void tma_splitter_role(const TcParams& P, unsigned char* ring, uint32_t landed0, uint32_t full0,
                                  volatile int* abort_flag, long long first_tile, long long tile_step, long long tiles) {
    constexpr int PPR = 8;                                // 16-byte pieces per 128-byte slab row
    constexpr int COUNT = TILE_M * PPR / PRODUCERS;       // pieces per thread and slab
    constexpr int ROW_STEP = PRODUCERS / PPR;
    constexpr uint32_t SMEM_STEP = (ROW_STEP / 8) * 1024;
    const int p = threadIdx.x;
    const uint32_t off0 = swz(p / PPR, (p % PPR) * 16);
    const int S = P.stages;
    const long long my_tiles = first_tile < tiles ? (tiles - first_tile + tile_step - 1) / tile_step : 0;
    const long long slabs = my_tiles * P.nchunks;
    for (long long c = 0; c < slabs; c++) {
        const int s = (int)(c % S);
        if (!mbar_wait(landed0 + 8 * s, (unsigned)((c / S) & 1), abort_flag, 5)) return;
        unsigned char* stage = ring + (size_t)s * STAGE_BYTES;
        float4 v[COUNT];
#pragma unroll
        for (int i = 0; i < COUNT; i++) v[i] = *reinterpret_cast<const float4*>(stage + off0 + i * SMEM_STEP);
#pragma unroll
        for (int i = 0; i < COUNT; i++) {
            const float* f = reinterpret_cast<const float*>(&v[i]);
            float h[4], l[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                h[e] = __uint_as_float(__float_as_uint(f[e]) & TF32_MASK);
                l[e] = __uint_as_float(__float_as_uint(f[e] - h[e]) & TF32_MASK);
            }
            // The hi half is NOT written back: the slab holds the raw fp32 values and the tensor core reads a
            // TF32 operand from the upper 19 bits of each 32-bit container, ignoring the lower 13: the
            // truncation that h stands for.  Only the lo half (the exact remainder v - h) is stored.
            if (!P.tf32) *reinterpret_cast<float4*>(stage + SLAB_BYTES + off0 + i * SMEM_STEP) = *reinterpret_cast<float4*>(l);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the tensor core
        mbar_arrive(full0 + 8 * s);
    }
}

__device__ void mma_role(const TcParams& P, uint32_t ring_base, uint32_t w_base, uint32_t full0,
                         uint32_t empty0, uint32_t tfull0, uint32_t tempty0, uint32_t tmem_base,
                         volatile int* abort_flag, long long first_tile, long long tile_step, long long tiles) {
    const int S = P.stages;
    const uint32_t panel = 2u * (uint32_t)P.Npad * 128u;     // hi rows then lo rows of one K chunk
    // instruction descriptor: D fp32, A/B TF32, both K-major, M = 128, N = 2*Npad (hi and lo columns of w side by
    // side in the accumulator) or Npad for the single-pass mode (hi only)
    const uint32_t ncols = (uint32_t)(P.tf32 ? P.Npad : 2 * P.Npad);
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((ncols >> 3) << 17) | ((uint32_t)(TILE_M >> 4) << 24);
    long long consumed = 0, t = 0;
    for (long long tile = first_tile; tile < tiles; tile += tile_step, t++) {
        const int buf = (int)(t & 1);
        const long long use_t = t >> 1;
        if (use_t >= 1 && !mbar_wait(tempty0 + 8 * buf, (unsigned)((use_t - 1) & 1), abort_flag, 4)) return;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * 2 * P.Npad);
        for (int kc = 0; kc < P.nchunks; kc++, consumed++) {
            const int s = (int)(consumed % S);
            if (!mbar_wait(full0 + 8 * s, (unsigned)((consumed / S) & 1), abort_flag, 1)) return;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_hi = ring_base + (uint32_t)s * STAGE_BYTES, a_lo = a_hi + SLAB_BYTES;
            const uint32_t b = w_base + (uint32_t)kc * panel;
#pragma unroll
            for (int ks = 0; ks < CHUNK_K / 8; ks++) {
                const uint32_t koff = (uint32_t)ks * 32u;   // 8 TF32 = 32 bytes along K inside the swizzled row
                const uint64_t db = umma_desc(b + koff);
                umma_tf32(d_tmem, umma_desc(a_hi + koff), db, idesc, (kc > 0 || ks > 0) ? 1u : 0u);   // x_hi * [w_hi | w_lo]
                if (!P.tf32) umma_tf32(d_tmem, umma_desc(a_lo + koff), db, idesc, 1u);                 // x_lo * [w_hi | w_lo]
            }
            umma_commit(empty0 + 8 * s);            // the slab may be overwritten once these MMAs are done
        }
        umma_commit(tfull0 + 8 * buf);              // the accumulator of this tile is complete
    }
}

// e^d for d <= 0 as 2^(d * log2 e) on the special-function unit (relative error below 1e-6 * max(1, |d| / 10), flushed to
// 0 below d = -87): the same exponential as the CUDA-core fused dense + softmax kernel
__device__ __forceinline__ float exp_neg(float d) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d * 1.4426950408889634f));
    return r;
}

__device__ void epilogue_role(const TcParams& P, float* out_stage, uint32_t tfull0, uint32_t tempty0, uint32_t tmem_base,
                              volatile int* abort_flag, long long first_tile, long long tile_step, long long tiles) {
    const int quarter = (threadIdx.x >> 5) & 3;   // a warp may only read tensor-memory lanes 32*(warp%4) ..
    const int lane = threadIdx.x & 31;
    long long t = 0;
    for (long long tile = first_tile; tile < tiles; tile += tile_step, t++) {
        const int buf = (int)(t & 1);
        // all lanes leave together: tcgen05.ld below needs the whole warp
        if (!__all_sync(0xffffffffu, mbar_wait(tfull0 + 8 * buf, (unsigned)((t >> 1) & 1), abort_flag, 3))) return;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const long long row = tile * TILE_M + quarter * 32 + lane;
        const float scale = (P.row_scale && row < P.n) ? P.row_scale[row] : 1.f;
        // 16 columns c0.. of this thread's row: columns c0.. of the accumulator hold x * w_hi, columns Npad + c0.. hold
        // x * w_lo, and the product is their sum
        auto load_chunk = [&](int c0, float (&v)[16]) {
            uint32_t r[16], q[16];
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * 2 * P.Npad + c0);
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                  "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                : "r"(taddr));
            if (!P.tf32) {
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                    : "=r"(q[0]), "=r"(q[1]), "=r"(q[2]), "=r"(q[3]), "=r"(q[4]), "=r"(q[5]), "=r"(q[6]), "=r"(q[7]),
                      "=r"(q[8]), "=r"(q[9]), "=r"(q[10]), "=r"(q[11]), "=r"(q[12]), "=r"(q[13]), "=r"(q[14]), "=r"(q[15])
                    : "r"(taddr + (uint32_t)P.Npad));
            }
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int j = 0; j < 16; j++) v[j] = P.tf32 ? __uint_as_float(r[j]) : __uint_as_float(r[j]) + __uint_as_float(q[j]);
        };
        if (P.softmax) {
            // Each thread owns a whole row of the accumulator, so the row's maximum and its sum of exponentials need no
            // exchange between threads: one pass over tensor memory for the maximum, a second for exp(v - max), which is
            // parked in the staging rows together with 1 / sum (in the pitch's spare column) for the coalesced store.
            float m = -3.402823466e38f;
            for (int c0 = 0; c0 < P.Npad; c0 += 16) {
                float v[16];
                load_chunk(c0, v);
#pragma unroll
                for (int j = 0; j < 16; j++)
                    if (c0 + j < P.M) m = fmaxf(m, v[j]);
            }
            float sum = 0.f;
            for (int c0 = 0; c0 < P.Npad; c0 += 16) {
                float v[16];
                load_chunk(c0, v);
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const float e = (c0 + j < P.M) ? exp_neg(v[j] - m) : 0.f;
                    sum += e;
                    out_stage[lane * (P.Npad + 1) + c0 + j] = e;
                }
            }
            out_stage[lane * (P.Npad + 1) + P.Npad] = 1.f / sum;
        }
        for (int c0 = 0; !P.softmax && c0 < P.Npad; c0 += 16) {
            float acc[16];
            load_chunk(c0, acc);
            if (row < P.n) {
                float v[16];
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    v[j] = acc[j] * scale;
                    if (P.relu) v[j] = fmaxf(v[j], 0.f);
                }
                const long long o = row * P.M + c0;
                if (out_stage != nullptr) {
                    // park the row in shared memory; the warp stores its 32 rows coalesced below
#pragma unroll
                    for (int j = 0; j < 16; j++) out_stage[lane * (P.Npad + 1) + c0 + j] = v[j];   // odd pitch: no bank conflicts
                } else if (P.vec_store && c0 + 16 <= P.M) {
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
        mbar_arrive(tempty0 + 8 * buf);   // the accumulator is in registers / shared memory: free it early
        if (out_stage != nullptr) {
            // The warp's 32 rows are one contiguous run of 32*M floats in the output (and in every
            // replica it publishes to): consecutive lanes store consecutive addresses, so a peer
            // receives full 128- to 512-byte writes instead of one 16-byte piece per row.
            __syncwarp();
            const long long first = tile * TILE_M + quarter * 32;
            const int total = (int)max(0LL, min(32LL, P.n - first)) * P.M;
            const long long o = first * P.M;
            const float inv_m = 1.0f / (float)P.M;   // (i + 0.5) * inv_m truncates to i / M exactly for i < 2^13
            if (P.vec_store) {
                for (int i = lane * 4; i < total; i += 128) {
                    const int r = (int)(((float)i + 0.5f) * inv_m);
                    const float* src = out_stage + r * (P.Npad + 1) + (i - r * P.M);
                    const float k = P.softmax ? out_stage[r * (P.Npad + 1) + P.Npad] : 1.f;
                    const float4 f = make_float4(src[0] * k, src[1] * k, src[2] * k, src[3] * k);
                    *reinterpret_cast<float4*>(P.out + o + i) = f;
                    for (int q = 0; q < P.pub.n; q++) *reinterpret_cast<float4*>(P.pub.dst[q] + o + i) = f;
                }
            } else {
                for (int i = lane; i < total; i += 32) {
                    const int r = (int)(((float)i + 0.5f) * inv_m);
                    const float f = out_stage[r * (P.Npad + 1) + (i - r * P.M)] * (P.softmax ? out_stage[r * (P.Npad + 1) + P.Npad] : 1.f);
                    P.out[o + i] = f;
                    for (int q = 0; q < P.pub.n; q++) P.pub.dst[q][o + i] = f;
                }
            }
            __syncwarp();
        }
    }
}

// G: bytes per piece of the loaders (8 or 16), or 0 for the TMA path (tmap then describes x).
template <int G>
__global__ void __launch_bounds__(G == 0 ? TMA_THREADS : THREADS, 1) dense_tc_kernel(const TcParams P, const __grid_constant__ CUtensorMap tmap) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // carve: [w_hi][w_lo][ring][barriers][tmem ptr]; every region a multiple of 1024 bytes
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // w: per K chunk one panel of [2*Npad rows x 32 floats]: rows 0..Npad-1 hold the hi part of w's
    // columns, rows Npad..2*Npad-1 the lo part, so ONE tensor-core instruction with N = 2*Npad multiplies a
    // slab by both and x's slabs are read from shared memory twice per k-step (hi, lo) instead of four times.
    const size_t w_bytes = (size_t)P.nchunks * P.Npad * 128;
    unsigned char* w_hi = base;
    unsigned char* ring = base + 2 * w_bytes;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(ring + (size_t)P.stages * STAGE_BYTES);
    // bars: full[MAX_STAGES], empty[MAX_STAGES], tmem_full[2], tmem_empty[2], landed[MAX_STAGES]
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;

    const int warp = threadIdx.x >> 5;
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * MAX_STAGES;
    const uint32_t tfull0 = empty0 + 8 * MAX_STAGES, tempty0 = tfull0 + 16, landed0 = tempty0 + 16;

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < MAX_STAGES; s++) {
            mbar_init(full0 + 8 * s, (G == 0 || UseProducer<G>::value) ? PRODUCERS : LOADERS);
            mbar_init(empty0 + 8 * s, 1);
            mbar_init(landed0 + 8 * s, G == 0 ? 1 : LOADERS);
        }
        for (int b = 0; b < 2; b++) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, 128); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2 * LOADER_WARPS + 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)), "r"(P.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // w, split into hi/lo, transposed into K-major swizzled panels of [Npad rows x 32 floats]
    for (int idx = threadIdx.x; idx < P.nchunks * CHUNK_K * P.Npad; idx += blockDim.x) {
        const int nn = idx % P.Npad, kk = (idx / P.Npad) % CHUNK_K, kc = idx / (P.Npad * CHUNK_K);
        const int k = kc * CHUNK_K + kk;
        const float v = (k < P.K && nn < P.M) ? __ldg(P.w + (long long)k * P.M + nn) : 0.f;
        const float h = __uint_as_float(__float_as_uint(v) & TF32_MASK);
        const uint32_t chunk0 = (uint32_t)kc * 2u * P.Npad * 128u;
        *reinterpret_cast<float*>(w_hi + chunk0 + swz(nn, kk * 4)) = h;
        *reinterpret_cast<float*>(w_hi + chunk0 + swz(P.Npad + nn, kk * 4)) = __uint_as_float(__float_as_uint(v - h) & TF32_MASK);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = s_tmem_base;

    const long long tiles = (P.n + TILE_M - 1) / TILE_M;
    if (G == 0 && warp < 2 * LOADER_WARPS) {
        tma_splitter_role(P, ring, landed0, full0, &s_abort, blockIdx.x, gridDim.x, tiles);
    } else if (G == 0 && warp == 2 * LOADER_WARPS + 5) {
        if ((threadIdx.x & 31) == 0)
            tma_issuer_role(P, &tmap, smem_u32(ring), landed0, empty0, &s_abort, blockIdx.x, gridDim.x, tiles);
    } else if (UseProducer<G>::value && warp < 2 * LOADER_WARPS) {
        producer_role<(G == 0 ? 8 : G)>(P, ring, full0, empty0, &s_abort, blockIdx.x, gridDim.x, tiles);
    } else if (G != 0 && warp < LOADER_WARPS) {
        loader_role<(G == 0 ? 16 : G)>(P, ring, landed0, empty0, &s_abort, blockIdx.x, gridDim.x, tiles);
    } else if (G != 0 && warp < 2 * LOADER_WARPS) {
        splitter_role<(G == 0 ? 16 : G)>(P, ring, landed0, full0, &s_abort, blockIdx.x, gridDim.x, tiles);
    } else if (warp < 2 * LOADER_WARPS + 4) {
        // staging rows (odd output widths, publishing calls): 32 rows x (Npad+1) floats per epilogue warp, after the barriers
        float* out_stage = P.stage_out ? reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(bars) + 256) +
                                             (size_t)(warp - 2 * LOADER_WARPS) * 32 * (P.Npad + 1) : nullptr;
        epilogue_role(P, out_stage, tfull0, tempty0, tmem_base, &s_abort, blockIdx.x, gridDim.x, tiles);
    } else if ((threadIdx.x & 31) == 0) {
        mma_role(P, smem_u32(ring), smem_u32(w_hi), full0, empty0, tfull0, tempty0, tmem_base,
                 &s_abort, blockIdx.x, gridDim.x, tiles);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 2 * LOADER_WARPS + 4) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(P.tmem_cols) : "memory");
    }
}

}  // namespace

namespace {

// cuTensorMapEncodeTiled, looked up through the runtime so that the library does not link against
// the driver library (machines that only build it have none).  NULL when the driver offers none.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static bool looked = false;
    if (!looked) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        looked = true;
    }
    return fn;
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
    if (Npad > 128) return MGGB_OK;     // the accumulator holds 2*Npad columns (x*w_hi | x*w_lo) and one instruction spans them
    const int nchunks = (dim1 + CHUNK_K - 1) / CHUNK_K;
    if (nchunks < 2) return MGGB_OK;   // one slab per tile leaves the four epilogue warps as the limit: the CUDA-core kernel is faster
    const size_t w_bytes = 2 * (size_t)nchunks * Npad * 128;
    const size_t budget = 225 * 1024;                                      // of the 227 KiB a CTA may use
    // coalescing buffer: for odd widths, and whenever rows are also published to peers
    const bool softmax = (flags & DENSE_TC_SOFTMAX) != 0;   // internal: the fused last layer
    // (staging every output, also rows of a multiple of 4 floats that nobody else receives, was measured slower than the
    // epilogue's strided 16-byte stores: 2,449,029 x 64 -> 64 in 0.41 ms against 0.29 ms)
    const size_t out_stage_bytes = (dim2 % 4 != 0 || num_publish > 0 || softmax) ? (size_t)4 * 32 * (Npad + 1) * sizeof(float) : 0;
    size_t fixed = w_bytes + 1024 /*alignment slack*/ + 256 /*barriers*/ + out_stage_bytes;
    bool stage_out = out_stage_bytes != 0;
    if (stage_out && fixed + 2 * STAGE_BYTES > budget) {
        if (softmax) return MGGB_OK;     // the softmax epilogue needs the staging rows
        fixed -= out_stage_bytes; stage_out = false;   // no room: strided stores
    }
    if (fixed + 2 * STAGE_BYTES > budget) return MGGB_OK;                  // needs at least a 2-stage ring
    const int stages = (int)std::min<size_t>(MAX_STAGES, (budget - fixed) / STAGE_BYTES);
    unsigned tmem_cols = 32;
    while (tmem_cols < 4u * Npad) tmem_cols <<= 1;      // two accumulators (double buffering) of 2*Npad columns
    if (tmem_cols > 512) return MGGB_OK;

    TcParams P{};
    P.out = out; P.x = x; P.w = w; P.row_scale = row_scale; P.n = n;
    P.K = dim1; P.M = dim2; P.Npad = Npad; P.nchunks = nchunks; P.stages = stages;
    P.relu = (flags & MGGB_DENSE_RELU) ? 1 : 0;
    P.tf32 = (flags & MGGB_DENSE_TF32) ? 1 : 0;
    P.stage_out = stage_out ? 1 : 0;
    P.softmax = softmax ? 1 : 0;
    // 128-bit stores need 16-byte aligned destinations (a view that starts at an odd float offset is
    // not); otherwise the epilogue stores float by float.
    bool vec_store = (dim2 % 4 == 0) && ((uintptr_t)out % 16 == 0);
    for (int q = 0; q < num_publish; q++) vec_store = vec_store && ((uintptr_t)publish_out[q] % 16 == 0);
    P.vec_store = vec_store ? 1 : 0;
    P.tmem_cols = tmem_cols;
    P.pub.n = num_publish;
    for (int q = 0; q < num_publish; q++) P.pub.dst[q] = publish_out[q];

    const size_t smem = fixed + (size_t)stages * STAGE_BYTES;
    const int sms = mggb::sm_count();
    const long long tiles = (n + TILE_M - 1) / TILE_M;
    const int grid = (int)std::min<long long>(tiles, sms);
    const bool wide = (dim1 % 4 == 0) && ((uintptr_t)x % 16 == 0);
    CUtensorMap tmap;
    memset(&tmap, 0, sizeof(tmap));
    if (wide && encode_tiled() != nullptr) {
        // x as a 2-D tensor [n rows][dim1 floats] (row stride dim1 * 4 bytes, a multiple of 16); one box = one slab
        const cuuint64_t gdim[2] = {(cuuint64_t)dim1, (cuuint64_t)n};
        const cuuint64_t gstride[1] = {(cuuint64_t)dim1 * sizeof(float)};
        const cuuint32_t box[2] = {(cuuint32_t)CHUNK_K, (cuuint32_t)TILE_M};
        const cuuint32_t estride[2] = {1, 1};
        CUresult r = encode_tiled()(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(x), gdim, gstride, box, estride,
                                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return mggb::fail(MGGB_ERR_CUDA, "dense_forward: cuTensorMapEncodeTiled failed with CUresult %d (n=%lld dim1=%d)", (int)r, (long long)n, dim1);
        MGGB_CUDA(cudaFuncSetAttribute(dense_tc_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        dense_tc_kernel<0><<<grid, TMA_THREADS, smem, st>>>(P, tmap);
    } else if (wide) {      // a driver without the tensor-map entry point: the cp.async loader / splitter pair
        MGGB_CUDA(cudaFuncSetAttribute(dense_tc_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        dense_tc_kernel<16><<<grid, THREADS, smem, st>>>(P, tmap);
    } else {
        MGGB_CUDA(cudaFuncSetAttribute(dense_tc_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        dense_tc_kernel<8><<<grid, THREADS, smem, st>>>(P, tmap);
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
