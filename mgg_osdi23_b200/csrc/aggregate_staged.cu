// Neighbor aggregation with rows staged through shared memory by bulk asynchronous copies (sm_100a).
//
// Same operator and the same work map as aggregate.cu (one block per node, `wpb` warps, a warp takes
// `dist*ps` consecutive neighbors per turn: include/neighbor_utils.cuh:1395-1400, :1432-1437), but a
// neighbor's row is not loaded into registers by the warp's lanes: each lane asks the copy engine
// for one whole row (cp.async.bulk global -> shared, completion counted on an mbarrier), 32 rows per
// batch, into a per-warp ring of stages.  The warp then adds the rows up from shared memory.
//
// Why it exists.  A row gathered through the load/store unit holds registers and an L1 miss slot for
// as long as it is in flight; rows that come over NVLink from a peer's memory (the reference's
// blocking nvshmemx_float_get_warp, include/neighbor_utils.cuh:1445) are in flight for microseconds.
// Bulk copies are queued in the copy engine, cost the warp nothing while they fly, and land in
// shared memory.  The copies for the first stages of the REMOTE list are issued before the warp
// walks its LOCAL list, so remote latency hides behind the local gather; later remote batches are
// double-buffered (stage k+1 in flight while stage k is added up).
// What measuring it on B200 showed (MGGB_AGG_STAGE_ROWS selects it; it is NOT the default): 64-byte
// rows pulled from a peer arrive at 530 GB/s per GPU with either path (the link's rate for reads of
// that size; 670 GB/s from 128-byte rows up), so for remote rows it is a tie; for rows of this GPU's
// own memory it is 3.7x slower than register loads (2.5 ms against 0.68 ms on 115 M 64-byte rows that
// sit in L2; 15.7 ms against 4.8 ms on 124 M 256-byte rows from HBM): an SM's copy engine keeps only
// about a hundred row-sized copies in flight, far fewer bytes than its warps' loads do.
//
// STAGE bit 0: the remote list (owner lookup, REMOTE_MODE 1) is staged; bit 1: the directly
// addressed lists are staged too (wide rows, where registers limit the bytes in flight).
// No copy here uses cluster multicast, and no tensor map: plain 1-D bulk copies of one row each,
// from this GPU's memory or a peer-mapped pointer.  Every mbarrier wait is bounded; on expiry the
// block raises a status word (mggb_agg_device_status), lets its pending copies drain for a bounded
// time and returns.
#include <algorithm>
#include "aggregate_core.cuh"

namespace {

__device__ int g_agg_status = 0;   // 0 ok; 1 = a staged batch never arrived within the wait limit

constexpr unsigned WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool mbar_try(uint32_t bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// One neighbor list as this warp sees it: its share of the edges [beg, end), chunk after chunk, as
// one virtual sequence of `total` edges; edge k of the sequence sits at pos(k).
struct WarpList {
    const int32_t* ci;
    unsigned beg, chunk, stride_chunks, warp, total;
    bool remote;   // owner lookup (peer table) or direct addressing
    const char* base;
    __device__ __forceinline__ unsigned pos(unsigned k) const {
        const unsigned q = k / chunk;
        return beg + (q * stride_chunks + warp) * chunk + (k - q * chunk);
    }
};

__device__ __forceinline__ WarpList make_list(const int32_t* ci, int beg, int end, unsigned chunk, int warp, int nwarps,
                                              bool remote, const char* base) {
    WarpList L;
    L.ci = ci; L.beg = (unsigned)beg; L.chunk = chunk; L.stride_chunks = (unsigned)nwarps; L.warp = (unsigned)warp;
    L.remote = remote; L.base = base;
    const unsigned len = (unsigned)(end - beg), full = len / chunk, rem = len - full * chunk;
    const unsigned mine = full / nwarps + ((unsigned)warp < full % nwarps ? 1u : 0u);
    L.total = mine * chunk + ((unsigned)warp == full % nwarps ? rem : 0u);
    return L;
}

// Asks the copy engine for the rows of batch `b` (edges 32b .. 32b+31 of the warp's sequence) into
// ring stage `stage`; lane k's row lands in slot k.
template <bool REMOTE_LOOKUP>
__device__ __forceinline__ void issue_batch(const AggParams& P, const float* const* s_peer, const WarpList& L, unsigned b,
                                            unsigned char* stage, uint32_t bar, unsigned row_bytes, int lane) {
    const unsigned k = b * 32u + (unsigned)lane;
    const unsigned cnt = min(32u, L.total - b * 32u);
    if (lane == 0)
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(cnt * row_bytes) : "memory");
    __syncwarp();
    if (k < L.total) {
        const int nid = __ldcs(L.ci + L.pos(k));
        const void* src;
        if (REMOTE_LOOKUP && L.remote) {
            const unsigned owner = (unsigned)(((unsigned long long)(unsigned)nid * P.div_magic) >> P.div_shift);
            src = s_peer[owner] + (long long)(nid - (int)owner * P.node_per_pe) * P.dim;
        } else {
            src = L.base + (long long)nid * row_bytes;
        }
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(smem_addr(stage + (size_t)lane * row_bytes)), "l"(src), "r"(row_bytes), "r"(bar) : "memory");
    }
}

// Waits (bounded) for a stage and adds its `cnt` rows into acc: sub-warp g reads row r*G+g, lane l of
// it the row's l-th 16 bytes.
template <int LPR>
__device__ __forceinline__ bool consume_batch(Vec<4>& acc, const unsigned char* stage, uint32_t bar, unsigned parity,
                                              unsigned cnt, unsigned row_bytes, int lane) {
    bool ok = false;
    for (unsigned i = 0; i < WAIT_LIMIT; i++)
        if (mbar_try(bar, parity)) { ok = true; break; }
    if (!__all_sync(0xffffffffu, ok)) return false;      // the warp gives up together
    constexpr int G = 32 / LPR;
    constexpr int U = LPR < MGGB_AGG_MAX_ROUNDS ? LPR : MGGB_AGG_MAX_ROUNDS;
    const int g = lane / LPR, l = lane % LPR;
#pragma unroll 1
    for (int r0 = 0; r0 < LPR; r0 += U) {
        if ((unsigned)(r0 * G) >= cnt) break;
        float4 v[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const unsigned j = (unsigned)((r0 + u) * G + g);
            v[u] = j < cnt ? *reinterpret_cast<const float4*>(stage + (size_t)j * row_bytes + l * 16) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < U; u++) { acc.v.x += v[u].x; acc.v.y += v[u].y; acc.v.z += v[u].z; acc.v.w += v[u].w; }
    }
    return true;
}

// One block per node, dim == 4 * LPR.  Dynamic shared memory: [nwarps * dim floats of partial rows]
// [nwarps rings of S stages x 32 rows]; the mbarriers are static.
//   REMOTE_MODE as in aggregate.cu (0 one PE, 1 owner lookup, 2 one replica matrix);
//   STAGE bit 0: remote list staged (REMOTE_MODE 1); bit 1: directly addressed lists staged.
constexpr int MAX_WARPS = 16;
constexpr int MAX_STAGES = 4;

template <int LPR, int REMOTE_MODE, int STAGE>
__global__ void __launch_bounds__(512, 1) sag_staged_kernel(const AggParams P, const int stages) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long s_bar[MAX_WARPS * MAX_STAGES];
    __shared__ const float* s_peer[MGGB_MAX_PES];
    __shared__ int s_deferred;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const unsigned row_bytes = (unsigned)P.dim * 4u;
    float* s_part = reinterpret_cast<float*>(smem_raw);
    // rings start on a 128-byte boundary after the partial rows
    unsigned char* rings = smem_raw + (((size_t)nwarps * row_bytes + 127) & ~(size_t)127);
    unsigned char* ring = rings + (size_t)warp * stages * 32 * row_bytes;
    const uint32_t bar0 = smem_addr(&s_bar[warp * MAX_STAGES]);

    const int row = P.row_order ? P.row_order[blockIdx.x] : (int)blockIdx.x;
    if (threadIdx.x < MGGB_MAX_PES) s_peer[threadIdx.x] = P.peer[threadIdx.x < P.num_pes ? threadIdx.x : 0];
    if (lane == 0)
        for (int s = 0; s < stages; s++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar0 + 8 * s));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();

    const int lbeg = P.rp_l[row], lend = P.rp_l[row + 1];
    const int rbeg = P.rp_r[row], rend = P.rp_r[row + 1];
    if (P.hub_count != nullptr && (lend - lbeg) + (rend - rbeg) > P.hub_min_edges) {
        if (threadIdx.x == 0) s_deferred = defer_row(P, row, (lend - lbeg) + (rend - rbeg));
        __syncthreads();
        if (s_deferred) return;      // no copy has been issued yet
    }

    const unsigned chunk = (unsigned)P.chunk;
    const int l = lane % LPR;
    // the remote list's chunks are dealt to the warps continuing from where the local list's stopped (as in aggregate.cu)
    const int rwarp = (warp + nwarps - (int)(((unsigned)(lend - lbeg) + chunk - 1) / chunk % nwarps)) % nwarps;
    const char* lbase = reinterpret_cast<const char*>(P.peer[P.pe]) - (long long)P.lb * row_bytes;
    const char* rbase = reinterpret_cast<const char*>(P.peer[0]);      // REMOTE_MODE 2: one matrix indexed by global id
    WarpList lists[2];
    int nlists = 0;
    if (STAGE & 2) lists[nlists++] = make_list(P.ci_l, lbeg, lend, chunk, warp, nwarps, false, lbase);
    if (REMOTE_MODE == 1 && (STAGE & 1)) lists[nlists++] = make_list(P.ci_r, rbeg, rend, chunk, rwarp, nwarps, true, nullptr);
    if (REMOTE_MODE == 2 && (STAGE & 2)) lists[nlists++] = make_list(P.ci_r, rbeg, rend, chunk, rwarp, nwarps, false, rbase);
    unsigned nb[2] = {0, 0};
    for (int i = 0; i < nlists; i++) nb[i] = (lists[i].total + 31u) / 32u;
    const unsigned T = nb[0] + nb[1];                 // batches of this warp, list 0 first

    auto issue = [&](unsigned t) {
        const unsigned s = t % (unsigned)stages;
        const int li = t < nb[0] ? 0 : 1;
        issue_batch<REMOTE_MODE == 1>(P, s_peer, lists[li], t - (li ? nb[0] : 0u), ring + (size_t)s * 32 * row_bytes, bar0 + 8 * s, row_bytes, lane);
    };
    for (unsigned t = 0; t < min(T, (unsigned)stages); t++) issue(t);

    Vec<4> acc;
    acc.zero();
    // lists that are not staged go through the register path while the first copies fly
    if (!(STAGE & 2)) {
        const char* lb_col = lbase + l * 16;
        gather_list<LPR, 4, false, 2>(acc, P, s_peer, P.ci_l, lbeg, lend, lb_col, warp, nwarps, lane, l * 4, true);
        if (REMOTE_MODE == 2 && rend > rbeg)
            gather_list<LPR, 4, false, 2>(acc, P, s_peer, P.ci_r, rbeg, rend, rbase + l * 16, rwarp, nwarps, lane, l * 4, true);
    }
    if (REMOTE_MODE == 1 && !(STAGE & 1) && rend > rbeg)
        gather_list<LPR, 4, true, 2>(acc, P, s_peer, P.ci_r, rbeg, rend, nullptr, rwarp, nwarps, lane, l * 4, true);

    bool alive = true;
    for (unsigned t = 0; t < T; t++) {
        const unsigned s = t % (unsigned)stages;
        const int li = t < nb[0] ? 0 : 1;
        const unsigned b = t - (li ? nb[0] : 0u);
        const unsigned cnt = min(32u, lists[li].total - b * 32u);
        if (alive && !consume_batch<LPR>(acc, ring + (size_t)s * 32 * row_bytes, bar0 + 8 * s, (t / (unsigned)stages) & 1u, cnt, row_bytes, lane)) {
            alive = false;
            atomicCAS(&g_agg_status, 0, 1);
        }
        __syncwarp();                                  // every lane has read the stage before it is refilled
        if (alive && t + (unsigned)stages < T) issue(t + (unsigned)stages);
    }
    if (!alive) {
        // copies may still be on their way into this block's shared memory: give them a bounded time
        // to land before the block (and its shared memory) goes away
        for (unsigned i = 0; i < (1u << 16); i++) __nanosleep(100);
    }

#pragma unroll
    for (int off = LPR; off < 32; off <<= 1) acc.xor_reduce(off);
    if (lane < LPR) acc.store_smem(s_part + warp * P.dim + l * 4);
    __syncthreads();
    store_row(P, row, s_part, nwarps);
}

template <int LPR, int REMOTE_MODE, int STAGE>
int launch_staged(const AggParams& P, int wpb, int stages, size_t smem, cudaStream_t st) {
    MGGB_CUDA(cudaFuncSetAttribute(sag_staged_kernel<LPR, REMOTE_MODE, STAGE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    sag_staged_kernel<LPR, REMOTE_MODE, STAGE><<<P.num_rows, wpb * 32, smem, st>>>(P, stages);
    MGGB_CUDA(cudaGetLastError());
    return MGGB_OK;
}

template <int LPR>
int launch_lpr(const AggParams& P, int wpb, int remote_mode, int stage, int stages, size_t smem, cudaStream_t st) {
    if (remote_mode == 1) {
        if (stage == 1) return launch_staged<LPR, 1, 1>(P, wpb, stages, smem, st);
        return launch_staged<LPR, 1, 3>(P, wpb, stages, smem, st);
    }
    if (remote_mode == 2) return launch_staged<LPR, 2, 2>(P, wpb, stages, smem, st);
    return launch_staged<LPR, 0, 2>(P, wpb, stages, smem, st);
}

}  // namespace

namespace mggb {

// Launches the staged kernel for the rows of P (hub rows are appended to P's hub list exactly as the
// register-path kernels do; the caller runs the hub kernel afterwards).  stage: bit 0 remote list,
// bit 1 directly addressed lists.  *launched = false (and MGGB_OK) when the shape is not served:
// dim not one of 4..128 in powers of two, or no room for at least two stages per warp.
int aggregate_staged(const void* params, int wpb, int remote_mode, int stage, void* stream, bool* launched) {
    const AggParams& P = *static_cast<const AggParams*>(params);
    *launched = false;
    const int q = P.dim / 4;
    if (P.dim % 4 != 0 || q < 1 || q > 32 || (q & (q - 1)) != 0 || wpb > MAX_WARPS) return MGGB_OK;
    if (remote_mode != 1) stage = 2;               // no owner-lookup list: the directly addressed lists are all there is
    else if ((stage & 1) == 0) stage |= 1;
    const size_t row_bytes = (size_t)P.dim * 4;
    const size_t part = ((size_t)wpb * row_bytes + 127) & ~(size_t)127;
    // Ring depth: as many stages as fit a per-block budget that still lets several blocks share an SM.
    const size_t budget = row_bytes <= 64 ? 24 * 1024 : (row_bytes <= 128 ? 40 * 1024 : 72 * 1024);
    int stages = (int)std::min<size_t>(MAX_STAGES, budget / ((size_t)wpb * 32 * row_bytes));
    if (stages < 2) stages = 2;
    const size_t smem = part + (size_t)wpb * stages * 32 * row_bytes;
    if (smem > 200 * 1024) return MGGB_OK;
    cudaStream_t st = (cudaStream_t)stream;
    int rc;
    switch (q) {
        case 1: rc = launch_lpr<1>(P, wpb, remote_mode, stage, stages, smem, st); break;
        case 2: rc = launch_lpr<2>(P, wpb, remote_mode, stage, stages, smem, st); break;
        case 4: rc = launch_lpr<4>(P, wpb, remote_mode, stage, stages, smem, st); break;
        case 8: rc = launch_lpr<8>(P, wpb, remote_mode, stage, stages, smem, st); break;
        case 16: rc = launch_lpr<16>(P, wpb, remote_mode, stage, stages, smem, st); break;
        default: rc = launch_lpr<32>(P, wpb, remote_mode, stage, stages, smem, st); break;
    }
    if (rc == MGGB_OK) *launched = true;
    return rc;
}

}  // namespace mggb

extern "C" int mggb_agg_device_status(int* status, int reset) {
    MGGB_REQUIRE(status, "agg_device_status: NULL output");
    MGGB_CUDA(cudaMemcpyFromSymbol(status, g_agg_status, sizeof(int)));
    if (reset) {
        const int zero = 0;
        MGGB_CUDA(cudaMemcpyToSymbol(g_agg_status, &zero, sizeof(int)));
    }
    return MGGB_OK;
}
