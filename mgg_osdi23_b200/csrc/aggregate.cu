// Neighbor aggregation over a node shard with in-kernel remote fetch (sm_100a).
//
// Stands in for the reference's np_div kernels (include/neighbor_utils.cuh:1351-1460 for the plain
// sum, :1554-1667 for the GIN form) and keeps their work decomposition: one thread block per node
// of the shard, `wpb` warps per block, and each warp taking `dist*ps` consecutive neighbors per
// turn with a block stride of `dist*wpb*ps` (:1395-1400 for the local list, :1432-1437 for the
// remote list; the local list is walked first).
//
// What is different from the reference:
//   * a row of `dim` floats is read by a SUB-WARP of LPR lanes with one 128-bit load per lane, so
//     a warp gathers 32/LPR neighbor rows per load instruction (8 rows at dim 16) and keeps up to
//     32 independent row loads in flight, instead of one row per iteration with half the lanes idle;
//   * the running sum lives in registers, not in shared memory that is read-modify-written per
//     element (:1409);
//   * a remote neighbor's row is read straight from the owner's memory through a peer-mapped
//     pointer (owner = id / nodePerPE, row = id % nodePerPE, :1440-1441) with the same vector loads,
//     so remote and local rows are in flight together; there is no blocking per-neighbor get (:1445);
//   * the warps' partial sums meet in shared memory and ONE thread group stores the output row.
//     No atomics (:1456-1458 uses a spin on atomicExch), so the result is reproducible for fixed
//     knobs, and the epilogue (accumulate / GIN combine / row scale) is applied exactly once.
#include <algorithm>
#include <climits>
#include <map>
#include <mutex>
#include <utility>
#include "aggregate_core.cuh"

// Compile-time tuning, per row width (LPR = lanes that read one row).  Chosen by measurement on
// B200: narrow rows (dim <= 16) are served mostly from L2 and want many resident warps, so registers
// are capped (3 blocks of 512 threads -> 40 registers); wide rows stream from HBM, run one batch
// per node on typical graphs, and do better without the cap.
//   MGGB_AGG_MIN_BLOCKS_NARROW  second argument of __launch_bounds__(512, .) for LPR <= 4.  Measured on 115 M 64-byte
//   rows (232,965 nodes): 2 (64 registers, 32 warps per SM) 0.783 ms; 3 (40 registers, 48 warps) 0.655 ms;
//   4 (32 registers, 64 warps) 0.685 ms.
#ifndef MGGB_AGG_MIN_BLOCKS_NARROW
#define MGGB_AGG_MIN_BLOCKS_NARROW 3
#endif

namespace mggb {
int aggregate_staged(const void* params, int wpb, int remote_mode, int stage, void* stream, bool* launched);
}

namespace {

// Sums the neighbor rows of the list ranges [lbeg, lend) (local) and [rbeg, rend) (remote) with all warps of
// the block: on return (past a __syncthreads()) s_part[w * dim + c] holds warp w's partial sums.
// s_part: nwarps * dim floats of shared memory.
template <int LPR, int VEC, bool EXACT, int REMOTE_MODE, int WALK>
__device__ __forceinline__ void aggregate_range(const AggParams& P, int lbeg, int lend, int rbeg, int rend,
                                                float* s_part, const float* const* s_peer) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwarps = blockDim.x >> 5;
    const int l = lane % LPR;
    constexpr int COLS = LPR * VEC;  // columns covered per pass

    for (int cb = 0; cb < (EXACT ? 1 : P.dim); cb += COLS) {
        const int col = cb + l * VEC;
        const bool col_ok = EXACT || col < P.dim;
        Vec<VEC> acc;
        acc.zero();
        accumulate_row<LPR, VEC, REMOTE_MODE, WALK>(acc, P, s_peer, lbeg, lend, rbeg, rend, warp, nwarps, lane, col, col_ok);
        // fold the 32/LPR sub-warps together; the lanes left holding final sums store them
        const Folded<LPR, VEC> f = fold_subwarps<LPR, VEC>(acc, lane);
        if (f.owner && col_ok) {
#pragma unroll
            for (int j = 0; j < VEC; j++)
                if (j < f.n) s_part[warp * P.dim + col + f.first + j] = f.out[j];
        }
    }
    __syncthreads();
}

// Aggregates one node with all warps of the block and stores its output row.  A caller that loops over
// rows must synchronise before reusing s_part.
template <int LPR, int VEC, bool EXACT, int REMOTE_MODE, int WALK>
__device__ __forceinline__ void aggregate_row(const AggParams& P, const int row, float* s_part,
                                              const float* const* s_peer) {
    aggregate_range<LPR, VEC, EXACT, REMOTE_MODE, WALK>(P, P.rp_l[row], P.rp_l[row + 1], P.rp_r[row], P.rp_r[row + 1], s_part, s_peer);
    store_row(P, row, s_part, blockDim.x >> 5);
}

// One block per node.  Dynamic shared memory: nwarps * dim floats (the warps' partial rows).
template <int LPR, int VEC, bool EXACT, int REMOTE_MODE, int WALK>
__global__ void __launch_bounds__(512, (LPR <= 4 ? MGGB_AGG_MIN_BLOCKS_NARROW : 1)) sag_np_div_kernel(const AggParams P) {
    extern __shared__ __align__(16) float s_part[];
    __shared__ const float* s_peer[MGGB_MAX_PES];
    __shared__ int s_deferred;

    const int row = P.row_order ? P.row_order[blockIdx.x] : (int)blockIdx.x;
    // Only the owner lookup reads the pointer table from shared memory; the other modes skip the
    // fill and its barrier.
    if (REMOTE_MODE == 1) {
        if (threadIdx.x < MGGB_MAX_PES) s_peer[threadIdx.x] = P.peer[threadIdx.x < P.num_pes ? threadIdx.x : 0];
        __syncthreads();
    }
    // Every thread reads the row's bounds, so "is this a hub" is known block-wide without a barrier;
    // only an actual hub pays for the hand-over (atomic slot, shared flag, barrier).
    if (P.hub_count != nullptr) {
        const int edges = (P.rp_l[row + 1] - P.rp_l[row]) + (P.rp_r[row + 1] - P.rp_r[row]);
        if (edges > P.hub_min_edges) {
            // handed to the wide-block kernel if its lists still have room; otherwise this block
            // aggregates the row after all (slower, same result)
            if (threadIdx.x == 0) s_deferred = defer_row(P, row, edges);
            __syncthreads();
            if (s_deferred) return;
        }
    }
    aggregate_row<LPR, VEC, EXACT, REMOTE_MODE, WALK>(P, row, s_part, s_peer);
}

// warp_per_block == 1: a warp owns its node outright, so nothing has to meet in shared memory and no
// block barrier is needed.  Eight such warps share a CUDA block (consecutive entries of the
// schedule), which cuts the number of blocks eightfold on graphs whose nodes have a few dozen
// neighbors.  Same edge-to-lane mapping and summation order as the one-warp block above: identical bits.
constexpr int ROW_WARPS = 8;

template <int LPR, int VEC, bool EXACT, int REMOTE_MODE, int WALK>
__global__ void __launch_bounds__(ROW_WARPS * 32, (LPR <= 4 ? 6 : 2)) sag_row_per_warp_kernel(const AggParams P) {
    __shared__ const float* s_peer[MGGB_MAX_PES];
    if (REMOTE_MODE == 1) {
        if (threadIdx.x < MGGB_MAX_PES) s_peer[threadIdx.x] = P.peer[threadIdx.x < P.num_pes ? threadIdx.x : 0];
        __syncthreads();
    }
    const int lane = threadIdx.x & 31;
    const long long slot_idx = (long long)blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
    if (slot_idx >= P.num_rows) return;
    const int row = P.row_order ? P.row_order[slot_idx] : (int)slot_idx;
    const int lbeg = P.rp_l[row], lend = P.rp_l[row + 1];
    const int rbeg = P.rp_r[row], rend = P.rp_r[row + 1];
    if (P.hub_count != nullptr && (lend - lbeg) + (rend - rbeg) > P.hub_min_edges) {
        int deferred = 0;
        if (lane == 0) deferred = defer_row(P, row, (lend - lbeg) + (rend - rbeg));
        if (__shfl_sync(0xffffffffu, deferred, 0)) return;
    }
    const int l = lane % LPR;
    constexpr int COLS = LPR * VEC;
    for (int cb = 0; cb < (EXACT ? 1 : P.dim); cb += COLS) {
        const int col = cb + l * VEC;
        const bool col_ok = EXACT || col < P.dim;
        Vec<VEC> acc;
        acc.zero();
        accumulate_row<LPR, VEC, REMOTE_MODE, WALK>(acc, P, s_peer, lbeg, lend, rbeg, rend, 0, 1, lane, col, col_ok);
        // the same fold and the same arithmetic as a one-warp block of the kernel above (store_row adds the single
        // partial row to 0.f), so the two kernels give identical bits
        const Folded<LPR, VEC> f = fold_subwarps<LPR, VEC>(acc, lane);
        if (f.owner && col_ok) {
#pragma unroll
            for (int j = 0; j < VEC; j++)
                if (j < f.n) finish_element(P, row, col + f.first + j, 0.f + f.out[j]);
        }
    }
}

// MGGB_AGG_GROUP_PER_NODE, dim == 16: a node is aggregated by ONE group of 4 lanes (one float4 of the
// row each), so a warp works on 8 nodes at once, each group walking its own neighbor lists 4 ids at
// a time (4 row loads in flight per lane, 32 per warp, as in the other kernels).  Nothing is reduced
// across lanes and the per-node fixed cost (bounds, loop set-up, epilogue) is paid by 4 lanes instead
// of 32: on graphs whose nodes have a few dozen neighbors that cost, not memory, is the limit.
// Nodes above hub_min_edges still go to the wide-block kernel.  The chunk knobs do not apply.
constexpr int GROUP_LANES = 4;
constexpr int GROUP_BLOCK = 256;
constexpr int GROUP_ROWS_PER_BLOCK = GROUP_BLOCK / GROUP_LANES;

template <int REMOTE_MODE>
__device__ __forceinline__ void group_gather_list(float4& acc, const AggParams& P, const float* const* s_peer,
                                                  const int32_t* __restrict__ ci, int beg, int end,
                                                  const char* base, bool remote, int l, unsigned group_mask) {
    const unsigned row_bytes = 64u;
    // every group of the warp keeps stepping until the longest list among them is done.  The ids of
    // step t+1 are requested before the rows of step t, so the two dependent latencies (id, then row)
    // of consecutive steps overlap instead of adding up.
    int nxt = (beg + l < end) ? __ldcs(ci + beg + l) : -1;
    for (int e = beg; __any_sync(0xffffffffu, e < end); e += GROUP_LANES) {
        const int my = nxt;
        const int en = e + GROUP_LANES;
        nxt = (en + l < end) ? __ldcs(ci + en + l) : -1;
        float4 v[GROUP_LANES];
        bool ok[GROUP_LANES];
#pragma unroll
        for (int j = 0; j < GROUP_LANES; j++) {
            const int got = __shfl_sync(0xffffffffu, my, j, GROUP_LANES);
            ok[j] = got >= 0;
            const int nid = max(got, 0);
            const float* src;
            if (REMOTE_MODE == 1 && remote) {
                const unsigned owner = (unsigned)(((unsigned long long)(unsigned)nid * P.div_magic) >> P.div_shift);
                src = s_peer[owner] + (long long)(nid - (int)owner * P.node_per_pe) * 16 + l * 4;
            } else {
                src = reinterpret_cast<const float*>(base + (long long)nid * row_bytes);
            }
            if (ok[j]) v[j] = __ldg(reinterpret_cast<const float4*>(src));
        }
#pragma unroll
        for (int j = 0; j < GROUP_LANES; j++)
            if (ok[j]) { acc.x += v[j].x; acc.y += v[j].y; acc.z += v[j].z; acc.w += v[j].w; }
    }
    (void)group_mask;
}

template <int REMOTE_MODE>
__global__ void __launch_bounds__(GROUP_BLOCK, 4) sag_group_per_node_kernel(const AggParams P) {
    __shared__ const float* s_peer[MGGB_MAX_PES];
    if (REMOTE_MODE == 1) {
        if (threadIdx.x < MGGB_MAX_PES) s_peer[threadIdx.x] = P.peer[threadIdx.x < P.num_pes ? threadIdx.x : 0];
        __syncthreads();
    }
    const int l = threadIdx.x & (GROUP_LANES - 1);
    const long long slot = (long long)blockIdx.x * GROUP_ROWS_PER_BLOCK + (threadIdx.x / GROUP_LANES);
    const bool active = slot < P.num_rows;
    int row = 0, lbeg = 0, lend = 0, rbeg = 0, rend = 0;
    if (active) {
        row = P.row_order ? P.row_order[slot] : (int)slot;
        lbeg = P.rp_l[row]; lend = P.rp_l[row + 1];
        rbeg = P.rp_r[row]; rend = P.rp_r[row + 1];
    }
    // A node above the hub threshold is handed to the wide-block kernel by its group's leader (if the
    // list has room).  The decision is shared with an unconditional group-wide shuffle.
    const bool hub = active && P.hub_count != nullptr && (lend - lbeg) + (rend - rbeg) > P.hub_min_edges;
    int handed = 0;
    if (hub && l == 0) handed = defer_row(P, row, (lend - lbeg) + (rend - rbeg));
    handed = __shfl_sync(0xffffffffu, handed, 0, GROUP_LANES);
    const bool mine = active && !handed;   // false: nothing to aggregate or store here
    if (!mine) { lbeg = lend = rbeg = rend = 0; }
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const char* lbase = reinterpret_cast<const char*>(P.peer[P.pe] + l * 4) - (long long)P.lb * 64;
    const char* rbase = reinterpret_cast<const char*>(P.peer[0] + l * 4);
    group_gather_list<REMOTE_MODE>(acc, P, s_peer, P.ci_l, lbeg, lend, lbase, false, l, 0);
    if (REMOTE_MODE != 0)
        group_gather_list<REMOTE_MODE>(acc, P, s_peer, P.ci_r, rbeg, rend, rbase, true, l, 0);
    if (!mine) return;
    const long long o = (long long)row * 16 + l * 4;
    if (P.row_scale) { const float sc = P.row_scale[row]; acc.x *= sc; acc.y *= sc; acc.z *= sc; acc.w *= sc; }
    if (P.mode == MODE_GIN) {
        const float4 x = *reinterpret_cast<const float4*>(P.peer[P.pe] + o);
        acc.x += P.self_scale * x.x; acc.y += P.self_scale * x.y; acc.z += P.self_scale * x.z; acc.w += P.self_scale * x.w;
    } else if (P.mode == MODE_ACCUMULATE) {
        const float4 x = *reinterpret_cast<const float4*>(P.out + o);
        acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
    }
    *reinterpret_cast<float4*>(P.out + o) = acc;
    for (int k = 0; k < P.num_publish; k++) *reinterpret_cast<float4*>(P.publish[k] + o) = acc;
}

// Hub rows: a fixed grid of 16-warp blocks walks the lists the kernel above filled.  First the segments of
// the giant rows, one block per segment: the block sums its segment into a partial row in global memory,
// and the block that finishes a row's last segment adds the row's partial rows in segment order and
// stores the output row (so the result depends neither on which block came last nor on the order in
// which rows were appended).  Then the hub list proper: each listed row is aggregated by ONE block with
// the same warp/chunk mapping as a one-node block (just more warps).  The next batch of neighbor ids is
// prefetched here: a hub's warps run hundreds of batches back to back.
template <int LPR, int VEC, bool EXACT, int REMOTE_MODE, int WALK>
__global__ void __launch_bounds__(512, 2) sag_hub_rows_kernel(const AggParams P) {
    extern __shared__ __align__(16) float s_part[];
    __shared__ const float* s_peer[MGGB_MAX_PES];
    __shared__ GiantRow s_giant;
    __shared__ int s_giant_index, s_last;
    if (threadIdx.x < MGGB_MAX_PES) s_peer[threadIdx.x] = P.peer[threadIdx.x < P.num_pes ? threadIdx.x : 0];
    if (threadIdx.x == 0) s_giant_index = -1;
    __syncthreads();
    const int nwarps = blockDim.x >> 5;
    const int giants = P.giant_rows != nullptr ? min(P.hub_count[1], P.giant_row_cap) : 0;
    const int items = giants > 0 ? min(P.hub_count[2], P.giant_item_cap) : 0;
    for (int j = blockIdx.x; j < items; j += gridDim.x) {
        // whose segment is partial row j?  (entries that did not get their partial rows have row < 0)
        for (int g = threadIdx.x; g < giants; g += blockDim.x) {
            const GiantRow r = P.giant_rows[g];
            if (r.row >= 0 && j >= r.first && j < r.first + r.nseg) { s_giant = r; s_giant_index = g; }
        }
        __syncthreads();
        const int gi = s_giant_index;
        const GiantRow r = s_giant;
        __syncthreads();   // everyone has read the match before it is cleared for the next round
        if (threadIdx.x == 0) s_giant_index = -1;
        if (gi >= 0) {
            const int lbeg = P.rp_l[r.row], lend = P.rp_l[r.row + 1];
            const int rbeg = P.rp_r[r.row], rend = P.rp_r[r.row + 1];
            // neighbors [a, b) of the row's local list followed by its remote list
            const long long a = (long long)(j - r.first) * r.seg_edges, b = a + r.seg_edges;
            const int nl = lend - lbeg, nr = rend - rbeg;
            const int la = (int)min((long long)nl, a), lb_ = (int)min((long long)nl, b);
            const int ra = (int)min((long long)nr, max(0LL, a - nl)), rb = (int)min((long long)nr, max(0LL, b - nl));
            aggregate_range<LPR, VEC, EXACT, REMOTE_MODE, WALK>(P, lbeg + la, lbeg + lb_, rbeg + ra, rbeg + rb, s_part, s_peer);
            float* mine = P.giant_part + (long long)j * P.dim;
            for (int c = threadIdx.x; c < P.dim; c += blockDim.x) {
                float s = 0.f;
                for (int w = 0; w < nwarps; w++) s += s_part[w * P.dim + c];
                mine[c] = s;
            }
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) s_last = (atomicAdd(P.giant_done + gi, 1) == r.nseg - 1);
            __syncthreads();
            if (s_last) {
                __threadfence();
                const float* parts = P.giant_part + (long long)r.first * P.dim;
                for (int c = threadIdx.x; c < P.dim; c += blockDim.x) {
                    float s = 0.f;
                    for (int q = 0; q < r.nseg; q++) s += __ldcg(parts + (long long)q * P.dim + c);
                    finish_element(P, r.row, c, s);
                }
                if (threadIdx.x == 0) P.giant_done[gi] = 0;   // zero again for the next call
            }
        }
        __syncthreads();   // s_part, s_giant and s_last are reused
    }
    __syncthreads();
    const int count = min(*P.hub_count, P.hub_cap);
    // blocks that took no (or fewer) segments start the list
    const int shift = items % gridDim.x;
    for (int i = (blockIdx.x + gridDim.x - shift) % gridDim.x; i < count; i += gridDim.x) {
        aggregate_row<LPR, VEC, EXACT, REMOTE_MODE, WALK>(P, P.hub_list[i], s_part, s_peer);
        __syncthreads();   // s_part is reused by the next row
    }
}

constexpr int HUB_COUNTERS = 4;   // ints cleared before every call: [0] hub rows, [1] giant rows, [2] partial rows handed out
constexpr int GROUP_HUB_MIN_EDGES = 1024;   // group-per-node kernel: longer lists would leave one 4-lane group as the kernel's tail

// Neighbor count above which a row is handed to the wide-block kernel, or -1 when these knobs use no
// hub list at all.  One definition for the launch code, the allocation-free entry point's size
// check and mggb_hub_threshold().
long long hub_threshold(int ps, int wpb, int dist, int dim, int flags) {
    if ((flags & MGGB_AGG_NO_HUB_SPLIT) || wpb > HUB_WARPS / 2 || (size_t)HUB_WARPS * dim * sizeof(float) > 200 * 1024) return -1;
    if ((flags & MGGB_AGG_GROUP_PER_NODE) && dim == 16) return GROUP_HUB_MIN_EDGES;
    const long long chunk = std::min<long long>((long long)ps * dist, 1 << 24);
    return std::max<long long>(HUB_MIN_EDGES, 64 * chunk * wpb);
}

template <int LPR, int VEC, bool EXACT>
int launch_exact(const AggParams& P, int wpb, cudaStream_t st);

// The wide-block kernel over whatever the first kernel appended to the hub list.
template <int LPR, int VEC, bool EXACT, int REMOTE_MODE, int WALK>
int launch_hub(const AggParams& P, cudaStream_t st) {
    const size_t hub_smem = (size_t)HUB_WARPS * P.dim * sizeof(float);
    if (hub_smem > 48 * 1024)
        MGGB_CUDA(cudaFuncSetAttribute(sag_hub_rows_kernel<LPR, VEC, EXACT, REMOTE_MODE, WALK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)hub_smem));
    sag_hub_rows_kernel<LPR, VEC, EXACT, REMOTE_MODE, WALK><<<HUB_BLOCKS_PER_SM * mggb::sm_count(), HUB_WARPS * 32, hub_smem, st>>>(P);
    MGGB_CUDA(cudaGetLastError());
    return MGGB_OK;
}

// The same for the staged kernels (dim == 4 * LPR, 128-bit loads), by run-time row width and mode.
template <int LPR>
int launch_hub_mode(const AggParams& P, int remote_mode, cudaStream_t st) {
    if (P.chunk < 32) {
        if (remote_mode == 0) return launch_hub<LPR, 4, true, 0, 2>(P, st);
        if (remote_mode == 1) return launch_hub<LPR, 4, true, 1, 2>(P, st);
        return launch_hub<LPR, 4, true, 2, 2>(P, st);
    }
    if (remote_mode == 0) return launch_hub<LPR, 4, true, 0, 1>(P, st);
    if (remote_mode == 1) return launch_hub<LPR, 4, true, 1, 1>(P, st);
    return launch_hub<LPR, 4, true, 2, 1>(P, st);
}

int launch_hub_for(const AggParams& P, int remote_mode, cudaStream_t st) {
    switch (P.dim / 4) {
        case 1: return launch_hub_mode<1>(P, remote_mode, st);
        case 2: return launch_hub_mode<2>(P, remote_mode, st);
        case 4: return launch_hub_mode<4>(P, remote_mode, st);
        case 8: return launch_hub_mode<8>(P, remote_mode, st);
        case 16: return launch_hub_mode<16>(P, remote_mode, st);
        default: return launch_hub_mode<32>(P, remote_mode, st);
    }
}

// 0 = one PE; 2 = the PEs' buffers are consecutive slots of one matrix (a local replica); 1 = buffers anywhere.
int remote_mode_of(const AggParams& P) {
    if (P.num_pes == 1 || P.no_remote) return 0;
    bool one_matrix = true;   // peer[p] == peer[0] + p * node_per_pe * dim for every p
    for (int p = 1; p < P.num_pes; p++)
        one_matrix = one_matrix && (P.peer[p] == P.peer[0] + (long long)p * P.node_per_pe * P.dim);
    return one_matrix ? 2 : 1;
}
template <int LPR, int VEC, bool EXACT, int REMOTE_MODE>
int launch_kernel(const AggParams& P, int wpb, cudaStream_t st);

template <int LPR, int VEC>
int launch(const AggParams& P, int wpb, cudaStream_t st) {
    if (P.dim == LPR * VEC) return launch_exact<LPR, VEC, true>(P, wpb, st);
    return launch_exact<LPR, VEC, false>(P, wpb, st);
}

// A single PE has no remote half: that instantiation drops the owner lookup altogether.
template <int LPR, int VEC, bool EXACT>
int launch_exact(const AggParams& P, int wpb, cudaStream_t st) {
    const int mode = remote_mode_of(P);
    if (mode == 0) return launch_kernel<LPR, VEC, EXACT, 0>(P, wpb, st);
    if (mode == 2) return launch_kernel<LPR, VEC, EXACT, 2>(P, wpb, st);
    return launch_kernel<LPR, VEC, EXACT, 1>(P, wpb, st);
}

template <int LPR, int VEC, bool EXACT, int REMOTE_MODE, int WALK>
int launch_walk(const AggParams& P, int wpb, cudaStream_t st) {
    const size_t smem = (size_t)wpb * P.dim * sizeof(float);
    if (smem > 48 * 1024)
        MGGB_CUDA(cudaFuncSetAttribute(sag_np_div_kernel<LPR, VEC, EXACT, REMOTE_MODE, WALK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (P.hub_count != nullptr) MGGB_CUDA(cudaMemsetAsync(P.hub_count, 0, HUB_COUNTERS * sizeof(int), st));
    if (wpb == 1 && LPR <= 4)   // wide rows stream from HBM and measured no better this way
        sag_row_per_warp_kernel<LPR, VEC, EXACT, REMOTE_MODE, WALK><<<(P.num_rows + ROW_WARPS - 1) / ROW_WARPS, ROW_WARPS * 32, 0, st>>>(P);
    else
        sag_np_div_kernel<LPR, VEC, EXACT, REMOTE_MODE, WALK><<<P.num_rows, wpb * 32, smem, st>>>(P);
    MGGB_CUDA(cudaGetLastError());
    if (P.hub_count != nullptr) return launch_hub<LPR, VEC, EXACT, REMOTE_MODE, (WALK == 2 ? 2 : 1)>(P, st);
    return MGGB_OK;
}

// Chunks shorter than one 32-id batch get the walk that packs several chunks into a batch.
template <int LPR, int VEC, bool EXACT, int REMOTE_MODE>
int launch_kernel(const AggParams& P, int wpb, cudaStream_t st) {
    if (P.chunk < 32) return launch_walk<LPR, VEC, EXACT, REMOTE_MODE, 2>(P, wpb, st);
    return launch_walk<LPR, VEC, EXACT, REMOTE_MODE, 0>(P, wpb, st);
}

// Hub work list: per (device, stream) so that calls ordered on one stream reuse it safely and calls
// on different streams never share one.  Allocated on first use, kept until the process exits.
struct HubScratch {
    int* count; int* list;
    GiantRow* giant_rows; int* giant_done; float* giant_part;   // giant_rows NULL: giant rows are not cut
    int giant_row_cap; long long giant_part_floats;
};

constexpr long long GIANT_PART_FLOATS = 4 << 20;   // 16 MiB of partial rows per (device, stream)

int hub_scratch(cudaStream_t st, HubScratch* out) {
    static std::mutex mu;
    static std::map<std::pair<int, cudaStream_t>, HubScratch> table;
    int dev = 0;
    MGGB_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> g(mu);
    auto key = std::make_pair(dev, st);
    auto it = table.find(key);
    if (it == table.end()) {
        // one block: [64 counters][HUB_CAP rows][GIANT_ROWS_CAP descriptors][GIANT_ROWS_CAP counters][partial rows]
        const size_t ints = 64 + (size_t)HUB_CAP + 4 * (size_t)GIANT_ROWS_CAP + GIANT_ROWS_CAP;
        int* base = nullptr;
        MGGB_CUDA(cudaMalloc((void**)&base, sizeof(int) * ints + sizeof(float) * (size_t)GIANT_PART_FLOATS));
        HubScratch hs{};
        hs.count = base; hs.list = base + 64;
        hs.giant_rows = reinterpret_cast<GiantRow*>(base + 64 + HUB_CAP);
        hs.giant_done = base + 64 + HUB_CAP + 4 * GIANT_ROWS_CAP;
        hs.giant_part = reinterpret_cast<float*>(base + ints);
        hs.giant_row_cap = GIANT_ROWS_CAP; hs.giant_part_floats = GIANT_PART_FLOATS;
        // the segment counters start at zero and every call leaves them at zero
        MGGB_CUDA(cudaMemset(hs.giant_done, 0, sizeof(int) * GIANT_ROWS_CAP));
        it = table.emplace(key, hs).first;
    }
    *out = it->second;
    return MGGB_OK;
}

// The group-per-node kernel, then the hub kernel for whatever it deferred.
int launch_group_per_node(const AggParams& P, cudaStream_t st) {
    const int mode = remote_mode_of(P);
    if (P.hub_count != nullptr) MGGB_CUDA(cudaMemsetAsync(P.hub_count, 0, HUB_COUNTERS * sizeof(int), st));
    const int grid = (P.num_rows + GROUP_ROWS_PER_BLOCK - 1) / GROUP_ROWS_PER_BLOCK;
    const size_t hub_smem = (size_t)HUB_WARPS * P.dim * sizeof(float);
    if (mode == 0) sag_group_per_node_kernel<0><<<grid, GROUP_BLOCK, 0, st>>>(P);
    else if (mode == 1) sag_group_per_node_kernel<1><<<grid, GROUP_BLOCK, 0, st>>>(P);
    else sag_group_per_node_kernel<2><<<grid, GROUP_BLOCK, 0, st>>>(P);
    MGGB_CUDA(cudaGetLastError());
    if (P.hub_count != nullptr) {
        if (mode == 0) sag_hub_rows_kernel<4, 4, true, 0, 1><<<HUB_BLOCKS_PER_SM * mggb::sm_count(), HUB_WARPS * 32, hub_smem, st>>>(P);
        else if (mode == 1) sag_hub_rows_kernel<4, 4, true, 1, 1><<<HUB_BLOCKS_PER_SM * mggb::sm_count(), HUB_WARPS * 32, hub_smem, st>>>(P);
        else sag_hub_rows_kernel<4, 4, true, 2, 1><<<HUB_BLOCKS_PER_SM * mggb::sm_count(), HUB_WARPS * 32, hub_smem, st>>>(P);
        MGGB_CUDA(cudaGetLastError());
    }
    return MGGB_OK;
}

int aggregate(float* output, const float* const* peer_input, int num_pes, const int32_t* rp_l,
              const int32_t* ci_l, const int32_t* rp_r, const int32_t* ci_r, int32_t lb, int32_t ub,
              int dim, int32_t node_per_pe, int pe, int ps, int wpb, int dist, const float* row_scale,
              int mode, float self_scale, float* const* publish_out, int num_publish, int flags, void* stream,
              const HubScratch* caller_scratch = nullptr, int caller_scratch_cap = 0, const int32_t* row_order = nullptr,
              int64_t row_count = -1) {
    MGGB_REQUIRE(num_publish >= 0 && num_publish <= MGGB_MAX_PES && (num_publish == 0 || publish_out),
                 "aggregate: num_publish must be in [0,%d] with a non-NULL table (got %d)", MGGB_MAX_PES, num_publish);
    for (int k = 0; k < num_publish; k++)
        MGGB_REQUIRE(publish_out[k] != nullptr, "aggregate: publish_out[%d] is NULL", k);
    MGGB_REQUIRE(output && peer_input && rp_l && rp_r, "aggregate: NULL argument");
    MGGB_REQUIRE(num_pes >= 1 && num_pes <= MGGB_MAX_PES, "aggregate: num_pes must be in [1,%d] (got %d)", MGGB_MAX_PES, num_pes);
    MGGB_REQUIRE(pe >= 0 && pe < num_pes, "aggregate: pe %d outside [0,%d)", pe, num_pes);
    MGGB_REQUIRE(lb >= 0 && ub >= lb, "aggregate: need 0 <= lb <= ub (lb=%d ub=%d)", lb, ub);
    MGGB_REQUIRE(dim >= 1, "aggregate: dim must be >= 1 (got %d)", dim);
    MGGB_REQUIRE(node_per_pe >= 1 && ub - lb <= node_per_pe, "aggregate: shard [%d,%d) larger than node_per_pe=%d", lb, ub, node_per_pe);
    MGGB_REQUIRE((long long)lb == (long long)pe * node_per_pe || ub == lb, "aggregate: lb=%d is not pe*node_per_pe (%d*%d)", lb, pe, node_per_pe);
    MGGB_REQUIRE(ps >= 1 && dist >= 1 && wpb >= 1 && wpb <= 16, "aggregate: need part_size >= 1, interleaved_dist >= 1, 1 <= warp_per_block <= 16 (ps=%d wpb=%d dist=%d)", ps, wpb, dist);
    MGGB_REQUIRE((long long)ps * dist <= (1 << 30), "aggregate: part_size*interleaved_dist too large");
    for (int p = 0; p < num_pes; p++)
        MGGB_REQUIRE(peer_input[p] != nullptr, "aggregate: peer_input[%d] is NULL", p);
    MGGB_REQUIRE(mode != MODE_GIN || output != peer_input[pe], "gin_np_div: output must not alias this PE's input buffer");
    if ((size_t)wpb * dim * sizeof(float) > 200 * 1024)
        return mggb::fail(MGGB_ERR_UNSUPPORTED, "aggregate: warp_per_block*dim*4 = %zu bytes of shared memory exceeds 200 KiB", (size_t)wpb * dim * sizeof(float));
    if (ub == lb) return MGGB_OK;

    AggParams P{};
    P.out = output;
    for (int p = 0; p < MGGB_MAX_PES; p++) P.peer[p] = peer_input[p < num_pes ? p : 0];
    P.rp_l = rp_l; P.ci_l = ci_l; P.rp_r = rp_r; P.ci_r = ci_r;
    P.row_scale = row_scale;
    P.row_order = row_order;
    P.num_publish = num_publish;
    for (int k = 0; k < num_publish; k++) P.publish[k] = publish_out[k];
    P.lb = lb; P.num_rows = ub - lb; P.node_per_pe = node_per_pe;
    if (row_count >= 0) {   // only the listed rows (ids relative to lb)
        if (row_count == 0) return MGGB_OK;
        MGGB_REQUIRE(row_order != nullptr && row_count <= ub - lb, "aggregate: row_count needs a row list of at most ub-lb rows (got %lld)", (long long)row_count);
        P.num_rows = (int32_t)row_count;
    }
    P.dim = dim; P.pe = pe; P.num_pes = num_pes;
    P.no_remote = (flags & MGGB_AGG_NO_REMOTE) ? 1 : 0;
    P.chunk = (int)std::min<long long>((long long)ps * dist, 1 << 24);  // larger than any useful chunk: same walk
    make_divider((uint32_t)node_per_pe, &P.div_magic, &P.div_shift);
    P.mode = mode; P.self_scale = self_scale;
    // Hub rows get wide blocks unless the caller asked for none, already runs wide blocks, or the wide
    // block's partial rows would not fit in shared memory (then every node stays on its own block).
    P.hub_count = nullptr; P.hub_list = nullptr; P.hub_cap = 0;
    P.giant_rows = nullptr; P.giant_done = nullptr; P.giant_part = nullptr; P.giant_row_cap = 0; P.giant_item_cap = 0;
    const HubScratch* scratch = nullptr;
    HubScratch own{};
    const long long hub_min = hub_threshold(ps, wpb, dist, dim, caller_scratch ? (flags & ~MGGB_AGG_GROUP_PER_NODE) : flags);
    P.hub_min_edges = (int)std::min<long long>(std::max<long long>(hub_min, 0), INT_MAX);
    if (hub_min >= 0 && caller_scratch != nullptr) {
        scratch = caller_scratch;
        P.hub_cap = caller_scratch_cap;
    } else if (hub_min >= 0) {
        int st_ = hub_scratch((cudaStream_t)stream, &own);
        if (st_ != MGGB_OK) return st_;
        scratch = &own;
        P.hub_cap = HUB_CAP;
    }
    if (scratch != nullptr) {
        P.hub_count = scratch->count; P.hub_list = scratch->list;
        if (scratch->giant_rows != nullptr) {
            P.giant_rows = scratch->giant_rows; P.giant_done = scratch->giant_done; P.giant_part = scratch->giant_part;
            P.giant_row_cap = scratch->giant_row_cap;
            P.giant_item_cap = (int)std::min<long long>(scratch->giant_part_floats / dim, (long long)GIANT_ROWS_CAP * GIANT_MAX_SEG);
        }
    }

    cudaStream_t st = (cudaStream_t)stream;
    if ((flags & MGGB_AGG_GROUP_PER_NODE) && dim == 16 && caller_scratch == nullptr) {
        bool aligned = ((uintptr_t)output % 16 == 0);
        for (int p = 0; p < num_pes; p++) aligned = aligned && ((uintptr_t)peer_input[p] % 16 == 0);
        for (int k = 0; k < num_publish; k++) aligned = aligned && ((uintptr_t)publish_out[k] % 16 == 0);
        if (aligned)   // hub_threshold() already gave this kernel its own, lower threshold
            return launch_group_per_node(P, st);
        if (P.hub_count != nullptr) {   // not taken after all: back to the wide-row threshold
            P.hub_min_edges = (int)std::min<long long>(hub_threshold(ps, wpb, dist, dim, flags & ~MGGB_AGG_GROUP_PER_NODE), INT_MAX);
        }
    }
    bool vec4 = (dim % 4 == 0);
    for (int p = 0; p < num_pes && vec4; p++) vec4 = ((uintptr_t)peer_input[p] % 16 == 0);
    // On request, rows staged through shared memory by bulk copies: the remote list when remote rows are
    // fetched from the owners' buffers, every list otherwise.
    const int remote_mode = remote_mode_of(P);
    if (vec4 && (flags & MGGB_AGG_STAGE_ROWS)) {
        if (P.hub_count != nullptr) MGGB_CUDA(cudaMemsetAsync(P.hub_count, 0, HUB_COUNTERS * sizeof(int), st));
        bool launched = false;
        int rc = mggb::aggregate_staged(&P, wpb, remote_mode, remote_mode == 1 ? 1 : 2, st, &launched);
        if (rc != MGGB_OK) return rc;
        if (launched) return P.hub_count != nullptr ? launch_hub_for(P, remote_mode, st) : MGGB_OK;
    }
    if (vec4) {
        const int q = dim / 4;
        // (64-byte rows read by TWO lanes with one 256-bit load each, 16 rows per load instruction, were measured slower
        // than four lanes with 128-bit loads: 0.728 ms against 0.676 ms per aggregation of 115 M rows)
        if (q <= 1) return launch<1, 4>(P, wpb, st);
        if (q <= 2) return launch<2, 4>(P, wpb, st);
        if (q <= 4) return launch<4, 4>(P, wpb, st);
        if (q <= 8) return launch<8, 4>(P, wpb, st);
        if (q <= 16) return launch<16, 4>(P, wpb, st);
        return launch<32, 4>(P, wpb, st);
    }
    if (dim <= 1) return launch<1, 1>(P, wpb, st);
    if (dim <= 2) return launch<2, 1>(P, wpb, st);
    if (dim <= 4) return launch<4, 1>(P, wpb, st);
    if (dim <= 8) return launch<8, 1>(P, wpb, st);
    if (dim <= 16) return launch<16, 1>(P, wpb, st);
    return launch<32, 1>(P, wpb, st);
}

// ---- hub work list that needs no allocation ---------------------------------------------------------
// Backing store of mggb_sag_np_div_static: lives in the library's device image, so every GPU that
// loads the library holds these bytes until the process exits.  [0] is the counter, the list
// starts 64 ints in (256-byte aligned like the array).
constexpr int STATIC_HUB_CAP = 8192;
static __device__ __align__(256) int g_static_hub[64 + STATIC_HUB_CAP];
// Giant rows of the same entry point: descriptors, segment counters (zero in the image, left at zero by
// every call) and 256 KiB of partial rows (4096 segments at dim 16, 1024 at dim 64).
constexpr int STATIC_GIANT_ROWS = 256;
constexpr int STATIC_GIANT_FLOATS = 64 * 1024;
static __device__ __align__(16) int g_static_giant_rows[4 * STATIC_GIANT_ROWS];
static __device__ int g_static_giant_done[STATIC_GIANT_ROWS];
static __device__ __align__(16) float g_static_giant_part[STATIC_GIANT_FLOATS];

// The array's name is only a host-side handle; the kernels need its device address, which differs
// per device.  Looked up once per device (with that device current) and cached.
int static_hub_scratch(HubScratch* out) {
    constexpr int MAX_DEVICES = 64;
    static std::mutex mu;
    static int* base[MAX_DEVICES] = {nullptr};
    static int* giant_rows[MAX_DEVICES] = {nullptr};
    static int* giant_done[MAX_DEVICES] = {nullptr};
    static float* giant_part[MAX_DEVICES] = {nullptr};
    int dev = 0;
    MGGB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES)
        return mggb::fail(MGGB_ERR_UNSUPPORTED, "sag_np_div_static: device ordinal %d is beyond %d", dev, MAX_DEVICES);
    std::lock_guard<std::mutex> g(mu);
    if (base[dev] == nullptr) {
        int* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&p, g_static_hub);
        if (e != cudaSuccess || p == nullptr)
            return mggb::fail(MGGB_ERR_CUDA, "sag_np_div_static: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
        int *rows = nullptr, *done = nullptr;
        float* part = nullptr;
        if (cudaGetSymbolAddress((void**)&rows, g_static_giant_rows) != cudaSuccess || cudaGetSymbolAddress((void**)&done, g_static_giant_done) != cudaSuccess ||
            cudaGetSymbolAddress((void**)&part, g_static_giant_part) != cudaSuccess)
            return mggb::fail(MGGB_ERR_CUDA, "sag_np_div_static: cudaGetSymbolAddress failed on device %d", dev);
        giant_rows[dev] = rows; giant_done[dev] = done; giant_part[dev] = part;
        base[dev] = p;
    }
    out->count = base[dev];
    out->list = base[dev] + 64;
    out->giant_rows = reinterpret_cast<GiantRow*>(giant_rows[dev]);
    out->giant_done = giant_done[dev];
    out->giant_part = giant_part[dev];
    out->giant_row_cap = STATIC_GIANT_ROWS;
    out->giant_part_floats = STATIC_GIANT_FLOATS;
    return MGGB_OK;
}

}  // namespace

extern "C" {

// Same aggregation as mggb_sag_np_div for callers that cannot let the library allocate device memory
// (a pool that owns the whole GPU, a loop that must not hit cudaMalloc's implicit synchronisation, a
// process with a frozen footprint).  The hub work list is the fixed array g_static_hub instead of a
// heap block, so nothing is allocated or freed here.  The price: a shard may have at most
// STATIC_HUB_CAP * (hub threshold + 1) edges, checked below; the first call on a device resolves the
// array's address and should be made outside stream capture; and all calls on one device share the
// array, so calls whose kernels could overlap must be ordered by the caller.  The counter is cleared
// at the start of every call; stale list entries are never read because the hub kernel stops at the
// counter.
int mggb_sag_np_div_static(float* output, const float* const* peer_input, int num_pes,
                           const int32_t* row_ptr_l, const int32_t* col_idx_l, const int32_t* row_ptr_r,
                           const int32_t* col_idx_r, int32_t lb, int32_t ub, int64_t shard_edges, int dim,
                           int32_t node_per_pe, int pe, int part_size, int warp_per_block,
                           int interleaved_dist, const float* row_scale, int flags,
                           float* const* publish_out, int num_publish, void* stream) {
    MGGB_REQUIRE(shard_edges >= 0, "sag_np_div_static: shard_edges must be >= 0");
    MGGB_REQUIRE(part_size >= 1 && interleaved_dist >= 1 && warp_per_block >= 1 && warp_per_block <= HUB_WARPS / 2,
                 "sag_np_div_static: need part_size >= 1, interleaved_dist >= 1 and 1 <= warp_per_block <= %d", HUB_WARPS / 2);
    // Every listed row has more than hub_min neighbors, so at most shard_edges / (hub_min + 1) rows
    // can be listed; refuse shards for which that bound does not fit the fixed list.  (The group-per-node
    // kernel is not offered here: its threshold of 1024 neighbors would shrink that bound sixteenfold.)
    const int eff_flags = flags & ~(MGGB_AGG_NO_HUB_SPLIT | MGGB_AGG_GROUP_PER_NODE);
    const long long hub_min = hub_threshold(part_size, warp_per_block, interleaved_dist, dim, eff_flags);
    const long long max_edges = hub_min < 0 ? LLONG_MAX : (long long)STATIC_HUB_CAP * (hub_min + 1);
    if (shard_edges > max_edges)
        return mggb::fail(MGGB_ERR_UNSUPPORTED,
                          "sag_np_div_static: a shard of %lld edges may hold more than %d hub rows (limit %lld edges at these knobs); "
                          "use mggb_sag_np_div, which sizes its work list on the heap", (long long)shard_edges, STATIC_HUB_CAP, max_edges);
    HubScratch hs{};
    int st = static_hub_scratch(&hs);
    if (st != MGGB_OK) return st;
    return aggregate(output, peer_input, num_pes, row_ptr_l, col_idx_l, row_ptr_r, col_idx_r, lb, ub, dim,
                     node_per_pe, pe, part_size, warp_per_block, interleaved_dist, row_scale,
                     (flags & MGGB_AGG_ACCUMULATE) ? MODE_ACCUMULATE : MODE_OVERWRITE, 0.f, publish_out,
                     num_publish, eff_flags, stream, &hs, STATIC_HUB_CAP);
}

int mggb_hub_threshold(int part_size, int warp_per_block, int interleaved_dist, int dim, int flags, int64_t* threshold) {
    MGGB_REQUIRE(threshold, "hub_threshold: NULL output");
    MGGB_REQUIRE(part_size >= 1 && interleaved_dist >= 1 && warp_per_block >= 1 && dim >= 1, "hub_threshold: knobs and dim must be >= 1");
    *threshold = hub_threshold(part_size, warp_per_block, interleaved_dist, dim, flags);
    return MGGB_OK;
}

int mggb_sag_np_div(float* output, const float* const* peer_input, int num_pes,
                    const int32_t* row_ptr_l, const int32_t* col_idx_l, const int32_t* row_ptr_r,
                    const int32_t* col_idx_r, int32_t lb, int32_t ub, int dim, int32_t node_per_pe,
                    int pe, int part_size, int warp_per_block, int interleaved_dist,
                    const float* row_scale, int flags, float* const* publish_out, int num_publish,
                    void* stream) {
    return aggregate(output, peer_input, num_pes, row_ptr_l, col_idx_l, row_ptr_r, col_idx_r, lb, ub, dim,
                     node_per_pe, pe, part_size, warp_per_block, interleaved_dist, row_scale,
                     (flags & MGGB_AGG_ACCUMULATE) ? MODE_ACCUMULATE : MODE_OVERWRITE, 0.f, publish_out,
                     num_publish, flags, stream);
}

int mggb_gin_np_div(float* output, const float* const* peer_input, int num_pes,
                    const int32_t* row_ptr_l, const int32_t* col_idx_l, const int32_t* row_ptr_r,
                    const int32_t* col_idx_r, int32_t lb, int32_t ub, int dim, int32_t node_per_pe,
                    int pe, int part_size, int warp_per_block, int interleaved_dist, float eps,
                    int flags, void* stream) {
    return aggregate(output, peer_input, num_pes, row_ptr_l, col_idx_l, row_ptr_r, col_idx_r, lb, ub, dim,
                     node_per_pe, pe, part_size, warp_per_block, interleaved_dist, nullptr, MODE_GIN,
                     1.0f + eps, nullptr, 0, flags, stream);
}

int mggb_sag_np_div_ordered(float* output, const float* const* peer_input, int num_pes,
                            const int32_t* row_ptr_l, const int32_t* col_idx_l, const int32_t* row_ptr_r,
                            const int32_t* col_idx_r, int32_t lb, int32_t ub, int dim, int32_t node_per_pe,
                            int pe, int part_size, int warp_per_block, int interleaved_dist,
                            const float* row_scale, int flags, float* const* publish_out, int num_publish,
                            const int32_t* row_order, void* stream) {
    return aggregate(output, peer_input, num_pes, row_ptr_l, col_idx_l, row_ptr_r, col_idx_r, lb, ub, dim,
                     node_per_pe, pe, part_size, warp_per_block, interleaved_dist, row_scale,
                     (flags & MGGB_AGG_ACCUMULATE) ? MODE_ACCUMULATE : MODE_OVERWRITE, 0.f, publish_out,
                     num_publish, flags, stream, nullptr, 0, row_order);
}

int mggb_gin_np_div_ordered(float* output, const float* const* peer_input, int num_pes,
                            const int32_t* row_ptr_l, const int32_t* col_idx_l, const int32_t* row_ptr_r,
                            const int32_t* col_idx_r, int32_t lb, int32_t ub, int dim, int32_t node_per_pe,
                            int pe, int part_size, int warp_per_block, int interleaved_dist, float eps,
                            int flags, const int32_t* row_order, void* stream) {
    return aggregate(output, peer_input, num_pes, row_ptr_l, col_idx_l, row_ptr_r, col_idx_r, lb, ub, dim,
                     node_per_pe, pe, part_size, warp_per_block, interleaved_dist, nullptr, MODE_GIN,
                     1.0f + eps, nullptr, 0, flags, stream, nullptr, 0, row_order);
}

int mggb_sag_np_div_rows(float* output, const float* const* peer_input, int num_pes,
                         const int32_t* row_ptr_l, const int32_t* col_idx_l, const int32_t* row_ptr_r,
                         const int32_t* col_idx_r, int32_t lb, int32_t ub, int dim, int32_t node_per_pe,
                         int pe, int part_size, int warp_per_block, int interleaved_dist,
                         const float* row_scale, int flags, float* const* publish_out, int num_publish,
                         const int32_t* row_list, int64_t row_count, void* stream) {
    MGGB_REQUIRE(row_count >= 0, "sag_np_div_rows: row_count must be >= 0 (got %lld)", (long long)row_count);
    return aggregate(output, peer_input, num_pes, row_ptr_l, col_idx_l, row_ptr_r, col_idx_r, lb, ub, dim,
                     node_per_pe, pe, part_size, warp_per_block, interleaved_dist, row_scale,
                     (flags & MGGB_AGG_ACCUMULATE) ? MODE_ACCUMULATE : MODE_OVERWRITE, 0.f, publish_out,
                     num_publish, flags, stream, nullptr, 0, row_list, row_count);
}

int mggb_gin_np_div_rows(float* output, const float* const* peer_input, int num_pes,
                         const int32_t* row_ptr_l, const int32_t* col_idx_l, const int32_t* row_ptr_r,
                         const int32_t* col_idx_r, int32_t lb, int32_t ub, int dim, int32_t node_per_pe,
                         int pe, int part_size, int warp_per_block, int interleaved_dist, float eps,
                         int flags, const int32_t* row_list, int64_t row_count, void* stream) {
    MGGB_REQUIRE(row_count >= 0, "gin_np_div_rows: row_count must be >= 0 (got %lld)", (long long)row_count);
    return aggregate(output, peer_input, num_pes, row_ptr_l, col_idx_l, row_ptr_r, col_idx_r, lb, ub, dim,
                     node_per_pe, pe, part_size, warp_per_block, interleaved_dist, nullptr, MODE_GIN,
                     1.0f + eps, nullptr, 0, flags, stream, nullptr, 0, row_list, row_count);
}

}  // extern "C"
