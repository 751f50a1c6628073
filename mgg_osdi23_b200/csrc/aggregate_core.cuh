// Shared device code of the aggregation kernels: parameters, the per-lane vector type, and the
// register-path gather (ids held one per lane, rows loaded with 128-bit read-only loads).  Included by
// aggregate.cu (block-per-node, row-per-warp, group-per-node and hub kernels) and by
// aggregate_staged.cu (rows staged through shared memory with bulk copies).  Everything here has
// internal linkage (anonymous namespace) in each translation unit.
#pragma once
#include "common.h"

#ifndef MGGB_AGG_MAX_ROUNDS
#define MGGB_AGG_MAX_ROUNDS 4   // load rounds issued back to back (rows in flight per warp = rounds * 32/LPR)
#endif

namespace {

constexpr int HUB_WARPS = 16;        // warps of a hub row's block
constexpr int HUB_BLOCKS_PER_SM = 2;  // blocks walking the hub list, per SM of the device
constexpr int HUB_MIN_EDGES = 16384; // smallest neighbor count treated as a hub (a 4-warp block needs > 100 us for it)
constexpr int HUB_CAP = 1 << 18;     // list entries: enough for every row above 16384 edges of a 2^32-edge shard
// Giant rows: one 16-warp block needs about 25 us per 16384 neighbors of 64 bytes, so a row of 10^5 or more
// neighbors would be the kernel's tail.  Such a row is cut into segments of consecutive neighbors, each
// summed by a block of its own into a partial row; the block that finishes last adds the partial rows in
// segment order and stores the output row.
constexpr int GIANT_MIN_EDGES = 16384;  // rows above this are cut
constexpr int GIANT_SEG_EDGES = 4096;   // shortest segment
constexpr int GIANT_MAX_SEG = 64;       // most segments per row (longer rows get longer segments)
constexpr int GIANT_ROWS_CAP = 1024;    // giant rows per call; further ones stay whole on the hub list

struct GiantRow { int row, first, nseg, seg_edges; };   // partial rows first .. first+nseg-1; row < 0: not taken

struct AggParams {
    float* out;
    const float* peer[MGGB_MAX_PES];
    const int32_t* rp_l;
    const int32_t* ci_l;
    const int32_t* rp_r;
    const int32_t* ci_r;
    const float* row_scale;
    const int32_t* row_order;       // NULL, or the row each block takes (a permutation of 0..num_rows-1)
    float* publish[MGGB_MAX_PES];   // extra destinations of every output row (peers' replicas)
    int num_publish;
    int32_t lb;
    int32_t num_rows;
    int32_t node_per_pe;
    int dim;
    int pe;
    int num_pes;
    int no_remote;         // 1: the remote lists are not read (every neighbor is in the local list, one matrix holds all rows)
    int chunk;             // dist * ps: neighbors a warp takes per turn
    unsigned long long div_magic;  // owner = (id * div_magic) >> div_shift
    int div_shift;
    int mode;              // 0 overwrite, 1 accumulate, 2 GIN combine
    float self_scale;      // 1 + eps (GIN)
    // Hub rows (more than hub_min_edges neighbors) are not aggregated by their one-node block: that
    // block appends the row to hub_list and a second kernel gives each listed row a 16-warp block.
    int* hub_count;        // number of rows appended (may exceed hub_cap); NULL = no hub handling
    int* hub_list;
    int hub_cap;
    int hub_min_edges;
    // Giant rows (NULL giant_rows = none are cut).  hub_count[1] counts the rows appended, hub_count[2]
    // the partial rows handed out; giant_done[g] counts row g's finished segments and is zero between calls.
    GiantRow* giant_rows;
    int* giant_done;
    float* giant_part;     // giant_item_cap partial rows of dim floats
    int giant_row_cap;
    int giant_item_cap;
};

enum { MODE_OVERWRITE = 0, MODE_ACCUMULATE = 1, MODE_GIN = 2 };

template <int VEC> struct Vec;
template <> struct Vec<4> {
    float4 v;
    __device__ __forceinline__ void zero() { v = make_float4(0.f, 0.f, 0.f, 0.f); }
    __device__ __forceinline__ void load(const float* p) { v = __ldg(reinterpret_cast<const float4*>(p)); }
    __device__ __forceinline__ void add(const Vec& o) { v.x += o.v.x; v.y += o.v.y; v.z += o.v.z; v.w += o.v.w; }
    __device__ __forceinline__ void xor_reduce(int off) {
        v.x += __shfl_xor_sync(0xffffffffu, v.x, off);
        v.y += __shfl_xor_sync(0xffffffffu, v.y, off);
        v.z += __shfl_xor_sync(0xffffffffu, v.z, off);
        v.w += __shfl_xor_sync(0xffffffffu, v.w, off);
    }
    __device__ __forceinline__ void store_smem(float* p) const { *reinterpret_cast<float4*>(p) = v; }
    __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = v; }   // 16-byte aligned destination
    __device__ __forceinline__ float get(int j) const { return j == 0 ? v.x : j == 1 ? v.y : j == 2 ? v.z : v.w; }
};
template <> struct Vec<1> {
    float v;
    __device__ __forceinline__ void zero() { v = 0.f; }
    __device__ __forceinline__ void load(const float* p) { v = __ldg(p); }
    __device__ __forceinline__ void add(const Vec& o) { v += o.v; }
    __device__ __forceinline__ void xor_reduce(int off) { v += __shfl_xor_sync(0xffffffffu, v, off); }
    __device__ __forceinline__ void store_smem(float* p) const { *p = v; }
    __device__ __forceinline__ void store(float* p) const { *p = v; }
    __device__ __forceinline__ float get(int) const { return v; }
};

// Adds up the 32/LPR sub-warps' partial rows (each lane holds VEC columns of its sub-warp's sum).  A plain butterfly
// would shuffle all VEC values at every one of its log2(32/LPR) steps; here a lane sends, at each step, the half of its
// values that its partner keeps and keeps the other half, until one value is left (then the steps are plain
// exchanges): VEC - 1 + (steps beyond log2 VEC) shuffles instead of VEC * steps (4 instead of 12 at 16 columns).
// On return out[0 .. n) are final sums of columns first .. first+n-1 of the lane's VEC columns, and `owner` says whether
// this lane is the one that should store them (lanes that differ only in the plain-exchange bits hold copies).
template <int LPR, int VEC>
struct Folded { float out[VEC]; int first; int n; bool owner; };

template <int LPR, int VEC>
__device__ __forceinline__ Folded<LPR, VEC> fold_subwarps(const Vec<VEC>& acc, int lane) {
    Folded<LPR, VEC> f;
#pragma unroll
    for (int j = 0; j < VEC; j++) f.out[j] = acc.get(j);
    f.first = 0; f.n = VEC; f.owner = true;
    int n = VEC;
#pragma unroll
    for (int off = 16; off >= LPR; off >>= 1) {
        const bool up = (lane & off) != 0;
        if (n > 1) {
            n >>= 1;
#pragma unroll
            for (int j = 0; j < VEC / 2; j++) {
                if (j < n) {
                    const float keep = up ? f.out[j + n] : f.out[j];
                    const float send = up ? f.out[j] : f.out[j + n];
                    f.out[j] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                }
            }
            f.first += up ? n : 0;
        } else {
            f.out[0] += __shfl_xor_sync(0xffffffffu, f.out[0], off);
            f.owner = f.owner && !up;
        }
    }
    f.n = n;
    return f;
}

// Adds the rows of up to 32 neighbors (ids held one per lane in `my`, -1 = none) into acc.
// FULL: all 32 ids are valid, so no per-row predicate is needed.
template <int LPR, int VEC, bool REMOTE, bool FULL>
__device__ __forceinline__ void gather_batch(Vec<VEC>& acc, const AggParams& P, const float* const* s_peer,
                                             const char* lbase, unsigned row_bytes, int my, int cnt,
                                             int g, int col, bool col_ok) {
    constexpr int G = 32 / LPR;             // neighbor rows per load round
    constexpr int U = LPR < MGGB_AGG_MAX_ROUNDS ? LPR : MGGB_AGG_MAX_ROUNDS;  // rounds issued back to back
#pragma unroll 1
    for (int r0 = 0; r0 < LPR; r0 += U) {
        if (!FULL && r0 * G >= cnt) break;
        Vec<VEC> v[U];
        bool ok[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int got = __shfl_sync(0xffffffffu, my, (r0 + u) * G + g);
            ok[u] = col_ok && (FULL || got >= 0);
            const int nid = FULL ? got : max(got, 0);   // absent lanes hold -1: keep every address and the owner index in range
            const float* src;
            if (REMOTE) {
                const unsigned owner = (unsigned)(((unsigned long long)(unsigned)nid * P.div_magic) >> P.div_shift);
                const int row = nid - (int)owner * P.node_per_pe;
                src = s_peer[owner] + (long long)row * P.dim + col;
            } else {
                src = reinterpret_cast<const float*>(lbase + (long long)nid * row_bytes);
            }
            if (ok[u]) v[u].load(src);
        }
#pragma unroll
        for (int u = 0; u < U; u++)
            if (ok[u]) acc.add(v[u]);
    }
}

// Gathers the edges [beg, end) of one neighbor list that belong to this warp and adds their rows
// (columns [col, col+VEC) of each) into acc.  REMOTE selects the owner lookup.
// The warp's share is walked as a sequence of batches of up to 32 ids: chunk q of the warp starts
// at beg + (q*nwarps + warp)*chunk.  The ids of batch t+1 are requested before the rows of batch t
// are gathered, so the id fetch (from HBM) overlaps the row fetch (mostly from L2).
// WALK: 0 chunk by chunk; 1 the same with the next batch of ids requested early; 2 chunks shorter than a batch
template <int LPR, int VEC, bool REMOTE, int WALK>
__device__ __forceinline__ void gather_list(Vec<VEC>& acc, const AggParams& P, const float* const* s_peer,
                                            const int32_t* __restrict__ ci, int beg, int end, const char* lbase,
                                            int warp, int nwarps, int lane, int col, bool col_ok) {
    const int g = lane / LPR;
    const unsigned row_bytes = (unsigned)P.dim * 4u;
    // directly addressed rows (REMOTE == false): address = lbase + id * row_bytes
    // Edge positions fit 32 bits (a shard half has < 2^31 edges and the chunk is clamped to 2^24),
    // so the walk uses unsigned arithmetic.
    const unsigned uend = (unsigned)end, chunk = (unsigned)P.chunk;
    const unsigned block_stride = chunk * (unsigned)nwarps;
    if (WALK == 2) {
        // Chunks shorter than a batch: the warp's edges, chunk after chunk, form one virtual sequence
        // and every batch takes its next 32 of them (lane k's edge sits in the warp's chunk k / chunk),
        // so that small part_size * interleaved_dist settings still gather 32 rows per batch.
        for (unsigned k0 = 0;; k0 += 32) {
            const unsigned k = k0 + (unsigned)lane, q = k / chunk;
            const unsigned pos = (unsigned)beg + (q * (unsigned)nwarps + (unsigned)warp) * chunk + (k - q * chunk);
            const unsigned valid = __ballot_sync(0xffffffffu, pos < uend);   // positions grow with k: a prefix of the lanes
            if (valid == 0u) break;
            const int cnt = __popc(valid);
            const int my = pos < uend ? __ldcs(ci + pos) : -1;
            if (cnt == 32) gather_batch<LPR, VEC, REMOTE, true>(acc, P, s_peer, lbase, row_bytes, my, cnt, g, col, col_ok);
            else           gather_batch<LPR, VEC, REMOTE, false>(acc, P, s_peer, lbase, row_bytes, my, cnt, g, col, col_ok);
            if (cnt < 32) break;
        }
        return;
    }
    unsigned cstart = (unsigned)beg + (unsigned)warp * chunk;         // start of the current chunk
    if (cstart >= uend) return;
    unsigned r = 0;                                                   // offset of the batch in its chunk
    int cnt = (int)min(32u, min(chunk, uend - cstart));
    int my = (lane < cnt) ? __ldcs(ci + cstart + lane) : -1;
    while (true) {
        unsigned ncs = cstart, nr = r + 32;
        if (nr >= chunk || ncs + nr >= uend) { ncs += block_stride; nr = 0; }
        const bool more = ncs < uend;
        int ncnt = 0, nxt = -1;
        if (more) {
            ncnt = (int)min(32u, min(chunk - nr, uend - (ncs + nr)));
            if (WALK == 1 && lane < ncnt) nxt = __ldcs(ci + ncs + nr + lane);
        }
        if (cnt == 32) gather_batch<LPR, VEC, REMOTE, true>(acc, P, s_peer, lbase, row_bytes, my, cnt, g, col, col_ok);
        else           gather_batch<LPR, VEC, REMOTE, false>(acc, P, s_peer, lbase, row_bytes, my, cnt, g, col, col_ok);
        if (!more) break;
        if (WALK != 1 && lane < ncnt) nxt = __ldcs(ci + ncs + nr + lane);
        cstart = ncs; r = nr; cnt = ncnt; my = nxt;
    }
}

// REMOTE_MODE: 0 = one PE, no remote half; 1 = remote rows found through the owner lookup (peers'
// buffers anywhere); 2 = the PEs' buffers are the consecutive slots of ONE matrix indexed by global id
// (a local replica), so remote rows are addressed like local ones.
//
// Adds into acc this warp's share (warp `warp` of `nwarps`) of one node's neighbor rows, columns
// [col, col+VEC).
template <int LPR, int VEC, int REMOTE_MODE, int WALK>
__device__ __forceinline__ void accumulate_row(Vec<VEC>& acc, const AggParams& P, const float* const* s_peer,
                                               int lbeg, int lend, int rbeg, int rend,
                                               int warp, int nwarps, int lane, int col, bool col_ok) {
    const unsigned row_bytes = (unsigned)P.dim * 4u;
    // the shard's first id, lb, is folded into the base of the local rows
    const char* lbase = reinterpret_cast<const char*>(P.peer[P.pe] + col) - (long long)P.lb * row_bytes;
    // The remote list's chunks are dealt to the warps starting where the local list's chunks
    // stopped, so a short remote list does not always land on warp 0 (the reference restarts at
    // warp 0, include/neighbor_utils.cuh:1432-1437; only the fp32 summation order differs).
    const int rwarp = (warp + nwarps - (int)(((unsigned)(lend - lbeg) + P.chunk - 1) / P.chunk % nwarps)) % nwarps;
    if (REMOTE_MODE == 1) {
        gather_list<LPR, VEC, false, WALK>(acc, P, s_peer, P.ci_l, lbeg, lend, lbase, warp, nwarps, lane, col, col_ok);
        if (rend > rbeg)
            gather_list<LPR, VEC, true, WALK>(acc, P, s_peer, P.ci_r, rbeg, rend, nullptr, rwarp, nwarps, lane, col, col_ok);
    } else {
        // both halves are directly addressed: one copy of the gather code walks them in turn
#pragma unroll 1
        for (int half = 0; half < (REMOTE_MODE == 2 ? 2 : 1); half++) {
            const int32_t* ci = half ? P.ci_r : P.ci_l;
            const int beg = half ? rbeg : lbeg, end = half ? rend : lend;
            const char* base = half ? reinterpret_cast<const char*>(P.peer[0] + col) : lbase;
            if (end > beg)
                gather_list<LPR, VEC, false, WALK>(acc, P, s_peer, ci, beg, end, base, half ? rwarp : warp, nwarps, lane, col, col_ok);
        }
    }
}

// Exact unsigned division by a runtime constant d for every 32-bit numerator:
// q = (n * magic) >> shift with shift = 32 + ceil(log2 d), magic = ceil(2^shift / d) < 2^33.
inline void make_divider(uint32_t d, unsigned long long* magic, int* shift) {
    int lg = 0;
    while ((1ull << lg) < d) lg++;
    *shift = 32 + lg;
    const unsigned __int128 one = 1;
    *magic = (unsigned long long)(((one << *shift) + d - 1) / d);
}

// Hands a row with `edges` neighbors (more than hub_min_edges) to the wide-block kernel: as a giant row cut
// into segments when it is long enough and the tables have room, else whole on the hub list.  Called by
// ONE thread.  False: no room anywhere, the caller aggregates the row itself.
__device__ __forceinline__ bool defer_row(const AggParams& P, int row, int edges) {
    if (P.giant_rows != nullptr && edges > GIANT_MIN_EDGES) {
        const int seg_edges = max(GIANT_SEG_EDGES, (edges + GIANT_MAX_SEG - 1) / GIANT_MAX_SEG);
        const int nseg = (edges + seg_edges - 1) / seg_edges;
        const int g = atomicAdd(P.hub_count + 1, 1);
        if (g < P.giant_row_cap) {
            const int first = atomicAdd(P.hub_count + 2, nseg);
            if (first >= 0 && first + nseg <= P.giant_item_cap) {
                P.giant_rows[g] = GiantRow{row, first, nseg, seg_edges};
                return true;
            }
            P.giant_rows[g] = GiantRow{-1, 0, 0, 0};   // no partial rows left: the row goes on the hub list whole
        }
    }
    const int slot = atomicAdd(P.hub_count, 1);
    if (slot < P.hub_cap) P.hub_list[slot] = row;
    return slot < P.hub_cap;
}

// One output element: epilogue (row scale, accumulate / GIN combine) and the stores, also to every publish
// destination.
__device__ __forceinline__ void finish_element(const AggParams& P, int row, int c, float s) {
    const long long o = (long long)row * P.dim + c;
    if (P.row_scale) s *= P.row_scale[row];
    if (P.mode == MODE_GIN) s += P.self_scale * P.peer[P.pe][o];
    else if (P.mode == MODE_ACCUMULATE) s += P.out[o];
    P.out[o] = s;
    for (int k = 0; k < P.num_publish; k++) P.publish[k][o] = s;
}

// Single writer per output element: sums the warps' partial rows (s_part[w * dim + c], complete and
// visible to the block) in warp order, applies the epilogue and stores the row, also to every publish
// destination.  Called by all threads of the block.
__device__ __forceinline__ void store_row(const AggParams& P, int row, const float* s_part, int nwarps) {
    for (int c = threadIdx.x; c < P.dim; c += blockDim.x) {
        float s = 0.f;
        for (int w = 0; w < nwarps; w++) s += s_part[w * P.dim + c];
        finish_element(P, row, c, s);
    }
    // No fence here: the pushed rows only have to be visible to kernels that peers launch after the
    // next barrier, and a kernel's stores are complete, system-wide, when the kernel has finished.
}

}  // namespace
