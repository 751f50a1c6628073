// Neighbor aggregation over EXPLICIT neighbor partitions: one warp per `interleaved_dist` partitions
// of at most `part_size` edges each, grid proportional to the number of partitions (sm_100a).
//
// Stands in for the reference's partition-array kernels (SAG_cuda_kernel_fused_interleaved,
// include/neighbor_utils.cuh:2598-2760, launched by SAG_host_fused_interleaved, :593-676, from
// src/test_neighbor_part.cu:93-211) and consumes exactly what build_part returns (:411-460):
// part_ptr (first edge of each partition), part2node (the row a partition belongs to) and node2part
// (first partition of each row).  Where the block-per-node kernels give every node a block however
// short or long its list is, here the unit of work is a partition, so a node with 10^5 neighbors is
// spread over thousands of warps and a node with 3 neighbors costs one short partition.
//
// The reference adds every partition's partial row into the output with its exchange-spin float atomic
// (:2683-2686, atomicAdd_F :28-32) and has its remote half commented out (:2693-2759).  Here:
//   kernel 1  warp w takes partitions [w*dist, (w+1)*dist) of the local half and the same range of
//             the remote half (the reference's warp-to-partition map, :2636-2640), gathers each
//             partition's rows (sub-warp 128-bit loads, register sums, remote rows through the peer
//             table) and writes the partition's partial row to a scratch matrix [partitions x dim];
//   kernel 2  one thread per output element adds its row's partial rows in partition order (local half
//             first), applies the epilogue and stores the element: one writer per row, no atomics,
//             the same bits on every run.
// A partition ends at min(part_ptr[p] + part_size, end of its row): part_ptr[p+1] is not used, so
// the reference's unwritten closing sentinel (:453-454) does no harm.
#include <algorithm>
#include "aggregate_core.cuh"

namespace {

struct PartHalf {
    const int32_t* rp;
    const int32_t* ci;
    const int32_t* part_ptr;
    const int32_t* part2node;
    const int32_t* node2part;
    long long num_parts;
    float* partial;            // [num_parts x dim]
};

struct PartParams {
    AggParams A;               // output, peer table, epilogue, shard bounds (rp/ci fields unused)
    PartHalf half[2];          // 0 local, 1 remote
    int ps, dist;
};

// Sum of the rows of edges [beg, end) of one partition, columns [col, col+VEC), into the sub-warps'
// registers, folded across sub-warps; valid in lanes < LPR on return.
template <int LPR, int VEC, bool REMOTE>
__device__ __forceinline__ Vec<VEC> partition_sum(const AggParams& P, const float* const* s_peer, const int32_t* __restrict__ ci,
                                                  int beg, int end, const char* lbase, int lane, int col, bool col_ok) {
    Vec<VEC> acc;
    acc.zero();
    const int g = lane / LPR;
    const unsigned row_bytes = (unsigned)P.dim * 4u;
    for (int e = beg; e < end; e += 32) {
        const int cnt = min(32, end - e);
        const int my = lane < cnt ? __ldcs(ci + e + lane) : -1;
        if (cnt == 32) gather_batch<LPR, VEC, REMOTE, true>(acc, P, s_peer, lbase, row_bytes, my, cnt, g, col, col_ok);
        else           gather_batch<LPR, VEC, REMOTE, false>(acc, P, s_peer, lbase, row_bytes, my, cnt, g, col, col_ok);
    }
#pragma unroll
    for (int off = LPR; off < 32; off <<= 1) acc.xor_reduce(off);
    return acc;
}

// REMOTE_MODE as in aggregate.cu: 0 one PE, 1 owner lookup, 2 one replica matrix.
template <int LPR, int VEC, int REMOTE_MODE>
__global__ void __launch_bounds__(512) sag_part_kernel(const PartParams Q) {
    __shared__ const float* s_peer[MGGB_MAX_PES];
    const AggParams& P = Q.A;
    if (REMOTE_MODE == 1) {
        if (threadIdx.x < MGGB_MAX_PES) s_peer[threadIdx.x] = P.peer[threadIdx.x < P.num_pes ? threadIdx.x : 0];
        __syncthreads();
    }
    const int lane = threadIdx.x & 31, l = lane % LPR;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const unsigned row_bytes = (unsigned)P.dim * 4u;
    constexpr int COLS = LPR * VEC;
#pragma unroll 1
    for (int h = 0; h < (REMOTE_MODE == 0 ? 1 : 2); h++) {
        const PartHalf& H = Q.half[h];
        const long long p0 = warp * Q.dist, p1 = min(p0 + Q.dist, H.num_parts);
        for (long long p = p0; p < p1; p++) {
            const int node = H.part2node[p];
            const int beg = H.part_ptr[p];
            const int end = min(beg + Q.ps, H.rp[node + 1]);
            for (int cb = 0; cb < P.dim; cb += COLS) {
                const int col = cb + l * VEC;
                const bool col_ok = col < P.dim;
                Vec<VEC> acc;
                if (h == 0) {
                    const char* lbase = reinterpret_cast<const char*>(P.peer[P.pe] + col) - (long long)P.lb * row_bytes;
                    acc = partition_sum<LPR, VEC, false>(P, s_peer, H.ci, beg, end, lbase, lane, col, col_ok);
                } else if (REMOTE_MODE == 1) {
                    acc = partition_sum<LPR, VEC, true>(P, s_peer, H.ci, beg, end, nullptr, lane, col, col_ok);
                } else {
                    acc = partition_sum<LPR, VEC, false>(P, s_peer, H.ci, beg, end, reinterpret_cast<const char*>(P.peer[0] + col), lane, col, col_ok);
                }
                if (lane < LPR && col_ok) acc.store(H.partial + p * P.dim + col);
            }
        }
    }
}

// One thread per (node, column): adds the node's partial rows, local half first, in partition order
// (long lists: in LANES interleaved running sums).
constexpr int LANES = 16;
__global__ void __launch_bounds__(256) sag_part_reduce_kernel(const PartParams Q, const int halves) {
    const AggParams& P = Q.A;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)P.num_rows * P.dim;
    if (idx >= total) return;
    const int row = (int)(idx / P.dim), c = (int)(idx - (long long)row * P.dim);
    float s = 0.f;
    for (int h = 0; h < halves; h++) {
        const PartHalf& H = Q.half[h];
        const int a = H.node2part[row], b = H.node2part[row + 1];
        const float* src = H.partial + (long long)a * P.dim + c;
        const long long step = P.dim;
        int p = a;
        if (b - a >= 2 * LANES) {
            // a long list (a hub row cut into thousands of partitions): LANES running sums, folded pairwise at
            // the end, keep LANES loads in flight and the rounding error LANES times below one running sum's
            float acc[LANES];
#pragma unroll
            for (int j = 0; j < LANES; j++) acc[j] = 0.f;
            for (; p + LANES <= b; p += LANES, src += LANES * step) {
#pragma unroll
                for (int j = 0; j < LANES; j++) acc[j] += src[j * step];
            }
#pragma unroll
            for (int w = LANES / 2; w >= 1; w >>= 1)
#pragma unroll
                for (int j = 0; j < w; j++) acc[j] += acc[j + w];
            s += acc[0];
        }
        for (; p < b; p++, src += step) s += *src;
    }
    if (P.row_scale) s *= P.row_scale[row];
    const long long o = (long long)row * P.dim + c;
    if (P.mode == MODE_GIN) s += P.self_scale * P.peer[P.pe][o];
    else if (P.mode == MODE_ACCUMULATE) s += P.out[o];
    P.out[o] = s;
    for (int k = 0; k < P.num_publish; k++) P.publish[k][o] = s;
}

template <int LPR, int VEC>
int launch_part(const PartParams& Q, int remote_mode, int grid, int block, cudaStream_t st) {
    if (remote_mode == 0) sag_part_kernel<LPR, VEC, 0><<<grid, block, 0, st>>>(Q);
    else if (remote_mode == 1) sag_part_kernel<LPR, VEC, 1><<<grid, block, 0, st>>>(Q);
    else sag_part_kernel<LPR, VEC, 2><<<grid, block, 0, st>>>(Q);
    MGGB_CUDA(cudaGetLastError());
    return MGGB_OK;
}

}  // namespace

extern "C" {

int mggb_sag_np_part_scratch_bytes(int64_t num_parts_l, int64_t num_parts_r, int dim, size_t* bytes) {
    MGGB_REQUIRE(bytes, "sag_np_part_scratch_bytes: NULL output");
    MGGB_REQUIRE(num_parts_l >= 0 && num_parts_r >= 0 && dim >= 1, "sag_np_part_scratch_bytes: need counts >= 0 and dim >= 1");
    *bytes = (size_t)(num_parts_l + num_parts_r) * (size_t)dim * sizeof(float);
    return MGGB_OK;
}

int mggb_sag_np_part(float* output, const float* const* peer_input, int num_pes,
                     const int32_t* row_ptr_l, const int32_t* col_idx_l, const int32_t* part_ptr_l,
                     const int32_t* part2node_l, const int32_t* node2part_l, int64_t num_parts_l,
                     const int32_t* row_ptr_r, const int32_t* col_idx_r, const int32_t* part_ptr_r,
                     const int32_t* part2node_r, const int32_t* node2part_r, int64_t num_parts_r,
                     int32_t lb, int32_t ub, int dim, int32_t node_per_pe, int pe,
                     int part_size, int warp_per_block, int interleaved_dist,
                     const float* row_scale, int flags, float eps,
                     float* scratch, size_t scratch_bytes, void* stream) {
    MGGB_REQUIRE(output && peer_input && row_ptr_l && node2part_l, "sag_np_part: NULL argument");
    MGGB_REQUIRE(num_pes >= 1 && num_pes <= MGGB_MAX_PES, "sag_np_part: num_pes must be in [1,%d] (got %d)", MGGB_MAX_PES, num_pes);
    MGGB_REQUIRE(pe >= 0 && pe < num_pes, "sag_np_part: pe %d outside [0,%d)", pe, num_pes);
    MGGB_REQUIRE(lb >= 0 && ub >= lb && dim >= 1, "sag_np_part: need 0 <= lb <= ub and dim >= 1");
    MGGB_REQUIRE(node_per_pe >= 1 && ub - lb <= node_per_pe, "sag_np_part: shard [%d,%d) larger than node_per_pe=%d", lb, ub, node_per_pe);
    MGGB_REQUIRE((long long)lb == (long long)pe * node_per_pe || ub == lb, "sag_np_part: lb=%d is not pe*node_per_pe (%d*%d)", lb, pe, node_per_pe);
    MGGB_REQUIRE(part_size >= 1 && interleaved_dist >= 1 && warp_per_block >= 1 && warp_per_block <= 16,
                 "sag_np_part: need part_size >= 1, interleaved_dist >= 1, 1 <= warp_per_block <= 16");
    MGGB_REQUIRE(num_parts_l >= 0 && num_parts_r >= 0, "sag_np_part: partition counts must be >= 0");
    MGGB_REQUIRE(num_parts_l == 0 || (col_idx_l && part_ptr_l && part2node_l), "sag_np_part: local partitions without their arrays");
    MGGB_REQUIRE(num_parts_r == 0 || (row_ptr_r && col_idx_r && part_ptr_r && part2node_r && node2part_r), "sag_np_part: remote partitions without their arrays");
    MGGB_REQUIRE(num_pes > 1 || num_parts_r == 0, "sag_np_part: one PE cannot have remote partitions");
    for (int p = 0; p < num_pes; p++) MGGB_REQUIRE(peer_input[p] != nullptr, "sag_np_part: peer_input[%d] is NULL", p);
    const bool gin = (flags & MGGB_AGG_GIN_COMBINE) != 0;
    MGGB_REQUIRE(!gin || output != peer_input[pe], "sag_np_part: with the GIN combine output must not alias this PE's input buffer");
    const size_t need = (size_t)(num_parts_l + num_parts_r) * (size_t)dim * sizeof(float);
    MGGB_REQUIRE(scratch_bytes >= need && (need == 0 || scratch != nullptr),
                 "sag_np_part: scratch of %zu bytes is smaller than the %zu needed (see mggb_sag_np_part_scratch_bytes)", scratch_bytes, need);
    if (ub == lb) return MGGB_OK;

    PartParams Q{};
    AggParams& P = Q.A;
    P.out = output;
    for (int p = 0; p < MGGB_MAX_PES; p++) P.peer[p] = peer_input[p < num_pes ? p : 0];
    P.row_scale = row_scale;
    P.lb = lb; P.num_rows = ub - lb; P.node_per_pe = node_per_pe;
    P.dim = dim; P.pe = pe; P.num_pes = num_pes;
    make_divider((uint32_t)node_per_pe, &P.div_magic, &P.div_shift);
    P.mode = gin ? MODE_GIN : ((flags & MGGB_AGG_ACCUMULATE) ? MODE_ACCUMULATE : MODE_OVERWRITE);
    P.self_scale = 1.0f + eps;
    Q.ps = part_size; Q.dist = interleaved_dist;
    Q.half[0] = PartHalf{row_ptr_l, col_idx_l, part_ptr_l, part2node_l, node2part_l, num_parts_l, scratch};
    Q.half[1] = PartHalf{row_ptr_r, col_idx_r, part_ptr_r, part2node_r, node2part_r, num_parts_r, scratch + (size_t)num_parts_l * dim};

    int remote_mode = 1;
    if (num_pes == 1) remote_mode = 0;
    else {
        bool one_matrix = true;
        for (int p = 1; p < num_pes; p++) one_matrix = one_matrix && (P.peer[p] == P.peer[0] + (long long)p * node_per_pe * dim);
        if (one_matrix) remote_mode = 2;
    }
    const int halves = (remote_mode == 0 || num_parts_r == 0) ? 1 : 2;
    if (halves == 1) Q.half[1].num_parts = 0;

    cudaStream_t st = (cudaStream_t)stream;
    const long long parts = std::max<long long>(num_parts_l, Q.half[1].num_parts);
    if (parts > 0) {
        const long long warps = (parts + interleaved_dist - 1) / interleaved_dist;
        const long long grid = (warps + warp_per_block - 1) / warp_per_block;
        MGGB_REQUIRE(grid <= 0x7fffffffLL, "sag_np_part: %lld blocks exceed the grid limit", grid);
        bool vec4 = (dim % 4 == 0);
        for (int p = 0; p < num_pes && vec4; p++) vec4 = ((uintptr_t)peer_input[p] % 16 == 0);
        vec4 = vec4 && ((uintptr_t)scratch % 16 == 0);
        int rc;
        const int block = warp_per_block * 32;
        if (vec4) {
            const int q = dim / 4;
            if (q <= 1) rc = launch_part<1, 4>(Q, remote_mode, (int)grid, block, st);
            else if (q <= 2) rc = launch_part<2, 4>(Q, remote_mode, (int)grid, block, st);
            else if (q <= 4) rc = launch_part<4, 4>(Q, remote_mode, (int)grid, block, st);
            else if (q <= 8) rc = launch_part<8, 4>(Q, remote_mode, (int)grid, block, st);
            else if (q <= 16) rc = launch_part<16, 4>(Q, remote_mode, (int)grid, block, st);
            else rc = launch_part<32, 4>(Q, remote_mode, (int)grid, block, st);
        } else {
            rc = launch_part<32, 1>(Q, remote_mode, (int)grid, block, st);
        }
        if (rc != MGGB_OK) return rc;
    }
    const long long total = (long long)P.num_rows * dim;
    sag_part_reduce_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(Q, halves);
    MGGB_CUDA(cudaGetLastError());
    return MGGB_OK;
}

}  // extern "C"
