// Host partitioner: node-range shards, the local/remote CSR split and the explicit
// neighbor-partition arrays.
//
// Same results, bit for bit, as the reference's split_CSR / build_part
// (include/neighbor_utils.cuh:381-405, :411-460), produced differently: the reference grows
// std::vectors with push_back on one thread; here every array is sized by a counting pass and then
// filled by all host threads, rows being independent once the per-row offsets are known.
#include <algorithm>
#include <climits>
#include <cstring>
#include <vector>
#include "common.h"

namespace {

template <typename PtrT>
int split_count(const PtrT* row_ptr, const int32_t* col, int32_t lb, int32_t ub,
                int64_t* n_local, int64_t* n_remote) {
    MGGB_REQUIRE(row_ptr && n_local && n_remote, "split_csr_count: NULL argument");
    MGGB_REQUIRE(lb >= 0 && ub >= lb, "split_csr_count: need 0 <= lb <= ub (lb=%d ub=%d)", lb, ub);
    MGGB_REQUIRE(col || row_ptr[ub] == row_ptr[lb], "split_csr_count: NULL col_idx");
    int64_t nl = 0, total = (int64_t)row_ptr[ub] - (int64_t)row_ptr[lb];
#pragma omp parallel for schedule(static) reduction(+ : nl)
    for (int32_t i = lb; i < ub; i++) {
        int64_t c = 0;
        for (PtrT j = row_ptr[i]; j < row_ptr[i + 1]; j++) c += (lb <= col[j] && col[j] < ub);
        nl += c;
    }
    *n_local = nl;
    *n_remote = total - nl;
    if (nl > INT32_MAX || total - nl > INT32_MAX)
        return mggb::fail(MGGB_ERR_UNSUPPORTED,
                          "split_csr: a shard half has more than 2^31-1 edges (local %lld remote %lld)",
                          (long long)nl, (long long)(total - nl));
    return MGGB_OK;
}

template <typename PtrT>
int split_fill(const PtrT* row_ptr, const int32_t* col, int32_t lb, int32_t ub, int32_t* local_ptr,
               int32_t* remote_ptr, int32_t* local_col, int32_t* remote_col) {
    MGGB_REQUIRE(row_ptr && local_ptr && remote_ptr, "split_csr_fill: NULL argument");
    MGGB_REQUIRE(lb >= 0 && ub >= lb, "split_csr_fill: need 0 <= lb <= ub (lb=%d ub=%d)", lb, ub);
    const int32_t rows = ub - lb;
    // Pass 1: per-row local counts, written one slot to the right so the prefix sum is in place.
    local_ptr[0] = 0;
    remote_ptr[0] = 0;
#pragma omp parallel for schedule(static)
    for (int32_t i = 0; i < rows; i++) {
        int32_t c = 0;
        const PtrT b = row_ptr[lb + i], e = row_ptr[lb + i + 1];
        for (PtrT j = b; j < e; j++) c += (lb <= col[j] && col[j] < ub);
        local_ptr[i + 1] = c;
        remote_ptr[i + 1] = (int32_t)(e - b) - c;
    }
    int64_t al = 0, ar = 0;
    for (int32_t i = 0; i < rows; i++) {
        al += local_ptr[i + 1];
        ar += remote_ptr[i + 1];
        if (al > INT32_MAX || ar > INT32_MAX)
            return mggb::fail(MGGB_ERR_UNSUPPORTED, "split_csr_fill: shard half exceeds 2^31-1 edges");
        local_ptr[i + 1] = (int32_t)al;
        remote_ptr[i + 1] = (int32_t)ar;
    }
    MGGB_REQUIRE((al == 0 || local_col) && (ar == 0 || remote_col), "split_csr_fill: NULL column buffer");
    // Pass 2: stable scatter of each row into its two halves.
#pragma omp parallel for schedule(dynamic, 256)
    for (int32_t i = 0; i < rows; i++) {
        int32_t pl = local_ptr[i], pr = remote_ptr[i];
        for (PtrT j = row_ptr[lb + i]; j < row_ptr[lb + i + 1]; j++) {
            const int32_t nid = col[j];
            if (lb <= nid && nid < ub) local_col[pl++] = nid;
            else remote_col[pr++] = nid;
        }
    }
    return MGGB_OK;
}

}  // namespace

extern "C" {

int mggb_shard_range(int64_t num_nodes, int num_pes, int pe, int64_t* nodes_per_pe, int64_t* lb,
                     int64_t* ub) {
    MGGB_REQUIRE(num_nodes >= 0 && num_pes >= 1 && pe >= 0 && pe < num_pes,
                 "shard_range: need num_nodes >= 0 and 0 <= pe < num_pes (N=%lld G=%d pe=%d)",
                 (long long)num_nodes, num_pes, pe);
    MGGB_REQUIRE(nodes_per_pe && lb && ub, "shard_range: NULL output");
    const int64_t npp = (num_nodes + num_pes - 1) / num_pes;
    int64_t l = npp * pe;
    if (l > num_nodes) l = num_nodes;  // trailing PEs of a tiny graph own nothing
    *nodes_per_pe = npp;
    *lb = l;
    *ub = (l + npp) < num_nodes ? (l + npp) : num_nodes;
    return MGGB_OK;
}

int mggb_split_csr_count(const int32_t* row_ptr, const int32_t* col_idx, int32_t lb, int32_t ub,
                         int64_t* n_local, int64_t* n_remote) {
    return split_count<int32_t>(row_ptr, col_idx, lb, ub, n_local, n_remote);
}
int mggb_split_csr_fill(const int32_t* row_ptr, const int32_t* col_idx, int32_t lb, int32_t ub,
                        int32_t* local_ptr, int32_t* remote_ptr, int32_t* local_col,
                        int32_t* remote_col) {
    return split_fill<int32_t>(row_ptr, col_idx, lb, ub, local_ptr, remote_ptr, local_col, remote_col);
}
int mggb_split_csr_count_i64(const int64_t* row_ptr, const int32_t* col_idx, int32_t lb, int32_t ub,
                             int64_t* n_local, int64_t* n_remote) {
    return split_count<int64_t>(row_ptr, col_idx, lb, ub, n_local, n_remote);
}
int mggb_split_csr_fill_i64(const int64_t* row_ptr, const int32_t* col_idx, int32_t lb, int32_t ub,
                            int32_t* local_ptr, int32_t* remote_ptr, int32_t* local_col,
                            int32_t* remote_col) {
    return split_fill<int64_t>(row_ptr, col_idx, lb, ub, local_ptr, remote_ptr, local_col, remote_col);
}

int mggb_build_part_count(const int32_t* indptr, int32_t num_nodes, int32_t part_size,
                          int64_t* num_parts) {
    MGGB_REQUIRE(indptr && num_parts, "build_part_count: NULL argument");
    MGGB_REQUIRE(num_nodes >= 0 && part_size >= 1, "build_part_count: need num_nodes >= 0, part_size >= 1");
    int64_t total = 0;
#pragma omp parallel for schedule(static) reduction(+ : total)
    for (int32_t i = 0; i < num_nodes; i++) {
        const int64_t deg = (int64_t)indptr[i + 1] - indptr[i];
        total += (deg + part_size - 1) / part_size;
    }
    *num_parts = total;
    if (total > INT32_MAX)
        return mggb::fail(MGGB_ERR_UNSUPPORTED, "build_part: more than 2^31-1 partitions");
    return MGGB_OK;
}

int mggb_build_part_fill(const int32_t* indptr, int32_t num_nodes, int32_t part_size,
                         int exact_sentinel, int32_t* part_ptr, int32_t* part2node,
                         int32_t* node2part) {
    MGGB_REQUIRE(indptr && part_ptr && node2part, "build_part_fill: NULL argument");
    MGGB_REQUIRE(num_nodes >= 0 && part_size >= 1, "build_part_fill: need num_nodes >= 0, part_size >= 1");
    // node2part: exclusive prefix of the per-node partition counts, total appended twice.
    int64_t total = 0;
    node2part[0] = 0;
    for (int32_t i = 0; i < num_nodes; i++) {
        const int64_t deg = (int64_t)indptr[i + 1] - indptr[i];
        total += (deg + part_size - 1) / part_size;
        if (total > INT32_MAX)
            return mggb::fail(MGGB_ERR_UNSUPPORTED, "build_part: more than 2^31-1 partitions");
        node2part[i + 1] = (int32_t)total;
    }
    node2part[num_nodes + 1] = (int32_t)total;
    MGGB_REQUIRE(total == 0 || part2node, "build_part_fill: NULL part2node");
#pragma omp parallel for schedule(dynamic, 256)
    for (int32_t i = 0; i < num_nodes; i++) {
        const int32_t first = node2part[i], cnt = node2part[i + 1] - first;
        for (int32_t p = 0; p < cnt; p++) {
            part_ptr[first + p] = indptr[i] + p * part_size;
            part2node[first + p] = i;
        }
    }
    // Closing sentinel.  The reference writes it only while visiting the last node, so it stays 0
    // when that node has no edges (or when there are no nodes at all).
    int32_t sentinel = 0;
    if (num_nodes > 0 && (exact_sentinel || indptr[num_nodes] > indptr[num_nodes - 1]))
        sentinel = indptr[num_nodes];
    part_ptr[total] = sentinel;
    return MGGB_OK;
}

int mggb_degree_order(const int32_t* row_ptr_l, const int32_t* row_ptr_r, int32_t num_rows, int32_t* order) {
    MGGB_REQUIRE(row_ptr_l && order, "degree_order: NULL argument");
    MGGB_REQUIRE(num_rows >= 0, "degree_order: need num_rows >= 0");
    if (num_rows == 0) return MGGB_OK;
    // Counting sort on the degree (stable, so ties stay in row order): degrees are small integers
    // with many repeats, and a comparison sort of 10^7 rows takes seconds.
    std::vector<int32_t> deg((size_t)num_rows);
    int64_t max_deg = 0;
#pragma omp parallel for schedule(static) reduction(max : max_deg)
    for (int32_t i = 0; i < num_rows; i++) {
        int64_t d = (int64_t)row_ptr_l[i + 1] - row_ptr_l[i];
        if (row_ptr_r) d += (int64_t)row_ptr_r[i + 1] - row_ptr_r[i];
        if (d < 0) d = 0;
        if (d > INT32_MAX) d = INT32_MAX;
        deg[i] = (int32_t)d;
        if (d > max_deg) max_deg = d;
    }
    if (max_deg > (int64_t)64 * num_rows + (1 << 20)) {
        // a histogram that large would cost more than sorting: compare instead
        for (int32_t i = 0; i < num_rows; i++) order[i] = i;
        std::stable_sort(order, order + num_rows, [&](int32_t a, int32_t b) { return deg[a] > deg[b]; });
        return MGGB_OK;
    }
    std::vector<int64_t> start((size_t)max_deg + 2, 0);
    for (int32_t i = 0; i < num_rows; i++) start[(size_t)(max_deg - deg[i]) + 1]++;   // bucket 0 = longest rows
    for (int64_t b = 0; b <= max_deg; b++) start[b + 1] += start[b];
    for (int32_t i = 0; i < num_rows; i++) order[start[(size_t)(max_deg - deg[i])]++] = i;
    return MGGB_OK;
}

}  // extern "C"
