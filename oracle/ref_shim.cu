/* Oracle-side binding of the reference's own HOST code (test infrastructure, never shipped).
 *
 * This translation unit includes the reference's headers from where they lie (the include path is
 * given on the command line by oracle/Makefile) and re-exports three of its host functions through
 * a C ABI so that tests and the CPU-baseline leg of the benchmark can call them with ctypes:
 *   - SAG_ref            include/utils.cuh:71-86           CPU CSR aggregation (fp32, sequential)
 *   - split_CSR<int>     include/neighbor_utils.cuh:381-405  local/remote split of a node shard
 *   - build_part<int>    include/neighbor_utils.cuh:411-460  explicit neighbor-partition arrays
 * No reference source is copied: the functions are called, not restated.
 */
#include <string>
#include <vector>
#include <cstdio>
#include <cstring>
#include <iostream>
#include <unistd.h>
#include <fcntl.h>
#include "utils.cuh"
#include "neighbor_utils.cuh"

extern "C" {

void mggref_sag_ref(float* update, float* input, int* node_ptr, int* column_index,
                    int num_node, int num_edges, int dim) {
    SAG_ref(update, input, node_ptr, column_index, num_node, num_edges, dim);
}

/* Two-call protocol: sizes first (out arrays NULL), then fill. */
void mggref_split_csr(const int* row_ptr, long long n_ptr, const int* col_idx, long long n_col,
                      int lb, int ub, long long* n_local, long long* n_remote,
                      int* local_ptr, int* remote_ptr, int* local_col, int* remote_col) {
    std::vector<int> p(row_ptr, row_ptr + n_ptr), c(col_idx, col_idx + n_col);
    auto r = split_CSR<int>(p, c, lb, ub);
    *n_local = (long long)r[2].size();
    *n_remote = (long long)r[3].size();
    if (local_ptr)  std::memcpy(local_ptr,  r[0].data(), r[0].size() * sizeof(int));
    if (remote_ptr) std::memcpy(remote_ptr, r[1].data(), r[1].size() * sizeof(int));
    if (local_col && !r[2].empty())  std::memcpy(local_col,  r[2].data(), r[2].size() * sizeof(int));
    if (remote_col && !r[3].empty()) std::memcpy(remote_col, r[3].data(), r[3].size() * sizeof(int));
}

/* build_part prints one line to stdout; it is silenced here by pointing fd 1 at /dev/null for the
 * duration of the call. */
void mggref_build_part(const int* indptr, int num_nodes, int part_size, long long* n_parts,
                       int* part_ptr, int* part2node, int* node2part) {
    std::vector<int> p(indptr, indptr + num_nodes + 1);
    fflush(stdout);
    int saved = dup(1), devnull = open("/dev/null", O_WRONLY);
    if (devnull >= 0) dup2(devnull, 1);
    auto r = build_part<int>(std::string("oracle"), p, num_nodes, part_size);
    fflush(stdout);
    if (saved >= 0) { dup2(saved, 1); close(saved); }
    if (devnull >= 0) close(devnull);
    *n_parts = (long long)r[1].size();
    if (part_ptr)  std::memcpy(part_ptr,  r[0].data(), r[0].size() * sizeof(int));
    if (part2node && !r[1].empty()) std::memcpy(part2node, r[1].data(), r[1].size() * sizeof(int));
    if (node2part) std::memcpy(node2part, r[2].data(), r[2].size() * sizeof(int));
}

}  // extern "C"
