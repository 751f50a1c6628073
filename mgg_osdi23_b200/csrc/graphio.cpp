// Binary CSR files in the reference's on-disk layout (include/graph.hpp:9-129):
//   <name>_beg_pos.bin  N+1 int64 row offsets
//   <name>_csr.bin      E   int64 neighbor ids
//   <name>_weight.bin   E   int32 edge weights (the reference loads them and never reads them)
// The reference narrows both to int in memory on every rank; here row offsets stay 64-bit and ids
// are narrowed to int32, streamed in blocks so that no second full-size copy is held.
#include <sys/stat.h>
#include <sys/types.h>
#include <climits>
#include <cstdio>
#include <vector>
#include "common.h"

namespace {
int64_t file_size(const char* path) {
    struct stat st;
    return stat(path, &st) == 0 ? (int64_t)st.st_size : -1;
}
}  // namespace

extern "C" {

int mggb_graph_file_info(const char* beg_file, const char* csr_file, int64_t* num_nodes, int64_t* num_edges) {
    MGGB_REQUIRE(beg_file && csr_file && num_nodes && num_edges, "graph_file_info: NULL argument");
    const int64_t sb = file_size(beg_file), sc = file_size(csr_file);
    if (sb < 8 || sb % 8) return mggb::fail(MGGB_ERR_IO, "graph_file_info: %s missing or not a multiple of 8 bytes", beg_file);
    if (sc < 0 || sc % 8) return mggb::fail(MGGB_ERR_IO, "graph_file_info: %s missing or not a multiple of 8 bytes", csr_file);
    *num_nodes = sb / 8 - 1;
    *num_edges = sc / 8;
    return MGGB_OK;
}

int mggb_graph_file_load(const char* beg_file, const char* csr_file, int64_t num_nodes, int64_t num_edges,
                         int64_t* row_ptr64, int32_t* col_idx) {
    MGGB_REQUIRE(beg_file && csr_file && row_ptr64, "graph_file_load: NULL argument");
    MGGB_REQUIRE(num_edges == 0 || col_idx, "graph_file_load: NULL col_idx");
    FILE* f = fopen(beg_file, "rb");
    if (!f) return mggb::fail(MGGB_ERR_IO, "graph_file_load: cannot open %s", beg_file);
    size_t got = fread(row_ptr64, sizeof(int64_t), (size_t)num_nodes + 1, f);
    fclose(f);
    if (got != (size_t)num_nodes + 1) return mggb::fail(MGGB_ERR_IO, "graph_file_load: %s is short", beg_file);
    if (row_ptr64[num_nodes] != num_edges)
        return mggb::fail(MGGB_ERR_IO, "graph_file_load: last offset %lld != edge count %lld", (long long)row_ptr64[num_nodes], (long long)num_edges);
    f = fopen(csr_file, "rb");
    if (!f) return mggb::fail(MGGB_ERR_IO, "graph_file_load: cannot open %s", csr_file);
    std::vector<int64_t> buf(1 << 20);
    int64_t done = 0;
    while (done < num_edges) {
        const size_t want = (size_t)((num_edges - done) < (int64_t)buf.size() ? (num_edges - done) : (int64_t)buf.size());
        got = fread(buf.data(), sizeof(int64_t), want, f);
        if (got != want) { fclose(f); return mggb::fail(MGGB_ERR_IO, "graph_file_load: %s is short", csr_file); }
        for (size_t i = 0; i < got; i++) {
            if (buf[i] < 0 || buf[i] >= num_nodes || buf[i] > INT32_MAX) {
                fclose(f);
                return mggb::fail(MGGB_ERR_IO, "graph_file_load: neighbor id %lld out of range at edge %lld", (long long)buf[i], (long long)(done + (int64_t)i));
            }
            col_idx[done + (int64_t)i] = (int32_t)buf[i];
        }
        done += (int64_t)got;
    }
    fclose(f);
    return MGGB_OK;
}

// A shard's rows only: reads offsets [lb, ub] and the ids between them, so that a rank which owns
// 1/G of a graph touches 1/G of the files (the reference loads the whole graph on every rank,
// src/mgg_np_div_mem.cu:54-56).
int mggb_graph_file_rows_info(const char* beg_file, int64_t lb, int64_t ub, int64_t* first_edge, int64_t* num_edges) {
    MGGB_REQUIRE(beg_file && first_edge && num_edges, "graph_file_rows_info: NULL argument");
    const int64_t sb = file_size(beg_file);
    if (sb < 8 || sb % 8) return mggb::fail(MGGB_ERR_IO, "graph_file_rows_info: %s missing or not a multiple of 8 bytes", beg_file);
    const int64_t num_nodes = sb / 8 - 1;
    MGGB_REQUIRE(lb >= 0 && lb <= ub && ub <= num_nodes, "graph_file_rows_info: need 0 <= lb <= ub <= %lld (lb=%lld ub=%lld)",
                 (long long)num_nodes, (long long)lb, (long long)ub);
    FILE* f = fopen(beg_file, "rb");
    if (!f) return mggb::fail(MGGB_ERR_IO, "graph_file_rows_info: cannot open %s", beg_file);
    int64_t ends[2] = {0, 0};
    bool ok = fseeko(f, (off_t)lb * 8, SEEK_SET) == 0 && fread(&ends[0], 8, 1, f) == 1 &&
              fseeko(f, (off_t)ub * 8, SEEK_SET) == 0 && fread(&ends[1], 8, 1, f) == 1;
    fclose(f);
    if (!ok) return mggb::fail(MGGB_ERR_IO, "graph_file_rows_info: %s is short", beg_file);
    if (ends[0] < 0 || ends[1] < ends[0])
        return mggb::fail(MGGB_ERR_IO, "graph_file_rows_info: offsets of rows %lld and %lld are not ascending", (long long)lb, (long long)ub);
    *first_edge = ends[0];
    *num_edges = ends[1] - ends[0];
    return MGGB_OK;
}

int mggb_graph_file_load_rows(const char* beg_file, const char* csr_file, int64_t lb, int64_t ub,
                              int64_t* row_ptr64, int32_t* col_idx) {
    MGGB_REQUIRE(beg_file && csr_file && row_ptr64, "graph_file_load_rows: NULL argument");
    int64_t first = 0, count = 0;
    const int st = mggb_graph_file_rows_info(beg_file, lb, ub, &first, &count);
    if (st != MGGB_OK) return st;
    MGGB_REQUIRE(count == 0 || col_idx, "graph_file_load_rows: NULL col_idx");
    const int64_t num_nodes = file_size(beg_file) / 8 - 1;
    const int64_t rows = ub - lb;
    FILE* f = fopen(beg_file, "rb");
    if (!f) return mggb::fail(MGGB_ERR_IO, "graph_file_load_rows: cannot open %s", beg_file);
    bool ok = fseeko(f, (off_t)lb * 8, SEEK_SET) == 0 && fread(row_ptr64, 8, (size_t)rows + 1, f) == (size_t)rows + 1;
    fclose(f);
    if (!ok) return mggb::fail(MGGB_ERR_IO, "graph_file_load_rows: %s is short", beg_file);
    for (int64_t i = 0; i <= rows; i++) {
        row_ptr64[i] -= first;                       // the shard's pointers start at 0
        if (row_ptr64[i] < 0 || row_ptr64[i] > count || (i > 0 && row_ptr64[i] < row_ptr64[i - 1]))
            return mggb::fail(MGGB_ERR_IO, "graph_file_load_rows: offsets are not ascending at row %lld", (long long)(lb + i));
    }
    if (file_size(csr_file) < (first + count) * 8)
        return mggb::fail(MGGB_ERR_IO, "graph_file_load_rows: %s is short", csr_file);
    f = fopen(csr_file, "rb");
    if (!f) return mggb::fail(MGGB_ERR_IO, "graph_file_load_rows: cannot open %s", csr_file);
    if (fseeko(f, (off_t)first * 8, SEEK_SET) != 0) { fclose(f); return mggb::fail(MGGB_ERR_IO, "graph_file_load_rows: cannot seek in %s", csr_file); }
    std::vector<int64_t> buf(1 << 20);
    for (int64_t done = 0; done < count;) {
        const size_t want = (size_t)((count - done) < (int64_t)buf.size() ? (count - done) : (int64_t)buf.size());
        if (fread(buf.data(), sizeof(int64_t), want, f) != want) { fclose(f); return mggb::fail(MGGB_ERR_IO, "graph_file_load_rows: %s is short", csr_file); }
        for (size_t i = 0; i < want; i++) {
            if (buf[i] < 0 || buf[i] >= num_nodes || buf[i] > INT32_MAX) {
                fclose(f);
                return mggb::fail(MGGB_ERR_IO, "graph_file_load_rows: neighbor id %lld out of range at edge %lld", (long long)buf[i], (long long)(first + done + (int64_t)i));
            }
            col_idx[done + (int64_t)i] = (int32_t)buf[i];
        }
        done += (int64_t)want;
    }
    fclose(f);
    return MGGB_OK;
}

int mggb_graph_file_write(const char* beg_file, const char* csr_file, const char* weight_file,
                          const int64_t* row_ptr64, const int32_t* col_idx, int64_t num_nodes) {
    MGGB_REQUIRE(beg_file && csr_file && row_ptr64, "graph_file_write: NULL argument");
    const int64_t num_edges = row_ptr64[num_nodes];
    MGGB_REQUIRE(num_edges == 0 || col_idx, "graph_file_write: NULL col_idx");
    FILE* f = fopen(beg_file, "wb");
    if (!f) return mggb::fail(MGGB_ERR_IO, "graph_file_write: cannot create %s", beg_file);
    size_t put = fwrite(row_ptr64, sizeof(int64_t), (size_t)num_nodes + 1, f);
    fclose(f);
    if (put != (size_t)num_nodes + 1) return mggb::fail(MGGB_ERR_IO, "graph_file_write: short write to %s", beg_file);
    f = fopen(csr_file, "wb");
    if (!f) return mggb::fail(MGGB_ERR_IO, "graph_file_write: cannot create %s", csr_file);
    std::vector<int64_t> buf(1 << 20);
    for (int64_t done = 0; done < num_edges;) {
        const size_t m = (size_t)((num_edges - done) < (int64_t)buf.size() ? (num_edges - done) : (int64_t)buf.size());
        for (size_t i = 0; i < m; i++) buf[i] = col_idx[done + (int64_t)i];
        if (fwrite(buf.data(), sizeof(int64_t), m, f) != m) { fclose(f); return mggb::fail(MGGB_ERR_IO, "graph_file_write: short write to %s", csr_file); }
        done += (int64_t)m;
    }
    fclose(f);
    if (weight_file) {
        f = fopen(weight_file, "wb");
        if (!f) return mggb::fail(MGGB_ERR_IO, "graph_file_write: cannot create %s", weight_file);
        std::vector<int32_t> ones(1 << 20, 1);
        for (int64_t done = 0; done < num_edges;) {
            const size_t m = (size_t)((num_edges - done) < (int64_t)ones.size() ? (num_edges - done) : (int64_t)ones.size());
            if (fwrite(ones.data(), sizeof(int32_t), m, f) != m) { fclose(f); return mggb::fail(MGGB_ERR_IO, "graph_file_write: short write to %s", weight_file); }
            done += (int64_t)m;
        }
        fclose(f);
    }
    return MGGB_OK;
}

}  // extern "C"
