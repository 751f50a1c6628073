// Shared host code of the command-line drivers: graph loading, per-PE state, peer tables, the
// inter-stage barrier and the timing / stdout protocol.
//
// The reference runs one MPI process per GPU (bench_MGG.py:34-35) and NVSHMEM joins them.  Neither
// exists here; these drivers run ONE process that drives `num_GPUs` PEs from one host thread.  PE p
// runs on device p % (visible devices), so a 4- or 8-PE partition can also be walked on fewer GPUs
// (the PEs then take turns on a device; stdout says so).  Kernels of different PEs never wait on one
// another; ordering between stages is by CUDA events.
#pragma once

#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <ctime>
#include <iostream>
#include <string>
#include <vector>

#include "mgg_compat.hpp"

#define CLI_CUDA(call)                                                                           \
    do {                                                                                         \
        cudaError_t e__ = (call);                                                                \
        if (e__ != cudaSuccess) {                                                                \
            printf("CUDA error @%s: %s\n", #call, cudaGetErrorString(e__));                       \
            exit(-1);                                                                            \
        }                                                                                        \
    } while (0)

namespace cli {

struct Args {
    const char *beg_file, *csr_file, *weight_file;
    int num_GPUs, partSize, warpPerBlock, interleaved_dist, dim, hiddenSize, outdim;
};

// Same ten positional arguments, same order, as src/mgg_np_div_mem.cu:40-49.
inline Args parse(int argc, char** argv) {
    if (argc < 11) {
        printf("Usage: %s beg_file csr_file weight_file num_GPUs partSize warpPerBlock interleaved_dist dim hidden outdim\n", argv[0]);
        exit(-1);
    }
    Args a{argv[1], argv[2], argv[3], atoi(argv[4]), atoi(argv[5]), atoi(argv[6]), atoi(argv[7]), atoi(argv[8]), atoi(argv[9]), atoi(argv[10])};
    if (a.num_GPUs < 1 || a.num_GPUs > MGGB_MAX_PES) { printf("num_GPUs must be in [1,%d]\n", MGGB_MAX_PES); exit(-1); }
    return a;
}

struct Graph {
    std::vector<int64_t> row_ptr;
    std::vector<int32_t> col;
    int64_t n = 0, e = 0;
};

inline Graph load_graph(const Args& a) {
    Graph g;
    MGG_COMPAT_CHECK(mggb_graph_file_info(a.beg_file, a.csr_file, &g.n, &g.e));
    g.row_ptr.resize(g.n + 1);
    g.col.resize(std::max<int64_t>(g.e, 1));
    MGG_COMPAT_CHECK(mggb_graph_file_load(a.beg_file, a.csr_file, g.n, g.e, g.row_ptr.data(), g.col.data()));
    std::cout << "Graph load (success): " << g.n << " verts, " << g.e << " edges\n";
    std::cout << "Complete loading graphs !!" << std::endl;
    return g;
}

// One PE: its device, stream, shard bounds and the split CSR on the device.
struct PE {
    int pe = 0, device = 0;
    cudaStream_t stream = nullptr;
    cudaEvent_t stage_done = nullptr;
    int64_t nodesPerPE = 0, lb = 0, ub = 0;
    int64_t e_local = 0, e_remote = 0;
    int32_t *rp_l = nullptr, *ci_l = nullptr, *rp_r = nullptr, *ci_r = nullptr;
    int rows() const { return (int)(ub - lb); }
};

struct Cluster {
    std::vector<PE> pes;
    int devices = 1;
    bool emulated = false;   // more PEs than devices
    double preproc_ms = 0;

    void use(const PE& p) const { CLI_CUDA(cudaSetDevice(p.device)); }

    // All PEs wait until every PE's work enqueued so far has finished (event-based, no host block).
    void barrier() {
        for (auto& p : pes) { use(p); CLI_CUDA(cudaEventRecord(p.stage_done, p.stream)); }
        for (auto& p : pes) {
            use(p);
            for (auto& q : pes)
                if (q.pe != p.pe) CLI_CUDA(cudaStreamWaitEvent(p.stream, q.stage_done, 0));
        }
    }
    void sync_all() {
        for (auto& p : pes) { use(p); CLI_CUDA(cudaStreamSynchronize(p.stream)); }
    }
};

inline Cluster make_cluster(const Args& a, const Graph& g) {
    Cluster c;
    CLI_CUDA(cudaGetDeviceCount(&c.devices));
    if (c.devices < 1) { printf("no CUDA device\n"); exit(-1); }
    c.emulated = a.num_GPUs > c.devices;
    if (c.emulated)
        printf("note: %d PEs on %d device(s): PEs share devices and run in turn (timings are not multi-GPU timings)\n", a.num_GPUs, c.devices);
    c.pes.resize(a.num_GPUs);
    std::clock_t t0 = std::clock();
    auto w0 = std::chrono::steady_clock::now();
    std::vector<std::vector<int32_t>> lp(a.num_GPUs), rp(a.num_GPUs), lc(a.num_GPUs), rc(a.num_GPUs);
    for (int pe = 0; pe < a.num_GPUs; pe++) {
        PE& p = c.pes[pe];
        p.pe = pe; p.device = pe % c.devices;
        MGG_COMPAT_CHECK(mggb_shard_range(g.n, a.num_GPUs, pe, &p.nodesPerPE, &p.lb, &p.ub));
        MGG_COMPAT_CHECK(mggb_split_csr_count_i64(g.row_ptr.data(), g.col.data(), (int32_t)p.lb, (int32_t)p.ub, &p.e_local, &p.e_remote));
        lp[pe].resize(p.rows() + 1); rp[pe].resize(p.rows() + 1);
        lc[pe].resize(std::max<int64_t>(p.e_local, 1)); rc[pe].resize(std::max<int64_t>(p.e_remote, 1));
        MGG_COMPAT_CHECK(mggb_split_csr_fill_i64(g.row_ptr.data(), g.col.data(), (int32_t)p.lb, (int32_t)p.ub,
                                                 lp[pe].data(), rp[pe].data(), lc[pe].data(), rc[pe].data()));
    }
    (void)t0;
    c.preproc_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - w0).count() / a.num_GPUs;
    printf("Preproc (ms): %.3f\n", c.preproc_ms);   // per PE, as the reference prints its own shard's time
    for (int pe = 0; pe < a.num_GPUs; pe++) {
        PE& p = c.pes[pe];
        c.use(p);
        CLI_CUDA(cudaStreamCreate(&p.stream));
        CLI_CUDA(cudaEventCreateWithFlags(&p.stage_done, cudaEventDisableTiming));
        auto up = [&](int32_t** d, const std::vector<int32_t>& h) {
            CLI_CUDA(cudaMalloc((void**)d, h.size() * sizeof(int32_t)));
            CLI_CUDA(cudaMemcpy(*d, h.data(), h.size() * sizeof(int32_t), cudaMemcpyHostToDevice));
        };
        up(&p.rp_l, lp[pe]); up(&p.ci_l, lc[pe]); up(&p.rp_r, rp[pe]); up(&p.ci_r, rc[pe]);
    }
    for (int a_ = 0; a_ < std::min(c.devices, a.num_GPUs); a_++)
        for (int b_ = 0; b_ < std::min(c.devices, a.num_GPUs); b_++)
            if (a_ != b_) MGG_COMPAT_CHECK(mggb_enable_peer_access(a_, b_));
    return c;
}

// A symmetric buffer: one allocation per PE plus the table every PE passes to the aggregation.
struct Symmetric {
    std::vector<float*> ptr;
    std::vector<const float*> table() const { return std::vector<const float*>(ptr.begin(), ptr.end()); }
};

inline Symmetric alloc_symmetric(Cluster& c, size_t floats) {
    Symmetric s;
    for (auto& p : c.pes) { c.use(p); s.ptr.push_back((float*)mgg_symmetric_malloc(std::max<size_t>(floats, 4) * sizeof(float))); }
    auto t = s.table();
    for (auto& p : c.pes) mgg_register_symmetric(s.ptr[p.pe], t.data(), (int)t.size());
    return s;
}

inline float* alloc_filled(Cluster& c, const PE& p, size_t floats, float value) {
    c.use(p);
    float* d = nullptr;
    floats = std::max<size_t>(floats, 4);
    CLI_CUDA(cudaMalloc((void**)&d, floats * sizeof(float)));
    std::vector<float> h(floats, value);
    CLI_CUDA(cudaMemcpy(d, h.data(), floats * sizeof(float), cudaMemcpyHostToDevice));
    return d;
}

// Times `num_profiles` runs of `body` the way the reference does (src/mgg_np_div_mem.cu:206-234):
// barrier, wall clock, loop, barrier; prints the per-PE CPU-clock line and the "MPI time (ms)" line
// that analysis_MGG.py scrapes.  Unlike the reference it does warm-up passes first.
template <typename F>
double time_loop(Cluster& c, int num_profiles, int warmup, F body) {
    for (int i = 0; i < warmup; i++) body();
    c.sync_all();
    std::clock_t c0 = std::clock();
    auto w0 = std::chrono::steady_clock::now();
    for (int i = 0; i < num_profiles; i++) body();
    c.sync_all();
    double wall_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - w0).count() / num_profiles;
    double cpu_ms = 1000.0 * (std::clock() - c0) / CLOCKS_PER_SEC / num_profiles;
    for (auto& p : c.pes) printf("PE-%d, Total (ms): %.3f\n", p.pe, cpu_ms);
    printf("MPI time (ms) %.3f\n", wall_ms);
    return wall_ms;
}

// MGG_VALIDATE=1 in the environment: with the reference's all-ones inputs and weights every column of a
// layer's output holds the same number per node, which the host can follow through the layers in double
// precision from the graph alone.  Compares `width` columns of each PE's rows in d_buf with want[node]
// (exactly when rel == 0, as the reference's check_equal does, include/utils.cuh:130-138) and prints the
// reference's "Validation status" line.
inline bool validate_enabled() { const char* v = getenv("MGG_VALIDATE"); return v && atoi(v); }

inline bool validate_rows(Cluster& c, const std::vector<float*>& d_buf, int width, const std::vector<double>& want, double rel) {
    bool ok = true;
    for (auto& p : c.pes) {
        c.use(p);
        std::vector<float> h((size_t)p.rows() * width);
        CLI_CUDA(cudaMemcpy(h.data(), d_buf[p.pe], h.size() * sizeof(float), cudaMemcpyDeviceToHost));
        for (int r = 0; r < p.rows() && ok; r++) {
            const double w = want[p.lb + r];
            for (int d = 0; d < width; d++) {
                const double got = h[(size_t)r * width + d];
                const bool same = rel == 0.0 ? got == w : std::fabs(got - w) <= rel * std::fabs(w) + 1e-4;
                if (!same) { printf("[PE %d row %d] ref: %.6g -- out: %.6g\n", p.pe, r, w, got); ok = false; break; }
            }
        }
    }
    printf("Validation status: %s\n", ok ? "True" : "False");
    return ok;
}

// sum over the neighbors j of node i of v[j], for every node (host, double)
inline std::vector<double> neighbor_sums(const Graph& g, const std::vector<double>& v) {
    std::vector<double> out(g.n, 0.0);
    for (int64_t i = 0; i < g.n; i++)
        for (int64_t e = g.row_ptr[i]; e < g.row_ptr[i + 1]; e++) out[i] += v[g.col[e]];
    return out;
}

inline void report(const Cluster& c, const Args& a, const Graph& g, double ms, int aggregations, int agg_dim) {
    int64_t el = 0, er = 0, max_l = 0, max_r = 0;
    for (auto& p : c.pes) { el += p.e_local; er += p.e_remote; max_l = std::max(max_l, p.e_local); max_r = std::max(max_r, p.e_remote); }
    printf("{\"ms\": %.4f, \"edges_per_s\": %.4e, \"num_GPUs\": %d, \"devices\": %d, \"emulated\": %s, \"ps\": %d, \"wpb\": %d, \"dist\": %d, "
           "\"nodes\": %lld, \"edges\": %lld, \"aggregations\": %d, \"aggregated_width\": %d, \"remote_fraction\": %.4f, "
           "\"max_local_gather_bytes\": %lld, \"max_remote_gather_bytes\": %lld}\n",
           ms, aggregations * (double)g.e / (ms * 1e-3), a.num_GPUs, c.devices, c.emulated ? "true" : "false", a.partSize, a.warpPerBlock,
           a.interleaved_dist, (long long)g.n, (long long)g.e, aggregations, agg_dim, g.e ? (double)er / g.e : 0.0,
           (long long)(4LL * agg_dim * max_l), (long long)(4LL * agg_dim * max_r));
    printf("===================================\n");
}

}  // namespace cli
