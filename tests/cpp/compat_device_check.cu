// Device half of the C++ shim, driven the way the reference's single-aggregation driver drives its
// headers (src/mgg_np_div_kernel.cu:85-188): per PE, shard bounds, split_CSR, device copies of the four
// arrays, `new dense_param_beg("d-1", d_input, numNodes, dim, hiddenSize)` whose d_out is symmetric,
// then mgg_SAG_np_div(dsp_out, dp1->d_out, ...) with the reference's parameter list.  The reference
// runs one MPI process per PE; here one process walks the PEs (PE p on device p % devices) and
// mgg_set_pe stands in for the rank.  Inputs are all ones as in the reference (:120-123), so after
// dense_beg_forward every embedding element equals `dim` and the aggregation of a zeroed output must
// equal degree * dim exactly: the reference's own (disabled) validation idea (:169-171, utils.cuh:130-138).
// Also runs mgg_GIN_np_div, dense_hidden_forward and softmax_forward.  Prints "compat device check: ok".
#include <cmath>
#include <cstdio>
#include <vector>

#include "mgg_compat.hpp"

#define CK(call) do { cudaError_t e__ = (call); if (e__ != cudaSuccess) { printf("CUDA error %s: %s\n", #call, cudaGetErrorString(e__)); return 1; } } while (0)

int main() {
    const int num_GPUs = 2, dim = 8, hiddenSize = 16, partSize = 4, warpPerBlock = 2, interleaved_dist = 2;
    // a 300-node graph from a linear congruential sequence, plus one long row that crosses both shards
    std::vector<nidType> global_row_ptr = {0}, global_col_ind;
    unsigned state = 2024u;
    const nidType numNodes = 300;
    for (nidType i = 0; i < numNodes; i++) {
        state = state * 1664525u + 1013904223u;
        const int deg = (i == 17) ? 900 : (int)((state >> 24) % 23);
        for (int k = 0; k < deg; k++) {
            state = state * 1664525u + 1013904223u;
            global_col_ind.push_back((nidType)((state >> 12) % numNodes));
        }
        global_row_ptr.push_back((nidType)global_col_ind.size());
    }
    int devices = 0;
    CK(cudaGetDeviceCount(&devices));
    if (devices < 1) { printf("no CUDA device\n"); return 1; }
    if (devices >= 2) { MGG_COMPAT_CHECK(mggb_enable_peer_access(0, 1)); MGG_COMPAT_CHECK(mggb_enable_peer_access(1, 0)); }

    const nidType nodesPerPE = (numNodes + num_GPUs - 1) / num_GPUs;
    struct PerPE { nidType lb, ub; float *d_input, *dsp_out, *gin_out; nidType *rp_l, *ci_l, *rp_r, *ci_r; dense_param_beg* dp1; dense_param_hidden* dp2; softmax_param* smx; };
    std::vector<PerPE> pes(num_GPUs);
    for (int mype_node = 0; mype_node < num_GPUs; mype_node++) {
        PerPE& P = pes[mype_node];
        CK(cudaSetDevice(mype_node % devices));
        mgg_set_pe(mype_node, num_GPUs);
        P.lb = nodesPerPE * mype_node;
        P.ub = (P.lb + nodesPerPE) < numNodes ? (P.lb + nodesPerPE) : numNodes;
        auto split_output = split_CSR<nidType>(global_row_ptr, global_col_ind, P.lb, P.ub);
        auto up = [&](nidType** d, std::vector<nidType>& h) {
            if (h.empty()) h.push_back(0);
            if (cudaMalloc((void**)d, h.size() * sizeof(nidType)) != cudaSuccess) exit(1);
            cudaMemcpy(*d, h.data(), h.size() * sizeof(nidType), cudaMemcpyHostToDevice);
        };
        up(&P.rp_l, split_output[0]); up(&P.rp_r, split_output[1]); up(&P.ci_l, split_output[2]); up(&P.ci_r, split_output[3]);
        std::vector<float> ones((size_t)nodesPerPE * dim, 1.0f);
        CK(cudaMalloc((void**)&P.d_input, ones.size() * sizeof(float)));
        CK(cudaMemcpy(P.d_input, ones.data(), ones.size() * sizeof(float), cudaMemcpyHostToDevice));
        CK(cudaMalloc((void**)&P.dsp_out, (size_t)nodesPerPE * hiddenSize * sizeof(float)));
        CK(cudaMemset(P.dsp_out, 0, (size_t)nodesPerPE * hiddenSize * sizeof(float)));
        CK(cudaMalloc((void**)&P.gin_out, (size_t)nodesPerPE * hiddenSize * sizeof(float)));
        P.dp1 = new dense_param_beg("d-1", P.d_input, nodesPerPE, dim, hiddenSize);      // owns the symmetric d_out
        P.dp2 = new dense_param_hidden("d-2", P.dsp_out, nodesPerPE, hiddenSize, 4);
        P.smx = new softmax_param("smx", P.dp2->d_out, nodesPerPE, 4);
    }
    // stage 1 on every PE, then (all of it synchronised by the shim's launchers) the aggregations
    for (int pe = 0; pe < num_GPUs; pe++) { CK(cudaSetDevice(pe % devices)); dense_beg_forward(pes[pe].dp1); CK(cudaDeviceSynchronize()); }
    for (int mype_node = 0; mype_node < num_GPUs; mype_node++) {
        PerPE& P = pes[mype_node];
        CK(cudaSetDevice(mype_node % devices));
        mgg_SAG_np_div(P.dsp_out, P.dp1->d_out, P.rp_l, P.ci_l, P.rp_r, P.ci_r, P.lb, P.ub, hiddenSize, nodesPerPE, mype_node,
                       partSize, warpPerBlock, interleaved_dist);
        mgg_GIN_np_div(P.gin_out, P.dp1->d_out, P.rp_l, P.ci_l, P.rp_r, P.ci_r, P.lb, P.ub, hiddenSize, nodesPerPE, mype_node,
                       partSize, warpPerBlock, interleaved_dist, 0.5f);
        dense_hidden_forward(P.dp2);
        softmax_forward(P.smx);
    }
    long long bad = 0, remote_edges = 0;
    for (int pe = 0; pe < num_GPUs; pe++) {
        PerPE& P = pes[pe];
        CK(cudaSetDevice(pe % devices));
        const int rows = P.ub - P.lb;
        std::vector<float> sag((size_t)rows * hiddenSize), gin(sag.size()), sm((size_t)rows * 4);
        CK(cudaMemcpy(sag.data(), P.dsp_out, sag.size() * sizeof(float), cudaMemcpyDeviceToHost));
        CK(cudaMemcpy(gin.data(), P.gin_out, gin.size() * sizeof(float), cudaMemcpyDeviceToHost));
        CK(cudaMemcpy(sm.data(), P.smx->d_out, sm.size() * sizeof(float), cudaMemcpyDeviceToHost));
        for (int r = 0; r < rows; r++) {
            const int deg = global_row_ptr[P.lb + r + 1] - global_row_ptr[P.lb + r];
            for (int e = global_row_ptr[P.lb + r]; e < global_row_ptr[P.lb + r + 1]; e++)
                remote_edges += (global_col_ind[e] < P.lb || global_col_ind[e] >= P.ub);
            for (int c = 0; c < hiddenSize; c++) {
                bad += sag[(size_t)r * hiddenSize + c] != (float)(deg * dim);                  // exact, as the reference compares
                bad += gin[(size_t)r * hiddenSize + c] != (float)(deg * dim) + 1.5f * dim;
            }
            for (int c = 0; c < 4; c++) bad += std::fabs(sm[(size_t)r * 4 + c] - 0.25f) > 1e-6f;   // equal logits
        }
    }
    printf("PEs %d on %d device(s), remote edges %lld, mismatches %lld\n", num_GPUs, devices, remote_edges, bad);
    if (bad != 0 || remote_edges == 0) { printf("compat device check: FAILED\n"); return 1; }
    printf("compat device check: ok\n");
    return 0;
}
