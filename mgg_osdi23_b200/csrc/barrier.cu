// Barrier between the PEs of a multi-GPU pass, in peer-mapped memory (sm_100a).
//
// The reference has no synchronisation between its layers at all (src/mgg_np_div_mem.cu:213-226: a
// PE may gather from a peer's symmetric buffer while the owner's next dense product overwrites it).
// Here a stage that reads what peers published is preceded by a barrier.  A one-element NCCL
// all-reduce does the job but costs 20-30 us per barrier on 8 GPUs; this one is a single tiny kernel
// per PE:
//   every PE owns an array of MGGB_MAX_PES epoch slots in a symmetric (peer-mapped) buffer;
//   thread p of the kernel stores the barrier's epoch into slot [pe] of PE p's array (a plain peer
//   store over NVLink), then polls slot [p] of its OWN array until PE p's store of the same epoch
//   (or a later one) has landed.
// Epochs only grow, so nothing is ever reset and a fast PE that is already one barrier ahead does
// no harm.  The wait is bounded by a wall-clock limit: when it runs out the kernel records which PE
// never arrived in a status word the host can read and returns, so a missing peer can never hang the
// GPU.  The kernels of different PEs wait on one another, so each PE must run on its own GPU.
#include "common.h"

namespace {

__device__ int g_barrier_status = 0;   // 0 ok; otherwise 1 + the first PE whose epoch never arrived

struct BarrierParams {
    int* slots[MGGB_MAX_PES];   // PE p's slot array as addressable from this device
    int pe, num_pes, epoch;
    int* epoch_counter;         // NULL, or this PE's count of barriers so far: the epoch is that count + 1
    unsigned long long timeout_ns;
};

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__global__ void flag_barrier_kernel(const BarrierParams P) {
    const int p = threadIdx.x;
    // A launch recorded in a CUDA graph repeats its arguments, so there the epoch comes from device memory:
    // every lane reads the count, then lane 0 advances it (launches of one PE are ordered by their stream).
    int epoch = P.epoch;
    if (P.epoch_counter != nullptr) {
        epoch = *reinterpret_cast<volatile int*>(P.epoch_counter) + 1;
        __syncwarp();
        if (p == 0) *reinterpret_cast<volatile int*>(P.epoch_counter) = epoch;
    }
    if (p >= P.num_pes) return;
    // everything this PE wrote before the barrier (kernels earlier in the stream have completed) is
    // ordered before the announcement
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(P.slots[p] + P.pe), "r"(epoch) : "memory");
    const int* mine = P.slots[P.pe] + p;
    const unsigned long long t0 = global_ns();
    for (unsigned i = 0;; i++) {
        int seen;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
        if ((int)((unsigned)seen - (unsigned)epoch) >= 0) break;   // epochs may wrap: compare by difference
        if ((i & 63) == 63 && global_ns() - t0 > P.timeout_ns) {
            atomicCAS(&g_barrier_status, 0, 1 + p);
            break;
        }
        __nanosleep(20);
    }
}

}  // namespace

extern "C" {

static int flag_barrier(int* const* peer_slots, int num_pes, int pe, int epoch, int* epoch_counter, int64_t timeout_ns, void* stream) {
    MGGB_REQUIRE(peer_slots != nullptr, "flag_barrier: NULL slot table");
    MGGB_REQUIRE(num_pes >= 1 && num_pes <= MGGB_MAX_PES, "flag_barrier: num_pes must be in [1,%d] (got %d)", MGGB_MAX_PES, num_pes);
    MGGB_REQUIRE(pe >= 0 && pe < num_pes, "flag_barrier: pe %d outside [0,%d)", pe, num_pes);
    MGGB_REQUIRE(timeout_ns > 0 && timeout_ns <= 10000000000LL, "flag_barrier: timeout must be in (0, 10 s] (got %lld ns)", (long long)timeout_ns);
    BarrierParams P{};
    for (int p = 0; p < num_pes; p++) {
        MGGB_REQUIRE(peer_slots[p] != nullptr && ((uintptr_t)peer_slots[p] % 4) == 0, "flag_barrier: peer_slots[%d] is NULL or misaligned", p);
        P.slots[p] = peer_slots[p];
    }
    P.pe = pe; P.num_pes = num_pes; P.epoch = epoch; P.epoch_counter = epoch_counter; P.timeout_ns = (unsigned long long)timeout_ns;
    flag_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(P);
    MGGB_CUDA(cudaGetLastError());
    return MGGB_OK;
}

int mggb_flag_barrier(int* const* peer_slots, int num_pes, int pe, int epoch, int64_t timeout_ns, void* stream) {
    return flag_barrier(peer_slots, num_pes, pe, epoch, nullptr, timeout_ns, stream);
}

int mggb_flag_barrier_counted(int* const* peer_slots, int num_pes, int pe, int* epoch_counter, int64_t timeout_ns, void* stream) {
    MGGB_REQUIRE(epoch_counter != nullptr && ((uintptr_t)epoch_counter % 4) == 0, "flag_barrier_counted: epoch_counter is NULL or misaligned");
    return flag_barrier(peer_slots, num_pes, pe, 0, epoch_counter, timeout_ns, stream);
}

int mggb_flag_barrier_status(int* status, int reset) {
    MGGB_REQUIRE(status, "flag_barrier_status: NULL output");
    MGGB_CUDA(cudaMemcpyFromSymbol(status, g_barrier_status, sizeof(int)));
    if (reset) {
        const int zero = 0;
        MGGB_CUDA(cudaMemcpyToSymbol(g_barrier_status, &zero, sizeof(int)));
    }
    return MGGB_OK;
}

}  // extern "C"
