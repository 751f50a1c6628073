/* mggb200.h - C ABI of the B200-native MGG hot path (libmggb200.so).
 *
 * Every entry point replaces one piece of the reference's operator surface; the comment above each
 * declaration names the reference interface it stands in for (paths relative to the reference
 * project's root).  Conventions:
 *   - plain pointers and sizes only; no C++ or framework types cross this boundary;
 *   - every function returns an int status (MGGB_OK == 0); nothing exits or throws.  The reference
 *     instead prints and calls exit(-1) on a CUDA error (include/neighbor_utils.cuh:836-840) and
 *     validates nothing; mggb_last_error() returns the message of the calling thread's last failure;
 *   - the caller owns every buffer it passes and the library keeps no pointer to one after a call
 *     returns.  The library's own device memory is small and listed where it arises: the hub work
 *     lists of the aggregation (17 MiB per device and stream, allocated on first use and kept until the
 *     process exits; mggb_sag_np_div_static allocates nothing) and the barrier's status word;
 *   - device work is enqueued on the given stream (a cudaStream_t passed as void*, NULL = default
 *     stream) of the CURRENT device and is NOT synchronised (the reference synchronises the device
 *     after every launch, include/neighbor_utils.cuh:835);
 *   - node ids are int32 (the reference's nidType, include/neighbor_utils.cuh:15); element offsets
 *     into embedding buffers are computed in 64 bits.
 */
#ifndef MGGB200_H
#define MGGB200_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    MGGB_OK = 0,
    MGGB_ERR_INVALID_ARG = 1, /* bad size, NULL pointer, unsupported knob value */
    MGGB_ERR_CUDA = 2,        /* a CUDA runtime call or launch failed */
    MGGB_ERR_UNSUPPORTED = 3, /* valid request that this build cannot serve */
    MGGB_ERR_PEER = 4,        /* peer access / IPC mapping unavailable between two devices */
    MGGB_ERR_IO = 5           /* file missing, short or inconsistent */
};

/* Flags of the aggregation entry points. */
enum {
    MGGB_AGG_ACCUMULATE = 1, /* out += sum (what the reference does, include/neighbor_utils.cuh:1456-1458);
                                without it out = sum, which needs no zero-fill between passes */
    MGGB_AGG_NO_HUB_SPLIT = 2, /* keep every node on its own warp_per_block-warp block, as the reference does.
                                 By default a node with more than max(16384, 64*ps*dist*wpb) neighbors is passed,
                                 through a work list in library-owned device memory (allocated once per device
                                 and stream, on first use), to a second kernel that gives it a 16-warp block; a node
                                 with more than 16384 neighbors is cut there into up to 64 segments of at least 4096
                                 neighbors, each summed by a block of its own, and the block that finishes last adds
                                 the segments' partial rows in segment order (no atomics on the data: same bits on
                                 every call) */
    MGGB_AGG_STAGE_ROWS = 8, /* bring neighbor rows into shared memory with bulk copies (one cp.async.bulk per row into a
                                per-warp ring, completion on an mbarrier) and add them up from there, instead of
                                loading them into registers: the rows pulled from peers' buffers when there are any
                                (their copies are issued before the local list is walked), every row otherwise.
                                dim must be 4, 8, ..., 128 (a power of two); ignored otherwise.  Measured on B200 it
                                does not pay: remote 64-byte rows arrive at the same 530 GB/s either way (the link's
                                rate for reads of that size), and local rows come 3.7x slower than through the
                                load/store unit, because an SM's copy engine keeps only about a hundred row copies
                                in flight.  Kept as an option for other row widths and machines */
    MGGB_AGG_NO_REMOTE = 64,  /* the remote lists are not read: every neighbor of every row is in its LOCAL list (global ids)
                                 and peer_input[pe] - lb * dim addresses row 0 of one matrix that holds every PE's rows
                                 (a local replica: peer_input[p] = base + p * node_per_pe * dim).  This is how the
                                 aggregation is called in push mode with merged lists; it then runs the single-PE kernel,
                                 12 % faster per edge than the kernel that also walks (empty) remote lists */
    MGGB_AGG_GIN_COMBINE = 32, /* mggb_sag_np_part only: out = (1+eps) * x_self + sum, as mggb_gin_np_div computes */
    MGGB_AGG_GROUP_PER_NODE = 4 /* dim 16 only (ignored otherwise): a node is aggregated by one group of 4 lanes,
                                 8 nodes per warp, instead of by warp_per_block warps; part_size and
                                 interleaved_dist then do not apply, and nodes above 1024 neighbors take the
                                 hub path.  For graphs whose nodes have a few dozen neighbors, where the
                                 per-node fixed cost of a whole warp dominates.  Same sums up to fp32 order */
};

/* Flags of mggb_dense_forward. */
enum {
    MGGB_DENSE_RELU = 1,      /* clamp the result at 0 (the reference's timed path has no activation) */
    MGGB_DENSE_TF32 = 2,      /* single-pass TF32 tensor-core product (about 1e-3 relative) */
    MGGB_DENSE_SIMT = 4,      /* no tensor cores: the fp32 CUDA-core kernels only */
    MGGB_DENSE_TENSOR = 8     /* the tensor-core kernel also where the default is a CUDA-core kernel that streams x row by
                                 row: outputs of at most 16 columns from rows whose stride is not a multiple of 16 bytes
                                 (602 floats), which TMA cannot load and a slab-wise walk reads at a third of HBM's rate */
};

#define MGGB_MAX_PES 16

/* Library version (major*10000 + minor*100 + patch). */
int mggb_version(void);
/* Message of the calling thread's most recent failing call ("" if none). */
const char* mggb_last_error(void);

/* ---- node-range shard ------------------------------------------------------------------------
 * Replaces the inline arithmetic of src/mgg_np_div_mem.cu:85-88:
 * nodes_per_pe = ceil(N/G), lb = pe*nodes_per_pe, ub = min(lb+nodes_per_pe, N). */
int mggb_shard_range(int64_t num_nodes, int num_pes, int pe,
                     int64_t* nodes_per_pe, int64_t* lb, int64_t* ub);

/* ---- partitioner (host, parallel) ---------------------------------------------------------------
 * Replaces split_CSR<T> (include/neighbor_utils.cuh:381-405).  For rows [lb,ub) of the global CSR,
 * each neighbor list is split, order preserved, into ids inside [lb,ub) (local) and the rest
 * (remote); ids stay global; both pointer arrays start at 0 and have ub-lb+1 entries.
 * Two calls: _count returns the two column counts, _fill writes into caller buffers of those sizes.
 * The _i64 forms take 64-bit global row pointers (graphs whose edge count exceeds 2^31); the
 * shard-local pointer arrays stay int32 and _count fails with MGGB_ERR_UNSUPPORTED if a shard's
 * half would not fit. */
int mggb_split_csr_count(const int32_t* row_ptr, const int32_t* col_idx, int32_t lb, int32_t ub,
                         int64_t* n_local, int64_t* n_remote);
int mggb_split_csr_fill(const int32_t* row_ptr, const int32_t* col_idx, int32_t lb, int32_t ub,
                        int32_t* local_ptr, int32_t* remote_ptr,
                        int32_t* local_col, int32_t* remote_col);
int mggb_split_csr_count_i64(const int64_t* row_ptr, const int32_t* col_idx, int32_t lb, int32_t ub,
                             int64_t* n_local, int64_t* n_remote);
int mggb_split_csr_fill_i64(const int64_t* row_ptr, const int32_t* col_idx, int32_t lb, int32_t ub,
                            int32_t* local_ptr, int32_t* remote_ptr,
                            int32_t* local_col, int32_t* remote_col);

/* Replaces build_part<T> (include/neighbor_utils.cuh:411-460): explicit neighbor partitions of at
 * most part_size edges.  part_ptr has P+1 entries, part2node P, node2part num_nodes+2 (the
 * reference appends the total twice, :420-429).  With exact_sentinel == 0 the closing entry
 * part_ptr[P] reproduces the reference bit for bit, including its corner case (:453-454): when the
 * last node has no edges the sentinel is left 0.  exact_sentinel != 0 always writes indptr[num_nodes].
 * The reference also prints one line per call (:457-458); this function prints nothing. */
int mggb_build_part_count(const int32_t* indptr, int32_t num_nodes, int32_t part_size,
                          int64_t* num_parts);
int mggb_build_part_fill(const int32_t* indptr, int32_t num_nodes, int32_t part_size,
                         int exact_sentinel,
                         int32_t* part_ptr, int32_t* part2node, int32_t* node2part);

/* ---- symmetric (peer-readable) buffers ----------------------------------------------------------
 * Replace nvshmem_malloc (src/mgg_np_div_mem.cu:139; include/layer_new.cuh:314) and the address
 * translation hidden inside nvshmemx_float_get_warp (include/neighbor_utils.cuh:1445).  A symmetric
 * buffer is an ordinary device allocation of the same size on every PE; what makes it symmetric is
 * that every PE holds a table of all PEs' base pointers and hands it to the aggregation call.
 *   one process, several devices: mggb_enable_peer_access(a, b) once per ordered pair, then use
 *       the owners' pointers directly;
 *   one process per device: the owner exports a 64-byte handle, the other processes import it
 *       (CUDA IPC) and get a pointer valid in their own address space. */
int mggb_sym_alloc(size_t bytes, void** dev_ptr);            /* on the current device; zero-filled */
int mggb_sym_free(void* dev_ptr);
int mggb_sym_export(void* dev_ptr, unsigned char handle_out[64]);
int mggb_sym_import(const unsigned char handle[64], void** peer_ptr); /* maps a peer's buffer */
int mggb_sym_close(void* peer_ptr);                          /* unmaps an imported buffer */
int mggb_enable_peer_access(int device, int peer_device);    /* MGGB_ERR_PEER if impossible */

/* ---- barrier between PEs ---------------------------------------------------------------------------
 * The reference's layers are not separated by anything (src/mgg_np_div_mem.cu:213-226); a pass that
 * publishes in one stage and gathers in the next needs every PE to have finished the first.  Each
 * PE owns MGGB_MAX_PES int32 epoch slots in a zero-filled symmetric buffer (mggb_sym_alloc, exported
 * to / imported by its peers); peer_slots[p] is PE p's slot array as addressable from this device.
 * The call enqueues one small kernel that stores `epoch` into slot [pe] of every PE's array and then
 * waits until slot [p] of its own array holds `epoch` or a later value for every p.  Call it with
 * epoch = 1, 2, 3, ... in the same order on every PE; each PE on its own GPU (kernels that wait on
 * one another must not share a device).  The wait gives up after timeout_ns (at most 10 s) of wall
 * clock: the kernel then returns, the stream carries on, and mggb_flag_barrier_status reports
 * 1 + the first PE that never arrived (0 = no wait has expired since the last reset; the call
 * synchronises the device).  Nothing here can hang a GPU. */
int mggb_flag_barrier(int* const* peer_slots, int num_pes, int pe, int epoch, int64_t timeout_ns, void* stream);
/* The same barrier with the epoch kept on the device: epoch_counter points to one int32 in THIS PE's
 * device memory (zero before the first barrier, touched by nothing else); each launch uses its value + 1
 * as the epoch and stores that back.  This is the form to record in a CUDA graph, where a replayed
 * launch repeats its arguments: every replay still gets the next epoch.  Every PE must run the same
 * number of barriers, and a PE must not mix the two forms on one slot array. */
int mggb_flag_barrier_counted(int* const* peer_slots, int num_pes, int pe, int* epoch_counter, int64_t timeout_ns,
                              void* stream);
int mggb_flag_barrier_status(int* status, int reset);

/* ---- neighbor aggregation ----------------------------------------------------------------------
 * Replaces mgg_SAG_np_div (launcher include/neighbor_utils.cuh:787-841, kernel :1351-1460).
 *   output      [ub-lb, dim] on this device (may itself be a symmetric buffer)
 *   peer_input  HOST array of num_pes device pointers: PE p's symmetric embedding buffer
 *               [node_per_pe, dim] as addressable from this device; peer_input[pe] is this PE's own
 *               (the reference passes only the local address and lets NVSHMEM translate it)
 *   row_ptr_l/col_idx_l, row_ptr_r/col_idx_r  the split CSR of this shard, on this device
 *   part_size, warp_per_block, interleaved_dist  the reference's ps / wpb / dist knobs: one thread
 *               block of warp_per_block warps per node, each warp taking interleaved_dist*part_size
 *               consecutive neighbors per turn, local list first, then remote (:1395-1400, :1432-1437)
 *   row_scale   NULL, or [ub-lb] factors applied to each output row before it is stored (used for
 *               symmetric normalisation; not in the reference)
 *   flags       MGGB_AGG_*
 *   publish_out HOST array of num_publish device pointers (NULL / 0 for none): every output row is
 *               ALSO stored at publish_out[k] + row*dim for each k, whichever device that memory is
 *               on.  This is how a layer's result is pushed into the peers' replicas of the embedding
 *               matrix from the kernel's epilogue, with no separate all-gather pass (the reference
 *               has no counterpart: its peers pull rows one neighbor at a time).  Peers may read
 *               them in kernels launched after this kernel has finished (i.e. after a barrier that
 *               follows it in stream order).
 * Results do not depend on ps/wpb/dist except through fp32 summation order; for fixed knobs they
 * are bit-reproducible (one writer per output row, no atomics). */
int mggb_sag_np_div(float* output, const float* const* peer_input, int num_pes,
                    const int32_t* row_ptr_l, const int32_t* col_idx_l,
                    const int32_t* row_ptr_r, const int32_t* col_idx_r,
                    int32_t lb, int32_t ub, int dim, int32_t node_per_pe, int pe,
                    int part_size, int warp_per_block, int interleaved_dist,
                    const float* row_scale, int flags,
                    float* const* publish_out, int num_publish, void* stream);

/* Replaces mgg_GIN_np_div (launcher include/neighbor_utils.cuh:902-958, kernel :1554-1667):
 * output[b,:] = (1+eps) * x_self[b,:] + sum, where x_self is this PE's own symmetric buffer
 * (:1660-1665).  The output row is written once, so output must not alias peer_input[pe]. */
int mggb_gin_np_div(float* output, const float* const* peer_input, int num_pes,
                    const int32_t* row_ptr_l, const int32_t* col_idx_l,
                    const int32_t* row_ptr_r, const int32_t* col_idx_r,
                    int32_t lb, int32_t ub, int dim, int32_t node_per_pe, int pe,
                    int part_size, int warp_per_block, int interleaved_dist,
                    float eps, int flags, void* stream);

/* The two aggregations with a caller-chosen block schedule.  row_order (device, int32[ub-lb], a
 * permutation of 0..ub-lb-1, or NULL for the natural order) names the row each thread block takes,
 * in launch order.  The reference launches block b for node b (include/neighbor_utils.cuh:808-818),
 * so a high-degree node late in the shard sets the kernel's tail; with the longest rows first
 * (mggb_degree_order) the tail disappears.  Results are identical: only the order in which rows are
 * started changes, never which warp sums which edge. */
int mggb_sag_np_div_ordered(float* output, const float* const* peer_input, int num_pes,
                            const int32_t* row_ptr_l, const int32_t* col_idx_l,
                            const int32_t* row_ptr_r, const int32_t* col_idx_r,
                            int32_t lb, int32_t ub, int dim, int32_t node_per_pe, int pe,
                            int part_size, int warp_per_block, int interleaved_dist,
                            const float* row_scale, int flags,
                            float* const* publish_out, int num_publish,
                            const int32_t* row_order, void* stream);
int mggb_gin_np_div_ordered(float* output, const float* const* peer_input, int num_pes,
                            const int32_t* row_ptr_l, const int32_t* col_idx_l,
                            const int32_t* row_ptr_r, const int32_t* col_idx_r,
                            int32_t lb, int32_t ub, int dim, int32_t node_per_pe, int pe,
                            int part_size, int warp_per_block, int interleaved_dist,
                            float eps, int flags, const int32_t* row_order, void* stream);
/* The same two operators over a LIST of rows: row_list holds row_count distinct shard-relative row ids
 * (0 .. ub-lb-1); only those rows of `output` are written, block k taking row_list[k].  A caller that
 * cuts a shard into row blocks can hand each finished block to the next kernel (the dense update and
 * its push to the peers) while the aggregation of the following block is still running.  No
 * counterpart in the reference, which always launches the whole shard. */
int mggb_sag_np_div_rows(float* output, const float* const* peer_input, int num_pes,
                         const int32_t* row_ptr_l, const int32_t* col_idx_l,
                         const int32_t* row_ptr_r, const int32_t* col_idx_r,
                         int32_t lb, int32_t ub, int dim, int32_t node_per_pe, int pe,
                         int part_size, int warp_per_block, int interleaved_dist,
                         const float* row_scale, int flags,
                         float* const* publish_out, int num_publish,
                         const int32_t* row_list, int64_t row_count, void* stream);
int mggb_gin_np_div_rows(float* output, const float* const* peer_input, int num_pes,
                         const int32_t* row_ptr_l, const int32_t* col_idx_l,
                         const int32_t* row_ptr_r, const int32_t* col_idx_r,
                         int32_t lb, int32_t ub, int dim, int32_t node_per_pe, int pe,
                         int part_size, int warp_per_block, int interleaved_dist,
                         float eps, int flags, const int32_t* row_list, int64_t row_count, void* stream);
/* Copies in[0, count) floats to every publish_out[k][0, count) with consecutive threads on consecutive
 * addresses.  For rows that a kernel wrote in a scattered order (an aggregation walking its rows by
 * degree): pushing them to the peers' replicas afterwards, as one contiguous run, moves the same bytes
 * over NVLink in full-width writes instead of one row-sized write per row.  No counterpart in the
 * reference (its PEs pull rows; nothing is pushed). */
int mggb_publish_rows(const float* in, int64_t count, float* const* publish_out, int num_publish, void* stream);
/* Host helper: order[k] = the shard row with the k-th largest neighbor count (local + remote; ties
 * in row order).  row_ptr_r may be NULL.  No counterpart in the reference. */
int mggb_degree_order(const int32_t* row_ptr_l, const int32_t* row_ptr_r, int32_t num_rows, int32_t* order);

/* The aggregation over EXPLICIT neighbor partitions.  Replaces SAG_host_fused_interleaved /
 * SAG_cuda_kernel_fused_interleaved (include/neighbor_utils.cuh:593-676, :2598-2760; driver
 * src/test_neighbor_part.cu:93-211) and takes what mggb_build_part_* returns for each half of the split
 * CSR: part_ptr (first edge of each partition), part2node (its row), node2part (first partition of each
 * row, ub-lb+2 entries).  One warp serves interleaved_dist consecutive partitions of the local half and
 * the same range of the remote half (the reference's map, :2636-2640), warp_per_block warps per block, so
 * the grid grows with the number of partitions and a row with 10^5 neighbors is spread over thousands of
 * warps.  Each partition's partial row goes to `scratch` ([num_parts_l + num_parts_r] x dim floats, device
 * memory the CALLER provides: mggb_sag_np_part_scratch_bytes gives the size; contents need no
 * initialisation and are garbage afterwards); a second kernel adds each row's partial rows in partition
 * order and stores the output row once.  The reference instead adds every partial row into the output
 * with a spinning float atomic (:2683-2686) and has its remote half commented out (:2693-2759).
 * A partition ends at min(part_ptr[p] + part_size, end of its row); part_ptr[p+1] is never read, so both
 * sentinel conventions of mggb_build_part_fill work.  row_scale, MGGB_AGG_ACCUMULATE and the result are as
 * for mggb_sag_np_div (same sums up to fp32 order; bit-reproducible for fixed knobs);
 * MGGB_AGG_GIN_COMBINE with eps gives mggb_gin_np_div's combine.  Other flags are ignored. */
int mggb_sag_np_part_scratch_bytes(int64_t num_parts_l, int64_t num_parts_r, int dim, size_t* bytes);
int mggb_sag_np_part(float* output, const float* const* peer_input, int num_pes,
                     const int32_t* row_ptr_l, const int32_t* col_idx_l, const int32_t* part_ptr_l,
                     const int32_t* part2node_l, const int32_t* node2part_l, int64_t num_parts_l,
                     const int32_t* row_ptr_r, const int32_t* col_idx_r, const int32_t* part_ptr_r,
                     const int32_t* part2node_r, const int32_t* node2part_r, int64_t num_parts_r,
                     int32_t lb, int32_t ub, int dim, int32_t node_per_pe, int pe,
                     int part_size, int warp_per_block, int interleaved_dist,
                     const float* row_scale, int flags, float eps,
                     float* scratch, size_t scratch_bytes, void* stream);

/* Neighbor count above which the aggregation entry points hand a row to the wide-block kernel at
 * these knobs, dim and flags (MGGB_AGG_*); -1 when no row ever is.  A caller that knows its shard's
 * largest neighbor count can pass MGGB_AGG_NO_HUB_SPLIT when nothing exceeds the threshold and save
 * the second kernel's launch.  No counterpart in the reference. */
int mggb_hub_threshold(int part_size, int warp_per_block, int interleaved_dist, int dim, int flags,
                       int64_t* threshold);

/* mggb_sag_np_div for callers that must not trigger a device allocation.  It has no counterpart in
 * the reference.
 *
 * mggb_sag_np_div keeps its list of hub rows (see MGGB_AGG_NO_HUB_SPLIT) in device memory that it
 * allocates the first time a (device, stream) pair is used.  Some callers cannot afford that: code
 * running inside a memory pool that owns the whole device, a latency-critical loop where an implicit
 * device synchronisation inside cudaMalloc is not acceptable, or a process that is forbidden to
 * grow its footprint after start-up.  This variant computes exactly the same result with the same
 * kernels, but its work lists live in fixed arrays inside the library's device image (32 KiB + a
 * 256-byte header for the hub list, 5 KiB for 256 cut rows and 256 KiB for their segments' partial
 * rows, present on every GPU that loads the library, for the life of the process).  A shard with more
 * than 256 rows above 16384 neighbors, or more segments than 65536 / dim, leaves the rest whole on the
 * hub list: same sums, a different fp32 summation order for those rows than mggb_sag_np_div's.  It
 * calls no cudaMalloc / cudaFree and no allocating library routine.
 *
 *   shard_edges  stored edges of this shard (local + remote, what mggb_split_csr_count returned).
 *                The fixed list holds 8192 rows; since a listed row has more than
 *                max(16384, 64*part_size*interleaved_dist*warp_per_block) neighbors, shards of up to
 *                8192 times that many edges (134 M at the default knobs) can never overflow it.
 *                Larger shards are refused with MGGB_ERR_UNSUPPORTED and a message naming the limit.
 *   warp_per_block must be <= 8 (wider blocks do not use a hub list at all).
 *   Every other argument is as for mggb_sag_np_div; MGGB_AGG_NO_HUB_SPLIT and MGGB_AGG_GROUP_PER_NODE
 *   are ignored (the latter's hub threshold of 1024 neighbors would shrink the edge bound sixteenfold).
 *   Rows wider than 3200 floats keep every node on its own block, exactly as in mggb_sag_np_div.
 *
 * The first call on each device looks up the array's device address (one cudaGetSymbolAddress, done
 * with that device current, result cached); make that first call outside any stream capture.
 * All calls on a device share the one array: the list counter is reset at the start of each call
 * (stream-ordered), the list keeps the previous call's rows until overwritten, and two calls whose
 * kernels overlap on the same GPU (different streams) race on it - order them. */
int mggb_sag_np_div_static(float* output, const float* const* peer_input, int num_pes,
                           const int32_t* row_ptr_l, const int32_t* col_idx_l,
                           const int32_t* row_ptr_r, const int32_t* col_idx_r,
                           int32_t lb, int32_t ub, int64_t shard_edges, int dim, int32_t node_per_pe, int pe,
                           int part_size, int warp_per_block, int interleaved_dist,
                           const float* row_scale, int flags,
                           float* const* publish_out, int num_publish, void* stream);

/* ---- dense node update and softmax ---------------------------------------------------------------
 * Replaces dense_beg_new_forward / dense_hidden_new_forward (include/gnn_layer.cuh:42-52) on the
 * parameter structs of include/layer_new.cuh:272-393: row-major out[n, dim2] = x[n, dim1] * w[dim1, dim2],
 * alpha = 1, beta = 0, no bias.  The reference's call passes d_out as the B operand and never reads
 * d_in; this function computes the intended product from x.  row_scale (NULL or [n]) multiplies
 * output row i; publish_out / num_publish as for mggb_sag_np_div.  out and every publish_out[k] may
 * have any 4-byte alignment (16-byte aligned buffers get 128-bit stores).  Precision: fp32-equivalent
 * by default (each operand split into two TF32 terms on the tensor cores and the partial products
 * accumulated in fp32, or the fp32 CUDA-core kernel: about 1e-6 relative to an fp64 product);
 * MGGB_DENSE_TF32 selects a single TF32 pass (operands truncated to 10 mantissa bits: about 1e-3
 * relative, as cublasSgemm gives under CUBLAS_TF32_TENSOR_OP_MATH). */
int mggb_dense_forward(float* out, const float* x, const float* w,
                       int64_t n, int dim1, int dim2,
                       const float* row_scale, int flags,
                       float* const* publish_out, int num_publish, void* stream);

/* Reads (and with reset != 0 clears) the status word of the aggregation kernels that stage rows through
 * shared memory; synchronises the device.  0 = every launch so far ran to completion; 1 = a bounded wait
 * for staged rows expired in some block, whose output row is then incomplete.  The reference has no
 * counterpart (its blocking gets cannot time out). */
int mggb_agg_device_status(int* status, int reset);

/* Reads (and with reset != 0 clears) the status word of the tensor-core dense kernel on the current
 * device; synchronises the device.  0 = every launch so far ran to completion; 1..4 = a bounded wait
 * inside the kernel expired (1 input slab, 2 free slab, 3 accumulator ready, 4 accumulator free) and
 * that launch returned early with an incomplete output.  The reference has no counterpart (cuBLAS
 * reports nothing from the device). */
int mggb_dense_device_status(int* status, int reset);

/* Replaces softmax_new_forward (include/gnn_layer.cuh:36-40; descriptors include/layer_new.cuh:80-85):
 * max-subtracted softmax over the dim classes of each row; in and out may alias. */
int mggb_softmax_forward(float* out, const float* in, int64_t n, int dim, void* stream);

/* The last layer in one pass: out[n, dim2] = softmax over each row of x[n, dim1] * w[dim1, dim2].
 * Replaces the pair dense_hidden_new_forward + softmax_new_forward at the end of both models
 * (src/mgg_np_div_mem.cu:220-226, src/mgg_np_div_gin_mem.cu:220-222) without writing the logits to
 * memory and reading them back; pass a non-NULL `logits` [n, dim2] to keep them as well.  fp32 FMA
 * product as in the CUDA-core dense kernel, max-subtracted exp / sum with the exponential taken on
 * the special-function unit (relative error below 1e-5 for every term that is not flushed to 0).
 * Returns MGGB_ERR_UNSUPPORTED when dim2 > 256 or w and the staging rows need more than
 * 160 KiB of shared memory; call the two separate entry points then. */
int mggb_dense_softmax_forward(float* out, float* logits, const float* x, const float* w, int64_t n,
                               int dim1, int dim2, void* stream);

/* out[i,:] = scale[i] * in[i,:] (in and out may alias); scale[i] = 1/sqrt(row_ptr[i+1]-row_ptr[i]),
 * 0 for empty rows.  Helpers for symmetric normalisation; no counterpart in the reference, whose
 * aggregation is an unnormalised sum. */
int mggb_row_scale(float* out, const float* in, const float* scale, int64_t n, int dim, void* stream);
int mggb_inv_sqrt_degree(float* scale, const int32_t* row_ptr_l, const int32_t* row_ptr_r,
                         int64_t n, void* stream);

/* ---- binary CSR files ---------------------------------------------------------------------------
 * Replaces the loader graph<long,long,int,int,int,int> (include/graph.hpp:9-129): <name>_beg_pos.bin
 * holds N+1 int64 offsets, <name>_csr.bin E int64 neighbor ids, <name>_weight.bin E int32 weights
 * (read by the reference, never used).  _info returns the counts; _load narrows ids to int32 into
 * caller buffers (row_ptr64 N+1 entries, col_idx E entries); weights are not read. */
int mggb_graph_file_info(const char* beg_file, const char* csr_file, int64_t* num_nodes, int64_t* num_edges);
int mggb_graph_file_load(const char* beg_file, const char* csr_file, int64_t num_nodes, int64_t num_edges,
                         int64_t* row_ptr64, int32_t* col_idx);
/* A shard's rows only: _rows_info returns the position of row lb's first neighbor and the number of
 * neighbors of rows [lb, ub); _load_rows fills row_ptr64 (ub-lb+1 entries, rebased to start at 0) and
 * col_idx (that many int32 ids) by reading just those parts of the two files.  Feeds
 * mggb_split_csr_*_i64 with shard-local pointers.  The reference loads the whole graph on every rank
 * (src/mgg_np_div_mem.cu:54-56). */
int mggb_graph_file_rows_info(const char* beg_file, int64_t lb, int64_t ub, int64_t* first_edge, int64_t* num_edges);
int mggb_graph_file_load_rows(const char* beg_file, const char* csr_file, int64_t lb, int64_t ub,
                              int64_t* row_ptr64, int32_t* col_idx);
int mggb_graph_file_write(const char* beg_file, const char* csr_file, const char* weight_file,
                          const int64_t* row_ptr64, const int32_t* col_idx, int64_t num_nodes);

#ifdef __cplusplus
}
#endif
#endif /* MGGB200_H */
