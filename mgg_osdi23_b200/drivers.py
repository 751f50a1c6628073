"""Forward-pass orchestration: the host side of the reference's ``main()`` functions.

* :class:`GCN2Forward`   - ``src/mgg_np_div_mem.cu:211-227``  (2-layer GCN, the headline path)
* :class:`GIN5Forward`   - ``src/mgg_np_div_gin_mem.cu:193-223`` (5-layer GIN)
* :class:`SingleAggregation` - ``src/mgg_np_div_kernel.cu:183-188`` (one aggregation; the ps/wpb/dist sweeps)

One object serves one PE (GPU).  A forward pass is a list of *stages*; peers must not start stage
s+1 before every PE finished stage s, because stage s+1 reads what the peers published in stage s.
:func:`run_stages` runs the stages with a barrier between them.  (The reference has no barrier
between its layers, ``src/mgg_np_div_mem.cu:213-226``: a PE can read a peer's buffer while the owner
overwrites it.)  With one process per GPU the barrier is a one-element NCCL all-reduce enqueued on
the compute stream, so the host never blocks; several PEs emulated in one process on one stream
need none.

Differences from the reference's drivers that are deliberate:
* the dense step computes ``X*W`` from its input (the reference multiplies its output buffer in place);
* both GCN aggregations run at the hidden width, as in the reference (``:214-215, :221-222``), which is
  legitimate because layer 2 is evaluated as ``(A*H)*W2``;
* publishing alternates between symmetric buffers so that no PE overwrites a buffer a slower peer may
  still be reading, within a pass AND from one pass to the next: the buffer a pass writes first is
  never the one its last stage reads (the 5-layer GIN needs a third buffer for that; a model that
  cannot arrange it starts every pass with a barrier, ``leading_barrier``).

How peers see a layer's output is chosen by what is passed as ``sym_a`` / ``sym_b``:
* a :class:`symmem.SymmetricBuffer` (or :class:`LocalSym`): each PE keeps only its own rows and the
  aggregation kernel PULLS every remote neighbor's row from the owner's memory (the reference's scheme);
* a :class:`symmem.ReplicaBuffer` (or :class:`LocalReplica`): the producing kernel's epilogue PUSHES
  each output row into every peer's copy of the matrix, and the aggregation then reads local memory
  only.  One pushed row per node and peer instead of one pulled row per remote edge.  A dense layer
  pushes from its epilogue (contiguous runs of rows); an aggregation does so only for small outputs
  and otherwise writes locally and pushes the finished rows with ``api.publish_rows``; a pass can be cut
  into row blocks whose pushes overlap the next block's gather (``overlap_blocks``).
"""
from __future__ import annotations

import ctypes as C
from contextlib import contextmanager
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import numpy as np
import torch

from . import api, _lib
from .symmem import SymmetricBuffer


@dataclass
class Knobs:
    """The reference's command-line tuning knobs (``src/mgg_np_div_mem.cu:44-46``)."""
    partSize: int = 16
    warpPerBlock: int = 4
    interleaved_dist: int = 1
    flags: int = 0      # extra MGGB_AGG_* flags (e.g. _lib.AGG_GROUP_PER_NODE for graphs with short neighbor lists)


class Shard:
    """What one PE holds of the graph: its node range and the split CSR on the device."""

    def __init__(self, row_ptr, col_idx, pe: int, num_pes: int, device=None, num_nodes: Optional[int] = None,
                 order_rows: Optional[bool] = None, shard_local: bool = False):
        """row_ptr / col_idx: the whole graph's CSR (what every rank of the reference loads), or, with
        ``shard_local=True`` and ``num_nodes`` given, only this PE's rows (pointers starting at 0 for
        row lb): for graphs too large to replicate per rank."""
        row_ptr = np.ascontiguousarray(row_ptr)
        if shard_local and num_nodes is None:
            raise ValueError("shard_local needs num_nodes")
        n = len(row_ptr) - 1 if num_nodes is None else num_nodes
        self.pe, self.num_pes, self.num_nodes = pe, num_pes, n
        self.node_per_pe, self.lb, self.ub = api.shard_range(n, num_pes, pe)
        self.rows = self.ub - self.lb
        first_row = self.lb if shard_local else 0
        lp, rp, lc, rc = api.split_CSR(row_ptr, col_idx, self.lb, self.ub, first_row=first_row)
        # this shard's rows of the UNSPLIT lists (views, nothing copied): what a PE that holds a full
        # replica of the embedding matrix gathers from, see merged_lists()
        e0, e1 = int(row_ptr[self.lb - first_row]), int(row_ptr[self.ub - first_row])
        self._host_rows = (row_ptr[self.lb - first_row: self.ub - first_row + 1], np.asarray(col_idx)[e0:e1], e0)
        self._merged = None
        self.e_local, self.e_remote = int(lc.size), int(rc.size)
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.device = dev
        self.rp_l = torch.from_numpy(lp).to(dev)
        self.rp_r = torch.from_numpy(rp).to(dev)
        # never hand the kernel a NULL column array, even for an empty half
        self.ci_l = torch.from_numpy(lc if lc.size else np.zeros(1, np.int32)).to(dev)
        self.ci_r = torch.from_numpy(rc if rc.size else np.zeros(1, np.int32)).to(dev)
        # block schedule: rows by decreasing degree.  No high-degree row is left for the kernel's tail
        # (3-6 % on 2-8 PEs with a block per node), and the nodes that share a warp in the
        # group-per-node kernel have lists of the same length (2.3x on the skewed R-MAT shape,
        # where a warp otherwise runs as long as the longest of its eight lists).
        if order_rows is None:
            order_rows = True
        # longest neighbor list of the shard: when no row reaches the hub threshold the aggregation is
        # told so (NO_HUB_SPLIT) and the second kernel, which would find an empty list, is not launched
        deg = (lp[1:] - lp[:-1]) + (rp[1:] - rp[:-1])
        self.max_degree = int(deg.max()) if self.rows else 0
        self._order_host = api.degree_order(lp, rp) if (order_rows and self.rows) else None
        self.row_order = torch.from_numpy(self._order_host).to(dev) if self._order_host is not None else None
        self._blocks = {}
        self._parts = {}
        self._flag_cache = {}
        self.use_merged_lists = True   # False: a replica is gathered from through the two split lists as well
        self._dinv = None
        self.event_sink = None   # when a list: (start, end) CUDA events of every aggregation launch are appended
        self._in_span = False

    def row_blocks(self, count: int):
        """The shard cut into ``count`` contiguous row ranges: a list of (r0, r1, rows) with ``rows`` the
        int32 device list of the range's rows in the shard's block schedule (by decreasing degree, or in
        id order).  Aggregating the ranges one after the other gives the same output as one call."""
        if count not in self._blocks:
            step = (self.rows + count - 1) // count
            step = (step + 127) // 128 * 128        # whole tiles of the dense kernel
            out = []
            for r0 in range(0, self.rows, step):
                r1 = min(self.rows, r0 + step)
                if self._order_host is not None:
                    o = self._order_host
                    ids = o[(o >= r0) & (o < r1)]
                else:
                    ids = np.arange(r0, r1, dtype=np.int32)
                out.append((r0, r1, torch.from_numpy(np.ascontiguousarray(ids, dtype=np.int32)).to(self.device)))
            self._blocks[count] = out
        return self._blocks[count]

    @contextmanager
    def timed_span(self):
        """One (start, end) event pair around several aggregation launches on the current stream."""
        if self.event_sink is None or self._in_span:
            yield
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        self._in_span = True
        try:
            yield
        finally:
            self._in_span = False
            b.record()
            self.event_sink.append((a, b))

    def _timed(self, launch):
        if self.event_sink is None or self._in_span:
            return launch()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        launch()
        b.record()
        self.event_sink.append((a, b))

    @property
    def edges(self) -> int:
        return self.e_local + self.e_remote

    def inv_sqrt_degree(self) -> torch.Tensor:
        """1/sqrt(deg) of this shard's rows (deg = stored row length, local + remote)."""
        if self._dinv is None:
            self._dinv = torch.empty(max(self.rows, 1), dtype=torch.float32, device=self.device)[: self.rows]
            if self.rows:
                api.inv_sqrt_degree(self._dinv, self.rp_l, self.rp_r)
        return self._dinv

    def merged_lists(self):
        """(row_ptr, col_idx, empty row_ptr, dummy col_idx) on the device: each row's whole neighbor list,
        local and remote ids together in stored order, as the "local" half, and an empty "remote" half.
        For aggregating from a REPLICA of the embedding matrix: every id is then addressed the same way,
        so the split into two lists (two walks per node, two ragged tails) buys nothing."""
        if self._merged is None:
            rp, col, e0 = self._host_rows
            rp_m = np.ascontiguousarray(np.asarray(rp, dtype=np.int64) - e0, dtype=np.int32)
            ci_m = np.ascontiguousarray(col, dtype=np.int32)
            self._merged = (torch.from_numpy(rp_m).to(self.device),
                            torch.from_numpy(ci_m if ci_m.size else np.zeros(1, np.int32)).to(self.device),
                            torch.zeros(self.rows + 1, dtype=torch.int32, device=self.device),
                            torch.zeros(1, dtype=torch.int32, device=self.device))
        return self._merged

    def _lists_for(self, sym):
        if getattr(sym, "slot_elems", None) is not None and self.num_pes > 1 and self.use_merged_lists:
            return self.merged_lists()
        return self.rp_l, self.ci_l, self.rp_r, self.ci_r

    def partitions(self, part_size: int):
        """``build_part`` of both halves of this shard's split CSR at ``part_size``, on the device (cached):
        a dict with ``l`` and ``r`` = (part_ptr, part2node, node2part, num_parts)."""
        if part_size not in self._parts:
            out = {}
            for key, rp in (("l", self.rp_l), ("r", self.rp_r)):
                pp, p2n, n2p = api.build_part(key, rp.cpu().numpy(), self.rows, part_size)
                pad = lambda a: torch.from_numpy(a if a.size else np.zeros(1, np.int32)).to(self.device)
                out[key] = (pad(pp), pad(p2n), pad(n2p), int(p2n.size))
            self._parts[part_size] = out
        return self._parts[part_size]

    def aggregate_parts(self, out, sym, dim, knobs: Knobs, accumulate=False, row_scale_=None, gin_eps=None, scratch=None):
        """The same aggregation through the explicit-partition kernels (``api.SAG_host_fused_interleaved``):
        one warp per ``interleaved_dist`` partitions of ``partSize`` edges.  Returns the scratch tensor used."""
        parts = self.partitions(knobs.partSize)
        (pl, p2l, n2l, nl), (pr, p2r, n2r, nr) = parts["l"], parts["r"]
        box = []
        self._timed(lambda: box.append(api.SAG_host_fused_interleaved(
            out, sym, self.rp_l, self.ci_l, pl, p2l, nl, self.rp_r, self.ci_r, pr, p2r, nr if self.num_pes > 1 else 0,
            self.rows, self.lb, knobs.partSize, dim, min(dim, 32), knobs.warpPerBlock, knobs.interleaved_dist,
            local_node2Part=n2l, remote_node2Part=n2r, nodePerPE=self.node_per_pe, peid=self.pe, scratch=scratch,
            accumulate=accumulate, row_scale_=row_scale_, gin_eps=gin_eps)))
        return box[0]

    def agg_flags(self, knobs: Knobs, dim: int) -> int:
        """The knobs' flags, plus NO_HUB_SPLIT when no row of this shard exceeds the hub threshold."""
        key = (knobs.partSize, knobs.warpPerBlock, knobs.interleaved_dist, knobs.flags, dim)
        if key not in self._flag_cache:
            thr = api.hub_threshold(knobs.partSize, knobs.warpPerBlock, knobs.interleaved_dist, dim, knobs.flags)
            self._flag_cache[key] = knobs.flags | (_lib.AGG_NO_HUB_SPLIT if (thr < 0 or self.max_degree <= thr) else 0)
        return self._flag_cache[key]

    def _flags_for(self, lists, knobs: Knobs, dim: int) -> int:
        # merged lists (a replica is gathered from): nothing is left in the remote half, the single-PE kernel does
        merged = self._merged is not None and lists is self._merged
        return self.agg_flags(knobs, dim) | (_lib.AGG_NO_REMOTE if merged else 0)

    def aggregate(self, out, sym, dim, knobs: Knobs, accumulate=False, row_scale_=None, publish=None, rows=None):
        """``rows``: a row list from :meth:`row_blocks` (only those rows are computed); None = the whole shard."""
        lists = self._lists_for(sym)
        self._timed(lambda: api.mgg_SAG_np_div(
            out, sym, *lists, self.lb, self.ub, dim, self.node_per_pe, self.pe,
            knobs.partSize, knobs.warpPerBlock, knobs.interleaved_dist, accumulate=accumulate, row_scale_=row_scale_,
            publish=publish, row_order=self.row_order, rows=rows, flags=self._flags_for(lists, knobs, dim)))

    def aggregate_gin(self, out, sym, dim, knobs: Knobs, eps: float, rows=None):
        lists = self._lists_for(sym)
        self._timed(lambda: api.mgg_GIN_np_div(
            out, sym, *lists, self.lb, self.ub, dim, self.node_per_pe, self.pe,
            knobs.partSize, knobs.warpPerBlock, knobs.interleaved_dist, eps, row_order=self.row_order, rows=rows,
            flags=self._flags_for(lists, knobs, dim)))


def nccl_stream_barrier(group=None) -> Callable[[], None]:
    """Barrier for one-process-per-GPU runs: a one-element all-reduce on the current stream."""
    import torch.distributed as dist
    token = torch.zeros(1, dtype=torch.float32, device=torch.device("cuda", torch.cuda.current_device()))

    def barrier():
        dist.all_reduce(token, group=group)
    return barrier


class FlagBarrier:
    """Barrier for one-process-per-GPU runs without NCCL on the path: epoch flags in peer-mapped memory
    (``mggb_flag_barrier``).  Calling the object enqueues one small kernel on the current stream; the
    host never blocks.  The kernel's wait is bounded (``timeout_s``); ``status()`` synchronises and
    returns 0, or 1 + the PE that never arrived at some barrier since the last ``reset``."""

    def __init__(self, group, pe: int, num_pes: int, timeout_s: float = 2.0):
        self.pe, self.num_pes = pe, num_pes
        self.slots = SymmetricBuffer(_lib.MAX_PES, group, pe, num_pes)     # zero-filled 4-byte slots: epoch 0
        self.table = (C.c_void_p * num_pes)(*self.slots.peer_ptrs)
        self.timeout_ns = int(timeout_s * 1e9)
        # the epoch lives on the device (this PE's count of barriers so far), so a barrier recorded in a CUDA
        # graph gets the next epoch at every replay
        self.counter = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", torch.cuda.current_device()))

    def __call__(self):
        api.kernel_launches[0] += 1
        _lib.check(_lib.lib.mggb_flag_barrier_counted(self.table, self.num_pes, self.pe, C.c_void_p(self.counter.data_ptr()),
                                                      self.timeout_ns, C.c_void_p(torch.cuda.current_stream().cuda_stream)))

    @property
    def epoch(self) -> int:
        """Barriers this PE has run so far (synchronises)."""
        return int(self.counter.item())

    def status(self, reset: bool = False) -> int:
        st = C.c_int(0)
        _lib.check(_lib.lib.mggb_flag_barrier_status(C.byref(st), int(reset)))
        return st.value

    def close(self):
        self.slots.close()


def run_stages(models: Sequence, barrier: Optional[Callable[[], None]] = None, marks: Optional[list] = None):
    """Runs every model's stage s (all PEs held by this process), then the barrier, for each s.
    ``marks``: when a list, a CUDA event is recorded before the first stage and after every stage and
    barrier, and the events of this pass are appended as one list (for a time breakdown)."""
    n = len(models[0].stages)
    ev = None
    if marks is not None:
        ev = [torch.cuda.Event(enable_timing=True)]
        ev[0].record()
    if barrier is not None and any(getattr(m, "leading_barrier", False) for m in models):
        # stage 0 overwrites a buffer that a slower peer may still be reading in its previous pass
        barrier()
        if ev is not None:
            ev.append(torch.cuda.Event(enable_timing=True)); ev[-1].record()
    for s in range(n):
        for m in models:
            m.stages[s]()
        if ev is not None:
            ev.append(torch.cuda.Event(enable_timing=True)); ev[-1].record()
        if barrier is not None and s + 1 < n:
            barrier()
            if ev is not None:
                ev.append(torch.cuda.Event(enable_timing=True)); ev[-1].record()
    if marks is not None:
        marks.append(ev)


class _Forward:
    """Shared plumbing: symmetric buffers, sizes, the host-buffer entry point."""

    def __init__(self, shard: Shard, sym_a, sym_b, knobs: Knobs):
        self.shard, self.knobs = shard, knobs
        self.sym_a, self.sym_b = sym_a, sym_b
        self.stages: List[Callable[[], None]] = []
        self._h_out = None
        self._copy_stream = None
        self.first_dense = None     # set by models whose stage 0 is exactly one row-local dense product
        # True: the last dense layer's output (the logits) is stored as well as the probabilities, as the
        # reference's separate dense and softmax calls do; False saves that write.
        self.keep_logits = True
        # Row blocks per aggregation whose output is pushed to peers: with N > 1, block b's consumer (the
        # dense update that pushes, or the push itself) runs on a second, high-priority stream while block
        # b+1 is aggregated.  1 (the default) = one launch, no second stream: on 4 B200s with the
        # products-shaped GIN the cut gave no gain (11.7 ms per pass against 11.4 ms), because the
        # persistent dense kernel and the gather compete for the same SMs.
        self.overlap_blocks = 1
        self.overlap_min_rows = 8192      # rows per block below which cutting the shard does not pay
        self._side = None
        # True: a pass starts with a barrier, because its first stage overwrites the published buffer
        # that the previous pass's LAST stage reads (a slower peer may still be gathering from it).
        self.leading_barrier = False

    # An aggregation pushes its rows from its own epilogue only while that is a small transfer: the
    # epilogue writes one row per store, in the block schedule's (degree) order, and a peer then receives
    # row-sized writes.  Above this many bytes per pass the rows are pushed by a copy kernel instead.
    EPILOGUE_PUSH_MAX_BYTES = 16 << 20

    def _blocked(self, aggregate_rows: Callable, consume: Callable[[int, int], None]):
        """aggregate_rows(rows or None) launches the aggregation of a row list (None: the whole shard) on
        the current stream; consume(r0, r1) launches whatever reads rows [r0, r1) of its output."""
        sh = self.shard
        nblk = self.overlap_blocks
        if nblk <= 1 or sh.rows < self.overlap_min_rows * nblk:
            with sh.timed_span():
                aggregate_rows(None)
            consume(0, sh.rows)
            return
        cur = torch.cuda.current_stream()
        if self._side is None:
            self._side = torch.cuda.Stream(priority=-1)
        side = self._side
        side.wait_stream(cur)
        with sh.timed_span():
            for r0, r1, rows in sh.row_blocks(nblk):
                aggregate_rows(rows)
                done = torch.cuda.Event()
                done.record(cur)
                side.wait_event(done)
                with torch.cuda.stream(side):
                    consume(r0, r1)
        cur.wait_stream(side)

    def _sym_view(self, sym, dim):
        """Where this PE writes its rows of the published matrix (its own buffer, or its slot of a replica)."""
        return sym.own(self.shard.rows, dim)

    def forward(self, barrier=None, marks=None):
        run_stages([self], barrier, marks)
        return self.out

    def capture(self, barrier=None) -> int:
        """Records one forward pass (its kernels, memsets and barriers, in stream order) as a CUDA graph;
        :meth:`replay` then enqueues the whole pass with one launch, which is what an 8-GPU pass of a
        few hundred microseconds needs (a dozen launches from Python cost about as much as its kernels).
        Returns the number of kernels in the graph.

        The pass is run once on the capture stream first, so that everything the library allocates on first
        use for a (device, stream) pair exists before recording starts.  ``barrier`` must be recordable: a
        :class:`FlagBarrier` (its epoch is read from device memory) or None.  Every PE must capture, and
        later replay, the same number of times.  Buffers, weights and knobs are fixed at capture time."""
        if self.overlap_blocks > 1:
            raise ValueError("capture: row blocks on a second stream (overlap_blocks > 1) are not recorded")
        sink, self.shard.event_sink = self.shard.event_sink, None
        try:
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                self.forward(barrier)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            before = api.kernel_launches[0]
            # thread-local: other threads of the process (a collective library's watchdog, a clock sampler) keep working
            with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
                self.forward(barrier)
            self._graph, self._graph_kernels = graph, api.kernel_launches[0] - before
        finally:
            self.shard.event_sink = sink
        return self._graph_kernels

    def replay(self):
        """One captured pass on the current stream (see :meth:`capture`)."""
        self._graph.replay()
        api.kernel_launches[0] += self._graph_kernels
        return self.out

    def forward_host(self, x_host: torch.Tensor, barrier=None, chunks: int = 8, marks: Optional[list] = None) -> torch.Tensor:
        """The call a user with HOST data makes: uploads this PE's feature rows (pinned ``x_host``
        [rows, in_dim]), runs the forward pass and returns the class probabilities in pinned host
        memory.  Synchronises the stream before returning.

        The first layer's dense product is row-local, so the upload is cut into ``chunks`` row blocks
        on a copy stream and each block is multiplied as soon as it has arrived: the product (and the
        publication to peers) hides behind the PCIe transfer.  ``marks``: when a list, three CUDA events of
        this call (start, forward done, probabilities copied out) are appended to it as one list."""
        ev = None
        if marks is not None:
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            ev[0].record()
        first = getattr(self, "first_dense", None)
        rows = self.shard.rows
        if first is None or chunks <= 1 or rows < 4096 * chunks:
            self.d_in.copy_(x_host, non_blocking=True)
            self.forward(barrier)
        else:
            cur = torch.cuda.current_stream()
            if self._copy_stream is None:
                self._copy_stream = torch.cuda.Stream()
            if barrier is not None and self.leading_barrier:
                barrier()
            cs = self._copy_stream
            cs.wait_stream(cur)                 # the previous pass no longer reads d_in
            step = (rows + chunks - 1) // chunks
            for r0 in range(0, rows, step):
                r1 = min(rows, r0 + step)
                with torch.cuda.stream(cs):
                    self.d_in[r0:r1].copy_(x_host[r0:r1], non_blocking=True)
                    arrived = torch.cuda.Event()
                    arrived.record(cs)
                cur.wait_event(arrived)
                first._forward_rows(r0, r1)
            for s in range(1, len(self.stages)):
                if barrier is not None:
                    barrier()
                self.stages[s]()
        if self._h_out is None:
            self._h_out = torch.empty(self.out.shape, dtype=torch.float32, pin_memory=True)
        if ev is not None:
            ev[1].record()
        self._h_out.copy_(self.out, non_blocking=True)
        if ev is not None:
            ev[2].record()
            marks.append(ev)
        torch.cuda.current_stream().synchronize()
        return self._h_out


class GCN2Forward(_Forward):
    """softmax((A * (A * (X*W1))) * W2) on one PE's rows; both aggregations at the hidden width.

    norm: "none" (the reference: unnormalised sums) or "sym" (A scaled by 1/sqrt(deg_i*deg_j); the
    row factors are folded into the epilogues of the dense and aggregation kernels).
    Buffers per PE: d_in [rows, in], two symmetric [nodePerPE, hidden], d_agg [rows, hidden],
    logits/out [rows, out]."""

    def __init__(self, shard: Shard, in_dim: int, hidden: int, out_dim: int, sym_a, sym_b, knobs: Knobs,
                 w1: Optional[torch.Tensor] = None, w2: Optional[torch.Tensor] = None, norm: str = "none",
                 dense_flags: int = 0):
        super().__init__(shard, sym_a, sym_b, knobs)
        dev, rows = shard.device, max(shard.rows, 1)
        self.in_dim, self.hidden, self.out_dim = in_dim, hidden, out_dim
        self.d_in = torch.zeros(rows, in_dim, dtype=torch.float32, device=dev)[: shard.rows]
        self.d_agg = torch.zeros(rows, hidden, dtype=torch.float32, device=dev)[: shard.rows]
        self.logits = torch.zeros(rows, out_dim, dtype=torch.float32, device=dev)[: shard.rows]
        self.out = torch.zeros(rows, out_dim, dtype=torch.float32, device=dev)[: shard.rows]
        self.dp1 = api.dense_param_new_beg("d-1", self.d_in, self._sym_view(sym_a, hidden), shard.rows, in_dim, hidden)
        self.dp2 = api.dense_param_new_hidden("d-2", self.d_agg, self.logits, shard.rows, hidden, out_dim)
        self.smx = api.softmax_new_param("smx-2", self.logits, self.out, shard.rows, out_dim)
        self.dp1.flags = self.dp2.flags = dense_flags
        self.dp1.publish = sym_a.publish
        if w1 is not None:
            self.dp1.set_weight(w1)
        if w2 is not None:
            self.dp2.set_weight(w2)
        if norm not in ("none", "sym"):
            raise ValueError("norm must be 'none' or 'sym'")
        self.scale1 = self.scale2 = None
        if norm == "sym":
            dinv = shard.inv_sqrt_degree()
            self.dp1.row_scale = dinv          # H1' = dinv * (X W1)
            self.scale1 = dinv * dinv          # Z1' = dinv * (dinv * A H1')   (second factor pre-scales layer 2)
            self.scale2 = dinv                 # Z2  = dinv * A Z1'
        self.stages = [self._dense1, self._agg1, self._agg2_dense2_softmax]
        self.first_dense = self.dp1

    def _dense1(self):
        if self.shard.rows:
            api.dense_beg_new_forward(self.dp1)

    def _agg1(self):
        if not self.shard.rows:
            return
        own = self._sym_view(self.sym_b, self.hidden)
        pub = self.sym_b.publish
        if not pub or self.shard.rows * self.hidden * 4 * len(pub) <= self.EPILOGUE_PUSH_MAX_BYTES:
            self.shard.aggregate(own, self.sym_a, self.hidden, self.knobs, row_scale_=self.scale1, publish=pub)
            return
        self._blocked(
            lambda rows: self.shard.aggregate(own, self.sym_a, self.hidden, self.knobs, row_scale_=self.scale1, rows=rows),
            lambda r0, r1: api.publish_rows(own[r0:r1], pub, elem_offset=r0 * self.hidden))

    def _agg2_dense2_softmax(self):
        if self.shard.rows:
            self.shard.aggregate(self.d_agg, self.sym_b, self.hidden, self.knobs, row_scale_=self.scale2)
            api.dense_hidden_softmax_new_forward(self.dp2, self.smx, self.keep_logits)

    @property
    def kernels_per_forward(self):
        # dense, aggregate (+ its hub-row kernel), aggregate (+ hub), then dense+softmax as one kernel or two
        return 6 if api.dense_softmax_fits(self.hidden, self.out_dim) else 7
    aggregations_per_forward = 2


class GIN5Forward(_Forward):
    """dense(in->hidden), then five times [GIN aggregation, dense], the last dense hidden->out, softmax.
    Each "MLP" is one bias-free linear layer, as in the reference (``src/mgg_np_div_gin_mem.cu:195-222``)."""

    def __init__(self, shard: Shard, in_dim: int, hidden: int, out_dim: int, sym_a, sym_b, knobs: Knobs,
                 eps: float = 0.5, weights: Optional[Sequence[torch.Tensor]] = None, num_layers: int = 5,
                 dense_flags: int = 0, sym_c=None):
        super().__init__(shard, sym_a, sym_b, knobs)
        dev, rows = shard.device, max(shard.rows, 1)
        self.in_dim, self.hidden, self.out_dim, self.eps, self.num_layers = in_dim, hidden, out_dim, eps, num_layers
        self.d_in = torch.zeros(rows, in_dim, dtype=torch.float32, device=dev)[: shard.rows]
        self.d_agg = torch.zeros(rows, hidden, dtype=torch.float32, device=dev)[: shard.rows]
        self.logits = torch.zeros(rows, out_dim, dtype=torch.float32, device=dev)[: shard.rows]
        self.out = torch.zeros(rows, out_dim, dtype=torch.float32, device=dev)[: shard.rows]
        # Layer k reads what dense[k] published.  Consecutive layers must use different buffers, and so
        # must the first and the last of a pass (the next pass's first dense product may start while a
        # slower peer still gathers for the last layer): A B A B ... with the LAST one on the third
        # buffer when the count is odd.  Without a third buffer such a pass starts with a barrier.
        syms = [sym_a, sym_b][: 2 if sym_b is not None else 1]
        seq = [syms[k % len(syms)] for k in range(num_layers)]
        if seq[-1] is seq[0]:
            if sym_c is not None and num_layers > 1:
                seq[-1] = sym_c
            else:
                self.leading_barrier = True
        self.dense = [api.dense_param_new_beg("d-1", self.d_in, self._sym_view(seq[0], hidden), shard.rows, in_dim, hidden)]
        for k in range(1, num_layers):
            self.dense.append(api.dense_param_new_hidden(f"d-{k + 1}", self.d_agg, self._sym_view(seq[k], hidden),
                                                         shard.rows, hidden, hidden))
        self.dense.append(api.dense_param_new_hidden(f"d-{num_layers + 1}", self.d_agg, self.logits, shard.rows, hidden, out_dim))
        for k, dp in enumerate(self.dense):
            dp.flags = dense_flags
            if k < num_layers:
                dp.publish = seq[k].publish
        if weights is not None:
            for dp, w in zip(self.dense, weights):
                dp.set_weight(w)
        self.smx = api.softmax_new_param("smx", self.logits, self.out, shard.rows, out_dim)
        self._seq = seq
        self.stages = [self._first] + [self._layer(k) for k in range(num_layers)]
        self.first_dense = self.dense[0]

    def _first(self):
        if self.shard.rows:
            api.dense_beg_new_forward(self.dense[0])

    def _layer(self, k: int):
        def stage():
            if not self.shard.rows:
                return
            if k == self.num_layers - 1:
                self.shard.aggregate_gin(self.d_agg, self._seq[k], self.hidden, self.knobs, self.eps)
                api.dense_hidden_softmax_new_forward(self.dense[k + 1], self.smx, self.keep_logits)
            elif not self.dense[k + 1].publish:
                self.shard.aggregate_gin(self.d_agg, self._seq[k], self.hidden, self.knobs, self.eps)
                api.dense_hidden_new_forward(self.dense[k + 1])
            else:
                self._blocked(
                    lambda rows: self.shard.aggregate_gin(self.d_agg, self._seq[k], self.hidden, self.knobs,
                                                          self.eps, rows=rows),
                    lambda r0, r1: self.dense[k + 1]._forward_rows(r0, r1))
        return stage

    @property
    def kernels_per_forward(self):
        # dense x layers, aggregate + hub-row kernel per layer, then dense+softmax as one kernel or two
        fused = api.dense_softmax_fits(self.hidden, self.out_dim)
        return 3 * self.num_layers + (1 if fused else 2)

    @property
    def aggregations_per_forward(self):
        return self.num_layers


class SingleAggregation(_Forward):
    """One ``mgg_SAG_np_div`` over the shard (``src/mgg_np_div_kernel.cu:183-188``): what the
    ps / wpb / dist design-space sweeps time."""

    def __init__(self, shard: Shard, dim: int, sym_a, knobs: Knobs, norm: str = "none"):
        super().__init__(shard, sym_a, None, knobs)
        self.dim = dim
        rows = max(shard.rows, 1)
        self.d_in = self._sym_view(sym_a, dim)   # in replica mode the caller also fills the peers' slots
        self.out = torch.zeros(rows, dim, dtype=torch.float32, device=shard.device)[: shard.rows]
        self.scale = shard.inv_sqrt_degree() if norm == "sym" else None
        # push mode: the pass starts by pushing this PE's rows into the peers' replicas
        self.stages = [self._push, self._agg] if getattr(sym_a, "publish", None) else [self._agg]
        # the next pass's push lands in the replicas that slower peers are still aggregating from
        self.leading_barrier = len(self.stages) == 2

    def _push(self):
        if self.shard.rows:
            api.publish_rows(self.d_in, self.sym_a.publish)

    def _agg(self):
        if self.shard.rows:
            self.shard.aggregate(self.out, self.sym_a, self.dim, self.knobs, row_scale_=self.scale)

    @property
    def kernels_per_forward(self):
        return len(self.stages) + 1   # (the push,) the aggregation and its hub-row kernel

    aggregations_per_forward = 1


class LocalSym:
    """Symmetric buffers of several PEs emulated in ONE process: plain tensors plus the shared table."""
    publish = None

    def __init__(self, tensors: Sequence[torch.Tensor], pe: int):
        self.tensor = tensors[pe]
        self.peer_ptrs = [t.data_ptr() for t in tensors]

    def own(self, rows: int, dim: int) -> torch.Tensor:
        return self.tensor[: rows * dim].view(rows, dim)


class LocalReplica:
    """Replicated embedding matrices of several PEs emulated in ONE process (see symmem.ReplicaBuffer)."""

    def __init__(self, tensors: Sequence[torch.Tensor], pe: int, slot_elems: int):
        self.tensor, self.pe, self.slot_elems = tensors[pe], pe, slot_elems
        self.peer_ptrs = [tensors[pe].data_ptr() + p * slot_elems * 4 for p in range(len(tensors))]
        self.publish = [tensors[(pe + k) % len(tensors)].data_ptr() + pe * slot_elems * 4
                        for k in range(1, len(tensors))] or None

    def own(self, rows: int, dim: int) -> torch.Tensor:
        off = self.pe * self.slot_elems
        return self.tensor[off: off + rows * dim].view(rows, dim)


def local_replicas(num_pes: int, node_per_pe: int, dim: int, device=None) -> List[LocalReplica]:
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    slot = node_per_pe * dim
    tensors = [torch.zeros(max(num_pes * slot, 4), dtype=torch.float32, device=dev) for _ in range(num_pes)]
    return [LocalReplica(tensors, pe, slot) for pe in range(num_pes)]


def local_symmetric(num_pes: int, numel: int, device=None) -> List[LocalSym]:
    """One buffer per emulated PE, all on one device; returns the per-PE handles."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    tensors = [torch.zeros(max(numel, 4), dtype=torch.float32, device=dev) for _ in range(num_pes)]
    return [LocalSym(tensors, pe) for pe in range(num_pes)]
