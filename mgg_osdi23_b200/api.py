"""Host-side mirror of the reference's operator surface, on top of the C ABI.

Names, argument order and meaning follow the reference's header-defined functions and structs:

=============================  ==============================================================
here                           reference
=============================  ==============================================================
``split_CSR``                  ``include/neighbor_utils.cuh:381-405``
``build_part``                 ``include/neighbor_utils.cuh:411-460``
``mgg_SAG_np_div``             ``include/neighbor_utils.cuh:787-841``
``mgg_GIN_np_div``             ``include/neighbor_utils.cuh:902-958``
``dense_param_new_beg`` etc.   ``include/layer_new.cuh:59-103, 272-393``
``dense_*_new_forward`` etc.   ``include/gnn_layer.cuh:36-52``
=============================  ==============================================================

Device buffers are torch CUDA tensors (torch is used for memory and streams only); host arrays are
numpy.  Work is enqueued on torch's current stream and not synchronised.  There is no CPU path:
every compute function needs a CUDA device.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np
import torch

from . import _lib
from ._lib import lib, check

__all__ = [
    "shard_range", "split_CSR", "build_part", "mgg_SAG_np_div", "mgg_GIN_np_div", "SAG_host_fused_interleaved",
    "dense_param_new_beg", "dense_param_new_hidden", "softmax_new_param",
    "dense_beg_new_forward", "dense_hidden_new_forward", "softmax_new_forward", "dense_hidden_softmax_new_forward",
    "dense_forward", "softmax_forward", "dense_softmax_forward", "dense_softmax_fits", "publish_rows", "row_scale", "inv_sqrt_degree", "degree_order", "hub_threshold",
]


# Kernels launched through this module since import (each wrapper adds what its call launches):
# lets a benchmark report how many kernels one timed pass really issued.
kernel_launches = [0]


def _count_aggregation(dim: int, warpPerBlock: int, flags: int, rows) -> None:
    if rows is not None and rows.numel() == 0:
        return
    # the hub-row kernel follows whenever the library keeps a hub list (mggb_sag_np_div's default)
    hub = not (flags & _lib.AGG_NO_HUB_SPLIT) and warpPerBlock <= 8 and 16 * dim * 4 <= 200 * 1024
    kernel_launches[0] += 2 if hub else 1


# ---- helpers ------------------------------------------------------------------------------------

def _np_ptr(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _dev_ptr(t: torch.Tensor | None, dtype=None, name="tensor"):
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (this package has no CPU compute path)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise ValueError(f"{name} must have dtype {dtype}, got {t.dtype}")
    return C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _peer_table(input_) -> tuple:
    """Accepts a plain tensor (single PE), a sequence of tensors / raw pointers (one per PE), or an
    object with a ``peer_ptrs`` attribute (see symmem.SymmetricBuffer)."""
    if isinstance(input_, torch.Tensor):
        _dev_ptr(input_, torch.float32, "input")
        ptrs = [input_.data_ptr()]
    elif hasattr(input_, "peer_ptrs"):
        ptrs = list(input_.peer_ptrs)
    else:
        ptrs = [p.data_ptr() if isinstance(p, torch.Tensor) else int(p) for p in input_]
    return (C.c_void_p * len(ptrs))(*ptrs), len(ptrs)


def _publish_table(publish):
    """None, or a sequence of tensors / raw device addresses that also receive every output row."""
    if not publish:
        return None, 0
    ptrs = [p.data_ptr() if isinstance(p, torch.Tensor) else int(p) for p in publish]
    return (C.c_void_p * len(ptrs))(*ptrs), len(ptrs)


# ---- partitioner --------------------------------------------------------------------------------

def shard_range(num_nodes: int, num_gpus: int, pe: int):
    """(nodesPerPE, lb, ub) of PE ``pe``: ``src/mgg_np_div_mem.cu:85-88``."""
    a, b, c = C.c_int64(), C.c_int64(), C.c_int64()
    check(lib.mggb_shard_range(num_nodes, num_gpus, pe, C.byref(a), C.byref(b), C.byref(c)))
    return a.value, b.value, c.value


def split_CSR(origin_ptr, origin_col_idx, lb: int, ub: int, *, first_row: int = 0):
    """Returns ``[local_ptr, remote_ptr, local_col_idx, remote_col_idx]`` (int32 numpy arrays), in the
    reference's order.  ``origin_ptr`` may be int32 or int64.

    ``first_row``: ``origin_ptr[0]`` belongs to that global row.  The reference hands every rank the
    whole graph's pointers (first_row = 0); a rank that holds only its own rows' pointers (a graph
    too large to replicate) passes ``first_row = lb`` and gets the same four arrays."""
    ptr = np.ascontiguousarray(origin_ptr)
    if ptr.dtype not in (np.int32, np.int64):
        ptr = ptr.astype(np.int64)
    col = np.ascontiguousarray(origin_col_idx, dtype=np.int32)
    if lb < first_row or ub - first_row > len(ptr) - 1:
        raise ValueError(f"rows [{lb}, {ub}) are not inside the {len(ptr) - 1} rows held from row {first_row}")
    wide = ptr.dtype == np.int64
    count = lib.mggb_split_csr_count_i64 if wide else lib.mggb_split_csr_count
    fill = lib.mggb_split_csr_fill_i64 if wide else lib.mggb_split_csr_fill
    # the C entry points only read row_ptr[lb .. ub]: pass the address row 0 would have
    base = C.c_void_p(ptr.ctypes.data - first_row * ptr.itemsize)
    nl, nr = C.c_int64(), C.c_int64()
    check(count(base, _np_ptr(col), lb, ub, C.byref(nl), C.byref(nr)))
    local_ptr = np.empty(ub - lb + 1, np.int32)
    remote_ptr = np.empty(ub - lb + 1, np.int32)
    local_col = np.empty(nl.value, np.int32)
    remote_col = np.empty(nr.value, np.int32)
    check(fill(base, _np_ptr(col), lb, ub, _np_ptr(local_ptr), _np_ptr(remote_ptr),
               _np_ptr(local_col), _np_ptr(remote_col)))
    return [local_ptr, remote_ptr, local_col, remote_col]


def build_part(name: str, indptr, num_nodes: int, partSize: int, exact_sentinel: bool = False):
    """Returns ``[partPtr, part2Node, node2Part]`` exactly as the reference does (``node2Part`` has
    num_nodes+2 entries; the closing ``partPtr`` entry is 0 when the last node has no edges unless
    ``exact_sentinel``).  ``name`` is accepted for signature parity; nothing is printed."""
    del name
    indptr = np.ascontiguousarray(indptr, dtype=np.int32)
    if len(indptr) < num_nodes + 1:
        raise ValueError("indptr shorter than num_nodes+1")
    n = C.c_int64()
    check(lib.mggb_build_part_count(_np_ptr(indptr), num_nodes, partSize, C.byref(n)))
    part_ptr = np.empty(n.value + 1, np.int32)
    part2node = np.empty(n.value, np.int32)
    node2part = np.empty(num_nodes + 2, np.int32)
    check(lib.mggb_build_part_fill(_np_ptr(indptr), num_nodes, partSize, int(exact_sentinel),
                                   _np_ptr(part_ptr), _np_ptr(part2node), _np_ptr(node2part)))
    return [part_ptr, part2node, node2part]


def hub_threshold(np_size: int, warpPerBlock: int, interleaved_dist: int, dim: int, flags: int = 0) -> int:
    """Neighbor count above which the aggregations hand a row to their wide-block kernel at these knobs
    (-1: never).  A shard whose longest list stays below it can pass ``_lib.AGG_NO_HUB_SPLIT``."""
    t = C.c_int64()
    check(lib.mggb_hub_threshold(np_size, warpPerBlock, interleaved_dist, dim, flags, C.byref(t)))
    return t.value


def degree_order(row_ptr_l, row_ptr_r=None):
    """Host helper: shard rows sorted by neighbor count, longest first (int32 numpy array); pass it
    (on the device) as ``row_order`` to the aggregations so that long rows start first."""
    lp = np.ascontiguousarray(row_ptr_l, dtype=np.int32)
    rp = None if row_ptr_r is None else np.ascontiguousarray(row_ptr_r, dtype=np.int32)
    order = np.empty(len(lp) - 1, np.int32)
    check(lib.mggb_degree_order(_np_ptr(lp), _np_ptr(rp), len(lp) - 1, _np_ptr(order)))
    return order


# ---- aggregation --------------------------------------------------------------------------------

def mgg_SAG_np_div(output, input, row_pointers_l, column_index_l, row_pointers_r, column_index_r,
                   lb, ub, dim, nodePerPE, peid, np_size, warpPerBlock, interleaved_dist,
                   *, accumulate: bool = True, row_scale_: torch.Tensor | None = None, publish=None,
                   row_order: torch.Tensor | None = None, rows: torch.Tensor | None = None, flags: int = 0):
    """``output[b,:] (+)= sum of the local and remote neighbors' rows`` for the shard ``[lb, ub)``.
    ``rows`` (int32 device tensor of shard-relative row ids, each at most once): only those rows are
    computed, in that block order; ``output`` is still the whole shard's matrix.

    ``input`` is this PE's symmetric embedding buffer: a tensor when there is one PE, otherwise the
    table of all PEs' buffers (see ``_peer_table``).  ``accumulate=True`` is the reference's
    behaviour (it adds on top of ``output``'s contents).  ``publish``: buffers (local or peer-mapped)
    that also receive every output row, see ``mggb_sag_np_div``."""
    table, num_pes = _peer_table(input)
    pub, npub = _publish_table(publish)
    if ub > lb:
        _count_aggregation(dim, warpPerBlock, flags, rows)
    if rows is not None:
        check(lib.mggb_sag_np_div_rows(
            _dev_ptr(output, torch.float32, "output"), table, num_pes,
            _dev_ptr(row_pointers_l, torch.int32, "row_pointers_l"), _dev_ptr(column_index_l, torch.int32, "column_index_l"),
            _dev_ptr(row_pointers_r, torch.int32, "row_pointers_r"), _dev_ptr(column_index_r, torch.int32, "column_index_r"),
            lb, ub, dim, nodePerPE, peid, np_size, warpPerBlock, interleaved_dist,
            _dev_ptr(row_scale_, torch.float32, "row_scale"), (_lib.AGG_ACCUMULATE if accumulate else 0) | flags, pub, npub,
            _dev_ptr(rows, torch.int32, "rows"), rows.numel(), _stream()))
        return
    check(lib.mggb_sag_np_div_ordered(
        _dev_ptr(output, torch.float32, "output"), table, num_pes,
        _dev_ptr(row_pointers_l, torch.int32, "row_pointers_l"), _dev_ptr(column_index_l, torch.int32, "column_index_l"),
        _dev_ptr(row_pointers_r, torch.int32, "row_pointers_r"), _dev_ptr(column_index_r, torch.int32, "column_index_r"),
        lb, ub, dim, nodePerPE, peid, np_size, warpPerBlock, interleaved_dist,
        _dev_ptr(row_scale_, torch.float32, "row_scale"), (_lib.AGG_ACCUMULATE if accumulate else 0) | flags, pub, npub,
        _dev_ptr(row_order, torch.int32, "row_order"), _stream()))


def mgg_GIN_np_div(output, input, row_pointers_l, column_index_l, row_pointers_r, column_index_r,
                   lb, ub, dim, nodePerPE, peid, np_size, warpPerBlock, interleaved_dist, eps,
                   *, row_order: torch.Tensor | None = None, rows: torch.Tensor | None = None, flags: int = 0):
    """``output[b,:] = (1+eps) * input_self[b,:] + sum`` (``include/neighbor_utils.cuh:1660-1665``).
    ``rows``: as for ``mgg_SAG_np_div``."""
    table, num_pes = _peer_table(input)
    if ub > lb:
        _count_aggregation(dim, warpPerBlock, flags, rows)
    if rows is not None:
        check(lib.mggb_gin_np_div_rows(
            _dev_ptr(output, torch.float32, "output"), table, num_pes,
            _dev_ptr(row_pointers_l, torch.int32, "row_pointers_l"), _dev_ptr(column_index_l, torch.int32, "column_index_l"),
            _dev_ptr(row_pointers_r, torch.int32, "row_pointers_r"), _dev_ptr(column_index_r, torch.int32, "column_index_r"),
            lb, ub, dim, nodePerPE, peid, np_size, warpPerBlock, interleaved_dist, float(eps), flags,
            _dev_ptr(rows, torch.int32, "rows"), rows.numel(), _stream()))
        return
    check(lib.mggb_gin_np_div_ordered(
        _dev_ptr(output, torch.float32, "output"), table, num_pes,
        _dev_ptr(row_pointers_l, torch.int32, "row_pointers_l"), _dev_ptr(column_index_l, torch.int32, "column_index_l"),
        _dev_ptr(row_pointers_r, torch.int32, "row_pointers_r"), _dev_ptr(column_index_r, torch.int32, "column_index_r"),
        lb, ub, dim, nodePerPE, peid, np_size, warpPerBlock, interleaved_dist, float(eps), flags,
        _dev_ptr(row_order, torch.int32, "row_order"), _stream()))


def SAG_host_fused_interleaved(output, input, local_row_pointers, local_column_index, local_part_pointers, local_part2Node,
                               local_num_parts, remote_row_pointers, remote_column_index, remote_part_pointers, remote_part2Node,
                               remote_num_parts, num_nodes, lowbound, partSize, dim, dimWorker, warpPerBlock, interleaved_dist=1,
                               *, local_node2Part, remote_node2Part=None, nodePerPE=None, peid=0, scratch=None,
                               accumulate: bool = True, row_scale_=None, gin_eps=None):
    """The aggregation over explicit neighbor partitions, with the reference launcher's argument order
    (``include/neighbor_utils.cuh:593-616``): ``num_nodes`` rows starting at global row ``lowbound``;
    the ``*_part_pointers`` / ``*_part2Node`` device arrays are ``build_part``'s first two outputs for
    each half of the split CSR.  ``dimWorker`` is accepted for signature parity (the kernels choose
    their own lane mapping).  Beyond the reference's list: ``*_node2Part`` (``build_part``'s third
    output; the per-row reduce needs it where the reference uses atomics), ``nodePerPE`` / ``peid`` and
    a table ``input`` for several PEs, and an optional ``scratch`` tensor (allocated here when None)."""
    del dimWorker
    table, num_pes = _peer_table(input)
    npp = num_nodes if nodePerPE is None else nodePerPE
    need = C.c_size_t()
    check(lib.mggb_sag_np_part_scratch_bytes(local_num_parts, remote_num_parts, dim, C.byref(need)))
    if scratch is None:
        scratch = torch.empty(max(need.value // 4, 4), dtype=torch.float32, device=output.device)
    flags = (_lib.AGG_ACCUMULATE if accumulate and gin_eps is None else 0) | (_lib.AGG_GIN_COMBINE if gin_eps is not None else 0)
    kernel_launches[0] += 2 if num_nodes else 0
    check(lib.mggb_sag_np_part(
        _dev_ptr(output, torch.float32, "output"), table, num_pes,
        _dev_ptr(local_row_pointers, torch.int32), _dev_ptr(local_column_index, torch.int32), _dev_ptr(local_part_pointers, torch.int32),
        _dev_ptr(local_part2Node, torch.int32), _dev_ptr(local_node2Part, torch.int32), local_num_parts,
        _dev_ptr(remote_row_pointers, torch.int32), _dev_ptr(remote_column_index, torch.int32), _dev_ptr(remote_part_pointers, torch.int32),
        _dev_ptr(remote_part2Node, torch.int32), _dev_ptr(remote_node2Part, torch.int32), remote_num_parts,
        lowbound, lowbound + num_nodes, dim, npp, peid, partSize, warpPerBlock, interleaved_dist,
        _dev_ptr(row_scale_, torch.float32, "row_scale"), flags, float(gin_eps or 0.0),
        _dev_ptr(scratch, torch.float32, "scratch"), scratch.numel() * 4, _stream()))
    return scratch


# ---- dense update and softmax ---------------------------------------------------------------------

def dense_forward(out, x, w, row_scale_=None, relu=False, flags=0, publish=None):
    n, dim1 = x.shape
    dim2 = w.shape[1]
    if w.shape[0] != dim1 or tuple(out.shape) != (n, dim2):
        raise ValueError(f"shape mismatch: x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    kernel_launches[0] += 1 if n else 0
    check(lib.mggb_dense_forward(_dev_ptr(out, torch.float32, "out"), _dev_ptr(x, torch.float32, "x"),
                                 _dev_ptr(w, torch.float32, "w"), n, dim1, dim2,
                                 _dev_ptr(row_scale_, torch.float32, "row_scale"),
                                 flags | (_lib.DENSE_RELU if relu else 0), *_publish_table(publish), _stream()))


def softmax_forward(out, inp):
    n, dim = inp.shape
    kernel_launches[0] += 1 if n else 0
    check(lib.mggb_softmax_forward(_dev_ptr(out, torch.float32, "out"), _dev_ptr(inp, torch.float32, "in"),
                                   n, dim, _stream()))


def dense_softmax_forward(out, x, w, logits=None):
    """out = softmax_rows(x @ w) in one kernel (the models' last dense layer and softmax,
    ``src/mgg_np_div_mem.cu:220-226``); ``logits`` (optional) also receives x @ w.  Raises MggbError with
    status ERR_UNSUPPORTED for shapes the fused kernel does not take."""
    n, dim1 = x.shape
    dim2 = w.shape[1]
    if w.shape[0] != dim1 or tuple(out.shape) != (n, dim2) or (logits is not None and tuple(logits.shape) != (n, dim2)):
        raise ValueError(f"shape mismatch: x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    kernel_launches[0] += 1 if n else 0
    check(lib.mggb_dense_softmax_forward(_dev_ptr(out, torch.float32, "out"), _dev_ptr(logits, torch.float32, "logits"),
                                         _dev_ptr(x, torch.float32, "x"), _dev_ptr(w, torch.float32, "w"),
                                         n, dim1, dim2, _stream()))


def dense_softmax_fits(dim1: int, dim2: int) -> bool:
    """Whether ``dense_softmax_forward`` takes this shape (dim2 <= 256 and w plus the staging rows within 160 KiB)."""
    j = (dim2 + 31) // 32
    jp = (j + 1) // 2   # the kernel keeps w and the staged rows as pairs of floats
    return j <= 8 and (dim1 * 32 * jp + 64 * dim1) * 8 <= 160 * 1024


def publish_rows(src: torch.Tensor, publish, elem_offset: int = 0):
    """Copies the contiguous fp32 tensor ``src`` to ``base + elem_offset`` floats of every entry of
    ``publish`` (tensors or device addresses, e.g. ``ReplicaBuffer.publish``): pushes rows that a kernel
    wrote locally into the peers' replicas with full-width stores."""
    if not publish or src.numel() == 0:
        return
    if not src.is_contiguous():
        raise ValueError("publish_rows: src must be contiguous")
    dst = [(p.data_ptr() if isinstance(p, torch.Tensor) else int(p)) + 4 * elem_offset for p in publish]
    pub, npub = _publish_table(dst)
    kernel_launches[0] += 1
    check(lib.mggb_publish_rows(_dev_ptr(src, torch.float32, "src"), src.numel(), pub, npub, _stream()))


def row_scale(out, inp, scale):
    n, dim = inp.shape
    kernel_launches[0] += 1 if n else 0
    check(lib.mggb_row_scale(_dev_ptr(out, torch.float32, "out"), _dev_ptr(inp, torch.float32, "in"),
                             _dev_ptr(scale, torch.float32, "scale"), n, dim, _stream()))


def inv_sqrt_degree(scale, row_ptr_l, row_ptr_r=None):
    n = scale.numel()
    check(lib.mggb_inv_sqrt_degree(_dev_ptr(scale, torch.float32, "scale"), _dev_ptr(row_ptr_l, torch.int32, "row_ptr_l"),
                                   _dev_ptr(row_ptr_r, torch.int32, "row_ptr_r"), n, _stream()))


class _dense_param:
    """Common part of the reference's dense parameter structs: the caller supplies ``d_in`` and
    ``d_out`` (``[numNodes, dim1]`` and ``[numNodes, dim2]`` views are taken of them); the struct owns
    ``d_W`` ``[dim1, dim2]``, filled with 1.0 as in the reference (``include/layer_new.cuh:307``).
    ``set_weight`` uploads other values (the reference has no such entry point)."""

    def __init__(self, name_in: str, d_in_ext: torch.Tensor, d_out_ext: torch.Tensor, numNodes_in: int,
                 dim1_in: int, dim2_in: int):
        self.name = name_in[:8]
        self.numNodes, self.dim1, self.dim2 = numNodes_in, dim1_in, dim2_in
        self.m, self.n, self.k = dim2_in, numNodes_in, dim1_in
        self.ldx, self.ldw, self.ldout = dim1_in, dim2_in, dim2_in
        self.alpha, self.beta = 1.0, 0.0
        self.d_in, self.d_out = d_in_ext, d_out_ext
        if d_in_ext.numel() < numNodes_in * dim1_in or d_out_ext.numel() < numNodes_in * dim2_in:
            raise ValueError("d_in / d_out smaller than numNodes*dim1 / numNodes*dim2 floats")
        self.d_W = torch.ones(dim1_in, dim2_in, dtype=torch.float32, device=d_in_ext.device)
        self.row_scale = None
        self.relu = False
        self.flags = 0
        self.publish = None      # extra destinations of the output rows (peers' replicas)

    def set_weight(self, w: torch.Tensor):
        if tuple(w.shape) != (self.dim1, self.dim2):
            raise ValueError(f"weight must be [{self.dim1}, {self.dim2}]")
        self.d_W.copy_(w)

    def _forward(self):
        x = self.d_in.reshape(-1)[: self.numNodes * self.dim1].view(self.numNodes, self.dim1)
        o = self.d_out.reshape(-1)[: self.numNodes * self.dim2].view(self.numNodes, self.dim2)
        dense_forward(o, x, self.d_W, self.row_scale, self.relu, self.flags, self.publish)

    def _forward_rows(self, r0: int, r1: int):
        """The same product for rows [r0, r1) only (rows are independent): lets a caller overlap the
        upload of later rows with the product of earlier ones."""
        if r1 <= r0:
            return
        x = self.d_in.reshape(-1)[: self.numNodes * self.dim1].view(self.numNodes, self.dim1)[r0:r1]
        o = self.d_out.reshape(-1)[: self.numNodes * self.dim2].view(self.numNodes, self.dim2)[r0:r1]
        scale = None if self.row_scale is None else self.row_scale[r0:r1]
        pub = None
        if self.publish:
            off = r0 * self.dim2 * 4
            pub = [(p.data_ptr() if isinstance(p, torch.Tensor) else int(p)) + off for p in self.publish]
        dense_forward(o, x, self.d_W, scale, self.relu, self.flags, pub)


class dense_param_new_beg(_dense_param):
    """``include/layer_new.cuh:272-333``."""


class dense_param_new_hidden(_dense_param):
    """``include/layer_new.cuh:336-393``."""


class softmax_new_param:
    """``include/layer_new.cuh:59-103``: row softmax of ``d_in`` ``[numNodes, dim]`` into ``d_out``."""

    def __init__(self, name_in: str, d_in_input: torch.Tensor, d_out_ext: torch.Tensor, numNodes_in: int, dim_in: int):
        self.name = name_in[:8]
        self.numNodes, self.dim = numNodes_in, dim_in
        self.d_in, self.d_out = d_in_input, d_out_ext
        self.alpha, self.beta = 1.0, 0.0


def dense_beg_new_forward(dp: dense_param_new_beg):
    """``include/gnn_layer.cuh:42-46``.  Computes d_out = d_in * d_W (the reference's call passes d_out
    as the right-hand operand and never reads d_in; the intended product is computed here)."""
    dp._forward()


def dense_hidden_new_forward(dp: dense_param_new_hidden):
    """``include/gnn_layer.cuh:48-52``."""
    dp._forward()


def dense_hidden_softmax_new_forward(dp: dense_param_new_hidden, smx: softmax_new_param, keep_logits: bool = False):
    """``dense_hidden_new_forward(dp); softmax_new_forward(smx);`` (``src/mgg_np_div_mem.cu:220-226``) as one
    kernel when smx reads what dp writes and the shape fits; the two separate calls otherwise.  Without
    ``keep_logits`` the fused pass leaves dp.d_out untouched."""
    fused = (smx.d_in.data_ptr() == dp.d_out.data_ptr() and smx.numNodes == dp.numNodes and smx.dim == dp.dim2
             and dp.row_scale is None and not dp.publish and not dp.relu and not (dp.flags & _lib.DENSE_RELU)
             and dense_softmax_fits(dp.dim1, dp.dim2))
    if not fused:
        dp._forward()
        softmax_new_forward(smx)
        return
    n = dp.numNodes
    x = dp.d_in.reshape(-1)[: n * dp.dim1].view(n, dp.dim1)
    o = smx.d_out.reshape(-1)[: n * dp.dim2].view(n, dp.dim2)
    lg = dp.d_out.reshape(-1)[: n * dp.dim2].view(n, dp.dim2) if keep_logits else None
    dense_softmax_forward(o, x, dp.d_W, lg)


def softmax_new_forward(smx: softmax_new_param):
    """``include/gnn_layer.cuh:36-40``."""
    i = smx.d_in.reshape(-1)[: smx.numNodes * smx.dim].view(smx.numNodes, smx.dim)
    o = smx.d_out.reshape(-1)[: smx.numNodes * smx.dim].view(smx.numNodes, smx.dim)
    softmax_forward(o, i)
