"""Symmetric (peer-readable) embedding buffers for the Python host layer.

Replaces ``nvshmem_malloc`` (``src/mgg_np_div_mem.cu:139``): every PE allocates a buffer of the same
size and every PE ends up with the table of all PEs' base addresses, which the aggregation call
takes.  Allocation and mapping go through the C ABI (CUDA IPC between processes); torch only wraps
the local allocation as a tensor and carries the 64-byte handles between ranks.
"""
from __future__ import annotations

import ctypes as C

import torch

from ._lib import lib, check


class _RawCudaBuffer:
    """Exposes a raw device allocation through ``__cuda_array_interface__`` so torch can view it."""

    def __init__(self, ptr: int, numel: int):
        self.__cuda_array_interface__ = {
            "shape": (numel,), "typestr": "<f4", "data": (ptr, False), "version": 3, "strides": None}


def exchange_handles(handle: bytes, group, num_pes: int):
    """All-gathers one 64-byte export handle per PE (index = PE).  Works on any backend."""
    import torch.distributed as dist
    if len(handle) != 64:
        raise ValueError("an export handle is 64 bytes")
    handles = [None] * num_pes
    dist.all_gather_object(handles, handle, group=group)
    if any(h is None or len(h) != 64 for h in handles):
        raise RuntimeError("handle exchange returned a malformed handle")
    return handles


class SymmetricBuffer:
    """``numel`` fp32 elements on the current device, readable by every PE of ``group``.

    ``tensor``     1-D torch view of the local allocation.
    ``peer_ptrs``  base address of every PE's buffer as seen from this process (index = PE).
    With ``group=None`` (or a group of one) there is a single PE and nothing is exchanged.
    """

    def __init__(self, numel: int, group=None, pe: int = 0, num_pes: int = 1):
        self.numel = int(numel)
        self.pe, self.num_pes = pe, num_pes
        self._imported = []
        p = C.c_void_p()
        check(lib.mggb_sym_alloc(self.numel * 4, C.byref(p)))
        self.ptr = p.value
        self._raw = _RawCudaBuffer(self.ptr, self.numel)
        self.tensor = torch.as_tensor(self._raw, device=torch.device("cuda", torch.cuda.current_device()))
        self.peer_ptrs = [self.ptr]
        if num_pes > 1:
            handle = C.create_string_buffer(64)
            check(lib.mggb_sym_export(C.c_void_p(self.ptr), handle))
            handles = exchange_handles(handle.raw, group, num_pes)
            self.peer_ptrs = []
            for r, h in enumerate(handles):
                if r == pe:
                    self.peer_ptrs.append(self.ptr)
                else:
                    q = C.c_void_p()
                    check(lib.mggb_sym_import(h, C.byref(q)))
                    self._imported.append(q.value)
                    self.peer_ptrs.append(q.value)

    publish = None   # a directly shared buffer is written locally only; peers pull from it

    def view(self, rows: int, dim: int) -> torch.Tensor:
        return self.tensor[: rows * dim].view(rows, dim)

    def own(self, rows: int, dim: int) -> torch.Tensor:
        """Where this PE writes its rows."""
        return self.view(rows, dim)

    def close(self):
        """Unmaps the peers' buffers and frees the local one.  Every PE must have stopped reading it."""
        for q in self._imported:
            lib.mggb_sym_close(C.c_void_p(q))
        self._imported = []
        if self.ptr:
            self.tensor = None
            self._raw = None
            lib.mggb_sym_free(C.c_void_p(self.ptr))
            self.ptr = 0


class ReplicaBuffer:
    """A full copy of the [num_pes * node_per_pe, dim] embedding matrix on every PE.

    Slot p (rows p*node_per_pe ...) holds PE p's rows.  A PE's kernels write their output rows into
    their own slot of the local copy AND, through ``publish``, into the same slot of every peer's
    copy, so after the next barrier every aggregation reads local memory only.  It costs
    num_pes * node_per_pe * dim * 4 bytes per PE and one pushed row per (node, peer), instead of one
    pulled row per remote EDGE: cheaper whenever a node is referenced by more than one remote edge.
    Presents the same ``peer_ptrs`` / ``own`` / ``publish`` interface as :class:`SymmetricBuffer`.
    """

    def __init__(self, node_per_pe: int, dim: int, group=None, pe: int = 0, num_pes: int = 1):
        self.node_per_pe, self.dim, self.pe, self.num_pes = node_per_pe, dim, pe, num_pes
        self.slot_elems = node_per_pe * dim
        self.sym = SymmetricBuffer(num_pes * self.slot_elems, group, pe, num_pes)
        self.tensor = self.sym.tensor
        # reading: every slot of the LOCAL copy
        self.peer_ptrs = [self.sym.ptr + p * self.slot_elems * 4 for p in range(num_pes)]
        # writing: this PE's slot in every PEER's copy, nearest higher PE first.  Every kernel walks the
        # table in order for each tile it stores, so with this rotation the PEs aim at different
        # receivers at any one time instead of all at PE 0, then all at PE 1, ...
        self.publish = [self.sym.peer_ptrs[(pe + k) % num_pes] + pe * self.slot_elems * 4
                        for k in range(1, num_pes)] or None

    def own(self, rows: int, dim: int) -> torch.Tensor:
        off = self.pe * self.slot_elems
        return self.tensor[off: off + rows * dim].view(rows, dim)

    def close(self):
        self.tensor = None
        self.sym.close()
