"""The reference's binary CSR files (``include/graph.hpp:9-129``) through the C ABI.

``<name>_beg_pos.bin`` N+1 int64 offsets, ``<name>_csr.bin`` E int64 neighbor ids,
``<name>_weight.bin`` E int32 weights (written as ones; the reference never reads their values).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import lib, check


def graph_file_names(prefix: str):
    return prefix + "_beg_pos.bin", prefix + "_csr.bin", prefix + "_weight.bin"


def write_graph(prefix: str, row_ptr, col_idx, with_weights: bool = True):
    row_ptr = np.ascontiguousarray(row_ptr, dtype=np.int64)
    col_idx = np.ascontiguousarray(col_idx, dtype=np.int32)
    beg, csr, wt = graph_file_names(prefix)
    check(lib.mggb_graph_file_write(beg.encode(), csr.encode(), wt.encode() if with_weights else None,
                                    row_ptr.ctypes.data_as(C.c_void_p), col_idx.ctypes.data_as(C.c_void_p),
                                    len(row_ptr) - 1))
    return beg, csr, wt


def load_graph(beg_file: str, csr_file: str):
    """Returns (row_ptr int64 [N+1], col_idx int32 [E])."""
    n, e = C.c_int64(), C.c_int64()
    check(lib.mggb_graph_file_info(beg_file.encode(), csr_file.encode(), C.byref(n), C.byref(e)))
    row_ptr = np.empty(n.value + 1, np.int64)
    col = np.empty(e.value, np.int32)
    check(lib.mggb_graph_file_load(beg_file.encode(), csr_file.encode(), n.value, e.value,
                                   row_ptr.ctypes.data_as(C.c_void_p), col.ctypes.data_as(C.c_void_p)))
    return row_ptr, col


def load_graph_rows(beg_file: str, csr_file: str, lb: int, ub: int):
    """Rows [lb, ub) only: (row_ptr int64 [ub-lb+1] starting at 0, col_idx int32), read from just those
    parts of the files.  What ``drivers.Shard(..., shard_local=True)`` takes."""
    first, e = C.c_int64(), C.c_int64()
    check(lib.mggb_graph_file_rows_info(beg_file.encode(), lb, ub, C.byref(first), C.byref(e)))
    row_ptr = np.empty(ub - lb + 1, np.int64)
    col = np.empty(e.value, np.int32)
    check(lib.mggb_graph_file_load_rows(beg_file.encode(), csr_file.encode(), lb, ub,
                                        row_ptr.ctypes.data_as(C.c_void_p), col.ctypes.data_as(C.c_void_p)))
    return row_ptr, col
