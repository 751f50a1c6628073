"""ctypes binding of ``libmggb200.so``.

The library is the only compute path of this package: if it is missing or fails to load, importing
this module raises - there is no Python or CPU substitute behind it.
"""
from __future__ import annotations

import ctypes as C
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libmggb200.so")

OK, ERR_INVALID_ARG, ERR_CUDA, ERR_UNSUPPORTED, ERR_PEER, ERR_IO = range(6)
AGG_ACCUMULATE, AGG_NO_HUB_SPLIT, AGG_GROUP_PER_NODE, AGG_STAGE_ROWS, AGG_GIN_COMBINE, AGG_NO_REMOTE = 1, 2, 4, 8, 32, 64
DENSE_RELU, DENSE_TF32, DENSE_SIMT, DENSE_TENSOR = 1, 2, 4, 8
MAX_PES = 16


class MggbError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"mggb status {code}: {msg}")
        self.code = code


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python mgg_osdi23_b200/build.py` "
            "(nvcc, sm_100a). This package has no fallback path.")
    return C.CDLL(LIB_PATH)


lib = _load()

_vp, _i32, _i64, _int, _f = C.c_void_p, C.c_int32, C.c_int64, C.c_int, C.c_float
_pi64 = C.POINTER(C.c_int64)

# name -> argtypes; every function returns int status unless noted.
SIGNATURES = {
    "mggb_shard_range": [_i64, _int, _int, _pi64, _pi64, _pi64],
    "mggb_split_csr_count": [_vp, _vp, _i32, _i32, _pi64, _pi64],
    "mggb_split_csr_fill": [_vp, _vp, _i32, _i32, _vp, _vp, _vp, _vp],
    "mggb_split_csr_count_i64": [_vp, _vp, _i32, _i32, _pi64, _pi64],
    "mggb_split_csr_fill_i64": [_vp, _vp, _i32, _i32, _vp, _vp, _vp, _vp],
    "mggb_build_part_count": [_vp, _i32, _i32, _pi64],
    "mggb_build_part_fill": [_vp, _i32, _i32, _int, _vp, _vp, _vp],
    "mggb_sym_alloc": [C.c_size_t, C.POINTER(_vp)],
    "mggb_sym_free": [_vp],
    "mggb_sym_export": [_vp, C.c_char_p],
    "mggb_sym_import": [C.c_char_p, C.POINTER(_vp)],
    "mggb_sym_close": [_vp],
    "mggb_enable_peer_access": [_int, _int],
    "mggb_flag_barrier": [C.POINTER(_vp), _int, _int, _int, _i64, _vp],
    "mggb_flag_barrier_counted": [C.POINTER(_vp), _int, _int, _vp, _i64, _vp],
    "mggb_flag_barrier_status": [C.POINTER(_int), _int],
    "mggb_sag_np_div": [_vp, C.POINTER(_vp), _int, _vp, _vp, _vp, _vp, _i32, _i32, _int, _i32, _int,
                        _int, _int, _int, _vp, _int, C.POINTER(_vp), _int, _vp],
    "mggb_sag_np_div_static": [_vp, C.POINTER(_vp), _int, _vp, _vp, _vp, _vp, _i32, _i32, _i64, _int, _i32, _int,
                               _int, _int, _int, _vp, _int, C.POINTER(_vp), _int, _vp],
    "mggb_gin_np_div": [_vp, C.POINTER(_vp), _int, _vp, _vp, _vp, _vp, _i32, _i32, _int, _i32, _int,
                        _int, _int, _int, _f, _int, _vp],
    "mggb_sag_np_div_ordered": [_vp, C.POINTER(_vp), _int, _vp, _vp, _vp, _vp, _i32, _i32, _int, _i32, _int,
                                _int, _int, _int, _vp, _int, C.POINTER(_vp), _int, _vp, _vp],
    "mggb_gin_np_div_ordered": [_vp, C.POINTER(_vp), _int, _vp, _vp, _vp, _vp, _i32, _i32, _int, _i32, _int,
                                _int, _int, _int, _f, _int, _vp, _vp],
    "mggb_sag_np_div_rows": [_vp, C.POINTER(_vp), _int, _vp, _vp, _vp, _vp, _i32, _i32, _int, _i32, _int,
                             _int, _int, _int, _vp, _int, C.POINTER(_vp), _int, _vp, _i64, _vp],
    "mggb_gin_np_div_rows": [_vp, C.POINTER(_vp), _int, _vp, _vp, _vp, _vp, _i32, _i32, _int, _i32, _int,
                             _int, _int, _int, _f, _int, _vp, _i64, _vp],
    "mggb_sag_np_part_scratch_bytes": [_i64, _i64, _int, C.POINTER(C.c_size_t)],
    "mggb_sag_np_part": [_vp, C.POINTER(_vp), _int, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _i64,
                         _i32, _i32, _int, _i32, _int, _int, _int, _int, _vp, _int, _f, _vp, C.c_size_t, _vp],
    "mggb_publish_rows": [_vp, _i64, C.POINTER(_vp), _int, _vp],
    "mggb_degree_order": [_vp, _vp, _i32, _vp],
    "mggb_hub_threshold": [_int, _int, _int, _int, _int, _pi64],
    "mggb_dense_forward": [_vp, _vp, _vp, _i64, _int, _int, _vp, _int, C.POINTER(_vp), _int, _vp],
    "mggb_dense_device_status": [C.POINTER(_int), _int],
    "mggb_agg_device_status": [C.POINTER(_int), _int],
    "mggb_softmax_forward": [_vp, _vp, _i64, _int, _vp],
    "mggb_dense_softmax_forward": [_vp, _vp, _vp, _vp, _i64, _int, _int, _vp],
    "mggb_row_scale": [_vp, _vp, _vp, _i64, _int, _vp],
    "mggb_inv_sqrt_degree": [_vp, _vp, _vp, _i64, _vp],
    "mggb_graph_file_info": [C.c_char_p, C.c_char_p, _pi64, _pi64],
    "mggb_graph_file_load": [C.c_char_p, C.c_char_p, _i64, _i64, _vp, _vp],
    "mggb_graph_file_rows_info": [C.c_char_p, _i64, _i64, _pi64, _pi64],
    "mggb_graph_file_load_rows": [C.c_char_p, C.c_char_p, _i64, _i64, _vp, _vp],
    "mggb_graph_file_write": [C.c_char_p, C.c_char_p, C.c_char_p, _vp, _vp, _i64],
}

for _name, _args in SIGNATURES.items():
    if not hasattr(lib, _name):
        raise ImportError(f"{LIB_PATH} is stale (no symbol {_name}): rebuild it with `python mgg_osdi23_b200/build.py`. "
                          "This package has no fallback path.")
    _fn = getattr(lib, _name)
    _fn.argtypes = _args
    _fn.restype = C.c_int
lib.mggb_version.restype = C.c_int
lib.mggb_last_error.restype = C.c_char_p


def check(status: int) -> None:
    if status != OK:
        raise MggbError(status, lib.mggb_last_error().decode(errors="replace"))
