"""ctypes front-end of the CPU oracle.  TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark may import this
module; the shipped package never does.  Two libraries sit behind it:

* ``liboracle.so``  - our plain-C restatement (``mgg_oracle.c``), class :class:`Oracle`;
* ``_ref/libmggref.so`` - the reference's own host functions ``SAG_ref`` / ``split_CSR`` /
  ``build_part`` compiled from the reference's sources (``ref_shim.cu``), class :class:`Ref`.
  It is prebuilt where the reference sources exist and travels as a binary elsewhere.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_I32P = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_F32P = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")


def reference_root() -> str | None:
    """Where the reference project's sources lie: $MGG_REFERENCE_ROOT, else a directory named
    ``reference`` beside this repository.  None when neither exists."""
    cand = os.environ.get("MGG_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return cand if os.path.isdir(os.path.join(cand, "include")) else None


def build(verbose: bool = False, ref_root: str | None = None) -> None:
    """Run the Makefile (gcc for the restatement; nvcc for the reference shim when its sources are present)."""
    ref_root = ref_root or reference_root()
    cmd = ["make", "-C", _HERE] + ([f"REF_ROOT={ref_root}"] if ref_root else [])
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        print(r.stdout, r.stderr)
    if r.returncode != 0:
        raise RuntimeError("oracle build failed")


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _opt(a, dtype):
    """Pointer to an optional array (None -> NULL)."""
    if a is None:
        return None
    return a.ctypes.data_as(C.c_void_p)


class Oracle:
    """The plain-C restatement."""

    def __init__(self):
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        self.lib = L = C.CDLL(path)
        L.orc_sag_f32.argtypes = [_F32P, _F32P, _I32P, _I32P, C.c_int64, C.c_int]
        L.orc_sag_f64.argtypes = [_F32P, _F32P, _I32P, _I32P, C.c_int64, C.c_int]
        L.orc_sag_omp.argtypes = [_F32P, _F32P, _I32P, _I32P, C.c_int64, C.c_int]
        L.orc_sag_omp.restype = C.c_int
        L.orc_sag_f64_omp.argtypes = [_F32P, _F32P, _I32P, _I32P, C.c_int64, C.c_int]
        L.orc_set_threads.argtypes = [C.c_int]
        L.orc_get_threads.restype = C.c_int
        L.orc_shard_aggregate.argtypes = [_F32P, C.POINTER(C.c_void_p), C.c_int, C.c_int, _I32P, C.c_void_p,
                                          _I32P, C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_int64,
                                          C.c_int, C.c_int, C.c_float, C.c_void_p]
        L.orc_shard_range.argtypes = [C.c_int64, C.c_int, C.c_int] + [C.POINTER(C.c_int64)] * 3
        L.orc_split_csr.argtypes = [_I32P, C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.c_int64),
                                    C.POINTER(C.c_int64)] + [C.c_void_p] * 4
        L.orc_build_part.argtypes = [_I32P, C.c_int32, C.c_int32, C.POINTER(C.c_int64)] + [C.c_void_p] * 3
        L.orc_dense.argtypes = [_F32P, _F32P, _F32P, C.c_int64, C.c_int, C.c_int, C.c_void_p, C.c_int]
        L.orc_softmax.argtypes = [_F32P, _F32P, C.c_int64, C.c_int]
        L.orc_inv_sqrt_degree.argtypes = [_F32P, _I32P, C.c_int64]
        L.orc_row_scale.argtypes = [_F32P, _F32P, _F32P, C.c_int64, C.c_int]

    # -- aggregation -------------------------------------------------------------------------
    def sag_f32(self, x, row_ptr, col, update=None):
        """``SAG_ref`` arithmetic: fp32 sequential ``update += A @ x`` (update defaults to zeros)."""
        x, row_ptr, col = _f32(x), _i32(row_ptr), _i32(col)
        n, dim = len(row_ptr) - 1, x.shape[1]
        out = np.zeros((n, dim), np.float32) if update is None else _f32(update).copy()
        self.lib.orc_sag_f32(out, x, row_ptr, col, n, dim)
        return out

    def sag_f64(self, x, row_ptr, col):
        x, row_ptr, col = _f32(x), _i32(row_ptr), _i32(col)
        n, dim = len(row_ptr) - 1, x.shape[1]
        out = np.zeros((n, dim), np.float32)
        self.lib.orc_sag_f64(out, x, row_ptr, col, n, dim)
        return out

    def sag_f64_omp(self, x, row_ptr, col):
        """``sag_f64`` with the rows dealt to OpenMP threads (same values)."""
        x, row_ptr, col = _f32(x), _i32(row_ptr), _i32(col)
        n, dim = len(row_ptr) - 1, x.shape[1]
        out = np.zeros((n, dim), np.float32)
        self.lib.orc_sag_f64_omp(out, x, row_ptr, col, n, dim)
        return out

    def set_threads(self, threads: int) -> int:
        """Sets the thread count of the OpenMP routines (dense, softmax, sag_omp, sag_f64_omp) at run
        time, whatever OMP_NUM_THREADS said when the runtime was loaded; returns the count in effect."""
        self.lib.orc_set_threads(int(threads))
        return int(self.lib.orc_get_threads())

    def get_threads(self) -> int:
        return int(self.lib.orc_get_threads())

    def sag_omp(self, x, row_ptr, col, out=None):
        x, row_ptr, col = _f32(x), _i32(row_ptr), _i32(col)
        n, dim = len(row_ptr) - 1, x.shape[1]
        if out is None:
            out = np.empty((n, dim), np.float32)
        threads = self.lib.orc_sag_omp(out, x, row_ptr, col, n, dim)
        return out, threads

    def shard_aggregate(self, sym, pe, rp_l, ci_l, rp_r, ci_r, lb, ub, node_per_pe, out=None,
                        accumulate=False, gin=False, eps=0.0, row_scale=None):
        """One PE's rows from the per-PE symmetric buffers ``sym`` (list of [nodePerPE, dim] arrays)."""
        sym = [_f32(s) for s in sym]
        dim = sym[0].shape[1]
        rows = ub - lb
        rp_l, ci_l, rp_r, ci_r = _i32(rp_l), _i32(ci_l), _i32(rp_r), _i32(ci_r)
        res = np.zeros((rows, dim), np.float32) if out is None else _f32(out).copy()
        ptrs = (C.c_void_p * len(sym))(*[s.ctypes.data for s in sym])
        rs = None if row_scale is None else _f32(row_scale)
        self.lib.orc_shard_aggregate(res, ptrs, len(sym), pe, rp_l, _opt(ci_l, np.int32), rp_r,
                                     _opt(ci_r, np.int32), lb, ub, dim, node_per_pe,
                                     int(accumulate), int(gin), float(eps), _opt(rs, np.float32))
        return res

    # -- partitioner -------------------------------------------------------------------------
    def shard_range(self, num_nodes, num_gpus, pe):
        a, b, c = C.c_int64(), C.c_int64(), C.c_int64()
        self.lib.orc_shard_range(num_nodes, num_gpus, pe, C.byref(a), C.byref(b), C.byref(c))
        return a.value, b.value, c.value

    def split_csr(self, row_ptr, col, lb, ub):
        row_ptr, col = _i32(row_ptr), _i32(col)
        nl, nr = C.c_int64(), C.c_int64()
        colp = _opt(col, np.int32)
        self.lib.orc_split_csr(row_ptr, colp, lb, ub, C.byref(nl), C.byref(nr), None, None, None, None)
        lp = np.zeros(ub - lb + 1, np.int32)
        rp = np.zeros(ub - lb + 1, np.int32)
        lc = np.zeros(nl.value, np.int32)
        rc = np.zeros(nr.value, np.int32)
        self.lib.orc_split_csr(row_ptr, colp, lb, ub, C.byref(nl), C.byref(nr),
                               lp.ctypes.data, rp.ctypes.data, lc.ctypes.data, rc.ctypes.data)
        return lp, rp, lc, rc

    def build_part(self, indptr, num_nodes, ps):
        indptr = _i32(indptr)
        n = C.c_int64()
        self.lib.orc_build_part(indptr, num_nodes, ps, C.byref(n), None, None, None)
        pp = np.zeros(n.value + 1, np.int32)
        p2n = np.zeros(n.value, np.int32)
        n2p = np.zeros(num_nodes + 2, np.int32)
        self.lib.orc_build_part(indptr, num_nodes, ps, C.byref(n), pp.ctypes.data, p2n.ctypes.data,
                                n2p.ctypes.data)
        return pp, p2n, n2p

    # -- dense / softmax / norm --------------------------------------------------------------
    def dense(self, x, w, row_scale=None, relu=False):
        x, w = _f32(x), _f32(w)
        out = np.empty((x.shape[0], w.shape[1]), np.float32)
        rs = None if row_scale is None else _f32(row_scale)
        self.lib.orc_dense(out, x, w, x.shape[0], x.shape[1], w.shape[1], _opt(rs, np.float32), int(relu))
        return out

    def softmax(self, x):
        x = _f32(x)
        out = np.empty_like(x)
        self.lib.orc_softmax(out, x, x.shape[0], x.shape[1])
        return out

    def inv_sqrt_degree(self, row_ptr):
        row_ptr = _i32(row_ptr)
        out = np.empty(len(row_ptr) - 1, np.float32)
        self.lib.orc_inv_sqrt_degree(out, row_ptr, len(row_ptr) - 1)
        return out

    def row_scale(self, x, scale):
        x, scale = _f32(x), _f32(scale)
        out = np.empty_like(x)
        self.lib.orc_row_scale(out, x, scale, x.shape[0], x.shape[1])
        return out


class Ref:
    """The reference's own host functions (compiled from its sources; see ``ref_shim.cu``)."""

    PATH = os.path.join(_HERE, "_ref", "libmggref.so")

    @classmethod
    def available(cls) -> bool:
        return os.path.exists(cls.PATH)

    def __init__(self):
        if not self.available():
            raise FileNotFoundError(self.PATH)
        self.lib = L = C.CDLL(self.PATH)
        L.mggref_sag_ref.argtypes = [_F32P, _F32P, _I32P, _I32P, C.c_int, C.c_int, C.c_int]
        L.mggref_split_csr.argtypes = [_I32P, C.c_longlong, C.c_void_p, C.c_longlong, C.c_int, C.c_int,
                                       C.POINTER(C.c_longlong), C.POINTER(C.c_longlong)] + [C.c_void_p] * 4
        L.mggref_build_part.argtypes = [_I32P, C.c_int, C.c_int, C.POINTER(C.c_longlong)] + [C.c_void_p] * 3

    def sag_ref(self, x, row_ptr, col, update=None, threads: int = 1):
        """``SAG_ref`` (``include/utils.cuh:71-86``).  The function is a single loop over the nodes;
        with ``threads`` > 1 it is CALLED on that many disjoint node ranges at once (pointers offset
        to the range; column offsets stay absolute), which gives the same bits row for row."""
        x, row_ptr, col = _f32(x), _i32(row_ptr), _i32(col)
        n, dim = len(row_ptr) - 1, x.shape[1]
        out = np.zeros((n, dim), np.float32) if update is None else _f32(update).copy()
        if len(col) == 0:
            col = np.zeros(1, np.int32)
        if threads <= 1 or n < 4 * threads:
            self.lib.mggref_sag_ref(out, x, row_ptr, col, n, int(row_ptr[-1]), dim)
            return out
        from concurrent.futures import ThreadPoolExecutor
        # node ranges of about equal edge counts, four per thread
        cuts = np.searchsorted(row_ptr, np.linspace(0, int(row_ptr[-1]), 4 * threads + 1)[1:-1]).astype(np.int64)
        bounds = np.unique(np.concatenate([[0], np.clip(cuts, 0, n), [n]]))

        def run(k):
            r0, r1 = int(bounds[k]), int(bounds[k + 1])
            self.lib.mggref_sag_ref(out[r0:r1], x, row_ptr[r0:r1 + 1], col, r1 - r0, int(row_ptr[-1]), dim)

        with ThreadPoolExecutor(max_workers=threads) as pool:      # ctypes releases the GIL during the call
            list(pool.map(run, range(len(bounds) - 1)))
        return out

    def split_csr(self, row_ptr, col, lb, ub):
        row_ptr, col = _i32(row_ptr), _i32(col)
        nl, nr = C.c_longlong(), C.c_longlong()
        colp = col.ctypes.data_as(C.c_void_p)
        self.lib.mggref_split_csr(row_ptr, len(row_ptr), colp, len(col), lb, ub, C.byref(nl), C.byref(nr),
                                  None, None, None, None)
        lp = np.zeros(ub - lb + 1, np.int32)
        rp = np.zeros(ub - lb + 1, np.int32)
        lc = np.zeros(nl.value, np.int32)
        rc = np.zeros(nr.value, np.int32)
        self.lib.mggref_split_csr(row_ptr, len(row_ptr), colp, len(col), lb, ub, C.byref(nl), C.byref(nr),
                                  lp.ctypes.data, rp.ctypes.data, lc.ctypes.data, rc.ctypes.data)
        return lp, rp, lc, rc

    def build_part(self, indptr, num_nodes, ps):
        indptr = _i32(indptr)
        n = C.c_longlong()
        self.lib.mggref_build_part(indptr, num_nodes, ps, C.byref(n), None, None, None)
        pp = np.zeros(n.value + 1, np.int32)
        p2n = np.zeros(n.value, np.int32)
        n2p = np.zeros(num_nodes + 2, np.int32)
        self.lib.mggref_build_part(indptr, num_nodes, ps, C.byref(n), pp.ctypes.data, p2n.ctypes.data,
                                   n2p.ctypes.data)
        return pp, p2n, n2p
