"""Generates tests/golden/mgg_golden.npz by RUNNING THE REFERENCE'S OWN HOST CODE.

The reference ships no fixtures for this path, so these are made here: seeded inputs of ours are
pushed through the reference's SAG_ref, split_CSR<int> and build_part<int> (compiled from the
reference's sources into oracle/_ref/libmggref.so, see oracle/ref_shim.cu), and inputs and outputs
are stored together.  Needs the reference sources at build time; run from the repository root:

    make -C oracle && python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle.oracle import Ref  # noqa: E402
from mgg_osdi23_b200 import graphgen as gg  # noqa: E402

SPLITS = [(1, 0), (2, 0), (2, 1), (3, 0), (3, 2), (4, 1), (4, 3), (8, 5)]
PART_SIZES = [1, 2, 3, 16, 32]


def main():
    ref = Ref()
    out = {}

    # hand-sized known answers
    out["ka_sag_row_ptr"] = np.array([0, 2, 3, 5], np.int32)
    out["ka_sag_col"] = np.array([1, 2, 0, 0, 1], np.int32)
    out["ka_sag_x"] = np.array([[1, 2], [3, 4], [5, 6]], np.float32)
    out["ka_sag_out"] = ref.sag_ref(out["ka_sag_x"], out["ka_sag_row_ptr"], out["ka_sag_col"])
    for tag, ptr in (("a", [0, 3, 5, 6]), ("b", [0, 3, 5, 5]), ("c", [0, 0, 0, 0]), ("d", [0, 1, 1, 70])):
        ptr = np.array(ptr, np.int32)
        out[f"ka_part_{tag}_ptr"] = ptr
        for ps in (2, 16):
            pp, p2n, n2p = ref.build_part(ptr, len(ptr) - 1, ps)
            out[f"ka_part_{tag}_ps{ps}_partptr"] = pp
            out[f"ka_part_{tag}_ps{ps}_part2node"] = p2n
            out[f"ka_part_{tag}_ps{ps}_node2part"] = n2p

    # a small seeded R-MAT graph (scale 8: 256 nodes) with a few isolated rows
    g = gg.rmat_graph(8, 2048, 0.57, 0.19, 0.19, seed=3, symmetric=True, self_loops=False)
    rp = g.row_ptr.numpy().astype(np.int32)
    col = g.col_idx.numpy().astype(np.int32)
    n = g.num_nodes
    out["g_row_ptr"], out["g_col"] = rp, col
    for dim in (16, 5):
        x = gg.features(n, dim, seed=11).numpy()
        out[f"g_x{dim}"] = x
        out[f"g_sag{dim}"] = ref.sag_ref(x, rp, col)
    ones = np.ones((n, 4), np.float32)
    out["g_sag_ones"] = ref.sag_ref(ones, rp, col)           # = degree, exact in fp32
    out["g_sag_accum"] = ref.sag_ref(out["g_x16"], rp, col, update=out["g_sag16"])  # accumulates on top

    for (G, pe) in SPLITS:
        npp = (n + G - 1) // G
        lb = npp * pe
        ub = min(lb + npp, n)
        lp, rpp, lc, rc = ref.split_csr(rp, col, lb, ub)
        k = f"g_split_G{G}_pe{pe}"
        out[k + "_bounds"] = np.array([npp, lb, ub], np.int64)
        out[k + "_local_ptr"], out[k + "_remote_ptr"] = lp, rpp
        out[k + "_local_col"], out[k + "_remote_col"] = lc, rc
        for ps in PART_SIZES:
            for half, ptr in (("l", lp), ("r", rpp)):
                pp, p2n, n2p = ref.build_part(ptr, ub - lb, ps)
                out[f"{k}_{half}_ps{ps}_partptr"] = pp
                out[f"{k}_{half}_ps{ps}_part2node"] = p2n
                out[f"{k}_{half}_ps{ps}_node2part"] = n2p

    path = os.path.join(ROOT, "tests", "golden", "mgg_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
