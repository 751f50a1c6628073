"""The library's host partitioner (C ABI) against the oracle and the golden vectors: bit-exact."""
import ctypes as C

import numpy as np
import pytest

import mgg_osdi23_b200 as mgg
from mgg_osdi23_b200 import graphgen as gg

SPLITS = [(1, 0), (2, 0), (2, 1), (3, 0), (3, 2), (4, 1), (4, 3), (8, 5)]
PART_SIZES = [1, 2, 3, 16, 32]


@pytest.mark.parametrize("G,pe", SPLITS)
def test_golden(golden, G, pe):
    rp, col = golden["g_row_ptr"], golden["g_col"]
    k = f"g_split_G{G}_pe{pe}"
    assert list(mgg.shard_range(len(rp) - 1, G, pe)) == golden[k + "_bounds"].tolist()
    _, lb, ub = (int(v) for v in golden[k + "_bounds"])
    for ptr in (rp, rp.astype(np.int64)):
        lp, rpp, lc, rc = mgg.split_CSR(ptr, col, lb, ub)
        assert np.array_equal(lp, golden[k + "_local_ptr"]) and np.array_equal(rpp, golden[k + "_remote_ptr"])
        assert np.array_equal(lc, golden[k + "_local_col"]) and np.array_equal(rc, golden[k + "_remote_col"])
    for ps in PART_SIZES:
        for half, ptr in (("l", lp), ("r", rpp)):
            pp, p2n, n2p = mgg.build_part("t", ptr, ub - lb, ps)
            assert np.array_equal(pp, golden[f"{k}_{half}_ps{ps}_partptr"])
            assert np.array_equal(p2n, golden[f"{k}_{half}_ps{ps}_part2node"])
            assert np.array_equal(n2p, golden[f"{k}_{half}_ps{ps}_node2part"])


@pytest.mark.parametrize("tag", ["a", "b", "c", "d"])
def test_build_part_corner_cases(golden, tag):
    ptr = golden[f"ka_part_{tag}_ptr"]
    for ps in (2, 16):
        pp, p2n, n2p = mgg.build_part("t", ptr, len(ptr) - 1, ps)
        assert np.array_equal(pp, golden[f"ka_part_{tag}_ps{ps}_partptr"])
        assert np.array_equal(p2n, golden[f"ka_part_{tag}_ps{ps}_part2node"])
        assert np.array_equal(n2p, golden[f"ka_part_{tag}_ps{ps}_node2part"])
    # the opt-in fixed sentinel always closes the last partition
    pp, _, _ = mgg.build_part("t", [0, 3, 5, 5], 3, 2, exact_sentinel=True)
    assert pp.tolist() == [0, 2, 3, 5]


@pytest.mark.parametrize("G", [1, 2, 4, 8])
def test_config1_shape_vs_oracle(oracle, G):
    """A config-1-shaped R-MAT graph (smaller scale) split for every PE, every ps in 1..32."""
    g = gg.rmat_graph(11, 32768, seed=0)
    rp, col = g.row_ptr.numpy().astype(np.int32), g.col_idx.numpy()
    total = 0
    for pe in range(G):
        npp, lb, ub = mgg.shard_range(g.num_nodes, G, pe)
        got, want = mgg.split_CSR(rp, col, lb, ub), oracle.split_csr(rp, col, lb, ub)
        for u, v in zip(got, want):
            assert u.dtype == np.int32 and np.array_equal(u, v)
        total += got[2].size + got[3].size
        for ps in (1, 2, 5, 8, 16, 32):
            for ptr in got[:2]:
                for u, v in zip(mgg.build_part("t", ptr, ub - lb, ps), oracle.build_part(ptr, ub - lb, ps)):
                    assert np.array_equal(u, v)
    assert total == g.num_edges


def test_ragged_and_empty(oracle):
    # a graph with empty rows, a shard past the end (more PEs than nodes) and an empty graph
    rp = np.array([0, 0, 3, 3, 4], np.int32)
    col = np.array([0, 3, 1, 2], np.int32)
    for G in (1, 3, 8):
        for pe in range(G):
            npp, lb, ub = mgg.shard_range(4, G, pe)
            assert (npp, lb, ub) == oracle.shard_range(4, G, pe)
            for u, v in zip(mgg.split_CSR(rp, col, lb, ub), oracle.split_csr(rp, col, lb, ub)):
                assert np.array_equal(u, v)
    lp, rpp, lc, rc = mgg.split_CSR(np.zeros(1, np.int32), np.zeros(0, np.int32), 0, 0)
    assert lp.tolist() == [0] and rpp.tolist() == [0] and lc.size == 0 and rc.size == 0
    pp, p2n, n2p = mgg.build_part("t", [0], 0, 4)
    assert pp.tolist() == [0] and p2n.size == 0 and n2p.tolist() == [0, 0]


def test_argument_errors():
    with pytest.raises(mgg.MggbError):
        mgg.shard_range(10, 0, 0)
    with pytest.raises(mgg.MggbError):
        mgg.shard_range(10, 2, 2)
    with pytest.raises(mgg.MggbError):
        mgg.build_part("t", [0, 1], 1, 0)
    with pytest.raises(ValueError):
        mgg.split_CSR([0, 1], [0], 0, 5)
    from mgg_osdi23_b200._lib import lib
    assert lib.mggb_split_csr_count(None, None, 0, 0, None, None) != 0
    assert b"NULL" in lib.mggb_last_error()


def test_degree_order():
    lp = np.array([0, 2, 2, 9, 10, 10], np.int32)      # local degrees 2 0 7 1 0
    rp = np.array([0, 0, 5, 5, 6, 6], np.int32)        # remote degrees 0 5 0 1 0
    assert mgg.degree_order(lp, rp).tolist() == [2, 1, 0, 3, 4]      # totals 2 5 7 2 0; ties keep row order
    assert mgg.degree_order(lp).tolist() == [2, 0, 3, 1, 4]
    assert mgg.degree_order(np.zeros(1, np.int32)).size == 0
    # against a stable sort, on a skewed degree sequence, and on one whose largest degree dwarfs the row count
    rng = np.random.default_rng(3)
    deg = np.minimum(rng.zipf(1.7, size=20_000), 50_000)
    lp = np.zeros(deg.size + 1, np.int32); lp[1:] = np.cumsum(deg // 2)
    rp = np.zeros(deg.size + 1, np.int32); rp[1:] = np.cumsum(deg - deg // 2)
    assert np.array_equal(mgg.degree_order(lp, rp), np.argsort(-deg, kind="stable"))
    sparse = np.array([0, 5, 200_000_005, 200_000_006, 200_000_011], np.int32)
    assert mgg.degree_order(sparse).tolist() == [1, 0, 3, 2]


def test_split_from_shard_local_rows(oracle):
    """A rank that holds only its own rows' pointers (rebased to 0) gets the same split."""
    g = gg.rmat_graph(10, 8000, seed=6)
    rp, col = g.row_ptr.numpy(), g.col_idx.numpy()
    for G in (2, 3):
        for pe in range(G):
            npp, lb, ub = mgg.shard_range(g.num_nodes, G, pe)
            local_rp = (rp[lb:ub + 1] - rp[lb]).astype(np.int64)
            local_col = col[rp[lb]:rp[ub]]
            got = mgg.split_CSR(local_rp, local_col, lb, ub, first_row=lb)
            for u, v in zip(got, oracle.split_csr(rp.astype(np.int32), col, lb, ub)):
                assert np.array_equal(u, v)
    with pytest.raises(ValueError):
        mgg.split_CSR(np.zeros(3, np.int64), np.zeros(0, np.int32), 5, 9, first_row=6)
