"""Synthetic graph generators and the reference's binary CSR file format."""
import os

import numpy as np
import pytest
import torch

import mgg_osdi23_b200 as mgg
from mgg_osdi23_b200 import graphgen as gg, graphio


def _check_csr(g, symmetric, repeats=False):
    rp, col = g.row_ptr.numpy(), g.col_idx.numpy()
    assert rp[0] == 0 and rp[-1] == col.size and np.all(np.diff(rp) >= 0)
    assert col.min() >= 0 and col.max() < g.num_nodes
    rows = np.repeat(np.arange(g.num_nodes), np.diff(rp))
    keys = rows.astype(np.int64) * g.num_nodes + col
    if repeats:
        assert np.all(np.diff(keys) >= 0) and np.any(np.diff(keys) == 0)   # sorted; an edge list with repeated pairs
    else:
        assert np.all(np.diff(keys) > 0)             # sorted, no duplicates
    if symmetric:
        rev = np.sort(col.astype(np.int64) * g.num_nodes + rows)
        assert np.array_equal(rev, keys)


def test_config1_graph():
    g = gg.config1_graph()
    assert g.num_nodes == 16384 and 262144 < g.num_edges <= 2 * 262144 + 16384
    _check_csr(g, True)
    assert np.all(np.diff(g.row_ptr.numpy()) >= 1)   # self-loops
    g2 = gg.config1_graph()
    assert torch.equal(g.col_idx, g2.col_idx)        # seeded


def test_chung_lu_communities():
    g = gg.chung_lu_graph(4096, 200_000, 2.1, seed=1, communities=8, p_intra=0.7)
    _check_csr(g, True)
    assert abs(g.num_edges - 200_000) / 200_000 < 0.05
    rows = np.repeat(np.arange(g.num_nodes), np.diff(g.row_ptr.numpy()))
    same = (rows // 512) == (g.col_idx.numpy() // 512)
    assert 0.6 < same.mean() < 0.85
    deg = np.diff(g.row_ptr.numpy())
    assert deg.max() > 5 * deg.mean()                # heavy tail


def test_directed_rmat_subset():
    g = gg.config4_graph(scale_shift=8)
    _check_csr(g, False, repeats=True)
    assert g.num_nodes == 4_206_785 >> 8
    # every sampled pair is an edge (the shape's edge count and its skew both count repeated pairs)
    assert g.num_edges == 101_300_000 >> 8 and g.meta["repeated_pairs_kept"]
    assert g.meta["max_in_degree"] == int(np.diff(g.row_ptr.numpy()).max()) > 50 * g.num_edges // g.num_nodes


def test_features_are_shard_independent():
    full = gg.features(100, 16, seed=5)
    part = gg.features(30, 16, seed=5, first_row=40)
    assert torch.equal(full[40:70], part)
    assert full.min() >= -1 and full.max() < 1
    w = gg.glorot_uniform(602, 16, seed=1)
    assert w.abs().max() <= (6 / 618) ** 0.5


def test_binary_csr_roundtrip(tmp_path):
    g = gg.rmat_graph(8, 1000, seed=2)
    beg, csr, wt = graphio.write_graph(str(tmp_path / "g"), g.row_ptr.numpy(), g.col_idx.numpy())
    assert os.path.getsize(beg) == 8 * (g.num_nodes + 1)
    assert os.path.getsize(csr) == 8 * g.num_edges and os.path.getsize(wt) == 4 * g.num_edges
    assert np.array_equal(np.fromfile(csr, np.int64), g.col_idx.numpy().astype(np.int64))
    rp, col = graphio.load_graph(beg, csr)
    assert np.array_equal(rp, g.row_ptr.numpy()) and np.array_equal(col, g.col_idx.numpy())
    import mgg_osdi23_b200 as mgg
    with pytest.raises(mgg.MggbError):
        graphio.load_graph(str(tmp_path / "missing_beg_pos.bin"), csr)


def test_shard_local_generation_matches_whole_graph():
    """The config-5 path: each PE builds only its rows; together they are the whole symmetric graph."""
    scale, pairs, n = 10, 6000, 900
    whole = gg.rmat_graph(scale, pairs, seed=4, num_nodes=None)          # on all 1024 ids
    # same sampled pairs, ids >= n dropped, symmetrised, self-loops: assemble from three shards
    parts = []
    for pe in range(3):
        npp = (n + 2) // 3
        lb, ub = pe * npp, min(n, (pe + 1) * npp)
        sh = gg.rmat_shard(scale, pairs, n, lb, ub, seed=4, batch=1000)
        assert sh.row_ptr.numel() == ub - lb + 1 and sh.row_ptr[0] == 0
        rows = np.repeat(np.arange(lb, ub), np.diff(sh.row_ptr.numpy()))
        parts.append(rows.astype(np.int64) * n + sh.col_idx.numpy())
    got = np.concatenate(parts)
    wr = np.repeat(np.arange(whole.num_nodes), np.diff(whole.row_ptr.numpy()))
    wc = whole.col_idx.numpy()
    keep = (wr < n) & (wc < n)
    want = np.sort(wr[keep].astype(np.int64) * n + wc[keep])
    assert np.array_equal(np.sort(got), want)
    # the shard feeds the 64-bit-row-pointer split directly (local ids are rebased by the caller)
    sh = gg.config5_shard(1, 4, scale_shift=17)
    assert sh.num_nodes == 111_000_000 >> 17 and sh.row_ptr.dtype == torch.int64


def test_relabelling_is_a_permutation_and_balances_shards():
    for n in (1, 2, 7, 1000, 16433):
        p = gg.relabel_ids(torch.arange(n), n, seed=3)
        assert sorted(p.tolist()) == list(range(n))
    # relabelled shards assemble into the relabelled whole graph
    scale, pairs, n = 10, 6000, 900
    whole = gg.rmat_graph(scale, pairs, seed=4, num_nodes=None)
    wr = np.repeat(np.arange(whole.num_nodes), np.diff(whole.row_ptr.numpy()))
    wc = whole.col_idx.numpy().astype(np.int64)
    keep = (wr < n) & (wc < n)
    rr = gg.relabel_ids(torch.from_numpy(wr[keep]), n, seed=4).numpy()
    cc = gg.relabel_ids(torch.from_numpy(wc[keep]), n, seed=4).numpy()
    want = np.unique(rr * n + cc)
    parts = []
    for pe in range(3):
        lb, ub = pe * 300, (pe + 1) * 300
        sh = gg.rmat_shard(scale, pairs, n, lb, ub, seed=4, batch=1000, relabel=True)
        rows = np.repeat(np.arange(lb, ub), np.diff(sh.row_ptr.numpy()))
        parts.append(rows.astype(np.int64) * n + sh.col_idx.numpy())
    assert np.array_equal(np.sort(np.concatenate(parts)), want)
    # the skewed configurations give node-range shards of similar size
    g = gg.config4_graph(scale_shift=6)
    deg = np.diff(g.row_ptr.numpy())
    npp = (g.num_nodes + 7) // 8
    per = np.array([deg[i * npp:(i + 1) * npp].sum() for i in range(8)])
    assert per.max() < 1.25 * per.mean()
    g = gg.config3_graph(scale=0.02)
    deg = np.diff(g.row_ptr.numpy())
    npp = (g.num_nodes + 7) // 8
    per = np.array([deg[i * npp:(i + 1) * npp].sum() for i in range(8)])
    assert per.max() < 1.1 * per.mean()


def test_shard_rows_are_read_from_their_part_of_the_files(tmp_path):
    """load_graph_rows returns what slicing the whole graph gives, and feeds the shard-local split."""
    g = gg.rmat_graph(9, 5000, seed=8)
    rp, col = g.row_ptr.numpy(), g.col_idx.numpy()
    beg, csr, _ = graphio.write_graph(str(tmp_path / "g"), rp, col)
    n = g.num_nodes
    for lb, ub in ((0, n), (0, 100), (100, 371), (n - 7, n), (50, 50), (n, n)):
        srp, scol = graphio.load_graph_rows(beg, csr, lb, ub)
        assert srp.dtype == np.int64 and scol.dtype == np.int32 and srp[0] == 0
        assert np.array_equal(srp, rp[lb:ub + 1] - rp[lb])
        assert np.array_equal(scol, col[rp[lb]:rp[ub]])
    # the shard's rows go straight into the split with shard-local pointers
    G, pe = 3, 1
    npp, lb, ub = mgg.shard_range(n, G, pe)
    srp, scol = graphio.load_graph_rows(beg, csr, lb, ub)
    whole = mgg.split_CSR(rp.astype(np.int32), col, lb, ub)
    part = mgg.split_CSR(srp, scol, lb, ub, first_row=lb)
    assert all(np.array_equal(a, b) for a, b in zip(whole, part))
    # bad ranges and damaged files are refused with a message
    for lb, ub in ((-1, 5), (5, 4), (0, n + 1)):
        with pytest.raises(mgg.MggbError):
            graphio.load_graph_rows(beg, csr, lb, ub)
    short = str(tmp_path / "short_csr.bin")
    with open(csr, "rb") as f, open(short, "wb") as o:
        o.write(f.read()[: 8 * int(rp[200]) - 8])
    graphio.load_graph_rows(beg, short, 0, 100)                    # rows before the cut still load
    with pytest.raises(mgg.MggbError):
        graphio.load_graph_rows(beg, short, 150, 220)
    with pytest.raises(mgg.MggbError):
        graphio.load_graph_rows(str(tmp_path / "missing_beg_pos.bin"), csr, 0, 1)
