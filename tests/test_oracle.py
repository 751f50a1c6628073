"""The CPU oracle against (a) the committed golden vectors, which were produced by the reference's
own host code, and (b) that code itself where its compiled form is present."""
import numpy as np
import pytest

SPLITS = [(1, 0), (2, 0), (2, 1), (3, 0), (3, 2), (4, 1), (4, 3), (8, 5)]
PART_SIZES = [1, 2, 3, 16, 32]


def test_known_answers(oracle, golden):
    out = oracle.sag_f32(golden["ka_sag_x"], golden["ka_sag_row_ptr"], golden["ka_sag_col"])
    assert np.array_equal(out, golden["ka_sag_out"])
    assert np.array_equal(out, np.array([[8, 10], [1, 2], [4, 6]], np.float32))
    lp, rp, lc, rc = oracle.split_csr([0, 2, 3, 5, 6], [1, 2, 0, 0, 3, 2], 0, 2)
    assert lp.tolist() == [0, 1, 2] and rp.tolist() == [0, 1, 1]
    assert lc.tolist() == [1, 0] and rc.tolist() == [2]
    pp, p2n, n2p = oracle.build_part([0, 3, 5, 6], 3, 2)
    assert pp.tolist() == [0, 2, 3, 5, 6] and p2n.tolist() == [0, 0, 1, 2] and n2p.tolist() == [0, 2, 3, 4, 4]
    # last node without edges: the closing sentinel stays 0 (reference behaviour)
    pp, p2n, n2p = oracle.build_part([0, 3, 5, 5], 3, 2)
    assert pp.tolist() == [0, 2, 3, 0] and p2n.tolist() == [0, 0, 1] and n2p.tolist() == [0, 2, 3, 3, 3]


@pytest.mark.parametrize("tag", ["a", "b", "c", "d"])
@pytest.mark.parametrize("ps", [2, 16])
def test_build_part_golden_small(oracle, golden, tag, ps):
    ptr = golden[f"ka_part_{tag}_ptr"]
    pp, p2n, n2p = oracle.build_part(ptr, len(ptr) - 1, ps)
    assert np.array_equal(pp, golden[f"ka_part_{tag}_ps{ps}_partptr"])
    assert np.array_equal(p2n, golden[f"ka_part_{tag}_ps{ps}_part2node"])
    assert np.array_equal(n2p, golden[f"ka_part_{tag}_ps{ps}_node2part"])


@pytest.mark.parametrize("dim", [16, 5])
def test_sag_golden(oracle, golden, dim):
    rp, col, x = golden["g_row_ptr"], golden["g_col"], golden[f"g_x{dim}"]
    assert np.array_equal(oracle.sag_f32(x, rp, col), golden[f"g_sag{dim}"])          # same order: same bits
    out_omp, _ = oracle.sag_omp(x, rp, col)
    assert np.array_equal(out_omp, golden[f"g_sag{dim}"])
    np.testing.assert_allclose(oracle.sag_f64(x, rp, col), golden[f"g_sag{dim}"], rtol=1e-5, atol=1e-4)


def test_sag_all_ones_is_degree(oracle, golden):
    rp, col = golden["g_row_ptr"], golden["g_col"]
    ones = np.ones((len(rp) - 1, 4), np.float32)
    out = oracle.sag_f32(ones, rp, col)
    assert np.array_equal(out, golden["g_sag_ones"])
    assert np.array_equal(out[:, 0], np.diff(rp).astype(np.float32))


def test_sag_accumulates(oracle, golden):
    rp, col, x = golden["g_row_ptr"], golden["g_col"], golden["g_x16"]
    out = oracle.sag_f32(x, rp, col, update=golden["g_sag16"])
    assert np.array_equal(out, golden["g_sag_accum"])


@pytest.mark.parametrize("G,pe", SPLITS)
def test_split_and_parts_golden(oracle, golden, G, pe):
    rp, col = golden["g_row_ptr"], golden["g_col"]
    n = len(rp) - 1
    k = f"g_split_G{G}_pe{pe}"
    assert list(oracle.shard_range(n, G, pe)) == golden[k + "_bounds"].tolist()
    npp, lb, ub = golden[k + "_bounds"]
    lp, rpp, lc, rc = oracle.split_csr(rp, col, int(lb), int(ub))
    assert np.array_equal(lp, golden[k + "_local_ptr"]) and np.array_equal(rpp, golden[k + "_remote_ptr"])
    assert np.array_equal(lc, golden[k + "_local_col"]) and np.array_equal(rc, golden[k + "_remote_col"])
    for ps in PART_SIZES:
        for half, ptr in (("l", lp), ("r", rpp)):
            pp, p2n, n2p = oracle.build_part(ptr, int(ub - lb), ps)
            assert np.array_equal(pp, golden[f"{k}_{half}_ps{ps}_partptr"])
            assert np.array_equal(p2n, golden[f"{k}_{half}_ps{ps}_part2node"])
            assert np.array_equal(n2p, golden[f"{k}_{half}_ps{ps}_node2part"])


@pytest.mark.parametrize("G", [1, 2, 3, 4, 8])
def test_shard_aggregate_equals_whole_graph(oracle, golden, G):
    """Summing local + remote halves through the per-PE symmetric buffers (owner = id / nodePerPE,
    row = id % nodePerPE) reproduces the whole-graph aggregation restricted to the shard."""
    rp, col, x = golden["g_row_ptr"], golden["g_col"], golden["g_x16"]
    n, dim = x.shape
    want = oracle.sag_f64(x, rp, col)
    npp = (n + G - 1) // G
    sym = [np.zeros((npp, dim), np.float32) for _ in range(G)]
    for p in range(G):
        lo, hi = p * npp, min((p + 1) * npp, n)
        sym[p][: hi - lo] = x[lo:hi]
    for pe in range(G):
        _, lb, ub = oracle.shard_range(n, G, pe)
        lp, rpp, lc, rc = oracle.split_csr(rp, col, lb, ub)
        got = oracle.shard_aggregate(sym, pe, lp, lc, rpp, rc, lb, ub, npp)
        np.testing.assert_allclose(got, want[lb:ub], rtol=1e-6, atol=1e-6)
        gin = oracle.shard_aggregate(sym, pe, lp, lc, rpp, rc, lb, ub, npp, gin=True, eps=0.5)
        np.testing.assert_allclose(gin, want[lb:ub] + 1.5 * x[lb:ub], rtol=1e-6, atol=1e-5)


def test_dense_softmax_norm(oracle):
    rng = np.random.default_rng(0)
    x = rng.uniform(-1, 1, (37, 19)).astype(np.float32)
    w = rng.uniform(-1, 1, (19, 7)).astype(np.float32)
    np.testing.assert_allclose(oracle.dense(x, w), x.astype(np.float64) @ w.astype(np.float64), rtol=1e-6, atol=1e-6)
    s = oracle.softmax(oracle.dense(x, w))
    np.testing.assert_allclose(s.sum(1), 1.0, rtol=1e-6)
    z = x.astype(np.float64) @ w.astype(np.float64)
    e = np.exp(z - z.max(1, keepdims=True))
    np.testing.assert_allclose(s, e / e.sum(1, keepdims=True), rtol=1e-5, atol=1e-7)
    assert oracle.inv_sqrt_degree([0, 4, 4, 5]).tolist() == [0.5, 0.0, 1.0]


# ---- against the reference's own compiled host code (skipped where it is absent) ----------------

@pytest.mark.parametrize("seed", [0, 1, 2])
def test_oracle_matches_reference_host_code(oracle, ref, seed):
    rng = np.random.default_rng(seed)
    n = int(rng.integers(1, 200))
    deg = rng.integers(0, 12, n)
    deg[rng.integers(0, n)] = 90
    rp = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
    col = rng.integers(0, n, rp[-1]).astype(np.int32)
    x = rng.uniform(-1, 1, (n, 9)).astype(np.float32)
    assert np.array_equal(oracle.sag_f32(x, rp, col), ref.sag_ref(x, rp, col))
    for G in (1, 2, 5):
        for pe in range(G):
            _, lb, ub = oracle.shard_range(n, G, pe)
            a, b = oracle.split_csr(rp, col, lb, ub), ref.split_csr(rp, col, lb, ub)
            for u, v in zip(a, b):
                assert np.array_equal(u, v)
            for ps in (1, 4, 32):
                for ptr in a[:2]:
                    for u, v in zip(oracle.build_part(ptr, ub - lb, ps), ref.build_part(ptr, ub - lb, ps)):
                        assert np.array_equal(u, v)


def test_reference_aggregation_on_several_node_ranges_at_once_gives_the_same_bits():
    """The CPU arm of the benchmark calls SAG_ref on disjoint node ranges from several threads."""
    from oracle.oracle import Ref
    if not Ref.available():
        pytest.skip("the reference's host code was not compiled here")
    import numpy as np
    from mgg_osdi23_b200 import graphgen as gg
    ref = Ref()
    g = gg.chung_lu_graph(3000, 120_000, 2.1, seed=9)
    rp, col = g.row_ptr.numpy().astype(np.int32), g.col_idx.numpy()
    x = gg.features(g.num_nodes, 7, seed=1).numpy()
    one = ref.sag_ref(x, rp, col)
    for threads in (2, 3, 8):
        assert np.array_equal(one, ref.sag_ref(x, rp, col, threads=threads))
    start = gg.features(g.num_nodes, 7, seed=2).numpy()
    assert np.array_equal(ref.sag_ref(x, rp, col, update=start), ref.sag_ref(x, rp, col, update=start, threads=4))
