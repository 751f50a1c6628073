"""Parity of the CUDA aggregation (through the C ABI) with the CPU oracle and the golden vectors."""
import numpy as np
import pytest
import torch

import mgg_osdi23_b200 as mgg
from mgg_osdi23_b200 import drivers, graphgen as gg
from gpu_util import RTOL, ATOL, emulated_aggregate, random_graph

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("G", [1, 2, 3, 8])
@pytest.mark.parametrize("dim", [16, 5])
def test_golden_vectors(golden, G, dim):
    rp, col, x = golden["g_row_ptr"], golden["g_col"], golden[f"g_x{dim}"]
    got = emulated_aggregate(rp, col, x, G)
    np.testing.assert_allclose(got, golden[f"g_sag{dim}"], rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("G", [1, 2, 4])
def test_all_ones_is_exact_degree(golden, G):
    """The reference's only known-answer property: all-ones input gives the degree, exactly."""
    rp, col = golden["g_row_ptr"], golden["g_col"]
    ones = np.ones((len(rp) - 1, 16), np.float32)
    got = emulated_aggregate(rp, col, ones, G)
    assert np.array_equal(got, np.repeat(np.diff(rp)[:, None], 16, 1).astype(np.float32))
    assert np.array_equal(got[:, :4], golden["g_sag_ones"])


@pytest.mark.parametrize("dim", [1, 2, 4, 8, 12, 16, 32, 64, 100, 128, 200, 7, 33])
@pytest.mark.parametrize("G", [1, 4])
def test_widths(oracle, dim, G):
    rp, col = random_graph(300, 20, seed=dim, hubs=[(5, 700), (17, 0), (299, 0)])
    x = np.random.default_rng(dim).uniform(-1, 1, (300, dim)).astype(np.float32)
    got = emulated_aggregate(rp, col, x, G)
    np.testing.assert_allclose(got, oracle.sag_f64(x, rp, col), rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(got, oracle.sag_f32(x, rp, col), rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("ps", [1, 2, 4, 8, 16, 32])
@pytest.mark.parametrize("wpb,dist", [(1, 1), (2, 16), (4, 2), (8, 4), (16, 1), (3, 3)])
def test_knob_sweep(oracle, ps, wpb, dist):
    """Every ps x (wpb, dist) point of the design-space sweep gives the same sums."""
    rp, col = random_graph(200, 35, seed=1, hubs=[(0, 3000), (1, 1), (2, 0)])
    x = np.random.default_rng(2).uniform(-1, 1, (200, 16)).astype(np.float32)
    want = oracle.sag_f64(x, rp, col)
    for G in (1, 2):
        got = emulated_aggregate(rp, col, x, G, knobs=(ps, wpb, dist))
        np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL)


def test_accumulate_matches_reference_semantics(oracle, golden):
    """The reference adds on top of the output buffer; two calls double the sum."""
    rp, col, x = golden["g_row_ptr"], golden["g_col"], golden["g_x16"]
    first = emulated_aggregate(rp, col, x, 2, accumulate=True)
    second = emulated_aggregate(rp, col, x, 2, accumulate=True, init=first)
    np.testing.assert_allclose(second, golden["g_sag_accum"], rtol=RTOL, atol=ATOL)
    # overwrite mode ignores what was there
    again = emulated_aggregate(rp, col, x, 2, accumulate=False, init=np.full_like(first, 7.0))
    assert np.array_equal(again, first)


@pytest.mark.parametrize("G", [1, 3])
@pytest.mark.parametrize("eps", [0.0, 0.5])
def test_gin_combine(oracle, G, eps):
    rp, col = random_graph(257, 12, seed=4)
    x = np.random.default_rng(5).uniform(-1, 1, (257, 64)).astype(np.float32)
    got = emulated_aggregate(rp, col, x, G, gin_eps=eps)
    want = oracle.sag_f64(x, rp, col).astype(np.float64) + (1.0 + eps) * x
    np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL)


def test_row_scale_and_symmetric_norm_config1(oracle):
    """Config 1: one GCN aggregation with 1/sqrt(deg_i*deg_j) on the 16,384-node R-MAT graph, dim 16."""
    g = gg.config1_graph()
    rp, col = g.row_ptr.numpy().astype(np.int32), g.col_idx.numpy()
    x = gg.features(g.num_nodes, 16, seed=0).numpy()
    dinv = oracle.inv_sqrt_degree(rp)
    want = oracle.row_scale(oracle.sag_f64(oracle.row_scale(x, dinv), rp, col), dinv)
    for G in (1, 2):
        got = emulated_aggregate(rp, col, oracle.row_scale(x, dinv), G, row_scale=dinv)
        np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL)
    # the device-side helpers produce the same factors
    dev = torch.device("cuda")
    sh = drivers.Shard(rp, col, 0, 1, device=dev)
    np.testing.assert_allclose(sh.inv_sqrt_degree().cpu().numpy(), dinv, rtol=1e-6)
    xs = torch.empty(g.num_nodes, 16, device=dev)
    mgg.row_scale(xs, torch.from_numpy(x).to(dev), sh.inv_sqrt_degree())
    np.testing.assert_allclose(xs.cpu().numpy(), oracle.row_scale(x, dinv), rtol=1e-6)


def test_bit_reproducible_for_fixed_knobs():
    rp, col = random_graph(500, 60, seed=9, hubs=[(3, 5000)])
    x = np.random.default_rng(1).uniform(-1, 1, (500, 16)).astype(np.float32)
    a = emulated_aggregate(rp, col, x, 2, knobs=(16, 4, 2))
    b = emulated_aggregate(rp, col, x, 2, knobs=(16, 4, 2))
    assert np.array_equal(a, b)


def test_empty_graph_and_empty_shards():
    rp = np.zeros(5, np.int32)
    col = np.zeros(0, np.int32)
    x = np.ones((4, 16), np.float32)
    assert np.array_equal(emulated_aggregate(rp, col, x, 1), np.zeros((4, 16), np.float32))
    # more PEs than nodes: trailing PEs own nothing
    rp, col = random_graph(3, 2, seed=0)
    x = np.random.default_rng(0).uniform(-1, 1, (3, 16)).astype(np.float32)
    got = emulated_aggregate(rp, col, x, 8)
    want = np.zeros_like(x)
    for i in range(3):
        for e in range(rp[i], rp[i + 1]):
            want[i] += x[col[e]]
    np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL)


def test_errors_reported_not_fatal():
    dev = torch.device("cuda")
    rp, col = random_graph(8, 2, seed=0)
    sh = drivers.Shard(rp, col, 0, 1, device=dev)
    x = torch.zeros(8, 16, device=dev)
    o = torch.zeros(8, 16, device=dev)
    with pytest.raises(mgg.MggbError):
        sh.aggregate(o, x, 16, drivers.Knobs(16, 64, 1))
    with pytest.raises(mgg.MggbError):
        sh.aggregate_gin(x, x, 16, drivers.Knobs(), 0.0)      # output aliases the input
    with pytest.raises(ValueError):
        sh.aggregate(o.cpu(), x, 16, drivers.Knobs())
    sh.aggregate(o, x, 16, drivers.Knobs())                    # the context is still usable
    torch.cuda.synchronize()


def test_full_size_config2_properties():
    """At the benchmark's full size (232,965 nodes, ~114.6 M edges, dim 16): all-ones input gives the
    exact degree in every column, and the aggregation is linear (A(2x) = 2 A(x) bit for bit)."""
    dev = torch.device("cuda")
    g = gg.config2_graph(device=dev)
    assert g.num_nodes == 232_965 and abs(g.num_edges - 114.6e6) / 114.6e6 < 0.02
    sh = drivers.Shard(g.row_ptr.cpu().numpy(), g.col_idx.cpu().numpy(), 0, 1, device=dev)
    deg = (g.row_ptr[1:] - g.row_ptr[:-1]).to(torch.float32)
    ones = torch.ones(g.num_nodes, 16, device=dev)
    out = torch.empty_like(ones)
    sh.aggregate(out, ones, 16, drivers.Knobs(32, 4, 1))
    assert torch.equal(out, deg[:, None].expand(-1, 16))
    assert int(out[:, 0].double().sum().item()) == g.num_edges
    x = gg.features(g.num_nodes, 16, seed=1, device=dev)
    a, b = torch.empty_like(x), torch.empty_like(x)
    sh.aggregate(a, x, 16, drivers.Knobs(32, 4, 1))
    sh.aggregate(b, x * 2, 16, drivers.Knobs(32, 4, 1))
    assert torch.equal(b, a * 2)
    # spot rows against a float64 gather done with torch indexing (hub, median and tail rows)
    order = torch.argsort(deg)
    for r in [int(order[-1]), int(order[len(order) // 2]), int(order[0])]:
        nb = g.col_idx[g.row_ptr[r]:g.row_ptr[r + 1]].long()
        want = x[nb].double().sum(0)
        torch.testing.assert_close(a[r].double(), want, rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("G", [1, 2])
def test_hub_rows_every_epilogue(oracle, G):
    """Rows above the hub threshold take the wide-block path; every epilogue must agree with the
    one-block-per-node path (flag MGGB_AGG_NO_HUB_SPLIT) and with the oracle."""
    from mgg_osdi23_b200 import _lib
    n, dim = 400, 16
    rp, col = random_graph(n, 10, seed=11, hubs=[(0, 40000), (7, 16385), (150, 16384), (399, 20000), (398, 1025)])
    # small magnitudes: a 40,000-term fp32 sum of O(1) values is only good to ~1e-3 absolute
    x = np.random.default_rng(3).uniform(-0.02, 0.02, (n, dim)).astype(np.float32)
    want = oracle.sag_f64(x, rp, col)
    scale = np.random.default_rng(4).uniform(0.5, 1.5, n).astype(np.float32)
    np.testing.assert_allclose(emulated_aggregate(rp, col, x, G, knobs=(16, 2, 1)), want, rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(emulated_aggregate(rp, col, x, G, knobs=(16, 2, 1), row_scale=scale), want * scale[:, None], rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(emulated_aggregate(rp, col, x, G, knobs=(16, 2, 1), gin_eps=0.25), want + 1.25 * x, rtol=RTOL, atol=ATOL)
    init = np.random.default_rng(5).uniform(-1, 1, (n, dim)).astype(np.float32)
    np.testing.assert_allclose(emulated_aggregate(rp, col, x, G, knobs=(16, 2, 1), accumulate=True, init=init), want + init, rtol=RTOL, atol=ATOL)
    # the flag that keeps every node on its own block gives the same sums, and publish reaches hub rows too
    dev = torch.device("cuda")
    sh = drivers.Shard(rp, col, 0, 1, device=dev)
    xd = torch.from_numpy(x).to(dev)
    a, b, pub = (torch.zeros(n, dim, device=dev) for _ in range(3))
    mgg.mgg_SAG_np_div(a, xd, sh.rp_l, sh.ci_l, sh.rp_r, sh.ci_r, 0, n, dim, n, 0, 16, 2, 1, accumulate=False, publish=[pub])
    import ctypes as C
    table = (C.c_void_p * 1)(xd.data_ptr())
    _lib.check(_lib.lib.mggb_sag_np_div(b.data_ptr(), table, 1, sh.rp_l.data_ptr(), sh.ci_l.data_ptr(), sh.rp_r.data_ptr(),
                                        sh.ci_r.data_ptr(), 0, n, dim, n, 0, 16, 2, 1, None, 2, None, 0, None))
    torch.cuda.synchronize()
    np.testing.assert_allclose(a.cpu().numpy(), want, rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(b.cpu().numpy(), want, rtol=RTOL, atol=ATOL)
    assert torch.equal(a, pub)


@pytest.mark.parametrize("dim,G,knobs", [(16, 1, (16, 2, 1)), (16, 3, (32, 1, 1)), (64, 2, (16, 1, 2)), (7, 2, (8, 4, 1)), (128, 1, (16, 4, 2))])
def test_giant_rows_are_cut_into_segments(oracle, dim, G, knobs):
    """Rows above 16384 neighbors are summed segment by segment by several blocks (up to 64 segments per
    row); the sums agree with the oracle for every epilogue and are the same bits on every call and for
    every order in which the blocks take the rows."""
    n = 900
    hubs = [(0, 300_000), (1, 64 * 4096 + 1), (450, 16385), (451, 16384), (899, 70_000), (5, 20_000), (6, 0)]
    rp, col = random_graph(n, 12, seed=41, hubs=hubs)
    x = np.random.default_rng(13).uniform(-0.005, 0.005, (n, dim)).astype(np.float32)
    want = oracle.sag_f64(x, rp, col)
    got = emulated_aggregate(rp, col, x, G, knobs=knobs)
    np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL)
    scale = np.random.default_rng(14).uniform(0.5, 1.5, n).astype(np.float32)
    np.testing.assert_allclose(emulated_aggregate(rp, col, x, G, knobs=knobs, row_scale=scale), want * scale[:, None], rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(emulated_aggregate(rp, col, x, G, knobs=knobs, gin_eps=0.5), want + 1.5 * x, rtol=RTOL, atol=ATOL)
    init = np.random.default_rng(15).uniform(-1, 1, (n, dim)).astype(np.float32)
    np.testing.assert_allclose(emulated_aggregate(rp, col, x, G, knobs=knobs, accumulate=True, init=init), want + init, rtol=RTOL, atol=ATOL)
    assert np.array_equal(got, emulated_aggregate(rp, col, x, G, knobs=knobs))
    # another block order, a publish destination, and the group-per-node kernel's hand-over (dim 16)
    dev = torch.device("cuda")
    sh = drivers.Shard(rp, col, 0, 1, device=dev, order_rows=True)
    xd = torch.from_numpy(x).to(dev)
    a, b, pub = (torch.zeros(n, dim, device=dev) for _ in range(3))
    sh.aggregate(a, xd, dim, drivers.Knobs(*knobs))
    sh.row_order = torch.from_numpy(np.random.default_rng(16).permutation(n).astype(np.int32)).to(dev)
    sh.aggregate(b, xd, dim, drivers.Knobs(*knobs), publish=[pub])
    torch.cuda.synchronize()
    assert torch.equal(a, b) and torch.equal(b, pub)
    if G == 1:
        assert np.array_equal(a.cpu().numpy(), got)
    if dim == 16:
        from mgg_osdi23_b200 import _lib
        np.testing.assert_allclose(emulated_aggregate(rp, col, x, G, knobs=knobs, flags=_lib.AGG_GROUP_PER_NODE), want, rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("dim,knobs,flags", [(16, (32, 4, 2), 0), (16, (16, 1, 1), 4), (64, (16, 1, 2), 0), (7, (8, 2, 1), 0)])
def test_no_remote_flag_runs_the_single_pe_kernel_on_merged_lists(oracle, dim, knobs, flags):
    """MGGB_AGG_NO_REMOTE (what a shard passes when it gathers from a replica through merged lists): the remote
    lists are not read, and the sums are the bits of the call without the flag, for SAG and GIN, hub rows included."""
    from mgg_osdi23_b200 import _lib
    n, G, pe = 3000, 3, 1
    rp, col = random_graph(n, 25, seed=61, hubs=[(1000, 40_000), (1500, 17_000), (1999, 1500)])
    x = np.random.default_rng(62).uniform(-0.02, 0.02, (n, dim)).astype(np.float32)
    dev = torch.device("cuda")
    npp = (n + G - 1) // G
    reps = drivers.local_replicas(G, npp, dim, dev)
    for r in reps:
        r.tensor[: n * dim].copy_(torch.from_numpy(x).to(dev).reshape(-1))
    sh = drivers.Shard(rp, col, pe, G, device=dev)
    kn = drivers.Knobs(*knobs, flags=flags)
    lists = sh.merged_lists()
    assert sh._lists_for(reps[pe]) is lists and sh._flags_for(lists, kn, dim) & _lib.AGG_NO_REMOTE
    want = oracle.sag_f64(x, rp, col)[sh.lb:sh.ub]
    a, b = torch.zeros(sh.rows, dim, device=dev), torch.zeros(sh.rows, dim, device=dev)
    sh.aggregate(a, reps[pe], dim, kn)                                               # with the flag
    mgg.mgg_SAG_np_div(b, reps[pe], *lists, sh.lb, sh.ub, dim, sh.node_per_pe, pe, *knobs,
                       accumulate=False, row_order=sh.row_order, flags=sh.agg_flags(kn, dim))   # without it
    torch.cuda.synchronize()
    np.testing.assert_allclose(a.cpu().numpy(), want, rtol=RTOL, atol=ATOL)
    assert torch.equal(a, b)
    sh.aggregate_gin(a, reps[pe], dim, kn, 0.5)
    mgg.mgg_GIN_np_div(b, reps[pe], *lists, sh.lb, sh.ub, dim, sh.node_per_pe, pe, *knobs, 0.5,
                       row_order=sh.row_order, flags=sh.agg_flags(kn, dim))
    torch.cuda.synchronize()
    np.testing.assert_allclose(a.cpu().numpy(), want + 1.5 * x[sh.lb:sh.ub], rtol=RTOL, atol=ATOL)
    assert torch.equal(a, b)


def test_row_order_changes_schedule_not_results():
    """Blocks taking rows longest-first (or in any permutation) give bit-identical sums."""
    dev = torch.device("cuda")
    rp, col = random_graph(700, 25, seed=13, hubs=[(650, 6000), (3, 900)])
    x = torch.from_numpy(np.random.default_rng(2).uniform(-1, 1, (700, 16)).astype(np.float32)).to(dev)
    plain = drivers.Shard(rp, col, 0, 1, device=dev, order_rows=False)
    ordered = drivers.Shard(rp, col, 0, 1, device=dev, order_rows=True)
    assert plain.row_order is None and ordered.row_order[0].item() == 650
    a, b, c = (torch.zeros(700, 16, device=dev) for _ in range(3))
    plain.aggregate(a, x, 16, drivers.Knobs())
    ordered.aggregate(b, x, 16, drivers.Knobs())
    ordered.row_order = torch.from_numpy(np.random.default_rng(5).permutation(700).astype(np.int32)).to(dev)
    ordered.aggregate_gin(c, x, 16, drivers.Knobs(), 0.0)
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    torch.testing.assert_close(c, a + x, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("G", [1, 2, 3])
def test_group_per_node_kernel(oracle, G):
    """MGGB_AGG_GROUP_PER_NODE (dim 16): four lanes per node, eight nodes per warp; every epilogue,
    local and remote lists, empty nodes, nodes above its 1024-neighbor hub threshold."""
    from mgg_osdi23_b200 import _lib
    n, dim = 1000, 16
    rp, col = random_graph(n, 9, seed=31, hubs=[(0, 1500), (5, 1024), (6, 1025), (500, 3000), (999, 40), (998, 0), (2, 0)])
    x = np.random.default_rng(6).uniform(-0.1, 0.1, (n, dim)).astype(np.float32)
    want = oracle.sag_f64(x, rp, col)
    knobs = (16, 1, 1)
    flag = _lib.AGG_GROUP_PER_NODE

    def run(**kw):
        import gpu_util
        return gpu_util.emulated_aggregate(rp, col, x, G, knobs=knobs, flags=flag, **kw)

    np.testing.assert_allclose(run(), want, rtol=RTOL, atol=ATOL)
    scale = np.random.default_rng(7).uniform(0.5, 1.5, n).astype(np.float32)
    np.testing.assert_allclose(run(row_scale=scale), want * scale[:, None], rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(run(gin_eps=0.5), want + 1.5 * x, rtol=RTOL, atol=ATOL)
    init = np.random.default_rng(8).uniform(-1, 1, (n, dim)).astype(np.float32)
    np.testing.assert_allclose(run(accumulate=True, init=init), want + init, rtol=RTOL, atol=ATOL)
    # other widths ignore the flag and still give the right sums
    x8 = np.ascontiguousarray(x[:, :8])
    import gpu_util
    np.testing.assert_allclose(gpu_util.emulated_aggregate(rp, col, x8, G, knobs=knobs, flags=flag), oracle.sag_f64(x8, rp, col), rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("dim,knobs,flags", [(16, (16, 2, 2), 0), (16, (32, 1, 1), 4), (64, (16, 1, 2), 0), (7, (4, 4, 1), 0)])
def test_row_list_calls_cover_the_shard(dim, knobs, flags):
    """Aggregating a shard in three row-list calls gives the bits of one whole-shard call (SAG and GIN)."""
    from mgg_osdi23_b200 import drivers
    g = gg.chung_lu_graph(3000, 60_000, 2.2, seed=11)
    rp, col = g.row_ptr.numpy().astype(np.int32), g.col_idx.numpy()
    dev = torch.device("cuda")
    G, pe = 2, 1
    sh = drivers.Shard(rp, col, pe, G, device=dev)
    npp = sh.node_per_pe
    x = gg.features(G * npp, dim, seed=5, device=dev)
    table = [x[p * npp:(p + 1) * npp] for p in range(G)]
    kn = drivers.Knobs(*knobs, flags)
    whole = torch.zeros(sh.rows, dim, device=dev)
    sh.aggregate(whole, table, dim, kn)
    parts = torch.full((sh.rows, dim), 7.0, device=dev)
    blocks = sh.row_blocks(3)
    assert blocks[0][0] == 0 and blocks[-1][1] == sh.rows and sum(b[2].numel() for b in blocks) == sh.rows
    for r0, r1, rows in blocks:
        assert int(rows.min()) >= r0 and int(rows.max()) < r1
        sh.aggregate(parts, table, dim, kn, rows=rows)
    assert torch.equal(whole, parts)
    gin_whole = torch.zeros(sh.rows, dim, device=dev)
    gin_parts = torch.zeros(sh.rows, dim, device=dev)
    sh.aggregate_gin(gin_whole, table, dim, kn, 0.25)
    for _, _, rows in blocks:
        sh.aggregate_gin(gin_parts, table, dim, kn, 0.25, rows=rows)
    assert torch.equal(gin_whole, gin_parts)
    # an empty list is a no-op; a list longer than the shard is refused
    sh.aggregate(parts, table, dim, kn, rows=torch.zeros(0, dtype=torch.int32, device=dev))
    assert torch.equal(whole, parts)
    with pytest.raises(mgg.MggbError):
        sh.aggregate(parts, table, dim, kn, rows=torch.zeros(sh.rows + 1, dtype=torch.int32, device=dev))


def test_publish_rows_copies_to_every_destination():
    dev = torch.device("cuda")
    for count in (4096 * 16, 1001):
        src = gg.features(count, 1, seed=2, device=dev).reshape(-1)
        dst = [torch.zeros(count + 8, device=dev) for _ in range(3)]
        mgg.publish_rows(src, dst, elem_offset=4)
        for d in dst:
            assert torch.equal(d[4:4 + count], src) and float(d[:4].abs().sum()) == 0 and float(d[-4:].abs().sum()) == 0
    with pytest.raises(mgg.MggbError):
        mgg.publish_rows(src, [src])


@pytest.mark.parametrize("dim", [4, 8, 16, 32, 64, 128])
@pytest.mark.parametrize("G", [1, 2, 3])
def test_rows_staged_through_shared_memory_match_the_oracle(oracle, dim, G):
    """Rows brought in by bulk copies (AGG_STAGE_ROWS: the rows pulled from other PEs' buffers when there
    are peers, every row otherwise) against the register path and the fp64 oracle: short, long and
    empty lists, a hub row, chunk sizes below and above a 32-row batch, 1 to 8 warps."""
    import ctypes as C
    from mgg_osdi23_b200 import _lib
    rp, col = random_graph(700, 40, seed=10 * dim + G, hubs=[(5, 20000), (333, 3000), (7, 0), (699, 1)])
    x = np.random.default_rng(dim).uniform(-0.02, 0.02, (700, dim)).astype(np.float32)
    want = oracle.sag_f64(x, rp, col)
    for flags in (_lib.AGG_STAGE_ROWS, 0):
        for knobs in ((16, 4, 1), (3, 2, 2), (32, 1, 1), (8, 8, 4)):
            got = emulated_aggregate(rp, col, x, G, knobs, flags=flags)
            np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL, err_msg=f"flags={flags} knobs={knobs}")
    # the shared epilogue: GIN combine, accumulate and row scaling on the staged path
    got = emulated_aggregate(rp, col, x, G, (16, 4, 2), gin_eps=0.25, flags=_lib.AGG_STAGE_ROWS)
    np.testing.assert_allclose(got, want + 1.25 * x, rtol=RTOL, atol=ATOL)
    init = np.random.default_rng(1).uniform(-1, 1, x.shape).astype(np.float32)
    scale = np.random.default_rng(2).uniform(0.5, 1.5, 700).astype(np.float32)
    got = emulated_aggregate(rp, col, x, G, (16, 4, 2), accumulate=True, init=init, row_scale=scale, flags=_lib.AGG_STAGE_ROWS)
    np.testing.assert_allclose(got, want * scale[:, None] + init, rtol=RTOL, atol=ATOL)
    st = C.c_int(-1)
    _lib.check(_lib.lib.mggb_agg_device_status(C.byref(st), 0))
    assert st.value == 0


@pytest.mark.parametrize("G", [1, 2, 3])
@pytest.mark.parametrize("dim", [16, 64, 100, 7])
def test_explicit_partition_kernels_match_the_oracle(oracle, G, dim):
    """The warp-per-partition kernels over build_part's arrays (part_ptr / part2node / node2part of both
    halves): every part size and interleave distance gives the oracle's sums, bit-reproducibly, including
    a hub row that spans thousands of partitions, empty rows, and a last row with no edges (where the
    reference's build_part leaves the closing part_ptr entry at 0)."""
    rp, col = random_graph(500, 25, seed=3 * dim + G, hubs=[(5, 30000), (17, 0), (499, 0), (250, 1)])
    x = np.random.default_rng(dim).uniform(-0.02, 0.02, (500, dim)).astype(np.float32)
    want = oracle.sag_f64(x, rp, col)
    dev = torch.device("cuda")
    sym_np, npp = __import__("gpu_util").shard_inputs(x, G)
    sym = [torch.from_numpy(s_).to(dev) for s_ in sym_np]
    for ps, wpb, dist in ((16, 4, 1), (1, 2, 3), (32, 8, 16), (5, 1, 2)):
        got = np.zeros_like(want)
        again = np.zeros_like(want)
        for pe in range(G):
            sh = drivers.Shard(rp, col, pe, G, device=dev)
            if sh.rows == 0:
                continue
            for dst in (got, again):
                o = torch.full((sh.rows, dim), 3.0, device=dev)          # overwritten, not accumulated into
                sh.aggregate_parts(o, sym, dim, drivers.Knobs(ps, wpb, dist))
                dst[sh.lb:sh.ub] = o.cpu().numpy()
        np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL, err_msg=f"ps={ps} wpb={wpb} dist={dist}")
        assert np.array_equal(got, again)
    # epilogues: accumulate, row scale, GIN combine
    sh = drivers.Shard(rp, col, 0, 1, device=dev)
    xd = torch.from_numpy(x).to(dev)
    init = np.random.default_rng(1).uniform(-1, 1, x.shape).astype(np.float32)
    scale = np.random.default_rng(2).uniform(0.5, 1.5, 500).astype(np.float32)
    o = torch.from_numpy(init.copy()).to(dev)
    sh.aggregate_parts(o, xd, dim, drivers.Knobs(8, 4, 2), accumulate=True, row_scale_=torch.from_numpy(scale).to(dev))
    np.testing.assert_allclose(o.cpu().numpy(), want * scale[:, None] + init, rtol=RTOL, atol=ATOL)
    o = torch.zeros(500, dim, device=dev)
    sh.aggregate_parts(o, xd, dim, drivers.Knobs(8, 4, 2), gin_eps=0.5)
    np.testing.assert_allclose(o.cpu().numpy(), want + 1.5 * x, rtol=RTOL, atol=ATOL)


def test_explicit_partition_kernel_checks_its_scratch():
    from mgg_osdi23_b200 import _lib, api
    dev = torch.device("cuda")
    rp, col = random_graph(50, 5, seed=1)
    sh = drivers.Shard(rp, col, 0, 1, device=dev)
    x = torch.zeros(50, 16, device=dev)
    out = torch.zeros(50, 16, device=dev)
    small = torch.zeros(4, device=dev)
    with pytest.raises(_lib.MggbError) as e:
        sh.aggregate_parts(out, x, 16, drivers.Knobs(4, 4, 1), scratch=small)
    assert e.value.code == _lib.ERR_INVALID_ARG and "scratch" in str(e.value)
