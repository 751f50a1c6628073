"""2-layer GCN / 5-layer GIN forward passes (several PEs emulated on one device) against the oracle."""
import numpy as np
import pytest
import torch

import mgg_osdi23_b200 as mgg
from mgg_osdi23_b200 import drivers, graphgen as gg
from gpu_util import RTOL, ATOL

pytestmark = pytest.mark.gpu


def _oracle_gcn2(oracle, rp, col, x, w1, w2, norm):
    h = oracle.dense(x, w1)
    if norm == "sym":
        dinv = oracle.inv_sqrt_degree(rp)
        agg = lambda t: oracle.row_scale(oracle.sag_f64(oracle.row_scale(t, dinv), rp, col), dinv)
    else:
        agg = lambda t: oracle.sag_f64(t, rp, col)
    z = agg(agg(h))
    logits = oracle.dense(z, w2)
    return logits, oracle.softmax(logits)


def _run_cluster(make_model, G, n, x):
    models = [make_model(pe) for pe in range(G)]
    for m in models:
        m.d_in.copy_(torch.from_numpy(x[m.shard.lb:m.shard.ub]).to(m.d_in.device))
    drivers.run_stages(models)
    torch.cuda.synchronize()
    out = np.zeros((n, models[0].out.shape[1]), np.float32)
    logits = np.zeros_like(out)
    for m in models:
        out[m.shard.lb:m.shard.ub] = m.out.cpu().numpy()
        logits[m.shard.lb:m.shard.ub] = m.logits.cpu().numpy()
    return logits, out


def _published(G, npp, dim, dev, fetch):
    """Two publication buffers per PE: pulled-from symmetric shards, or pushed-into replicas."""
    if fetch == "replica":
        return drivers.local_replicas(G, npp, dim, dev), drivers.local_replicas(G, npp, dim, dev)
    return drivers.local_symmetric(G, npp * dim, dev), drivers.local_symmetric(G, npp * dim, dev)


@pytest.mark.parametrize("fetch", ["peer", "replica"])
@pytest.mark.parametrize("G", [1, 2, 4])
@pytest.mark.parametrize("norm", ["sym", "none"])
def test_gcn2_forward(oracle, G, norm, fetch):
    g = gg.chung_lu_graph(1500, 40_000, 2.1, seed=2, communities=4, p_intra=0.7)
    rp, col = g.row_ptr.numpy().astype(np.int32), g.col_idx.numpy()
    n, din, hid, dout = g.num_nodes, 602, 16, 41
    x = gg.features(n, din, seed=3).numpy()
    w1, w2 = gg.glorot_uniform(din, hid, 1), gg.glorot_uniform(hid, dout, 2)
    if norm == "none":
        w1 = w1 * 0.01          # keeps unnormalised sums of ~27^2 neighbors in a softmax-friendly range
    dev = torch.device("cuda")
    npp = (n + G - 1) // G
    sa, sb = _published(G, npp, hid, dev, fetch)

    def make(pe):
        sh = drivers.Shard(rp, col, pe, G, device=dev)
        return drivers.GCN2Forward(sh, din, hid, dout, sa[pe], sb[pe], drivers.Knobs(16, 4, 2),
                                   w1=w1.to(dev), w2=w2.to(dev), norm=norm)

    logits, probs = _run_cluster(make, G, n, x)
    want_logits, want_probs = _oracle_gcn2(oracle, rp, col, x, w1.numpy(), w2.numpy(), norm)
    np.testing.assert_allclose(logits, want_logits, rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(probs, want_probs, rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("fetch", ["peer", "replica"])
@pytest.mark.parametrize("G", [1, 3])
def test_gin5_forward(oracle, G, fetch):
    g = gg.chung_lu_graph(1200, 12_000, 2.3, seed=5)
    rp, col = g.row_ptr.numpy().astype(np.int32), g.col_idx.numpy()
    n, din, hid, dout, eps = g.num_nodes, 100, 64, 47, 0.0
    x = gg.features(n, din, seed=4).numpy()
    # scaled so that five unnormalised aggregations stay O(1)
    ws = [gg.glorot_uniform(din, hid, 10) * 0.1] + [gg.glorot_uniform(hid, hid, 11 + k) * 0.1 for k in range(4)] \
        + [gg.glorot_uniform(hid, dout, 20) * 0.1]
    dev = torch.device("cuda")
    npp = (n + G - 1) // G
    sa, sb = _published(G, npp, hid, dev, fetch)

    def make(pe):
        sh = drivers.Shard(rp, col, pe, G, device=dev)
        return drivers.GIN5Forward(sh, din, hid, dout, sa[pe], sb[pe], drivers.Knobs(8, 2, 2), eps=eps,
                                   weights=[w.to(dev) for w in ws])

    logits, probs = _run_cluster(make, G, n, x)
    h = oracle.dense(x, ws[0].numpy())
    for k in range(5):
        a = (oracle.sag_f64(h, rp, col).astype(np.float64) + (1 + eps) * h).astype(np.float32)
        h = oracle.dense(a, ws[k + 1].numpy())
    scale = max(1.0, float(np.abs(h).max()))
    np.testing.assert_allclose(logits / scale, h / scale, rtol=1e-4, atol=ATOL)   # 11 chained fp32 kernels
    np.testing.assert_allclose(probs, oracle.softmax(h), rtol=1e-3, atol=ATOL)


def test_forward_host_entry_point(oracle):
    """The host-buffer call: pinned features in, pinned probabilities out."""
    g = gg.rmat_graph(9, 4000, seed=7)
    rp, col = g.row_ptr.numpy().astype(np.int32), g.col_idx.numpy()
    n = g.num_nodes
    dev = torch.device("cuda")
    sa, sb = drivers.local_symmetric(1, n * 16, dev), drivers.local_symmetric(1, n * 16, dev)
    sh = drivers.Shard(rp, col, 0, 1, device=dev)
    w1, w2 = gg.glorot_uniform(32, 16, 1), gg.glorot_uniform(16, 8, 2)
    m = drivers.GCN2Forward(sh, 32, 16, 8, sa[0], sb[0], drivers.Knobs(), w1=w1.to(dev), w2=w2.to(dev), norm="sym")
    x = gg.features(n, 32, seed=1).pin_memory()
    probs = m.forward_host(x)
    assert probs.is_pinned() and not probs.is_cuda
    _, want = _oracle_gcn2(oracle, rp, col, x.numpy(), w1.numpy(), w2.numpy(), "sym")
    np.testing.assert_allclose(probs.numpy(), want, rtol=RTOL, atol=ATOL)


def test_single_aggregation_driver(oracle):
    g = gg.config4_graph(scale_shift=9)
    rp, col = g.row_ptr.numpy().astype(np.int32), g.col_idx.numpy()
    n = g.num_nodes
    dev = torch.device("cuda")
    x = gg.features(n, 16, seed=2).numpy()
    want = oracle.sag_f64(x, rp, col)
    for G in (1, 4):
        npp = (n + G - 1) // G
        syms = drivers.local_symmetric(G, npp * 16, dev)
        models = []
        for pe in range(G):
            sh = drivers.Shard(rp, col, pe, G, device=dev)
            m = drivers.SingleAggregation(sh, 16, syms[pe], drivers.Knobs(4, 8, 4))
            m.d_in.copy_(torch.from_numpy(x[sh.lb:sh.ub]).to(dev))
            models.append(m)
        drivers.run_stages(models)
        torch.cuda.synchronize()
        for m in models:
            np.testing.assert_allclose(m.out.cpu().numpy(), want[m.shard.lb:m.shard.ub], rtol=RTOL, atol=ATOL)


def test_symmetric_buffer_single_pe():
    """The library-allocated symmetric buffer viewed as a torch tensor, used as aggregation input."""
    from mgg_osdi23_b200.symmem import SymmetricBuffer
    dev = torch.device("cuda")
    s = SymmetricBuffer(64 * 16)
    assert s.tensor.is_cuda and s.tensor.numel() == 64 * 16 and s.tensor.data_ptr() == s.ptr
    assert float(s.tensor.abs().sum()) == 0.0            # zero-filled like the reference's buffers
    s.view(64, 16).fill_(1.0)
    rp = np.arange(0, 65 * 3, 3, dtype=np.int32)
    col = (np.arange(64 * 3) % 64).astype(np.int32)
    sh = drivers.Shard(rp, col, 0, 1, device=dev)
    out = torch.zeros(64, 16, device=dev)
    sh.aggregate(out, s, 16, drivers.Knobs())
    torch.cuda.synchronize()
    assert torch.equal(out, torch.full_like(out, 3.0))
    s.close()


def test_forward_host_overlapped_upload(oracle):
    """Enough rows for the chunked path: row blocks are uploaded on a copy stream and multiplied as
    they arrive; the result must equal the plain path bit for bit, on repeated calls."""
    g = gg.chung_lu_graph(40_000, 400_000, 2.3, seed=9)
    rp, col = g.row_ptr.numpy().astype(np.int32), g.col_idx.numpy()
    n = g.num_nodes
    dev = torch.device("cuda")
    sa, sb = drivers.local_symmetric(1, n * 16, dev), drivers.local_symmetric(1, n * 16, dev)
    sh = drivers.Shard(rp, col, 0, 1, device=dev)
    w1, w2 = gg.glorot_uniform(100, 16, 1), gg.glorot_uniform(16, 8, 2)
    m = drivers.GCN2Forward(sh, 100, 16, 8, sa[0], sb[0], drivers.Knobs(), w1=w1.to(dev), w2=w2.to(dev), norm="sym")
    x = gg.features(n, 100, seed=1).pin_memory()
    plain = m.forward_host(x, chunks=1).clone()
    for _ in range(3):
        chunked = m.forward_host(x, chunks=4)
        assert torch.equal(chunked, plain)
    _, want = _oracle_gcn2(oracle, rp, col, x.numpy(), w1.numpy(), w2.numpy(), "sym")
    np.testing.assert_allclose(plain.numpy(), want, rtol=RTOL, atol=ATOL)


def _force_overlap(m):
    """Cut every pushed aggregation into row blocks with the consumer on the second stream, whatever the size."""
    m.overlap_blocks, m.overlap_min_rows, m.EPILOGUE_PUSH_MAX_BYTES = 3, 1, 0
    return m


def test_overlapped_pushes_give_the_same_forward_pass(oracle):
    """Push mode with the aggregation cut into row blocks (block b pushed while block b+1 is gathered)
    matches the oracle and, bit for bit, the single-launch schedule."""
    dev = torch.device("cuda")
    G = 3
    # GCN-2
    g = gg.chung_lu_graph(1500, 40_000, 2.1, seed=2, communities=4, p_intra=0.7)
    rp, col = g.row_ptr.numpy().astype(np.int32), g.col_idx.numpy()
    n, din, hid, dout = g.num_nodes, 602, 16, 41
    x = gg.features(n, din, seed=3).numpy()
    w1, w2 = gg.glorot_uniform(din, hid, 1), gg.glorot_uniform(hid, dout, 2)
    npp = (n + G - 1) // G
    results = []
    for overlap in (False, True):
        sa, sb = _published(G, npp, hid, dev, "replica")

        def make(pe):
            sh = drivers.Shard(rp, col, pe, G, device=dev)
            m = drivers.GCN2Forward(sh, din, hid, dout, sa[pe], sb[pe], drivers.Knobs(16, 4, 2),
                                    w1=w1.to(dev), w2=w2.to(dev), norm="sym")
            return _force_overlap(m) if overlap else m

        results.append(_run_cluster(make, G, n, x))
    assert np.array_equal(results[0][0], results[1][0]) and np.array_equal(results[0][1], results[1][1])
    want_logits, want_probs = _oracle_gcn2(oracle, rp, col, x, w1.numpy(), w2.numpy(), "sym")
    np.testing.assert_allclose(results[1][0], want_logits, rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(results[1][1], want_probs, rtol=RTOL, atol=ATOL)
    # GIN-5
    g = gg.chung_lu_graph(1200, 12_000, 2.3, seed=5)
    rp, col = g.row_ptr.numpy().astype(np.int32), g.col_idx.numpy()
    n, din, hid, dout = g.num_nodes, 100, 64, 47
    x = gg.features(n, din, seed=4).numpy()
    ws = [gg.glorot_uniform(din, hid, 10) * 0.1] + [gg.glorot_uniform(hid, hid, 11 + k) * 0.1 for k in range(4)] \
        + [gg.glorot_uniform(hid, dout, 20) * 0.1]
    npp = (n + G - 1) // G
    results = []
    for overlap in (False, True):
        sa, sb = _published(G, npp, hid, dev, "replica")

        def make(pe):
            sh = drivers.Shard(rp, col, pe, G, device=dev)
            m = drivers.GIN5Forward(sh, din, hid, dout, sa[pe], sb[pe], drivers.Knobs(8, 2, 2), eps=0.0,
                                    weights=[w.to(dev) for w in ws])
            return _force_overlap(m) if overlap else m

        results.append(_run_cluster(make, G, n, x))
    assert np.array_equal(results[0][0], results[1][0]) and np.array_equal(results[0][1], results[1][1])


def test_single_aggregation_in_push_mode(oracle):
    g = gg.config4_graph(scale_shift=9)
    rp, col = g.row_ptr.numpy().astype(np.int32), g.col_idx.numpy()
    n, dim, G = g.num_nodes, 16, 4
    x = gg.features(n, dim, seed=8).numpy()
    dev = torch.device("cuda")
    npp = (n + G - 1) // G
    reps = drivers.local_replicas(G, npp, dim, dev)
    models = [drivers.SingleAggregation(drivers.Shard(rp, col, pe, G, device=dev), dim, reps[pe],
                                        drivers.Knobs(32, 1, 1, mgg._lib.AGG_GROUP_PER_NODE)) for pe in range(G)]
    assert len(models[0].stages) == 2
    for m in models:
        m.d_in.copy_(torch.from_numpy(x[m.shard.lb:m.shard.ub]).to(dev))
    drivers.run_stages(models)
    torch.cuda.synchronize()
    got = np.concatenate([m.out.cpu().numpy() for m in models])
    np.testing.assert_allclose(got, oracle.sag_f64(x, rp, col), rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("fetch", ["peer", "replica"])
def test_back_to_back_passes_never_overwrite_what_a_slow_peer_still_reads(oracle, fetch):
    """Two passes with DIFFERENT inputs, the PEs run in the worst order a barrier-separated schedule
    allows: PE 0 finishes pass 1 and runs the first stage of pass 2 (which publishes into its peers'
    view) BEFORE PE 1 runs the last stage of pass 1.  PE 1's pass-1 result must still be the oracle's:
    the first stage of a pass may not write the buffer the last stage reads.  The 5-layer GIN needs its
    third published buffer for that; without one the model asks for a barrier at the start of a pass."""
    g = gg.chung_lu_graph(1200, 12_000, 2.3, seed=5)
    rp, col = g.row_ptr.numpy().astype(np.int32), g.col_idx.numpy()
    n, din, hid, dout, G = g.num_nodes, 100, 64, 47, 2
    xs = [gg.features(n, din, seed=4).numpy(), gg.features(n, din, seed=44).numpy()]
    ws = [gg.glorot_uniform(din, hid, 10) * 0.1] + [gg.glorot_uniform(hid, hid, 11 + k) * 0.1 for k in range(4)] \
        + [gg.glorot_uniform(hid, dout, 20) * 0.1]
    dev = torch.device("cuda")
    npp = (n + G - 1) // G
    sa, sb = _published(G, npp, hid, dev, fetch)
    sc, _ = _published(G, npp, hid, dev, fetch)

    def want(x):
        h = oracle.dense(x, ws[0].numpy())
        for k in range(5):
            h = oracle.dense((oracle.sag_f64(h, rp, col).astype(np.float64) + h).astype(np.float32), ws[k + 1].numpy())
        return h

    models = [drivers.GIN5Forward(drivers.Shard(rp, col, pe, G, device=dev), din, hid, dout, sa[pe], sb[pe],
                                  drivers.Knobs(8, 2, 2), eps=0.0, weights=[w.to(dev) for w in ws], sym_c=sc[pe]) for pe in range(G)]
    assert not any(m.leading_barrier for m in models)
    for m in models:
        m.keep_logits = True
    load = lambda m, x: m.d_in.copy_(torch.from_numpy(x[m.shard.lb:m.shard.ub]).to(dev))
    last = len(models[0].stages) - 1
    for m in models:
        load(m, xs[0])
    for s in range(last):                       # pass 1 up to the last barrier
        for m in models:
            m.stages[s]()
    models[0].stages[last]()                    # PE 0 finishes pass 1 ...
    first = models[0].logits.clone()
    load(models[0], xs[1])
    models[0].stages[0]()                       # ... and starts pass 2 while PE 1 is still in pass 1
    models[1].stages[last]()
    torch.cuda.synchronize()
    h = want(xs[0])
    scale = max(1.0, float(np.abs(h).max()))
    got = np.concatenate([first.cpu().numpy(), models[1].logits.cpu().numpy()])
    np.testing.assert_allclose(got / scale, h / scale, rtol=1e-4, atol=ATOL)
    # without the third buffer the model says so instead of racing
    two = drivers.GIN5Forward(drivers.Shard(rp, col, 0, G, device=dev), din, hid, dout, sa[0], sb[0], drivers.Knobs(8, 2, 2))
    assert two.leading_barrier
    # a single aggregation that pushes starts its pass with a barrier too; the 2-layer GCN needs none
    reps = drivers.local_replicas(G, npp, 16, dev)
    assert drivers.SingleAggregation(drivers.Shard(rp, col, 0, G, device=dev), 16, reps[0], drivers.Knobs()).leading_barrier
    ga, gb = _published(G, npp, 16, dev, fetch)
    assert not drivers.GCN2Forward(drivers.Shard(rp, col, 0, G, device=dev), din, 16, dout, ga[0], gb[0], drivers.Knobs()).leading_barrier


@pytest.mark.parametrize("kind", ["gcn2", "gin5", "single"])
def test_captured_pass_replays_to_the_same_bits(oracle, kind):
    """A forward pass recorded as a CUDA graph: replaying it (with new inputs in the same buffers) gives exactly
    what launching the kernels one by one gives, replay after replay; rows above the hub threshold included
    (their work list is cleared by a memset node inside the graph)."""
    from gpu_util import random_graph
    n = 3000
    rp, col = random_graph(n, 20, seed=51, hubs=[(0, 40_000), (17, 17_000), (2999, 1500)])
    dev = torch.device("cuda")
    sh = drivers.Shard(rp, col, 0, 1, device=dev)
    din, hid, dout = 100, 16, 41
    sym = lambda d: drivers.LocalSym([torch.zeros(n * d, device=dev)], 0)
    if kind == "gcn2":
        m = drivers.GCN2Forward(sh, din, hid, dout, sym(hid), sym(hid), drivers.Knobs(16, 2, 1),
                                w1=(gg.glorot_uniform(din, hid, 1) * 0.01).to(dev), w2=gg.glorot_uniform(hid, dout, 2).to(dev))
    elif kind == "gin5":
        ws = [gg.glorot_uniform(din, 64, 10) * 0.01] + [gg.glorot_uniform(64, 64, 11 + k) * 0.01 for k in range(4)] + [gg.glorot_uniform(64, dout, 20)]
        m = drivers.GIN5Forward(sh, din, 64, dout, sym(64), sym(64), drivers.Knobs(16, 1, 2), eps=0.0, weights=[w.to(dev) for w in ws], sym_c=sym(64))
    else:
        m = drivers.SingleAggregation(sh, hid, sym(hid), drivers.Knobs(32, 1, 1, flags=4))
    inputs = [gg.features(n, m.d_in.shape[1], seed=s_, device=dev) * 0.05 for s_ in (3, 4)]
    eager = []
    for xi in inputs:
        m.d_in.copy_(xi)
        m.forward()
        eager.append(m.out.clone())
    kernels = m.capture()
    assert kernels >= 2
    for rnd in range(2):
        for xi, want in zip(inputs, eager):
            m.d_in.copy_(xi)
            m.out.fill_(-1.0)
            m.replay()
            torch.cuda.synchronize()
            assert torch.equal(m.out, want), (kind, rnd)
    assert not torch.equal(eager[0], eager[1])
