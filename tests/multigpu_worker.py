"""One rank of the real multi-GPU check (launched by torchrun from test_gpu_multiproc.py):
a GCN-2 forward and a single aggregation, each PE on its own GPU, remote rows read over peer
mappings of CUDA-IPC-shared symmetric buffers; every rank checks its shard against the CPU oracle."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from mgg_osdi23_b200 import drivers, graphgen as gg
    from mgg_osdi23_b200.symmem import SymmetricBuffer, ReplicaBuffer
    from oracle.oracle import Oracle
    orc = Oracle()

    g = gg.chung_lu_graph(6000, 300_000, 2.1, seed=1, communities=8, p_intra=0.6)
    rp, col = g.row_ptr.numpy().astype(np.int32), g.col_idx.numpy()
    n, din, hid, dout = g.num_nodes, 100, 16, 41
    x = gg.features(n, din, seed=3).numpy()
    w1, w2 = gg.glorot_uniform(din, hid, 1), gg.glorot_uniform(hid, dout, 2)
    sh = drivers.Shard(rp, col, rank, world, device=dev)
    assert world == 1 or sh.e_remote > 0
    nccl_barrier = drivers.nccl_stream_barrier()
    barrier = drivers.FlagBarrier(None, rank, world)       # epoch flags in peer memory: the two-sided wait on real peers
    xh = torch.from_numpy(x[sh.lb:sh.ub].copy()).pin_memory()
    dinv = orc.inv_sqrt_degree(rp)
    agg = lambda t: orc.row_scale(orc.sag_f64(orc.row_scale(t, dinv), rp, col), dinv)
    want = orc.softmax(orc.dense(agg(agg(orc.dense(x, w1.numpy()))), w2.numpy()))
    # pull mode (rows fetched from the owners inside the kernel), then push mode (replicas)
    sa = SymmetricBuffer(sh.node_per_pe * hid, None, rank, world)
    sb = SymmetricBuffer(sh.node_per_pe * hid, None, rank, world)
    ra = ReplicaBuffer(sh.node_per_pe, hid, None, rank, world)
    rb = ReplicaBuffer(sh.node_per_pe, hid, None, rank, world)
    for a, b in ((sa, sb), (ra, rb)):
        m = drivers.GCN2Forward(sh, din, hid, dout, a, b, drivers.Knobs(16, 4, 2), w1=w1.to(dev), w2=w2.to(dev), norm="sym")
        for _ in range(3):                   # repeated passes exercise the buffer alternation
            probs = m.forward_host(xh, barrier)
        np.testing.assert_allclose(probs.numpy(), want[sh.lb:sh.ub], rtol=1e-5, atol=1e-4)
        probs = m.forward_host(xh, nccl_barrier)                 # and once with the all-reduce barrier
        np.testing.assert_allclose(probs.numpy(), want[sh.lb:sh.ub], rtol=1e-5, atol=1e-4)
        # the same pass recorded as a CUDA graph (barriers included) and replayed: same bits as launched one by one
        m.d_in.copy_(xh.to(dev))
        m.forward(barrier)
        eager = m.out.clone()
        m.capture(barrier)
        for _ in range(3):
            m.out.zero_()
            m.replay()
        torch.cuda.synchronize()
        assert torch.equal(m.out, eager), "replayed pass differs"
        barrier()
    assert barrier.status() == 0, "a flag-barrier wait expired"

    # 5-layer GIN with the third published buffer: back-to-back passes with DIFFERENT inputs and no barrier
    # between passes; every pass must match the oracle for its own input
    ws = [gg.glorot_uniform(din, 64, 10) * 0.1] + [gg.glorot_uniform(64, 64, 11 + k) * 0.1 for k in range(4)] + [gg.glorot_uniform(64, dout, 20) * 0.1]
    for make in (lambda: SymmetricBuffer(sh.node_per_pe * 64, None, rank, world), lambda: ReplicaBuffer(sh.node_per_pe, 64, None, rank, world)):
        bufs = [make() for _ in range(3)]
        gin = drivers.GIN5Forward(sh, din, 64, dout, bufs[0], bufs[1], drivers.Knobs(8, 2, 2), eps=0.0, weights=[w.to(dev) for w in ws], sym_c=bufs[2])
        gin.keep_logits = True
        assert not gin.leading_barrier
        inputs = [x, gg.features(n, din, seed=33).numpy(), x]
        got = []
        for xi in inputs:
            gin.d_in.copy_(torch.from_numpy(xi[sh.lb:sh.ub].copy()).to(dev), non_blocking=True)
            gin.forward(barrier)
            got.append(gin.logits.clone())
        torch.cuda.synchronize()
        for xi, g_ in zip(inputs, got):
            h = orc.dense(xi, ws[0].numpy())
            for k in range(5):
                h = orc.dense((orc.sag_f64(h, rp, col).astype(np.float64) + h).astype(np.float32), ws[k + 1].numpy())
            scale = max(1.0, float(np.abs(h).max()))
            np.testing.assert_allclose(g_.cpu().numpy() / scale, h[sh.lb:sh.ub] / scale, rtol=1e-4, atol=1e-4)
        barrier()
        torch.cuda.synchronize(); dist.barrier()
        for b_ in bufs:
            b_.close()
    assert barrier.status() == 0, "a flag-barrier wait expired"

    # single aggregation, dim 64, GIN combine
    sc = SymmetricBuffer(sh.node_per_pe * 64, None, rank, world)
    x64 = gg.features(n, 64, seed=5).numpy()
    sc.view(sh.rows, 64).copy_(torch.from_numpy(x64[sh.lb:sh.ub]).to(dev))
    out = torch.zeros(sh.rows, 64, device=dev)
    barrier()
    sh.aggregate_gin(out, sc, 64, drivers.Knobs(8, 2, 1), 0.5)
    torch.cuda.synchronize()
    np.testing.assert_allclose(out.cpu().numpy(), (orc.sag_f64(x64, rp, col) + 1.5 * x64)[sh.lb:sh.ub], rtol=1e-5, atol=1e-4)

    dist.barrier()
    torch.cuda.synchronize()
    for s in (sa, sb, sc, ra, rb):
        s.close()
    barrier.close()
    dist.destroy_process_group()
    print(f"rank {rank}/{world} ok: local {sh.e_local} remote {sh.e_remote} edges")


if __name__ == "__main__":
    main()
