"""Host-side logic of the multi-PE path with two CPU ranks (gloo): shard coverage, the handle
exchange behind symmetric buffers, and stage/barrier ordering.  No GPU and no compute kernels."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import mgg_osdi23_b200 as mgg
        from mgg_osdi23_b200 import graphgen as gg, symmem, drivers
        from oracle.oracle import Oracle
        orc = Oracle()

        # every rank builds the same seeded graph and splits its own rows
        g = gg.rmat_graph(9, 6000, seed=4)
        rp, col = g.row_ptr.numpy().astype(np.int32), g.col_idx.numpy()
        npp, lb, ub = mgg.shard_range(g.num_nodes, world, rank)
        lp, rpp, lc, rc = mgg.split_CSR(rp, col, lb, ub)
        for u, v in zip((lp, rpp, lc, rc), orc.split_csr(rp, col, lb, ub)):
            assert np.array_equal(u, v)
        counts = torch.tensor([lc.size, rc.size, ub - lb], dtype=torch.int64)
        dist.all_reduce(counts)
        assert int(counts[0] + counts[1]) == g.num_edges and int(counts[2]) == g.num_nodes
        assert np.all((rc < lb) | (rc >= ub)) and np.all((lc >= lb) & (lc < ub))

        # the oracle's per-PE aggregation over exchanged shards equals the whole-graph result
        x = gg.features(g.num_nodes, 16, seed=2).numpy()
        mine = np.zeros((npp, 16), np.float32)
        mine[: ub - lb] = x[lb:ub]
        gathered = [torch.zeros(npp, 16) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(mine))
        got = orc.shard_aggregate([t.numpy() for t in gathered], rank, lp, lc, rpp, rc, lb, ub, npp)
        np.testing.assert_allclose(got, orc.sag_f64(x, rp, col)[lb:ub], rtol=1e-6, atol=1e-6)

        # handle exchange: index = PE, 64 opaque bytes each
        handles = symmem.exchange_handles(bytes([rank]) * 64, None, world)
        assert [h[0] for h in handles] == list(range(world)) and all(len(h) == 64 for h in handles)
        with pytest.raises(ValueError):
            symmem.exchange_handles(b"short", None, world)

        # stage ordering: a rank must see its peer's stage-s marker before it runs stage s+1
        class Model:
            def __init__(self):
                self.stages = [self._s(0), self._s(1), self._s(2)]
                self.seen = []

            def _s(self, k):
                def run():
                    if k > 0:
                        for r in range(world):
                            assert os.path.exists(os.path.join(tmp, f"s{k - 1}_r{r}")), f"stage {k} ran before peer {r} finished stage {k - 1}"
                    open(os.path.join(tmp, f"s{k}_r{rank}"), "w").close()
                    self.seen.append(k)
                return run

        m = Model()
        drivers.run_stages([m], barrier=dist.barrier)
        assert m.seen == [0, 1, 2]
    finally:
        dist.destroy_process_group()


def test_two_cpu_ranks(tmp_path):
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
