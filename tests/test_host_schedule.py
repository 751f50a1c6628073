"""Host-side logic of the block schedule and of push mode, on CPU tensors (no kernel is launched)."""
import numpy as np
import torch

import mgg_osdi23_b200 as mgg
from mgg_osdi23_b200 import drivers, graphgen as gg


def _graph():
    g = gg.chung_lu_graph(3000, 40_000, 2.2, seed=3)
    return g.row_ptr.numpy().astype(np.int32), g.col_idx.numpy()


def test_block_schedule_is_by_decreasing_degree_and_blocks_partition_it():
    rp, col = _graph()
    sh = drivers.Shard(rp, col, 1, 3, device="cpu")
    deg = (np.diff(sh.rp_l.numpy()) + np.diff(sh.rp_r.numpy()))
    order = sh.row_order.numpy()
    assert sorted(order.tolist()) == list(range(sh.rows))
    assert np.all(np.diff(deg[order]) <= 0)                       # longest rows first
    assert np.array_equal(order, mgg.degree_order(sh.rp_l.numpy(), sh.rp_r.numpy()))
    for count in (1, 2, 3, 7):
        blocks = sh.row_blocks(count)
        assert blocks[0][0] == 0 and blocks[-1][1] == sh.rows
        assert all(a[1] == b[0] for a, b in zip(blocks, blocks[1:]))          # contiguous ranges
        assert all(r0 % 128 == 0 for r0, _, _ in blocks)                      # whole dense tiles
        seen = np.concatenate([rows.numpy() for _, _, rows in blocks])
        assert sorted(seen.tolist()) == list(range(sh.rows))                  # every row exactly once
        for r0, r1, rows in blocks:
            ids = rows.numpy()
            assert ids.dtype == np.int32 and np.all((ids >= r0) & (ids < r1))
            assert np.all(np.diff(deg[ids]) <= 0)                             # each block keeps the order
    # in id order when the schedule is switched off
    plain = drivers.Shard(rp, col, 1, 3, device="cpu", order_rows=False)
    assert plain.row_order is None
    assert all(np.array_equal(rows.numpy(), np.arange(r0, r1)) for r0, r1, rows in plain.row_blocks(2))


def test_push_tables_rotate_and_cover_every_peer():
    G, npp, dim = 5, 40, 16
    reps = drivers.local_replicas(G, npp, dim, device="cpu")
    bases = [r.tensor.data_ptr() for r in reps]
    slot = npp * dim * 4
    for pe, r in enumerate(reps):
        # reading: slot p of the LOCAL copy; writing: the own slot of every PEER's copy
        assert r.peer_ptrs == [bases[pe] + p * slot for p in range(G)]
        assert r.publish == [bases[(pe + k) % G] + pe * slot for k in range(1, G)]
        assert r.own(7, dim).data_ptr() == bases[pe] + pe * slot
    # at every position of the tables the G PEs aim at G different receivers
    for k in range(G - 1):
        targets = {(reps[pe].publish[k] - pe * slot) for pe in range(G)}
        assert targets == set(bases)
    assert drivers.local_replicas(1, npp, dim, device="cpu")[0].publish is None


def test_models_choose_their_last_layer_and_launch_counts():
    rp, col = _graph()
    sh = drivers.Shard(rp, col, 0, 1, device="cpu")
    assert mgg.dense_softmax_fits(16, 41) and mgg.dense_softmax_fits(64, 47) and mgg.dense_softmax_fits(16, 172)
    assert not mgg.dense_softmax_fits(16, 257) and not mgg.dense_softmax_fits(1024, 172)
    sym = drivers.local_symmetric(1, sh.node_per_pe * 16, device="cpu")
    m = drivers.GCN2Forward(sh, 32, 16, 41, sym[0], sym[0], drivers.Knobs(16, 4, 2))
    assert m.kernels_per_forward == 6 and m.aggregations_per_forward == 2 and m.overlap_blocks == 1
    m = drivers.GCN2Forward(sh, 32, 16, 300, sym[0], sym[0], drivers.Knobs(16, 4, 2))
    assert m.kernels_per_forward == 7                               # dense and softmax stay two kernels
    one = drivers.SingleAggregation(sh, 16, sym[0], drivers.Knobs(16, 4, 2))
    assert len(one.stages) == 1 and one.kernels_per_forward == 2
    reps = drivers.local_replicas(2, (3000 + 1) // 2, 16, device="cpu")
    two = drivers.SingleAggregation(drivers.Shard(rp, col, 0, 2, device="cpu"), 16, reps[0], drivers.Knobs(16, 4, 2))
    assert len(two.stages) == 2 and two.kernels_per_forward == 3   # push, aggregation, hub rows


def test_row_of_flat_index_trick_of_the_dense_epilogue_is_exact():
    """dense_tc's staged epilogue finds the row of flat element i of a 32-row block of width M as
    int((float(i) + 0.5f) * (1.0f / M)).  Brute force in float32 over every width the kernel takes."""
    for m in range(1, 257):
        inv = np.float32(1.0) / np.float32(m)
        i = np.arange(32 * m, dtype=np.int64)
        r = ((i.astype(np.float32) + np.float32(0.5)) * inv).astype(np.int32)
        assert np.array_equal(r, i // m), m


def test_leading_barrier_is_issued_before_stage_zero():
    """run_stages calls the barrier once more, first, for a model that asks for it (host logic only)."""
    calls = []

    class M:
        leading_barrier = True
        stages = [lambda: calls.append("s0"), lambda: calls.append("s1")]

    drivers.run_stages([M()], barrier=lambda: calls.append("b"))
    assert calls == ["b", "s0", "b", "s1"]
    del calls[:]
    M.leading_barrier = False
    drivers.run_stages([M()], barrier=lambda: calls.append("b"))
    assert calls == ["s0", "b", "s1"]


def test_merged_lists_are_the_shard_rows_of_the_unsplit_graph():
    """What a PE gathers from a replica: each row's whole stored list as the "local" half, nothing in the
    "remote" half; the same arrays whether the shard was built from the whole graph or from its own rows."""
    rp, col = _graph()
    for pe in range(3):
        sh = drivers.Shard(rp, col, pe, 3, device="cpu")
        m = sh.merged_lists()
        assert np.array_equal(m[0].numpy(), rp[sh.lb:sh.ub + 1] - rp[sh.lb])
        assert np.array_equal(m[1].numpy(), col[rp[sh.lb]:rp[sh.ub]])
        assert m[2].numel() == sh.rows + 1 and int(m[2].abs().sum()) == 0
        local = drivers.Shard((rp[sh.lb:sh.ub + 1] - rp[sh.lb]).astype(np.int64), col[rp[sh.lb]:rp[sh.ub]], pe, 3, device="cpu",
                              num_nodes=len(rp) - 1, shard_local=True)
        assert all(torch.equal(a, b) for a, b in zip(m, local.merged_lists()))
        # only a replica (it has slots) gets them; a pulled symmetric buffer keeps the split lists
        rep = type("R", (), {"slot_elems": 4})()
        assert sh._lists_for(rep)[0] is m[0] and sh._lists_for(object())[0] is sh.rp_l
