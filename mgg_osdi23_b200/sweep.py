"""Design-space sweep of the single aggregation over partSize x warpPerBlock x interleaved_dist.

What the reference does with ``5_MGG_DSE_4GPU.py`` / ``5_MGG_DSE_8GPU.py`` (which run
``build/MGG_np_div_kernel`` once per point and scrape ``MPI time (ms)``) and
``extract_search_dist_ps.py`` / ``extract_search_dist_wpb.py`` (which arrange the times into the
dist x ps and dist x wpb tables of its README): here one process per GPU builds the graph once and
times every point in-process with CUDA events (max over ranks).

    python -m mgg_osdi23_b200.sweep --config cfg4                      # one GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        --master-port 29500 -m mgg_osdi23_b200.sweep --config cfg4 --csv sweep_8gpu.csv

Prints the full product as CSV rows ``ps,wpb,dist,ms`` (to --csv, or stdout) and the two 2-D slices
the reference tabulates (dist x ps at wpb=4; dist x wpb at ps=16).
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

from . import _lib, drivers, graphgen as gg
from .symmem import ReplicaBuffer, SymmetricBuffer

PS = (1, 2, 4, 8, 16, 32)
WPB = (1, 2, 4, 8, 16)
DIST = (1, 2, 4, 8, 16)


def _graph(name: str, device, scale: float):
    if name == "cfg1":
        return gg.config1_graph(device=device)
    if name == "cfg2":
        return gg.config2_graph(device=device, scale=scale)
    if name == "cfg3":
        return gg.config3_graph(device=device, scale=scale)
    shift = 0
    while scale < 1.0 and (1 << shift) * scale < 1.0:
        shift += 1
    return gg.config4_graph(device=device, scale_shift=shift)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", default="cfg4", choices=["cfg1", "cfg2", "cfg3", "cfg4"])
    ap.add_argument("--dim", type=int, default=16, help="aggregated width (the reference sweeps at hidden = 16)")
    ap.add_argument("--scale", type=float, default=1.0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--csv", default=None)
    ap.add_argument("--fetch", default="peer", choices=["peer", "replica"],
                    help="peer: remote rows are read from the owners' memory inside the kernel (the reference's scheme); "
                         "replica: every PE holds a copy of the whole matrix and the kernel reads local memory only")
    ap.add_argument("--kernel", default="node", choices=["node", "part"],
                    help="node: the block-per-node kernels (mggb_sag_np_div); part: the warp-per-partition kernels over "
                         "build_part's arrays (mggb_sag_np_part), whose grid grows with the number of partitions")
    ap.add_argument("--group-per-node", action="store_true",
                    help="also time the 4-lanes-per-node kernel (width 16 only; it ignores the three knobs)")
    args = ap.parse_args(argv)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("the sweep needs a CUDA device")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist_ = None
    if world > 1:
        import torch.distributed as dist_
        dist_.init_process_group("nccl", device_id=dev)

    g = _graph(args.config, dev, args.scale)
    shard = drivers.Shard(g.row_ptr.cpu().numpy(), g.col_idx.cpu().numpy(), rank, world, device=dev)
    edges, nodes = g.num_edges, g.num_nodes
    del g
    if args.fetch == "replica" and world > 1:
        # every PE fills its whole copy (the features depend only on seed, row and column)
        sym = ReplicaBuffer(shard.node_per_pe, args.dim, None, rank, world)
        for p in range(world):
            lo = min(nodes, p * shard.node_per_pe)
            hi = min(nodes, lo + shard.node_per_pe)
            if hi > lo:
                sym.tensor[p * sym.slot_elems: p * sym.slot_elems + (hi - lo) * args.dim].view(hi - lo, args.dim).copy_(
                    gg.features(hi - lo, args.dim, 1, device=dev, first_row=lo))
    else:
        sym = SymmetricBuffer(shard.node_per_pe * args.dim, None, rank, world)
        sym.view(shard.rows, args.dim).copy_(gg.features(shard.rows, args.dim, 1, device=dev, first_row=shard.lb))
    out = torch.zeros(max(shard.rows, 1), args.dim, device=dev)[: shard.rows]

    def sync():
        torch.cuda.synchronize()
        if world > 1:
            dist_.barrier()
            torch.cuda.synchronize()

    scratch = [None]

    def run_once(k):
        if not shard.rows:
            return
        if args.kernel == "part" and not (k.flags & _lib.AGG_GROUP_PER_NODE):
            scratch[0] = shard.aggregate_parts(out, sym, args.dim, k, scratch=scratch[0])
            if scratch[0].numel() * 4 > (8 << 30):       # part_size 1 on a large graph: do not keep 8 GB around
                scratch[0] = None
        else:
            shard.aggregate(out, sym, args.dim, k)

    def time_point(ps, wpb, dist, flags=0):
        k = drivers.Knobs(ps, wpb, dist, flags)
        scratch[0] = None
        for _ in range(args.warmup):
            run_once(k)
        sync()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.iters):
            run_once(k)
        b.record()
        sync()
        t = torch.tensor([a.elapsed_time(b) / args.iters], dtype=torch.float64, device=dev)
        if world > 1:
            dist_.all_reduce(t, op=dist_.ReduceOp.MAX)
        return float(t.item())

    results = {}
    for ps in PS:
        for wpb in WPB:
            for dist in DIST:
                results[(ps, wpb, dist)] = time_point(ps, wpb, dist)

    group_ms = time_point(32, 1, 1, _lib.AGG_GROUP_PER_NODE) if (args.group_per_node and args.dim == 16) else None

    if rank == 0:
        sink = open(args.csv, "w") if args.csv else sys.stdout
        print(f"# {args.config}: {nodes} nodes, {edges} edges, width {args.dim}, {world} GPU(s), fetch={args.fetch}; "
              f"ms per aggregation, max over ranks", file=sink)
        if group_ms is not None:
            print(f"# group-per-node kernel: {group_ms:.4f} ms", file=sink)
        print("ps,wpb,dist,ms", file=sink)
        for (ps, wpb, dist), ms in results.items():
            print(f"{ps},{wpb},{dist},{ms:.4f}", file=sink)
        if args.csv:
            sink.close()
        best = min(results, key=results.get)
        worst = max(results, key=results.get)
        print(f"\nbest  ps={best[0]} wpb={best[1]} dist={best[2]}: {results[best]:.4f} ms "
              f"({edges / results[best] / 1e6:.1f} G edges/s)")
        print(f"worst ps={worst[0]} wpb={worst[1]} dist={worst[2]}: {results[worst]:.4f} ms")
        if group_ms is not None:
            print(f"group-per-node kernel: {group_ms:.4f} ms ({edges / group_ms / 1e6:.1f} G edges/s)")
        print("\ndist \\ ps (wpb=4)   " + "".join(f"{ps:>9d}" for ps in PS))
        for dist in DIST:
            print(f"{dist:>18d}   " + "".join(f"{results[(ps, 4, dist)]:9.4f}" for ps in PS))
        print("\ndist \\ wpb (ps=16)  " + "".join(f"{w:>9d}" for w in WPB))
        for dist in DIST:
            print(f"{dist:>18d}   " + "".join(f"{results[(16, w, dist)]:9.4f}" for w in WPB))

    sync()
    sym.close()
    if world > 1:
        dist_.destroy_process_group()


if __name__ == "__main__":
    main()
