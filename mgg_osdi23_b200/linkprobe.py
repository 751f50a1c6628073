"""What the links between the GPUs give for MGG's access pattern: rows of ``dim`` floats gathered at
random from peers' symmetric buffers inside the aggregation kernel (every neighbor remote, none local).

The reference fetches each remote neighbor with one blocking ``nvshmemx_float_get_warp`` of ``dim``
floats (``include/neighbor_utils.cuh:1445``: 64 bytes at width 16, 256 bytes at width 64), so the
rate at which the fabric serves reads of that size is the ceiling of any pull-mode aggregation.  This
tool measures it with the library's own kernel, per row width, so that a measured pull-mode time can
be set against what the links can do rather than against their nominal 900 GB/s.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
        --master-port 29500 -m mgg_osdi23_b200.linkprobe

Prints one line per (row width, neighbors per row, path): ms per launch (max over ranks), GB/s of
gathered rows per GPU and rows/s.  ``--staged`` adds the path that stages rows through shared memory.
"""
from __future__ import annotations

import argparse
import os

import torch

from . import _lib, api
from .symmem import SymmetricBuffer


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--dims", default="16,32,64,128")
    ap.add_argument("--degrees", default="64,512", help="remote neighbors per output row")
    ap.add_argument("--rows", type=int, default=1 << 16, help="output rows per GPU")
    ap.add_argument("--table-rows", type=int, default=1 << 18, help="rows of every PE's symmetric buffer")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--staged", action="store_true", help="also time MGGB_AGG_STAGE_ROWS")
    args = ap.parse_args(argv)
    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0")))
    if world < 2:
        raise SystemExit("the link probe needs at least two GPUs (torchrun --nproc-per-node N)")
    import torch.distributed as dist
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    npp, rows = args.table_rows, args.rows
    paths = [("registers", _lib.AGG_NO_HUB_SPLIT)] + ([("staged", _lib.AGG_NO_HUB_SPLIT | _lib.AGG_STAGE_ROWS)] if args.staged else [])
    for dim in (int(d) for d in args.dims.split(",")):
        for deg in (int(d) for d in args.degrees.split(",")):
            sym = SymmetricBuffer(npp * dim, None, rank, world)
            sym.tensor.uniform_(-1, 1)
            g = torch.Generator(device="cpu")
            g.manual_seed(1000 * dim + rank)
            peer = (rank + 1 + torch.randint(0, world - 1, (rows * deg,), generator=g)) % world      # never this PE
            ids = (peer * npp + torch.randint(0, npp, (rows * deg,), generator=g)).to(torch.int32).to(dev)
            rp_r = (torch.arange(rows + 1, dtype=torch.int64) * deg).to(torch.int32).to(dev)
            rp_l = torch.zeros(rows + 1, dtype=torch.int32, device=dev)
            ci_l = torch.zeros(1, dtype=torch.int32, device=dev)
            out = torch.zeros(rows, dim, device=dev)
            lb = rank * npp
            for name, flags in paths:
                def run():
                    api.mgg_SAG_np_div(out, sym, rp_l, ci_l, rp_r, ids, lb, lb + rows, dim, npp, rank, 16, 4, 2,
                                       accumulate=False, flags=flags)
                for _ in range(3):
                    run()
                torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(args.iters):
                    run()
                e1.record()
                torch.cuda.synchronize()
                t = torch.tensor([e0.elapsed_time(e1) / args.iters], dtype=torch.float64, device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                if rank == 0:
                    ms = float(t)
                    print(f"{world} GPUs, rows of {4 * dim:4d} B, {deg:4d} remote neighbors per row, {name:9s}: {ms:8.3f} ms  "
                          f"{rows * deg * dim * 4 / ms / 1e6:7.1f} GB/s per GPU  {rows * deg / ms / 1e6:6.2f} G rows/s per GPU", flush=True)
            dist.barrier(); torch.cuda.synchronize()
            sym.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
