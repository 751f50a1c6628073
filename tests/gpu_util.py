"""Helpers shared by the GPU tests: several PEs emulated on one device, and oracle-side references."""
import numpy as np
import torch

import mgg_osdi23_b200 as mgg
from mgg_osdi23_b200 import drivers

RTOL, ATOL = 1e-5, 1e-4   # fp32 embeddings / logits: the tolerance the path is specified to


def shard_inputs(x: np.ndarray, G: int):
    """Lays the global feature matrix out as G symmetric buffers [nodePerPE, dim] (zero padded)."""
    n, dim = x.shape
    npp = (n + G - 1) // G
    sym = [np.zeros((npp, dim), np.float32) for _ in range(G)]
    for p in range(G):
        lo, hi = min(p * npp, n), min((p + 1) * npp, n)
        sym[p][: hi - lo] = x[lo:hi]
    return sym, npp


def emulated_aggregate(rp, col, x, G, knobs=(16, 4, 1), gin_eps=None, accumulate=False, init=None,
                       row_scale=None, flags=0):
    """Runs every PE's shard of the aggregation on the current device; returns the [N, dim] result."""
    n, dim = x.shape
    sym_np, npp = shard_inputs(x, G)
    dev = torch.device("cuda")
    sym = [torch.from_numpy(s).to(dev) for s in sym_np]
    out = np.zeros((n, dim), np.float32)
    for pe in range(G):
        sh = drivers.Shard(rp, col, pe, G, device=dev)
        if sh.rows == 0:
            continue
        o = torch.zeros(sh.rows, dim, device=dev) if init is None else torch.from_numpy(init[sh.lb:sh.ub].copy()).to(dev)
        k = drivers.Knobs(*knobs, flags=flags)
        if gin_eps is not None:
            sh.aggregate_gin(o, sym, dim, k, gin_eps)
        else:
            rs = None if row_scale is None else torch.from_numpy(row_scale[sh.lb:sh.ub].copy()).to(dev)
            sh.aggregate(o, sym, dim, k, accumulate=accumulate, row_scale_=rs)
        out[sh.lb:sh.ub] = o.cpu().numpy()
    torch.cuda.synchronize()
    return out


def random_graph(n, mean_deg, seed, hubs=()):
    rng = np.random.default_rng(seed)
    deg = rng.poisson(mean_deg, n)
    for i, d in hubs:
        deg[i] = d
    rp = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
    col = rng.integers(0, n, rp[-1]).astype(np.int32)
    return rp, col
