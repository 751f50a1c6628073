"""Seeded synthetic graphs, features and weights.

The reference is measured on downloaded datasets (Reddit, ogbn-products, enwiki-2013, paper100M;
``bench_MGG.py:21-29``) that are not available offline.  These generators produce graphs with the
same shapes (node and edge counts, degree skew, feature widths).  All randomness comes from a
counter-based integer hash evaluated with tensor ops, so a given seed yields the same graph on
the CPU and on a GPU, independent of the device's random-number generator.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

_MASK64 = (1 << 64) - 1


def _s64(v: int) -> int:
    """Python int -> the same 64 bits as a signed value."""
    v &= _MASK64
    return v - (1 << 64) if v >= (1 << 63) else v


_C1 = _s64(0xBF58476D1CE4E5B9)
_C2 = _s64(0x94D049BB133111EB)
_GOLD = _s64(0x9E3779B97F4A7C15)


def _lsr(x: torch.Tensor, s: int) -> torch.Tensor:
    """Logical right shift of int64 values."""
    return (x >> s) & ((1 << (64 - s)) - 1)


def hash64(counter: torch.Tensor, seed: int, stream: int = 0) -> torch.Tensor:
    """SplitMix64 finaliser of (counter, seed, stream); int64 in, int64 out (all 64 bits mixed)."""
    z = counter + _s64(seed * 0x9E3779B97F4A7C15 + stream * 0xD1B54A32D192ED03 + 0x2545F4914F6CDD1D)
    z = z * _GOLD
    z = (z ^ _lsr(z, 30)) * _C1
    z = (z ^ _lsr(z, 27)) * _C2
    return z ^ _lsr(z, 31)


def uniform01(counter: torch.Tensor, seed: int, stream: int = 0, dtype=torch.float64) -> torch.Tensor:
    """Uniform in [0, 1) from the top 53 (float64) or 24 (float32) bits of the hash."""
    h = hash64(counter, seed, stream)
    if dtype == torch.float64:
        return _lsr(h, 11).to(torch.float64) * (1.0 / (1 << 53))
    return _lsr(h, 40).to(torch.float32) * (1.0 / (1 << 24))


@dataclass
class Graph:
    """CSR graph with int64 row pointers and int32 column ids (sorted within a row)."""
    num_nodes: int
    row_ptr: torch.Tensor   # int64 [N+1]
    col_idx: torch.Tensor   # int32 [E]
    meta: dict = field(default_factory=dict)

    @property
    def num_edges(self) -> int:
        return int(self.col_idx.numel())

    def row_ptr32(self) -> torch.Tensor:
        assert self.num_edges < 2 ** 31
        return self.row_ptr.to(torch.int32)

    def cpu(self) -> "Graph":
        return Graph(self.num_nodes, self.row_ptr.cpu(), self.col_idx.cpu(), dict(self.meta))


def _csr_from_keys(keys: torch.Tensor, n: int, meta: dict) -> Graph:
    """keys = src * n + dst, already unique and sorted."""
    src = keys // n
    col = (keys - src * n).to(torch.int32)
    counts = torch.bincount(src, minlength=n)
    row_ptr = torch.zeros(n + 1, dtype=torch.int64, device=keys.device)
    torch.cumsum(counts, 0, out=row_ptr[1:])
    return Graph(n, row_ptr, col, meta)


def _finish(src: torch.Tensor, dst: torch.Tensor, n: int, symmetric: bool, self_loops: bool, dedup: bool = True) -> torch.Tensor:
    keys = src * n + dst
    if symmetric:
        keys = torch.cat([keys, dst * n + src])
    if self_loops:
        ids = torch.arange(n, dtype=torch.int64, device=src.device)
        keys = torch.cat([keys, ids * n + ids])
    if not dedup:       # a multigraph: every sampled pair is an edge, repeated pairs are repeated neighbors
        return torch.sort(keys).values
    return torch.unique(keys, sorted=True)


def _mix_bits(x: torch.Tensor, bits: int, seed: int) -> torch.Tensor:
    """A bijection of [0, 2^bits): odd multiplications and xor-shifts, each invertible modulo 2^bits."""
    mask = (1 << bits) - 1
    h = max(1, bits // 2)
    x = (x + (seed * 0x632BE5AB & mask)) & mask
    x = (x * _GOLD) & mask
    x = x ^ (x >> h)
    x = (x * _C1) & mask
    x = x ^ (x >> (h + 1 if h + 1 < bits else h))
    x = (x * _C2) & mask
    return x ^ (x >> h)


def relabel_ids(ids: torch.Tensor, n: int, seed: int = 0) -> torch.Tensor:
    """Pseudo-random permutation of [0, n) applied to ``ids`` (int64): the bit mixer above on the next
    power of two, walked along its cycle until it lands below n again (cycle walking keeps it a
    bijection).  Generators whose construction puts the heaviest nodes at the lowest ids (R-MAT) use it
    so that a node-range partition sees shards of similar size, as with a dataset's arbitrary ids."""
    bits = max(1, (n - 1).bit_length())
    out = _mix_bits(ids, bits, seed)
    bad = torch.nonzero(out >= n).flatten()
    while bad.numel():
        v = _mix_bits(out[bad], bits, seed)
        out[bad] = v
        bad = bad[v >= n]
    return out


def rmat_edges(scale: int, n_edges: int, a: float, b: float, c: float, seed: int, device="cpu",
               first: int = 0):
    """R-MAT endpoint pairs number [first, first+n_edges) on 2^scale ids (quadrant probabilities a, b, c, 1-a-b-c)."""
    e = torch.arange(first, first + n_edges, dtype=torch.int64, device=device)
    src = torch.zeros_like(e)
    dst = torch.zeros_like(e)
    for level in range(scale):
        u = uniform01(e, seed, stream=level + 1)
        right = ((u >= a) & (u < a + b)) | (u >= a + b + c)     # quadrants b and d set the dst bit
        down = u >= a + b                                       # quadrants c and d set the src bit
        src = src * 2 + down.to(torch.int64)
        dst = dst * 2 + right.to(torch.int64)
    return src, dst


def rmat_graph(scale: int, n_edges: int, a=0.57, b=0.19, c=0.19, seed=0, symmetric=True, self_loops=True,
               num_nodes: int | None = None, device="cpu", relabel: bool = False, dedup: bool = True) -> Graph:
    """R-MAT graph.  With num_nodes < 2^scale, sampled pairs with an endpoint >= num_nodes are dropped
    and sampling continues until n_edges pairs are kept (before symmetrisation / deduplication).
    relabel=True renumbers the nodes with ``relabel_ids`` (same graph up to isomorphism).
    dedup=False keeps repeated pairs (the edge list as an R-MAT generator emits it: a multigraph)."""
    n = num_nodes if num_nodes is not None else (1 << scale)
    if n == (1 << scale):
        src, dst = rmat_edges(scale, n_edges, a, b, c, seed, device)
    else:
        kept_s, kept_d, have, first = [], [], 0, 0
        while have < n_edges:
            batch = max(1024, int((n_edges - have) * 1.3 * ((1 << scale) / n) ** 2) + 1024)
            batch = min(batch, 1 << 26)
            s, d = rmat_edges(scale, batch, a, b, c, seed, device, first)
            first += batch
            ok = (s < n) & (d < n)
            s, d = s[ok], d[ok]
            take = min(int(s.numel()), n_edges - have)
            kept_s.append(s[:take]); kept_d.append(d[:take]); have += take
        src, dst = torch.cat(kept_s), torch.cat(kept_d)
    if relabel:
        src, dst = relabel_ids(src, n, seed), relabel_ids(dst, n, seed)
    keys = _finish(src, dst, n, symmetric, self_loops, dedup)
    meta = dict(kind="rmat", scale=scale, sampled_edges=n_edges, a=a, b=b, c=c, d=round(1 - a - b - c, 6),
                seed=seed, symmetric=symmetric, self_loops=self_loops, relabelled=relabel)
    if not dedup:
        meta["repeated_pairs_kept"] = True
    return _csr_from_keys(keys, n, meta)


def chung_lu_graph(num_nodes: int, target_edges: int, gamma: float, seed=0, communities: int = 1,
                   p_intra: float = 0.0, offset_frac: float = 1.0 / 256, self_loops=True, device="cpu",
                   max_rounds: int = 4) -> Graph:
    """Power-law (Chung-Lu style) symmetric graph with optional contiguous-id communities.

    Node weights follow w ~ (rank + i0)^(-1/(gamma-1)), ranks dealt round-robin to the communities so
    that each community has the same degree profile; node ids are NOT shuffled, so a contiguous range
    partition sees the community structure.  Both endpoints are drawn from the weights; with
    probability p_intra the second endpoint is drawn inside the first one's community.  Pairs are
    symmetrised and deduplicated; the number of sampled pairs is raised (at most max_rounds times, by
    extending the same random stream) until the stored edge count reaches about target_edges.
    """
    n = num_nodes
    alpha = 1.0 / (gamma - 1.0)
    csize = (n + communities - 1) // communities
    ids = torch.arange(n, dtype=torch.int64, device=device)
    rank = (ids % csize) * communities + ids // csize
    w = (rank.to(torch.float64) + offset_frac * n).pow(-alpha)
    cdf = torch.cumsum(w, 0)
    total = float(cdf[-1])
    cdf0 = torch.cat([torch.zeros(1, dtype=torch.float64, device=device), cdf])

    def sample(first: int, count: int):
        e = torch.arange(first, first + count, dtype=torch.int64, device=device)
        s = torch.searchsorted(cdf, uniform01(e, seed, 1) * total, right=True).clamp_(max=n - 1)
        comm = s // csize
        lo = cdf0[comm * csize]
        hi = cdf0[torch.clamp((comm + 1) * csize, max=n)]
        intra = uniform01(e, seed, 2) < p_intra
        u = uniform01(e, seed, 3)
        pos = torch.where(intra, lo + u * (hi - lo), u * total)
        d = torch.searchsorted(cdf, pos, right=True).clamp_(max=n - 1)
        return s, d

    want = target_edges - (n if self_loops else 0)
    pairs = max(1, want // 2)
    keys = None
    done = 0
    srcs, dsts = [], []
    for _ in range(max_rounds):
        s, d = sample(done, pairs - done)
        srcs.append(s); dsts.append(d); done = pairs
        keys = _finish(torch.cat(srcs), torch.cat(dsts), n, True, self_loops)
        got = int(keys.numel())
        if got >= 0.995 * target_edges:
            break
        grow = (target_edges - (n if self_loops else 0)) / max(1, got - (n if self_loops else 0))
        pairs = int(pairs * min(2.0, grow * 1.02)) + 1
    meta = dict(kind="chung_lu", gamma=gamma, communities=communities, p_intra=p_intra,
                offset_frac=offset_frac, sampled_pairs=done, seed=seed, self_loops=self_loops)
    return _csr_from_keys(keys, n, meta)


def features(num_rows: int, dim: int, seed: int, device="cpu", first_row: int = 0) -> torch.Tensor:
    """fp32 features ~ U[-1, 1); element (i, d) depends only on (seed, i, d), so shards can be generated independently."""
    idx = torch.arange(first_row * dim, (first_row + num_rows) * dim, dtype=torch.int64, device=device)
    return (uniform01(idx, seed, 7, torch.float32) * 2.0 - 1.0).reshape(num_rows, dim)


def glorot_uniform(fan_in: int, fan_out: int, seed: int, device="cpu") -> torch.Tensor:
    """[fan_in, fan_out] fp32 weight ~ U(-L, L), L = sqrt(6 / (fan_in + fan_out))."""
    lim = math.sqrt(6.0 / (fan_in + fan_out))
    idx = torch.arange(fan_in * fan_out, dtype=torch.int64, device=device)
    return ((uniform01(idx, seed, 11, torch.float32) * 2.0 - 1.0) * lim).reshape(fan_in, fan_out)


# ---- the named benchmark shapes -----------------------------------------------------------------

def config1_graph(device="cpu", seed=0) -> Graph:
    """16,384-node R-MAT (a=.57 b=.19 c=.19 d=.05), 262,144 sampled directed edges, symmetrised + self-loops."""
    return rmat_graph(14, 262_144, 0.57, 0.19, 0.19, seed=seed, device=device)


def config2_graph(device="cpu", seed=0, scale: float = 1.0) -> Graph:
    """Reddit-shaped: 232,965 nodes, ~114.6 M stored edges, power law 2.1, 16 contiguous communities.
    scale < 1 shrinks nodes and edges together (mean degree kept) for tests."""
    n = max(64, int(232_965 * scale))
    return chung_lu_graph(n, int(114_600_000 * scale), 2.1, seed=seed, communities=16, p_intra=0.7, device=device)


def config3_graph(device="cpu", seed=0, scale: float = 1.0) -> Graph:
    """ogbn-products-shaped: 2,449,029 nodes, ~123.7 M stored edges, power law 2.3.  The degree ranks are
    dealt round-robin to 64 contiguous id blocks (no preference for edges inside a block), so every
    node-range shard has the same degree profile and endpoints are spread over all shards."""
    n = max(64, int(2_449_029 * scale))
    return chung_lu_graph(n, int(123_700_000 * scale), 2.3, seed=seed, communities=64, p_intra=0.0, device=device)


def config4_graph(device="cpu", seed=0, scale_shift: int = 0) -> Graph:
    """enwiki-shaped skewed directed R-MAT (a=.6 b=.15 c=.15 d=.1): 4,206,785 nodes, 101.3 M edges, not
    symmetrised, node ids relabelled pseudo-randomly, largest neighbor list above 10^5 (checked at full
    size).  The 101.3 M sampled pairs are all kept, repeats included, as an R-MAT generator emits them:
    with repeats removed these parameters give 96.5 M edges and a largest list of 72 K, short of the
    shape's defining skew.  scale_shift > 0 halves ids and edges that many times for tests."""
    n = 4_206_785 >> scale_shift
    g = rmat_graph(23 - scale_shift, 101_300_000 >> scale_shift, 0.6, 0.15, 0.15, seed=seed,
                   symmetric=False, self_loops=False, num_nodes=n, device=device, relabel=True, dedup=False)
    g.meta["max_in_degree"] = int((g.row_ptr[1:] - g.row_ptr[:-1]).max())
    if scale_shift == 0 and g.meta["max_in_degree"] <= 100_000:
        raise AssertionError(f"config 4 needs a node with more than 10^5 in-edges, the generator gave {g.meta['max_in_degree']}")
    return g


def rmat_shard(scale: int, n_pairs: int, num_nodes: int, lb: int, ub: int, a=0.57, b=0.19, c=0.19, seed=0,
               device="cpu", batch: int = 1 << 25, relabel: bool = False) -> Graph:
    """The rows [lb, ub) of the symmetrised R-MAT graph on ``num_nodes`` ids, built WITHOUT
    materialising the whole graph: every rank walks the same ``n_pairs`` sampled pairs in batches
    (counter-based randomness, so all ranks see the same pairs) and keeps, in both directions, only
    the edges whose source row it owns.  Pairs with an endpoint >= num_nodes are dropped; relabel=True
    renumbers the endpoints with ``relabel_ids`` before the ownership test, as rmat_graph does.  Returns a
    Graph whose ``row_ptr`` (int64, ub-lb+1 entries, starting at 0) indexes the shard's rows and
    whose ``col_idx`` holds global ids; self-loops are added for the shard's own rows."""
    rows = ub - lb
    kept = []
    for first in range(0, n_pairs, batch):
        cnt = min(batch, n_pairs - first)
        s, d = rmat_edges(scale, cnt, a, b, c, seed, device, first)
        ok = (s < num_nodes) & (d < num_nodes)
        s, d = s[ok], d[ok]
        if relabel:
            s, d = relabel_ids(s, num_nodes, seed), relabel_ids(d, num_nodes, seed)
        fwd = (s >= lb) & (s < ub)
        bwd = (d >= lb) & (d < ub)
        kept.append(torch.cat([(s[fwd] - lb) * num_nodes + d[fwd], (d[bwd] - lb) * num_nodes + s[bwd]]))
        if len(kept) >= 8:       # keep the working set bounded: deduplicate as we go
            kept = [torch.unique(torch.cat(kept))]
    ids = torch.arange(lb, ub, dtype=torch.int64, device=device)
    kept.append((ids - lb) * num_nodes + ids)
    keys = torch.unique(torch.cat(kept), sorted=True)
    src = keys // num_nodes
    col = (keys - src * num_nodes).to(torch.int32)
    row_ptr = torch.zeros(rows + 1, dtype=torch.int64, device=keys.device)
    torch.cumsum(torch.bincount(src, minlength=rows), 0, out=row_ptr[1:])
    meta = dict(kind="rmat_shard", scale=scale, sampled_pairs=n_pairs, lb=lb, ub=ub, seed=seed, relabelled=relabel)
    return Graph(num_nodes, row_ptr, col, meta)


def config5_shard(pe: int, num_pes: int, device="cpu", seed=0, scale_shift: int = 0) -> Graph:
    """paper100M-shaped: 111 M nodes, ~3.2 B stored edges (1.6 B sampled pairs), symmetric R-MAT with node
    ids relabelled pseudo-randomly; only PE ``pe``'s rows are built (see rmat_shard).  scale_shift halves
    ids and pairs that many times."""
    n = 111_000_000 >> scale_shift
    npp = (n + num_pes - 1) // num_pes
    lb = min(n, pe * npp)
    ub = min(n, lb + npp)
    return rmat_shard(27 - scale_shift, 1_600_000_000 >> scale_shift, n, lb, ub, seed=seed, device=device, relabel=True)
