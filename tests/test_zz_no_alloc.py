"""The allocation-free aggregation entry point (mggb_sag_np_div_static) against the regular one.

Some users of this library run where a device allocation is off limits once the job is up: inside a
memory pool that has claimed the whole GPU, in a serving loop that cannot tolerate the implicit
synchronisation of cudaMalloc, or under a fixed memory budget.  For them the library offers a variant
whose only scratch memory (the list of hub rows) is a fixed array shipped inside the library.  This
file checks, through the C ABI, that the variant returns what the regular entry point returns, twice
in a row (the array is shared by all calls and keeps old contents), and that it refuses shards that
could overflow the fixed list.  It is named to be collected last, so a failure here cannot hide the
result of any other test; it must also pass when run on its own.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from mgg_osdi23_b200 import _lib, drivers
from gpu_util import RTOL, ATOL, random_graph

pytestmark = pytest.mark.gpu


def _call(fn, out, x, sh, dim, knobs, extra_edges=None, scale=None, flags=0):
    table = (C.c_void_p * 1)(x.data_ptr())
    head = [out.data_ptr(), table, 1, sh.rp_l.data_ptr(), sh.ci_l.data_ptr(), sh.rp_r.data_ptr(), sh.ci_r.data_ptr(), sh.lb, sh.ub]
    if extra_edges is not None:
        head.append(extra_edges)
    tail = [dim, sh.node_per_pe, 0, *knobs, None if scale is None else scale.data_ptr(), flags, None, 0, None]
    return fn(*head, *tail)


def test_static_scratch_variant_matches_regular_entry_point(oracle):
    dev = torch.device("cuda")
    n, dim = 600, 16
    # three rows above the hub threshold (16384 neighbors), so the shared list is really used
    rp, col = random_graph(n, 30, seed=21, hubs=[(3, 40000), (250, 17000), (599, 25000), (10, 16384)])
    x_np = np.random.default_rng(8).uniform(-0.02, 0.02, (n, dim)).astype(np.float32)   # keeps 40,000-term fp32 sums within 1e-4
    sh = drivers.Shard(rp, col, 0, 1, device=dev)
    x = torch.from_numpy(x_np).to(dev)
    scale = torch.from_numpy(np.random.default_rng(9).uniform(0.5, 1.5, n).astype(np.float32)).to(dev)
    want = oracle.sag_f64(x_np, rp, col)
    lib = _lib.lib
    knobs = (16, 4, 1)
    regular = torch.zeros(n, dim, device=dev)
    _lib.check(_call(lib.mggb_sag_np_div, regular, x, sh, dim, knobs))
    torch.cuda.synchronize()
    np.testing.assert_allclose(regular.cpu().numpy(), want, rtol=RTOL, atol=ATOL)

    # call 1: plain sum; call 2, straight after it on the same stream: another graph shape (row scaling,
    # different knobs), so the second call meets the list as the first one left it
    first = torch.full((n, dim), 7.0, device=dev)
    _lib.check(_call(lib.mggb_sag_np_div_static, first, x, sh, dim, knobs, extra_edges=sh.edges))
    second = torch.full((n, dim), -3.0, device=dev)
    _lib.check(_call(lib.mggb_sag_np_div_static, second, x, sh, dim, (32, 2, 2), extra_edges=sh.edges, scale=scale))
    third = torch.zeros(n, dim, device=dev)
    _lib.check(_call(lib.mggb_sag_np_div_static, third, x, sh, dim, knobs, extra_edges=sh.edges))
    torch.cuda.synchronize()
    np.testing.assert_allclose(first.cpu().numpy(), regular.cpu().numpy(), rtol=RTOL, atol=ATOL)
    assert torch.equal(first, regular) and torch.equal(third, regular)      # same kernels, same mapping: same bits
    regular_scaled = torch.zeros(n, dim, device=dev)
    _lib.check(_call(lib.mggb_sag_np_div, regular_scaled, x, sh, dim, (32, 2, 2), scale=scale))
    torch.cuda.synchronize()
    np.testing.assert_allclose(second.cpu().numpy(), regular_scaled.cpu().numpy(), rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(second.cpu().numpy(), want * scale.cpu().numpy()[:, None], rtol=RTOL, atol=ATOL)


def test_static_scratch_variant_with_more_giant_rows_than_its_tables_hold(oracle):
    """300 rows above 16384 neighbors at dim 64: the fixed tables take 256 rows and 1024 partial rows, so
    some rows are cut into segments, some run out of partial rows and some find the table full; those
    stay whole on the hub list.  Every row must still come out right, call after call."""
    dev = torch.device("cuda")
    n, dim = 320, 64
    rp, col = random_graph(n, 8, seed=23, hubs=[(i, 16385 + 37 * i) for i in range(300)])
    x_np = np.random.default_rng(24).uniform(-0.01, 0.01, (n, dim)).astype(np.float32)
    want = oracle.sag_f64(x_np, rp, col)
    sh = drivers.Shard(rp, col, 0, 1, device=dev)
    x = torch.from_numpy(x_np).to(dev)
    lib = _lib.lib
    outs = [torch.full((n, dim), float(k), device=dev) for k in range(3)]
    for o in outs:
        _lib.check(_call(lib.mggb_sag_np_div_static, o, x, sh, dim, (16, 2, 1), extra_edges=sh.edges))
    regular = torch.zeros(n, dim, device=dev)
    _lib.check(_call(lib.mggb_sag_np_div, regular, x, sh, dim, (16, 2, 1)))
    torch.cuda.synchronize()
    for o in outs:
        np.testing.assert_allclose(o.cpu().numpy(), want, rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(regular.cpu().numpy(), want, rtol=RTOL, atol=ATOL)


def test_static_scratch_variant_refuses_oversized_shards():
    dev = torch.device("cuda")
    rp, col = random_graph(50, 5, seed=1)
    sh = drivers.Shard(rp, col, 0, 1, device=dev)
    x = torch.zeros(50, 16, device=dev)
    out = torch.zeros(50, 16, device=dev)
    lib = _lib.lib
    too_many = 8192 * (16384 + 1) + 1           # one edge past what the 8192-entry list can cover
    st = _call(lib.mggb_sag_np_div_static, out, x, sh, 16, (16, 4, 1), extra_edges=too_many)
    assert st == _lib.ERR_UNSUPPORTED
    msg = lib.mggb_last_error().decode()
    assert "8192" in msg and "mggb_sag_np_div" in msg
    assert _call(lib.mggb_sag_np_div_static, out, x, sh, 16, (16, 4, 1), extra_edges=too_many - 1) == _lib.OK
    assert _call(lib.mggb_sag_np_div_static, out, x, sh, 16, (16, 16, 1), extra_edges=10) == _lib.ERR_INVALID_ARG
    torch.cuda.synchronize()


def test_static_scratch_variant_allocates_no_device_memory():
    """The point of the variant: after its first call on a device (which loads the kernels and looks the
    array's address up), further calls leave the device's free memory exactly as it was, hub rows
    included.  Run in a fresh process, where the regular entry point has never been called and so its
    heap work list does not exist: a variant that fell back to it would have to allocate it here."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = r'''
import ctypes as C, sys
import numpy as np, torch
sys.path.insert(0, %r); sys.path.insert(0, %r)
from mgg_osdi23_b200 import _lib, drivers
from gpu_util import random_graph
dev = torch.device("cuda")
rp, col = random_graph(600, 30, seed=21, hubs=[(3, 40000), (250, 17000)])
sh = drivers.Shard(rp, col, 0, 1, device=dev)
x = torch.rand(600, 16, device=dev) * 0.01
out = torch.zeros(600, 16, device=dev)
table = (C.c_void_p * 1)(x.data_ptr())
def call():
    _lib.check(_lib.lib.mggb_sag_np_div_static(out.data_ptr(), table, 1, sh.rp_l.data_ptr(), sh.ci_l.data_ptr(), sh.rp_r.data_ptr(),
                                               sh.ci_r.data_ptr(), sh.lb, sh.ub, sh.edges, 16, sh.node_per_pe, 0, 16, 4, 1, None, 0, None, 0, None))
call(); torch.cuda.synchronize()
free0 = torch.cuda.mem_get_info()[0]
for _ in range(4):
    call()
torch.cuda.synchronize()
free1 = torch.cuda.mem_get_info()[0]
assert free0 == free1, (free0, free1)
want = float(x[torch.from_numpy(col[rp[3]:rp[4]]).long().to(dev)].double().sum())
assert abs(float(out[3].double().sum()) - want) < 1e-4 * abs(want) + 1e-3
print("unchanged", free0)
''' % (root, os.path.join(root, "tests"))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "unchanged" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_static_scratch_variant_with_peers_and_a_publish_table(oracle):
    """Two PEs emulated on one device (separate symmetric buffers, so remote rows go through the owner
    lookup) and an extra destination for every output row: same bits as the regular entry point."""
    dev = torch.device("cuda")
    n, dim, G = 500, 16, 2
    rp, col = random_graph(n, 20, seed=5, hubs=[(7, 20000), (400, 18000)])
    x_np = np.random.default_rng(3).uniform(-0.02, 0.02, (n, dim)).astype(np.float32)
    npp = (n + G - 1) // G
    sym = [torch.from_numpy(np.ascontiguousarray(x_np[p * npp:(p + 1) * npp])).to(dev) for p in range(G)]
    table = (C.c_void_p * G)(*[s.data_ptr() for s in sym])
    want = oracle.sag_f64(x_np, rp, col)
    lib = _lib.lib
    for pe in range(G):
        sh = drivers.Shard(rp, col, pe, G, device=dev)
        outs, copies = [], []
        for fn, extra in ((lib.mggb_sag_np_div, []), (lib.mggb_sag_np_div_static, [sh.edges])):
            out = torch.zeros(sh.rows, dim, device=dev)
            copy = torch.zeros(sh.rows, dim, device=dev)
            pub = (C.c_void_p * 1)(copy.data_ptr())
            _lib.check(fn(out.data_ptr(), table, G, sh.rp_l.data_ptr(), sh.ci_l.data_ptr(), sh.rp_r.data_ptr(), sh.ci_r.data_ptr(),
                          sh.lb, sh.ub, *extra, dim, sh.node_per_pe, pe, 16, 4, 1, None, 0, pub, 1, None))
            outs.append(out); copies.append(copy)
        torch.cuda.synchronize()
        assert torch.equal(outs[0], outs[1]) and torch.equal(copies[1], outs[1]) and torch.equal(copies[0], outs[0])
        np.testing.assert_allclose(outs[1].cpu().numpy(), want[sh.lb:sh.ub], rtol=RTOL, atol=ATOL)
