"""The epoch-flag barrier (mggb_flag_barrier) on one device.

Two barrier kernels that wait on each other must never share a GPU, so the two-sided case runs in the
multi-process test on real peers.  Here the peer's side is played by the host: a flag that is already
set lets the wait through; a flag that nothing sets makes the bounded wait run out, and the kernel
must then return (the stream stays usable) and report which PE never arrived."""
import ctypes as C
import time

import pytest
import torch

from mgg_osdi23_b200 import _lib

pytestmark = pytest.mark.gpu


def _status(reset=False):
    st = C.c_int(-1)
    _lib.check(_lib.lib.mggb_flag_barrier_status(C.byref(st), int(reset)))
    return st.value


def test_wait_passes_when_the_peer_has_announced_and_expires_when_it_has_not():
    dev = torch.device("cuda")
    mine = torch.zeros(_lib.MAX_PES, dtype=torch.int32, device=dev)     # PE 0's slots
    peer = torch.zeros(_lib.MAX_PES, dtype=torch.int32, device=dev)     # PE 1's slots (PE 1 itself never runs here)
    table = (C.c_void_p * 2)(mine.data_ptr(), peer.data_ptr())
    _status(reset=True)
    # the peer "announced" epochs up to 3 already
    mine[1] = 3
    for epoch in (1, 2, 3):
        _lib.check(_lib.lib.mggb_flag_barrier(table, 2, 0, epoch, 50_000_000, None))
    torch.cuda.synchronize()
    assert _status() == 0
    assert int(mine[0]) == 3 and int(peer[0]) == 3                      # announced to itself and to the peer
    # epoch 4 never arrives: the wait gives up after ~20 ms, the kernel returns and says who was missing
    t0 = time.perf_counter()
    _lib.check(_lib.lib.mggb_flag_barrier(table, 2, 0, 4, 20_000_000, None))
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0
    assert _status() == 2                                               # 1 + PE 1
    assert int(peer[0]) == 4                                            # it still announced its own arrival
    # the context is intact: later work on the stream runs, and the status can be cleared
    assert float((torch.ones(8, device=dev) * 2).sum()) == 16.0
    assert _status(reset=True) == 2 and _status() == 0


def test_counted_form_takes_its_epoch_from_device_memory_also_when_replayed_from_a_graph():
    """mggb_flag_barrier_counted: every launch uses the device counter + 1 and stores it back, so a launch
    recorded in a CUDA graph announces a new epoch at every replay."""
    dev = torch.device("cuda")
    mine = torch.zeros(_lib.MAX_PES, dtype=torch.int32, device=dev)
    peer = torch.zeros(_lib.MAX_PES, dtype=torch.int32, device=dev)
    counter = torch.zeros(1, dtype=torch.int32, device=dev)
    table = (C.c_void_p * 2)(mine.data_ptr(), peer.data_ptr())
    _status(reset=True)
    mine[1] = 1000                                                      # the "peer" is far ahead: no wait ever blocks
    call = lambda: _lib.check(_lib.lib.mggb_flag_barrier_counted(table, 2, 0, counter.data_ptr(), 50_000_000,
                                                                 C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    call(); call()
    torch.cuda.synchronize()
    assert int(counter) == 2 and int(peer[0]) == 2 and int(mine[0]) == 2
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        call()
        call()
    assert int(counter) == 2                                            # recording runs nothing
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert int(counter) == 8 and int(peer[0]) == 8 and _status() == 0
    # a peer that stops announcing makes the bounded wait run out, from a graph as well
    mine[1] = 8
    t0 = time.perf_counter()
    graph.replay()
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0
    assert _status(reset=True) == 2 and int(counter) == 10
    assert _lib.lib.mggb_flag_barrier_counted(table, 2, 0, None, 1000, None) == _lib.ERR_INVALID_ARG


def test_arguments_are_checked_on_the_host():
    one = (C.c_void_p * 1)(16)
    for args in ((None, 1, 0, 1, 1000, None), (one, 0, 0, 1, 1000, None), (one, 1, 1, 1, 1000, None),
                 (one, 1, 0, 1, 0, None), (one, 1, 0, 1, 11_000_000_000, None), ((C.c_void_p * 1)(0), 1, 0, 1, 1000, None)):
        assert _lib.lib.mggb_flag_barrier(*args) == _lib.ERR_INVALID_ARG
