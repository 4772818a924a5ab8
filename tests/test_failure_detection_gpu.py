"""Failure detection on the GPU without a fault: a peer that never signals makes the bounded flag wait run out; the
kernel returns an error status that the host reads, and the CUDA context stays usable."""
from ctypes import c_double, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
MAX_RANKS = 8


def test_bounded_peer_wait_times_out_and_context_survives():
    from flextrain_b200.ops.cuda import load
    lib = load("comm")
    dev = "cuda:0"
    slots, slot = 16, 3
    # flag tables of "rank 0" (this process) and of a "rank 1" that never runs: both live on this GPU
    mine = torch.zeros(slots * MAX_RANKS, dtype=torch.int32, device=dev)
    peer = torch.zeros(slots * MAX_RANKS, dtype=torch.int32, device=dev)
    tables = (c_void_p * 2)(mine.data_ptr(), peer.data_ptr())
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    lib.ftb_comm_error()                                   # clear
    rc = lib.ftb_comm_signal_wait(tables, c_int(slot), c_int(0), c_int(2), c_int(1), c_double(0.2),
                                  c_void_p(status.data_ptr()), stream)
    assert rc == 0
    torch.cuda.synchronize()                               # returns after ~0.2 s: the wait gave up by itself
    assert int(status) == 2                                # 1 + the rank that never signalled
    assert int(peer[slot * MAX_RANKS + 0]) == 1            # our own signal did reach the peer's table
    err = lib.ftb_comm_error()
    assert err // 1000 == 2 and err % 1000 == slot * 100 + 1
    assert float(torch.ones(1000, device=dev).sum()) == 1000.0     # the context still works
    # the peer shows up: the same wait now completes cleanly
    status.zero_()
    mine[slot * MAX_RANKS + 1] = 2
    rc = lib.ftb_comm_signal_wait(tables, c_int(slot), c_int(0), c_int(2), c_int(2), c_double(5.0),
                                  c_void_p(status.data_ptr()), stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status) == 0 and lib.ftb_comm_error() == 0
