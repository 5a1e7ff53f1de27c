"""The bounded inter-rank barrier (snb_peer_barrier) on one GPU, called through the C ABI.

A barrier between real ranks is exercised by the two-GPU tests and by the benchmark's N > 1 runs;
here the two "ranks" are two flag arrays in the same device memory.  A wait that nothing satisfies
must run out: the kernel records which rank it gave up on, returns, and the context stays usable
(no trap, no hang)."""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptrs(*tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def test_barrier_passes_when_the_peer_has_signalled():
    from sortnet_b200 import _lib
    lib = _lib.load()
    mine = torch.zeros(4, dtype=torch.int32, device="cuda")
    peer = torch.zeros(4, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32).pin_memory()
    st = torch.cuda.current_stream().cuda_stream
    mine[1] = 3                                          # "rank 1" has already reached epoch 3
    rc = lib.snb_peer_barrier(_ptrs(mine, peer), 0, 2, 3, 2_000_000_000, status.data_ptr(), st)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    assert int(peer[0]) == 3                             # and rank 0's signal has landed in rank 1's flags
    # a later epoch in the flag also satisfies an earlier barrier
    mine[1] = 9
    assert lib.snb_peer_barrier(_ptrs(mine, peer), 0, 2, 4, 2_000_000_000, status.data_ptr(), st) == 0
    torch.cuda.synchronize()
    assert int(status[0]) == 0


def test_barrier_gives_up_after_its_time_limit_and_reports_the_missing_rank():
    from sortnet_b200 import _lib
    lib = _lib.load()
    flags = [torch.zeros(4, dtype=torch.int32, device="cuda") for _ in range(3)]
    status = torch.zeros(1, dtype=torch.int32).pin_memory()
    st = torch.cuda.current_stream().cuda_stream
    flags[0][1] = 1                                      # rank 1 arrives, rank 2 never does
    t0 = time.time()
    rc = lib.snb_peer_barrier(_ptrs(*flags), 0, 3, 1, 50_000_000, status.data_ptr(), st)   # 50 ms limit
    assert rc == 0
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0
    assert int(status[0]) == 1 + 2                       # gave up on rank 2
    # the context is still usable
    assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0


def test_barrier_argument_checks():
    from sortnet_b200 import _lib
    lib = _lib.load()
    a = torch.zeros(4, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32).pin_memory()
    assert lib.snb_peer_barrier(None, 0, 2, 1, 1000, status.data_ptr(), None) == 1
    assert lib.snb_peer_barrier(_ptrs(a, a), 2, 2, 1, 1000, status.data_ptr(), None) == 3
    assert lib.snb_peer_barrier(_ptrs(a, a), 0, 17, 1, 1000, status.data_ptr(), None) == 3
    assert lib.snb_peer_barrier(_ptrs(a), 0, 1, 1, 1000, status.data_ptr(), None) == 0     # one rank: nothing to do
