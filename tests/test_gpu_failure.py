"""Failure detection on the device: a bounded wait runs out, the kernel records
where it gave up and returns, and the CUDA context stays usable.

The failure is produced on the host: a two-rank communicator is created whose
second rank is never launched (both heaps live on this GPU, rank 1's kernels
simply do not exist), so the flag rank 0 waits for is one that nothing sets.
Nothing faults, traps or spins without a limit.
"""
import ctypes as C

import pytest
import torch

from configurable_hierarchical_allreduce_algorithms_b200 import _native as N
from configurable_hierarchical_allreduce_algorithms_b200.parallel import comm as cm

pytestmark = pytest.mark.gpu


def _half_world(timeout_us):
    """rank 0 of a P=2 world whose rank 1 never runs."""
    L = N.lib()
    c = cm.Communicator._new()
    P = 2
    ll, scratch, user = 64 << 10, 1 << 20, 1 << 20
    heap_bytes = int(L.chb_heap_bytes(P, ll, scratch, user))
    heap = torch.zeros(P * heap_bytes, dtype=torch.uint8, device="cuda")
    c._keep.append(heap)
    ptrs = (C.c_void_p * P)(*[heap.data_ptr() + p * heap_bytes for p in range(P)])
    c._finish(0, P, 1, ptrs, 0, ll, scratch, user, torch.cuda.current_device(), timeout_us)
    c.backend = "test"
    return c


def test_barrier_times_out_and_reports(cuda):
    c = _half_world(timeout_us=200_000)
    c.barrier()
    st = c.status()
    assert st["rc"] == N.ERR_TIMEOUT and st["code"] == 6
    assert st["rank"] == 0 and st["peer"] == 1 and st["expected"] == 1 and st["seen"] == 0
    with pytest.raises(cm.CollectiveError, match="timeout"):
        c.check()
    # the context is intact: ordinary work still runs and the error can be cleared
    x = torch.ones(1024, device="cuda")
    assert float(x.sum()) == 1024.0
    c.clear_error()
    assert c.status()["code"] == 0
    c.close()


def test_program_round_wait_times_out(cuda):
    c = _half_world(timeout_us=200_000)
    x = torch.ones(256, device="cuda")
    y = torch.zeros(256, device="cuda")
    prog = c.program("allreduce", "radix_batch", 256, 2, 1)
    c.run_program(prog, x, y)
    st = c.status()
    assert st["rc"] == N.ERR_TIMEOUT and st["code"] in (2, 3) and st["peer"] == 1
    c.close()


def test_flagged_line_wait_times_out(cuda):
    c = _half_world(timeout_us=200_000)
    x = torch.ones(64, device="cuda")
    y = torch.zeros(64, device="cuda")
    c.run_ll(0, x, y, 64)
    st = c.status()
    assert st["rc"] == N.ERR_TIMEOUT and st["code"] == 5 and st["peer"] == 1
    # an aborted communicator refuses further work quickly instead of waiting again
    c.run_ll(0, x, y, 64)
    assert c.status()["rc"] == N.ERR_TIMEOUT
    c.close()


def test_flagged_line_program_wait_times_out(cuda):
    """The push form of a step program: the line a missing peer owes never arrives, the poll gives up within its
    limit, the rank records which peer it waited for, and later levels and launches do no more work."""
    c = _half_world(timeout_us=200_000)
    x = torch.ones(256, device="cuda")
    y = torch.zeros(256, device="cuda")
    prog = c.program("allreduce", "radix_batch", 256, 2, 1, in_symmetric=True, out_symmetric=True)
    c.run_program(prog, x, y, mode="ll")
    st = c.status()
    assert st["rc"] == N.ERR_TIMEOUT and st["code"] == 5 and st["peer"] == 1
    c.run_program(prog, x, y, mode="ll")
    assert c.status()["rc"] == N.ERR_TIMEOUT
    z = torch.ones(1024, device="cuda")
    assert float(z.sum()) == 1024.0
    c.close()
