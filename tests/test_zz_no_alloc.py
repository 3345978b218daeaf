"""The allocation-free one-shot allreduce (csrc/api/chb_noalloc.h).

Some users of this library have to run a small allreduce at a point where they
may not allocate device memory: their memory pool is frozen or nearly full, a
host framework owns the allocator and only hands them buffers, or a cudaMalloc
would synchronise the device in the middle of a latency-critical loop.  They
cannot build a communicator (it allocates a heap, control blocks and program
tables), so they call `chb_allreduce_oneshot_noalloc`, whose working memory is
a fixed array inside the library image.

The test calls that entry point through its exported C symbol, twice in a row
(the second call meets the first call's leftovers in the shared array), and
compares each result with the communicator-based flagged-line kernel, using
the tolerances of the other GPU tests.  It also checks that a request beyond
the fixed capacity is refused before anything is launched.
"""
import ctypes as C

import pytest
import torch

from configurable_hierarchical_allreduce_algorithms_b200 import _native as N
from configurable_hierarchical_allreduce_algorithms_b200.parallel.comm import DTYPES, OPS, Communicator
import configurable_hierarchical_allreduce_algorithms_b200 as chb

pytestmark = pytest.mark.gpu

MAX_RANKS, MAX_BYTES = 8, 8192


def _entry():
    lib = C.CDLL(str(N._LIB_PATH))   # the exported C symbol, no Python wrapper in between
    fn = lib.chb_allreduce_oneshot_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int64,
                   C.c_float, C.c_void_p, C.c_char_p, C.c_int]
    st = lib.chb_noalloc_status
    st.restype = C.c_int
    st.argtypes = [C.c_void_p]
    return fn, st


def _call(fn, ins, outs, op="sum", scale=1.0):
    P = len(ins)
    err = C.create_string_buffer(256)
    rc = fn(P, DTYPES[ins[0].dtype], OPS[op], (C.c_void_p * P)(*[t.data_ptr() for t in ins]),
            (C.c_void_p * P)(*[t.data_ptr() for t in outs]), ins[0].numel(), scale,
            torch.cuda.current_stream().cuda_stream, err, len(err))
    return rc, err.value.decode()


def _inputs(P, n, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if dtype == torch.int32:
        return [torch.randint(-50, 50, (n,), generator=g, device="cuda", dtype=dtype) for _ in range(P)]
    return [(torch.rand(n, generator=g, device="cuda") * 2 - 1).to(dtype) for _ in range(P)]


def test_matches_communicator_kernel_on_two_calls_in_a_row(cuda):
    fn, status = _entry()
    # buffers are made before the calls: the entry point itself allocates nothing
    cases = [(4, 1000, torch.float32, "sum", 1.0), (8, 2048, torch.float32, "sum", 0.125),
             (3, 777, torch.bfloat16, "sum", 1.0), (4, 64, torch.int32, "max", 1.0)]
    for P, n, dtype, op, scale in cases:
        comm = Communicator.emulated(P, scratch_bytes=1 << 20, user_bytes=1 << 20)
        for call in range(2):   # second call sees the first call's lines and control words
            ins = _inputs(P, n - call * 5, dtype, seed=100 + call)
            outs = [torch.full_like(x, 7) for x in ins]
            before = torch.cuda.memory_allocated()
            rc, msg = _call(fn, ins, outs, op, scale)
            assert rc == 0, msg
            assert status(torch.cuda.current_stream().cuda_stream) == 0
            assert torch.cuda.memory_allocated() == before
            want = chb.all_reduce(comm, ins, op=op, algo="ll", scale=scale)
            torch.cuda.synchronize()
            # an oracle that is none of this library's kernels: the same reduction in fp64 / int64 by PyTorch
            hi = torch.float64 if dtype.is_floating_point else torch.int64
            st = torch.stack([x.to(hi) for x in ins])
            oracle = (st.sum(0) if op == "sum" else st.max(0).values) * (scale if dtype.is_floating_point else 1)
            for r in range(P):
                if dtype.is_floating_point:
                    tol = {torch.float32: 1e-5, torch.bfloat16: 2e-2}[dtype]
                    torch.testing.assert_close(outs[r].double(), oracle, rtol=tol, atol=tol * P)
                else:
                    assert torch.equal(outs[r].to(hi), oracle)
            for r in range(P):
                if dtype.is_floating_point:
                    tol = {torch.float32: 1e-5, torch.bfloat16: 2e-2}[dtype]
                    torch.testing.assert_close(outs[r].float(), want[r].float(), rtol=tol, atol=tol * P)
                else:
                    assert torch.equal(outs[r], want[r])
        comm.check()
        comm.close()


def test_refuses_what_does_not_fit(cuda):
    fn, _ = _entry()
    too_long = MAX_BYTES // 4 + 1
    ins = _inputs(2, too_long, torch.float32, 1)
    outs = [torch.zeros_like(x) for x in ins]
    rc, msg = _call(fn, ins, outs)
    assert rc == N.ERR_COUNT and "exceed" in msg and str(MAX_BYTES) in msg
    assert all(float(o.abs().sum()) == 0.0 for o in outs)      # nothing ran
    many = _inputs(MAX_RANKS + 1, 8, torch.float32, 2)
    rc, msg = _call(fn, many, [torch.zeros_like(x) for x in many])
    assert rc == N.ERR_COUNT and "capacity" in msg
    # a count so large that count * element size wraps around is refused like any other, not taken for a small one
    small = _inputs(2, 8, torch.float32, 4)
    souts = [torch.zeros_like(x) for x in small]
    err = C.create_string_buffer(256)
    rc = fn(2, DTYPES[torch.float32], OPS["sum"], (C.c_void_p * 2)(*[t.data_ptr() for t in small]),
            (C.c_void_p * 2)(*[t.data_ptr() for t in souts]), 1 << 62, 1.0,
            torch.cuda.current_stream().cuda_stream, err, len(err))
    assert rc == N.ERR_COUNT and "exceed" in err.value.decode()
    # the largest request that fits works
    ins = _inputs(MAX_RANKS, MAX_BYTES // 4, torch.float32, 3)
    outs = [torch.zeros_like(x) for x in ins]
    rc, msg = _call(fn, ins, outs)
    assert rc == 0, msg
    torch.cuda.synchronize()
    torch.testing.assert_close(outs[5], torch.stack(ins).sum(0), rtol=1e-5, atol=1e-4)
