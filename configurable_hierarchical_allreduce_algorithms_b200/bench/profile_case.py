"""Small fixed workloads for profiler captures on ONE GPU (all ranks emulated
on it): a few launches of one kernel, inputs larger than L2, about a GB held.

    python -m configurable_hierarchical_allreduce_algorithms_b200.bench.profile_case --case interp_ar [--mib 32]
      interp_ar  8 emulated ranks, allreduce radix_batch k=2 b=1 on symmetric buffers (program interpreter)
      interp_kb  same with k=2 b=4 (hierarchical schedule: entry round + five rounds, pull interpreter)
      llprog_ar  8 emulated ranks, allreduce radix_batch k=2 b=2 of 256 KiB with flagged lines (four rounds, push)
      ll_ar      8 emulated ranks, one-shot flagged-line allreduce of 64 KiB
      ll2_ar     8 emulated ranks, two-shot flagged-line allreduce of 1 MiB
      fp8_rs     4 emulated ranks, fp8 block-scaled wire reduce-scatter, --mib MiB of bf16 per rank
      adam_flat  AdamW on a flat fp32 master of --mib MiB with bf16 parameter copy (data-parallel optimizer)
      noalloc    allocation-free one-shot allreduce, 8 ranks x 8 KiB
      copy1      single rank, allreduce of --mib MiB (degenerates to the local copy, HBM bound)
      bulk_ag    4 emulated ranks, allgather of --mib MiB per rank through the bulk-copy engine
      rs_adam    4 emulated ranks, reduce-scatter + AdamW on a shard of --mib MiB of gradients per rank
Prints the CUDA-event time per launch so the same command line can be checked without a profiler first.
"""
from __future__ import annotations

import argparse

import torch

from .. import all_reduce
from ..ops import fused
from ..parallel.comm import Communicator


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="interp_ar")
    ap.add_argument("--mib", type=int, default=32)
    ap.add_argument("--iters", type=int, default=5)
    a = ap.parse_args()
    torch.cuda.set_device(0)
    n = (a.mib << 20) // 4
    if a.case in ("interp_ar", "interp_kb", "ll_ar", "ll2_ar", "llprog_ar"):
        P = 8
        if a.case == "ll_ar":
            n = (64 << 10) // 4
        if a.case == "ll2_ar":
            n = (1 << 20) // 4
        if a.case == "llprog_ar":
            n = (256 << 10) // 4
        comm = Communicator.emulated(P, scratch_bytes=n * 4 + (8 << 20), user_bytes=2 * n * 4 + (1 << 20))
        xs, ys = comm.empty(n, torch.float32), comm.empty(n, torch.float32)
        for i, x in enumerate(xs):
            x.copy_(torch.rand(n, device="cuda") + i)
        kw = {"interp_ar": dict(algo="radix_batch:pull", k=2, b=1), "interp_kb": dict(algo="radix_batch:pull", k=2, b=4),
              "llprog_ar": dict(algo="radix_batch:ll", k=2, b=2),
              "ll_ar": dict(algo="ll"), "ll2_ar": dict(algo="ll2")}[a.case]
        fn = lambda: all_reduce(comm, xs, out=ys, **kw)
        nbytes = n * 4
    elif a.case == "bulk_ag":
        from .. import all_gather
        P = 4
        comm = Communicator.emulated(P, scratch_bytes=1 << 20, user_bytes=(P + 1) * n * 4 + (1 << 20))
        xs, ys = comm.empty(n, torch.float32), comm.empty(n * P, torch.float32)
        for i, x in enumerate(xs):
            x.copy_(torch.rand(n, device="cuda") + i)
        fn = lambda: all_gather(comm, xs, out=ys, algo="bulk")
        nbytes = n * 4 * P
    elif a.case == "copy1":
        comm = Communicator.emulated(1, scratch_bytes=1 << 20, user_bytes=2 * n * 4 + (1 << 20))
        x, y = comm.empty(n, torch.float32), comm.empty(n, torch.float32)
        x.copy_(torch.rand(n, device="cuda"))
        fn = lambda: all_reduce(comm, x, out=y)
        nbytes = n * 4
    elif a.case == "rs_adam":
        P = 4
        comm = Communicator.emulated(P, scratch_bytes=1 << 20, user_bytes=n * 4 + (1 << 20))
        shard = n // P // 4 * 4
        grads = comm.empty(shard * P, torch.float32)
        for g in grads:
            g.copy_(torch.randn(shard * P, device="cuda"))
        w = [torch.randn(shard, device="cuda") for _ in range(P)]
        m = [torch.zeros(shard, device="cuda") for _ in range(P)]
        v = [torch.zeros(shard, device="cuda") for _ in range(P)]
        p = [torch.zeros(shard, dtype=torch.bfloat16, device="cuda") for _ in range(P)]
        fn = lambda: fused.reduce_scatter_adam(comm, grads, w, m, v, p, lr=1e-3, step=1, grad_scale=0.25, use_multimem=False)
        nbytes = shard * P * 4
    elif a.case == "fp8_rs":
        P = 4
        nb = (a.mib << 20) // 2 // P // 128 * 128
        comm = Communicator.emulated(P, scratch_bytes=(a.mib << 20) + (1 << 20), user_bytes=1 << 20)
        xs = [torch.randn(nb * P, device="cuda").bfloat16() for _ in range(P)]
        ys = [torch.empty(nb, dtype=torch.bfloat16, device="cuda") for _ in range(P)]
        fn = lambda: fused.reduce_scatter_fp8(comm, xs, out=ys, scale=0.25)
        nbytes = nb * P * 2
    elif a.case == "adam_flat":
        comm = Communicator.emulated(1, scratch_bytes=1 << 20, user_bytes=1 << 20)
        g, w = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
        m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
        pb = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
        fn = lambda: fused.adam_flat(g, w, m, v, pb, lr=1e-3, step=1)
        nbytes = n * 4
    elif a.case == "noalloc":
        import ctypes as C
        from .. import _native as N
        from ..parallel.comm import DTYPES, OPS
        P, n = 8, 2048
        comm = Communicator.emulated(1, scratch_bytes=1 << 20, user_bytes=1 << 20)
        xs = [torch.randn(n, device="cuda") for _ in range(P)]
        ys = [torch.empty(n, device="cuda") for _ in range(P)]
        L = C.CDLL(str(N._LIB_PATH))
        L.chb_allreduce_oneshot_noalloc.argtypes = [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                                    C.c_int64, C.c_float, C.c_void_p, C.c_char_p, C.c_int]
        ip = (C.c_void_p * P)(*[t.data_ptr() for t in xs])
        op_ = (C.c_void_p * P)(*[t.data_ptr() for t in ys])
        fn = lambda: L.chb_allreduce_oneshot_noalloc(P, DTYPES[torch.float32], OPS["sum"], ip, op_, n, 1.0,
                                                     torch.cuda.current_stream().cuda_stream, None, 0)
        nbytes = n * 4
    else:
        raise SystemExit(f"unknown case {a.case}")
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    comm.check()
    print(f"case={a.case} bytes_per_rank={nbytes} ms_per_launch={e0.elapsed_time(e1) / a.iters:.4f}")
    comm.close()


if __name__ == "__main__":
    main()
