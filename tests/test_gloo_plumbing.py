"""CPU plumbing: 4 gloo ranks replay the schedules with two-sided messages.

Equivalent of the reference's test driver run on 4 MPI ranks with k=2, b=1
(testing/custom_implementations/work_dir/all_reduce/main.cpp:43-76): int32
buffers of 1024 elements per rank, rank r's element i = (seed*31 + r*1009 + i) mod 97,
checked against naive sum / concat.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from configurable_hierarchical_allreduce_algorithms_b200.parallel import gloo_exec


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _val(r, n, seed=5):
    return ((seed * 31 + r * 1009 + torch.arange(n)) % 97).to(torch.int32)


def _worker(rank, P, port, cases, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=P)
    ok = True
    try:
        for (coll, algo, n, k, b) in cases:
            if coll == "allreduce":
                x = _val(rank, n * P)
                out = gloo_exec.run_collective(coll, algo, x, n * P, k, b)
                exp = sum(_val(r, n * P) for r in range(P))
            elif coll == "reduce_scatter":
                x = _val(rank, n * P)
                out = gloo_exec.run_collective(coll, algo, x, n, k, b)
                exp = sum(_val(r, n * P) for r in range(P))[rank * n:(rank + 1) * n]
            else:
                x = _val(rank, n)
                out = gloo_exec.run_collective(coll, algo, x, n, k, b)
                exp = torch.cat([_val(r, n) for r in range(P)])
            if not torch.equal(out, exp):
                ok = False
                print(f"rank {rank}: MISMATCH {coll}/{algo} n={n} k={k} b={b}", flush=True)
        flag = torch.tensor([1 if ok else 0])
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)   # AND over ranks, like the reference's reduce-scatter driver
        if rank == 0:
            q.put(int(flag.item()))
    finally:
        dist.destroy_process_group()
    os._exit(0)                       # skip the interpreter's teardown: helper threads of the transport may still be alive


def _launch(P, cases):
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, P, port, cases, q)) for r in range(P)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0, f"worker exit code {p.exitcode}"
    return q.get()


@pytest.mark.timeout(300)
def test_config1_four_gloo_ranks_k2_b1():
    cases = [("allreduce", "radix_batch", 1024, 2, 1), ("reduce_scatter", "radix_batch", 1024, 2, 1),
             ("allgather", "radix_batch", 1024, 2, 1)]
    assert _launch(4, cases) == 1


@pytest.mark.timeout(300)
def test_hierarchical_and_baselines_over_gloo():
    cases = [("allreduce", "radix_batch", 6, 2, 2), ("allreduce", "radix_batch", 6, 4, 4),
             ("reduce_scatter", "radix_batch", 5, 3, 2), ("allgather", "radix_batch", 7, 2, 4),
             ("allreduce", "ring", 5, 2, 1), ("allreduce", "recursive_doubling", 5, 2, 1),
             ("allreduce", "reduce_scatter_allgather", 5, 2, 1), ("allgather", "k_brucks", 3, 3, 1),
             ("reduce_scatter", "recursive_halving", 3, 2, 1), ("reduce_scatter", "radix_block", 3, 2, 2)]
    assert _launch(4, cases) == 1
