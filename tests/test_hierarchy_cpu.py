"""Two physical levels on CPU: 4 and 6 gloo ranks arranged as boxes x ranks-per-box.

The intra-box level and the lane level are each run either as a step program over
two-sided messages or by the library's collectives; results are compared with the
definitions of the collectives.  Mirrors the reference's way of testing several
"nodes" on one machine (oversubscribed ranks with a virtual group size b,
testing/Makefile:83-95).
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from configurable_hierarchical_allreduce_algorithms_b200.parallel import hierarchy as H


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _val(r, n):
    return ((r * 1009 + torch.arange(n) * 31 + 7) % 97).to(torch.float32)


def _worker(rank, P, L, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=P)
    bad = []
    try:
        intra_g, inter_g = H.split_world(L)
        combos = {
            "program/program": H.TwoLevel(H.GlooLevel(intra_g, "radix_batch", 2, 1), H.GlooLevel(inter_g, "ring")),
            "program/library": H.TwoLevel(H.GlooLevel(intra_g, "ring"), H.LibraryLevel(inter_g)),
            "library/program": H.TwoLevel(H.LibraryLevel(intra_g), H.GlooLevel(inter_g, "radix_batch", 2, 1)),
        }
        for name, two in combos.items():
            assert two.P == P and two.rank == rank
            for n in (1, 5, 64):
                x = _val(rank, n * P)
                exp = sum(_val(r, n * P) for r in range(P))
                if not torch.equal(two.all_reduce(x), exp):
                    bad.append((name, "allreduce", n))
                if not torch.equal(two.all_reduce(x[:n * P - 1]), exp[:n * P - 1]):    # not a multiple of anything
                    bad.append((name, "allreduce ragged", n))
                if not torch.equal(two.reduce_scatter(x), exp[rank * n:(rank + 1) * n]):
                    bad.append((name, "reduce_scatter", n))
                if not torch.equal(two.all_gather(_val(rank, n)), torch.cat([_val(r, n) for r in range(P)])):
                    bad.append((name, "allgather", n))
            mx = two.all_reduce(_val(rank, 8), op="max")
            if not torch.equal(mx, torch.stack([_val(r, 8) for r in range(P)]).max(0).values):
                bad.append((name, "allreduce max", 8))
        flag = torch.tensor([0 if bad else 1])
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if bad:
            print(f"rank {rank}: {bad}", flush=True)
        if rank == 0:
            q.put(int(flag.item()))
    finally:
        dist.destroy_process_group()
    os._exit(0)                       # skip the interpreter's teardown: helper threads of the transport may still be alive


@pytest.mark.parametrize("P,L", [(4, 2), (6, 3), (6, 2), (4, 1), (4, 4)])
def test_two_level_collectives(P, L):
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, P, L, port, q)) for r in range(P)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0, f"worker exit code {p.exitcode}"
    assert q.get() == 1


def test_split_world_rejects_bad_box_size():
    with pytest.raises(Exception):
        # no process group: the argument check comes after the world lookup, either way it must raise
        H.split_world(3)
