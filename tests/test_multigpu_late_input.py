"""A peer-visible input that one rank produces late must never be read early.

Rank `late` queues a long sleep kernel and then the fill of its symmetric input on its stream before it
calls the collective; the other rank calls at once and is therefore inside the collective long before the
late rank's input exists.  The pull interpreter reads peers' symmetric inputs in place, so the result is
only right if readers wait for the owner to enter the collective.  Compared with NCCL on the same data
(bit for bit at two ranks: one fp32 addition, commutative).  Needs >= 2 GPUs.
"""
import os
import socket
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.multigpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, P, port, q):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=P, device_id=torch.device("cuda", rank))
        import configurable_hierarchical_allreduce_algorithms_b200 as chb

        comm = chb.Communicator.from_process_group(backend="ipc", scratch_bytes=64 << 20, user_bytes=64 << 20)
        n = 1 << 20
        xs, ys = comm.empty(n, torch.float32), comm.empty(n, torch.float32)
        bad = []
        for it in range(50):
            g = torch.Generator(device="cuda").manual_seed(7919 * it + rank)
            fresh = torch.rand(n, generator=g, device="cuda") * 2 - 1
            ref = fresh.clone()
            dist.all_reduce(ref)
            torch.cuda.synchronize()
            dist.barrier()
            if rank == it % P:
                torch.cuda._sleep(15_000_000)        # several milliseconds before this rank's input exists
            xs.copy_(fresh)
            algo = ("radix_batch:pull", "ring:pull", "recursive_doubling:pull")[it % 3]
            chb.all_reduce(comm, xs, out=ys, algo=algo, k=2, b=1)
            torch.cuda.synchronize()
            if not torch.equal(ys, ref) and not torch.allclose(ys, ref, rtol=1e-6, atol=1e-6):
                bad.append((it, algo, float((ys - ref).abs().max())))
        comm.check()
        dist.barrier()
        comm.close()
        dist.destroy_process_group()
        q.put((rank, "fail" if bad else "ok", repr(bad[:5])))
    except Exception:  # noqa: BLE001
        q.put((rank, "fail", traceback.format_exc()))


@pytest.mark.timeout(600)
def test_late_symmetric_input_is_not_read_early():
    P = 2
    if not torch.cuda.is_available() or torch.cuda.device_count() < P:
        pytest.skip("needs at least two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, P, port, q)) for r in range(P)]
    for p in procs:
        p.start()
    res = [q.get(timeout=500) for _ in range(P)]
    for p in procs:
        p.join(60)
    bad = [r for r in res if r[1] != "ok"]
    assert not bad, "\n".join(f"rank {r[0]}: {r[2]}" for r in bad)
