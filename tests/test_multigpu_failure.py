"""A rank that does not join a collective: the others' bounded waits run out,
the status names the missing peer, and every CUDA context stays usable.

The failure is made on the host (rank 1 simply skips the second call and stays
alive, so no peer memory disappears under a running kernel), NVLS is off in
NCCL and in this library, and nothing faults or hangs a GPU.
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


def _worker(rank, P, port, done, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", CHB_NVLS="0")
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=P, device_id=torch.device("cuda", rank))
        import configurable_hierarchical_allreduce_algorithms_b200 as chb

        comm = chb.Communicator.from_process_group(backend="ipc", scratch_bytes=8 << 20, user_bytes=1 << 20,
                                                   timeout_us=300_000)
        x = torch.full((4096,), float(rank + 1), device="cuda")
        y = chb.all_reduce(comm, x, algo="radix_batch")          # everybody joins: fine
        torch.cuda.synchronize()
        assert float(y[0]) == sum(range(1, P + 1))
        comm.check()
        dist.barrier()
        torch.cuda.synchronize()
        if rank == 1:
            done.wait(60)                                        # never joins the second call, stays alive
            result = "skipped"
        else:
            chb.all_reduce(comm, x, algo="radix_batch")          # peer 1 is missing
            st = comm.status()
            assert st["rc"] == 6 and st["peer"] == 1, st
            try:
                comm.check()
                raise AssertionError("expected a timeout")
            except chb.CollectiveError as e:
                assert "timeout" in str(e)
            z = torch.ones(1024, device="cuda").sum()            # the context still works
            assert float(z) == 1024.0
            result = f"timeout reported: code {st['code']} peer {st['peer']} round {st['round']}"
            dist.barrier() if P > 2 else None
            done.set()
        torch.cuda.synchronize()
        comm.close()
        q.put((rank, "ok", result))
        dist.destroy_process_group()
    except Exception:  # noqa: BLE001
        done.set()
        q.put((rank, "fail", traceback.format_exc()))


@pytest.mark.timeout(300)
def test_missing_rank_is_reported_not_hung():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    P = 2
    ctx = mp.get_context("spawn")
    q, done = ctx.Queue(), ctx.Event()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, P, port, done, q)) for r in range(P)]
    for p in procs:
        p.start()
    res = [q.get(timeout=200) for _ in range(P)]
    for p in procs:
        p.join(60)
    bad = [r for r in res if r[1] != "ok"]
    assert not bad, "\n".join(f"rank {r[0]}:\n{r[2]}" for r in bad)
