"""Two physical levels on GPUs: the box's GPUs are split into "boxes" of L ranks; inside
a box the collectives are this library's kernels on a sub-communicator, across boxes the
lanes use NCCL.  With 2 GPUs: 2 boxes of 1; with 4 or more also 2-rank boxes.  Needs >= 2 GPUs."""
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


def _inp(r, n):
    g = torch.Generator(device="cuda").manual_seed(77 + r)
    return torch.rand(n, generator=g, device="cuda") * 2 - 1


def _worker(rank, P, port, q):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=P, device_id=torch.device("cuda", rank))
        import configurable_hierarchical_allreduce_algorithms_b200 as chb
        from configurable_hierarchical_allreduce_algorithms_b200.parallel import hierarchy as H

        notes = []
        for L in [l for l in (1, 2, 4) if P % l == 0 and l < P]:
            intra_g, inter_g = H.split_world(L)
            comm = chb.Communicator.from_process_group(group=intra_g, backend="ipc", scratch_bytes=64 << 20, user_bytes=8 << 20)
            two = H.TwoLevel(H.DeviceLevel(comm), H.LibraryLevel(inter_g))
            assert (two.P, two.rank) == (P, rank)
            for n in (1, 1000, (1 << 18) + 5):
                ins = [_inp(r, n * P) for r in range(P)]
                exp = torch.stack([x.double() for x in ins]).sum(0)
                y = two.all_reduce(ins[rank])
                torch.testing.assert_close(y.double(), exp, rtol=1e-5, atol=1e-5 * P)
                y = two.reduce_scatter(ins[rank])
                torch.testing.assert_close(y.double(), exp[rank * n:(rank + 1) * n], rtol=1e-5, atol=1e-5 * P)
                y = two.all_gather(ins[rank][:n].contiguous())
                assert torch.equal(y, torch.cat([i[:n] for i in ins]))
            comm.check()
            torch.cuda.synchronize()
            dist.barrier()
            comm.close()
            notes.append(f"L={L} ok")
        dist.destroy_process_group()
        q.put((rank, "ok", "; ".join(notes)))
    except Exception:  # noqa: BLE001
        q.put((rank, "fail", traceback.format_exc()))


@pytest.mark.timeout(600)
def test_two_level_on_gpus():
    from conftest import gpus_for_test
    P = gpus_for_test(8)
    if P < 2:
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
    assert not bad, "\n".join(f"rank {r[0]}:\n{r[2]}" for r in bad)
    print(res[0][2])


def _native_worker(rank, P, name, q):
    try:
        torch.cuda.set_device(rank)
        import configurable_hierarchical_allreduce_algorithms_b200 as chb

        # no torch.distributed anywhere in this process
        comm = chb.Communicator.from_shared_memory(name, rank, P, scratch_bytes=64 << 20, user_bytes=8 << 20)
        assert (comm.P, comm.rank) == (P, rank) and comm.backend in ("ipc-native", "vmm-native")
        for n in (5, 4096, (1 << 18) + 1):
            ins = [_inp(r, n * P) for r in range(P)]
            exp = torch.stack([x.double() for x in ins]).sum(0)
            for algo in ("auto", "radix_batch", "ring"):
                y = chb.all_reduce(comm, ins[rank], algo=algo)
                torch.testing.assert_close(y.double(), exp, rtol=1e-5, atol=1e-5 * P)
            y = chb.all_gather(comm, ins[rank][:n].contiguous())
            assert torch.equal(y, torch.cat([i[:n] for i in ins]))
        # host buffers: chunked upload / allreduce / download pipeline
        ins = [_inp(r, (5 << 15) + 7) for r in range(P)]
        exp = torch.stack([x.double() for x in ins]).sum(0)
        hy = chb.all_reduce_host(comm, ins[rank].cpu().pin_memory(), chunk_elems=1 << 16, depth=2)
        torch.cuda.synchronize()
        torch.testing.assert_close(hy.double(), exp.cpu(), rtol=1e-5, atol=1e-5 * P)
        from configurable_hierarchical_allreduce_algorithms_b200.ops.host import HostAllReduce
        pipe = HostAllReduce(comm, torch.float32, chunk_elems=1 << 14, depth=2)
        n = (3 << 13) + 5                                   # several chunks with a ragged tail
        ins = [_inp(r, n * P) for r in range(P)]
        exp = torch.stack([x.double() for x in ins]).sum(0)
        part = pipe.reduce_scatter(ins[rank].cpu().pin_memory())
        full = pipe.all_gather(ins[rank][:n].cpu().pin_memory())
        torch.cuda.synchronize()
        torch.testing.assert_close(part.double(), exp[rank * n:(rank + 1) * n].cpu(), rtol=1e-5, atol=1e-5 * P)
        assert torch.equal(full, torch.cat([i[:n] for i in ins]).cpu())
        comm.barrier()
        comm.check()
        comm.close()
        q.put((rank, "ok", ""))
    except Exception:  # noqa: BLE001
        q.put((rank, "fail", traceback.format_exc()))


@pytest.mark.timeout(600)
def test_communicator_over_the_native_bootstrap():
    """One rank per GPU, rendezvous through POSIX shared memory: no process group is ever created."""
    from conftest import gpus_for_test
    P = gpus_for_test(4)
    if P < 2:
        pytest.skip("needs at least two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    name = f"/chb_test_{os.getpid()}"
    procs = [ctx.Process(target=_native_worker, args=(r, P, name, q)) for r in range(P)]
    for p in procs:
        p.start()
    res = [q.get(timeout=500) for _ in range(P)]
    for p in procs:
        p.join(60)
    bad = [r for r in res if r[1] != "ok"]
    assert not bad, "\n".join(f"rank {r[0]}:\n{r[2]}" for r in bad)
