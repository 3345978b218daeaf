"""Communicator on heaps from the native virtual-memory allocator: peers mapped through shareable
allocation handles (file descriptors over the bootstrap), NVLink multicast alias bound natively, the
multimem kernels running without torch's symmetric memory.  Needs >= 2 GPUs; skipped where the platform
has no shareable handles.  Ranks leave only after a final barrier, with nothing in flight."""
import os
import traceback

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.multigpu


def _inp(r, n, dtype=torch.float32):
    g = torch.Generator(device="cuda").manual_seed(4000 + r)
    return (torch.rand(n, generator=g, device="cuda") * 2 - 1).to(dtype)


def _worker(rank, P, name, q):
    comm = None
    try:
        torch.cuda.set_device(rank)
        import configurable_hierarchical_allreduce_algorithms_b200 as chb
        from configurable_hierarchical_allreduce_algorithms_b200 import _native as N

        try:
            comm = chb.Communicator.from_shared_memory(name, rank, P, scratch_bytes=64 << 20, user_bytes=32 << 20, heap="vmm")
        except chb.CollectiveError as e:
            q.put((rank, "skip" if e.code == N.ERR_UNSUPPORTED else "fail", str(e)))
            return
        assert comm.backend == "vmm-native"
        notes = [f"multicast={comm.has_multicast}"]
        n = 1 << 16
        xs, ys = comm.empty(n * P, torch.float32), comm.empty(n * P, torch.float32)
        ins = [_inp(r, n * P) for r in range(P)]
        exp = torch.stack([x.double() for x in ins]).sum(0)
        xs.copy_(ins[rank])
        for algo in ("radix_batch:pull", "radix_batch:ll", "ring:pull", "ll2"):     # peer-mapped heaps
            ys.zero_()
            chb.all_reduce(comm, xs, out=ys, algo=algo)
            torch.testing.assert_close(ys.double(), exp, rtol=1e-5, atol=1e-5 * P)
        if comm.has_multicast:                                                       # the natively bound alias
            for algo in ("nvls", "nvls1"):
                ys.zero_()
                chb.all_reduce(comm, xs, out=ys, algo=algo, scale=0.5)
                torch.testing.assert_close(ys.double(), exp * 0.5, rtol=1e-5, atol=1e-5 * P)
            part = chb.reduce_scatter(comm, xs, algo="nvls")
            torch.testing.assert_close(part.double(), exp[rank * n:(rank + 1) * n], rtol=1e-5, atol=1e-5 * P)
            ys.zero_()
            chb.all_gather(comm, xs[:n], out=ys, algo="nvls")
            torch.cuda.synchronize()
            assert torch.equal(ys, torch.cat([i[:n] for i in ins]))
            xb, yb = xs.view(torch.bfloat16), ys.view(torch.bfloat16)
            insb = [_inp(r, 2 * n * P, torch.bfloat16) for r in range(P)]
            xb.copy_(insb[rank])
            comm.barrier()
            chb.all_reduce(comm, xb, out=yb, algo="nvls")
            torch.testing.assert_close(yb.double(), torch.stack([x.double() for x in insb]).sum(0), rtol=2e-2, atol=2e-2 * P)
            notes.append("multimem kernels ok")
        comm.barrier()
        comm.check()
        q.put((rank, "ok", "; ".join(notes)))
    except Exception:  # noqa: BLE001
        q.put((rank, "fail", traceback.format_exc()))
    finally:
        # also after a failed check: leave in order (the ranks meet, unmap and unbind, meet again, release), so that no
        # rank's memory is still bound to the multicast object when a process goes away
        try:
            if comm is not None:
                torch.cuda.synchronize()
                comm.close()
        except Exception:  # noqa: BLE001
            pass


@pytest.mark.timeout(600)
def test_native_virtual_memory_heaps_and_multicast():
    from conftest import gpus_for_test
    P = gpus_for_test(4)
    if P < 2:
        pytest.skip("needs at least two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    name = f"/chb_vmm_{os.getpid()}"
    procs = [ctx.Process(target=_worker, args=(r, P, name, q)) for r in range(P)]
    for p in procs:
        p.start()
    res = [q.get(timeout=500) for _ in range(P)]
    for p in procs:
        p.join(60)
    if all(r[1] == "skip" for r in res):
        pytest.skip("no shareable allocation handles here: " + res[0][2])
    bad = [r for r in res if r[1] != "ok"]
    assert not bad, "\n".join(f"rank {r[0]}:\n{r[2]}" for r in bad)
    print(res[0][2])
