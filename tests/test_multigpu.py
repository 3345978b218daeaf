"""One rank per GPU over NVLink: heaps exchanged as cudaIpc handles or through
torch's symmetric memory (which adds the NVLS multicast alias), every kernel
family against a locally computed reference.  Needs >= 2 GPUs."""
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


def _inp(r, n, dtype):
    g = torch.Generator(device="cuda").manual_seed(1000 + r)
    return (torch.rand(n, generator=g, device="cuda") * 2 - 1).to(dtype)


def _worker(rank, P, port, backend, q):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=P, device_id=torch.device("cuda", rank))
        import configurable_hierarchical_allreduce_algorithms_b200 as chb

        try:
            comm = chb.Communicator.from_process_group(backend=backend, scratch_bytes=(48 << 20) * P, user_bytes=96 << 20)
        except Exception:  # noqa: BLE001
            if backend == "symm_mem":   # the VMM / multicast rendezvous is not available on every box
                q.put((rank, "skip", traceback.format_exc()))
                dist.destroy_process_group()
                return
            raise
        assert comm.backend == backend, (comm.backend, getattr(comm, "_symm_mem_error", None))
        notes = [f"backend={comm.backend} nvls={comm.has_multicast}"]
        tol = {torch.float32: 1e-5, torch.bfloat16: 2e-2}

        def close(a, b, dtype):
            torch.testing.assert_close(a.double(), b.double(), rtol=tol[dtype], atol=tol[dtype] * P)

        divs = [b for b in (1, 2, 4, 8) if P % b == 0]
        for dtype in (torch.float32, torch.bfloat16):
            for n in (1, 3, 1000, 1 << 16, (1 << 20) + 3):
                N = n * P
                ins = [_inp(r, N, dtype) for r in range(P)]
                exp = torch.stack([x.double() for x in ins]).sum(0)
                x = ins[rank]
                algos = [("ll", 2, 1)] if N * x.element_size() <= comm.ll_max_bytes else []
                algos += [("radix_batch", 2, b) for b in divs] + [("radix_batch", 4, divs[-1]), ("ring", 2, 1),
                                                                  ("recursive_doubling", 2, 1), ("auto", 2, 1)]
                for algo, k, b in algos:
                    y = chb.all_reduce(comm, x, algo=algo, k=k, b=b)
                    close(y, exp, dtype)
                    y = chb.reduce_scatter(comm, x, algo=algo if algo not in ("recursive_doubling",) else "radix", k=k, b=b)
                    close(y, exp[rank * n:(rank + 1) * n], dtype)
                    y = chb.all_gather(comm, x[:n].contiguous(), algo=algo if algo != "recursive_doubling" else "k_brucks", k=k, b=b)
                    assert torch.equal(y, torch.cat([i[:n] for i in ins]))
                comm.check()
        # symmetric buffers: zero-copy programs, NVLS kernels
        n = 1 << 18
        N = n * P
        xs = comm.empty(N, torch.float32)
        ys = comm.empty(N, torch.float32)
        ins = [_inp(r, N, torch.float32) for r in range(P)]
        exp = torch.stack([x.double() for x in ins]).sum(0)
        xs.copy_(ins[rank])
        torch.cuda.synchronize()
        dist.barrier()
        chb.all_reduce(comm, xs, out=ys, algo="radix_batch", k=2, b=1)
        close(ys, exp, torch.float32)
        if comm.has_multicast:
            for algo in ("nvls", "nvls1"):
                ys.zero_()
                chb.all_reduce(comm, xs, out=ys, algo=algo, scale=0.5)
                close(ys, exp * 0.5, torch.float32)
            y2 = chb.reduce_scatter(comm, xs, algo="nvls")
            close(y2, exp[rank * n:(rank + 1) * n], torch.float32)
            ys.zero_()
            chb.all_gather(comm, xs[:n], out=ys, algo="nvls")
            torch.cuda.synchronize()
            assert torch.equal(ys, torch.cat([i[:n] for i in ins]))
            xb, yb = xs.view(torch.bfloat16), ys.view(torch.bfloat16)
            insb = [_inp(r, 2 * N, torch.bfloat16) for r in range(P)]
            xb.copy_(insb[rank])
            torch.cuda.synchronize()
            dist.barrier()
            chb.all_reduce(comm, xb, out=yb, algo="nvls")
            close(yb, torch.stack([x.double() for x in insb]).sum(0), torch.bfloat16)
            notes.append("nvls kernels ok")
        # ---- the reference-compatible C entry points, called through their exported symbols
        import ctypes as C
        from configurable_hierarchical_allreduce_algorithms_b200 import _native as NN
        L = C.CDLL(str(NN._LIB_PATH))
        vp, i32, i64 = C.c_void_p, C.c_int, C.c_int64
        L.chb_set_stream.argtypes = [vp]
        L.chb_set_stream(torch.cuda.current_stream().cuda_stream)
        cnt = 4096 * P
        a = _inp(rank, cnt, torch.float32)
        full = torch.stack([_inp(r, cnt, torch.float32).double() for r in range(P)]).sum(0)
        o = torch.zeros(cnt, device="cuda")
        L.all_reduce_radix_batch.argtypes = [vp, vp, i32, i32, i32, vp, i32, i32]
        assert L.all_reduce_radix_batch(a.data_ptr(), o.data_ptr(), cnt, NN.F32, NN.SUM, comm.handle, 2, divs[-1]) == 0
        close(o, full, torch.float32)
        L.MPICH_Allreduce_ring.argtypes = [vp, vp, i32, i32, i32, vp]
        o.zero_()
        assert L.MPICH_Allreduce_ring(a.data_ptr(), o.data_ptr(), cnt, NN.F32, NN.SUM, comm.handle) == 0
        close(o, full, torch.float32)
        L.reduce_scatter_radix_batch.argtypes = [vp, vp, i64, i32, i32, vp, i32, i32]
        inplace = a.clone()
        assert L.reduce_scatter_radix_batch(C.c_void_p(-1), inplace.data_ptr(), 4096, NN.F32, NN.SUM, comm.handle, 2, 1) == 0   # CHB_IN_PLACE
        close(inplace[:4096], full[rank * 4096:(rank + 1) * 4096], torch.float32)
        L.allgather_radix_batch.argtypes = [vp, i32, i32, vp, vp, i32, i32]
        og = torch.zeros(cnt, device="cuda")
        assert L.allgather_radix_batch(a.data_ptr(), 4096, NN.F32, og.data_ptr(), comm.handle, 2, divs[-1]) == 0
        torch.cuda.synchronize()
        assert torch.equal(og, torch.cat([_inp(r, cnt, torch.float32)[:4096] for r in range(P)]))
        assert L.all_reduce_radix_batch(a.data_ptr(), o.data_ptr(), cnt - 1, NN.F32, NN.SUM, comm.handle, 2, 1) == NN.ERR_COUNT
        L.MPICH_reduce_scatter_k_nomial.argtypes = [vp, vp, i32, i32, i32, vp, i32]
        okn = torch.zeros(4096, device="cuda")
        assert L.MPICH_reduce_scatter_k_nomial(a.data_ptr(), okn.data_ptr(), 4096, NN.F32, NN.SUM, comm.handle, 3) == 0
        close(okn, full[rank * 4096:(rank + 1) * 4096], torch.float32)
        # all-to-all-v: rank s sends 100 * (s + 1) + 10 * d elements to rank d, packed
        cnt_of = lambda s_, d_: 100 * (s_ + 1) + 10 * d_
        sc = (C.c_int * P)(*[cnt_of(rank, d) for d in range(P)])
        rc_ = (C.c_int * P)(*[cnt_of(s_, rank) for s_ in range(P)])
        sd = (C.c_int * P)(*[sum(cnt_of(rank, d) for d in range(j)) for j in range(P)])
        rd = (C.c_int * P)(*[sum(cnt_of(s_, rank) for s_ in range(j)) for j in range(P)])
        src_of = lambda s_: torch.arange(sum(cnt_of(s_, d) for d in range(P)), device="cuda", dtype=torch.int32) + 100000 * s_
        mine = src_of(rank)
        got = torch.full((sum(cnt_of(s_, rank) for s_ in range(P)),), -1, device="cuda", dtype=torch.int32)
        L.tuna2_algorithm.argtypes = [i32, i32, vp, C.POINTER(C.c_int), C.POINTER(C.c_int), i32, vp, C.POINTER(C.c_int),
                                      C.POINTER(C.c_int), i32, vp]
        for radix, batch in ((2, 1), (3, 2)):
            got.fill_(-1)
            assert L.tuna2_algorithm(radix, batch, mine.data_ptr(), sc, sd, NN.I32, got.data_ptr(), rc_, rd, NN.I32, comm.handle) == 0
            torch.cuda.synchronize()
            exp_parts = []
            for s_ in range(P):
                off = sum(cnt_of(s_, d) for d in range(rank))
                exp_parts.append(src_of(s_)[off:off + cnt_of(s_, rank)])
            assert torch.equal(got, torch.cat(exp_parts)), (radix, batch)
        # ---- fp8 block-scaled wire reduce-scatter against the exact result
        from configurable_hierarchical_allreduce_algorithms_b200.ops import fused
        nb = 128 * 512
        ab = _inp(rank, nb * P, torch.bfloat16)
        exact = torch.stack([_inp(r, nb * P, torch.bfloat16).double() for r in range(P)]).sum(0)[rank * nb:(rank + 1) * nb]
        got = fused.reduce_scatter_fp8(comm, ab)
        rel = (got.double() - exact).norm() / exact.norm()
        assert rel < 0.05, rel
        notes.append(f"fp8 wire rel err {float(rel):.4f}")
        for _ in range(20):   # back-to-back mixed launches
            chb.all_reduce(comm, xs, out=ys)
            chb.all_reduce(comm, xs[:256], out=ys[:256])
        comm.barrier()
        comm.check()
        dist.barrier()
        comm.close()
        dist.destroy_process_group()
        q.put((rank, "ok", "; ".join(notes)))
    except Exception:  # noqa: BLE001
        q.put((rank, "fail", traceback.format_exc()))


def _launch(P, backend):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, P, port, backend, q)) for r in range(P)]
    for p in procs:
        p.start()
    res = []
    for _ in range(P):
        res.append(q.get(timeout=600))
    for p in procs:
        p.join(60)
    if all(r[1] == "skip" for r in res):
        pytest.skip("symmetric-memory rendezvous unavailable: " + res[0][2][-400:])
    bad = [r for r in res if r[1] != "ok"]
    assert not bad, "\n".join(f"rank {r[0]}:\n{r[2]}" for r in bad)
    return res


def _ngpus():
    """GPUs a test world uses: see conftest.gpus_for_test (CHB_TEST_MAX_GPUS widens it up to all eight)."""
    from conftest import gpus_for_test
    return gpus_for_test(8)


@pytest.mark.timeout(900)
@pytest.mark.parametrize("backend", ["ipc", "symm_mem"])
def test_all_gpus(backend):
    P = _ngpus()
    if P < 2:
        pytest.skip("needs at least two GPUs")
    os.environ.setdefault("NCCL_DEBUG", "WARN")
    res = _launch(P, backend)
    print(res[0][2])
