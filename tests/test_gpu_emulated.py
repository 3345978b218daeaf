"""Kernels on a real GPU with all ranks emulated on that one device.

Each kernel is compared against a plain PyTorch fp32 / fp64 reference of the
same collective.  The emulated world runs the same kernels as a multi-GPU
world: the peers' heaps are slices of one allocation and one cooperative
launch executes all ranks.
"""
import pytest
import torch

import configurable_hierarchical_allreduce_algorithms_b200 as chb
from configurable_hierarchical_allreduce_algorithms_b200.parallel.comm import Communicator

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def comms(cuda):
    made = {}

    def get(P):
        if P not in made:
            made[P] = Communicator.emulated(P, scratch_bytes=96 << 20, user_bytes=32 << 20)
        return made[P]

    yield get
    for c in made.values():
        c.close()


def make_inputs(P, n, dtype, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if dtype in (torch.int32, torch.int64):
        return [torch.randint(-50, 50, (n,), generator=g, device="cuda", dtype=dtype) for _ in range(P)]
    if dtype == torch.uint8:
        return [torch.randint(0, 8, (n,), generator=g, device="cuda", dtype=torch.int32).to(dtype) for _ in range(P)]
    return [(torch.rand(n, generator=g, device="cuda", dtype=torch.float32) * 2 - 1).to(dtype) for _ in range(P)]


def ref_reduce(ins, op):
    hi = torch.float64 if ins[0].dtype.is_floating_point else torch.int64
    st = torch.stack([x.to(hi) for x in ins])
    return {"sum": st.sum(0), "max": st.max(0).values, "min": st.min(0).values}[op]


def check(out, exp, dtype, P):
    if dtype.is_floating_point:
        tol = {torch.float32: 1e-5, torch.float64: 1e-12, torch.bfloat16: 2e-2, torch.float16: 2e-3}[dtype]
        torch.testing.assert_close(out.to(torch.float64), exp.to(torch.float64), rtol=tol, atol=tol * P)
    else:
        assert torch.equal(out.to(torch.int64), exp.to(torch.int64))


AR_CASES = [("radix_batch", 2, 1), ("radix_batch", 2, 2), ("radix_batch", 4, 4), ("radix_batch", 2, 8),
            ("radix_batch", 8, 8), ("radix_batch", 3, 4), ("ring", 2, 1), ("recursive_doubling", 2, 1),
            ("reduce_scatter_allgather", 2, 1), ("k_reduce_scatter_allgather", 4, 1),
            ("recursive_multiplying", 3, 1), ("recursive_exchange", 4, 1), ("inter_reduce_exchange_bcast", 2, 2),
            ("semi_radix_batch", 2, 2), ("custom", 2, 2)]


@pytest.mark.parametrize("algo,k,b", AR_CASES)
def test_allreduce_programs(comms, algo, k, b):
    P = 8
    comm = comms(P)
    if P % b:
        pytest.skip("b must divide P")
    for dtype, n in ((torch.float32, 8 * 1024), (torch.bfloat16, 8 * 33), (torch.int32, 8 * 3), (torch.float32, 8)):
        ins = make_inputs(P, n, dtype)
        outs = chb.all_reduce(comm, ins, algo=algo, k=k, b=b)
        exp = ref_reduce(ins, "sum")
        for r in range(P):
            check(outs[r], exp, dtype, P)
    comm.check()


@pytest.mark.parametrize("P", [2, 3, 4, 6, 8])
def test_three_collectives_radix_batch(comms, P):
    comm = comms(P)
    for b in [d for d in (1, 2, 3, 4, 8) if P % d == 0]:
        for k in (2, 4):
            for n in (1, 3, 31, 127, 2048):
                ins = make_inputs(P, n * P, torch.float32, seed=n)
                exp = ref_reduce(ins, "sum")
                outs = chb.all_reduce(comm, ins, algo="radix_batch", k=k, b=b)
                for r in range(P):
                    check(outs[r], exp, torch.float32, P)
                outs = chb.reduce_scatter(comm, ins, algo="radix_batch", k=k, b=b)
                for r in range(P):
                    check(outs[r], exp[r * n:(r + 1) * n], torch.float32, P)
                blocks = [x[:n].contiguous() for x in ins]
                outs = chb.all_gather(comm, blocks, algo="radix_batch", k=k, b=b)
                cat = torch.cat(blocks)
                for r in range(P):
                    assert torch.equal(outs[r], cat)
    comm.check()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.int32, torch.float64, torch.int64])
@pytest.mark.parametrize("op", ["sum", "max", "min"])
def test_dtypes_ops(comms, dtype, op):
    P = 4
    comm = comms(P)
    for n in (4, 1000):
        ins = make_inputs(P, n * P, dtype)
        exp = ref_reduce(ins, op)
        for algo, k, b in (("radix_batch", 2, 2), ("ll", 2, 1)):
            outs = chb.all_reduce(comm, ins, op=op, algo=algo, k=k, b=b)
            for r in range(P):
                check(outs[r], exp, dtype, P)
    comm.check()


@pytest.mark.parametrize("algo", ["pairwise", "ring", "recursive_halving", "recursive_doubling", "radix", "radix_block"])
def test_reduce_scatter_baselines(comms, algo):
    for P in (4, 6, 8):
        comm = comms(P)
        n = 257
        ins = make_inputs(P, n * P, torch.float32)
        exp = ref_reduce(ins, "sum")
        outs = chb.reduce_scatter(comm, ins, algo=algo, k=3, b=2)
        for r in range(P):
            check(outs[r], exp[r * n:(r + 1) * n], torch.float32, P)
        comm.check()


@pytest.mark.parametrize("algo", ["k_brucks", "ring", "recursive_doubling", "linear"])
def test_allgather_baselines(comms, algo):
    for P in (4, 8):
        comm = comms(P)
        blocks = make_inputs(P, 1001, torch.bfloat16)
        outs = chb.all_gather(comm, blocks, algo=algo, k=3)
        cat = torch.cat(blocks)
        for r in range(P):
            assert torch.equal(outs[r], cat)
        comm.check()


def test_all_to_all_and_gather(comms):
    P = 8
    comm = comms(P)
    n = 100
    ins = make_inputs(P, n * P, torch.float32)
    # every schedule in both execution modes, and as the library chooses (flagged lines at this size)
    for algo, k, b in (("tuna", 2, 1), ("tuna", 3, 2), ("linear", 2, 1)):
        for mode in ("", ":pull", ":ll"):
            outs = chb.all_to_all(comm, ins, algo=algo + mode, k=k, b=b)
            for r in range(P):
                exp = torch.cat([ins[s][r * n:(r + 1) * n] for s in range(P)])
                assert torch.equal(outs[r], exp), (algo, mode, r)
    blocks = [x[:n].contiguous() for x in ins]
    outs = chb.gather(comm, blocks, root=5, k=3)
    assert torch.equal(outs[5], torch.cat(blocks))
    comm.check()


@pytest.mark.parametrize("P", [2, 4, 8])
def test_flagged_line_kernels(comms, P):
    comm = comms(P)
    for dtype in (torch.float32, torch.bfloat16):
        for n in (1, 2, 3, 7, 64, 1000, 8192):
            ins = make_inputs(P, n * P, dtype, seed=n)
            exp = ref_reduce(ins, "sum")
            outs = chb.all_reduce(comm, ins, algo="ll")
            for r in range(P):
                check(outs[r], exp, dtype, P)
            # bit-identical on every rank: all ranks add in rank order
            for r in range(1, P):
                assert torch.equal(outs[r], outs[0])
            outs = chb.all_reduce(comm, ins, algo="ll2")      # two-shot flagged lines
            for r in range(P):
                check(outs[r], exp, dtype, P)
                assert torch.equal(outs[r], outs[0])
            outs = chb.reduce_scatter(comm, ins, algo="ll")
            for r in range(P):
                check(outs[r], exp[r * n:(r + 1) * n], dtype, P)
            blocks = [x[:n].contiguous() for x in ins]
            outs = chb.all_gather(comm, blocks, algo="ll")
            for r in range(P):
                assert torch.equal(outs[r], torch.cat(blocks))
    # back-to-back launches reuse the two inbox halves
    ins = make_inputs(P, 512, torch.float32)
    exp = ref_reduce(ins, "sum")
    for _ in range(7):
        outs = chb.all_reduce(comm, ins, algo="ll")
    for r in range(P):
        check(outs[r], exp, torch.float32, P)
    comm.check()


def test_large_multi_cta_and_scale(comms):
    P = 4
    comm = comms(P)
    n = (4 << 20) // 4 + 13  # 4 MiB per rank plus an odd tail
    ins = make_inputs(P, n * P, torch.float32)
    exp = ref_reduce(ins, "sum")
    for nctas in (1, 4, 16):
        outs = chb.all_reduce(comm, ins, algo="radix_batch", k=2, b=1, nctas=nctas, scale=0.25)
        for r in range(P):
            check(outs[r], exp * 0.25, torch.float32, P)
        outs = chb.all_reduce(comm, ins, algo="radix_batch", k=2, b=2, nctas=nctas)
        for r in range(P):
            check(outs[r], exp, torch.float32, P)
    comm.check()


def test_symmetric_buffers_zero_copy(comms):
    P = 4
    comm = comms(P)
    n = 4096
    xs = comm.empty(n * P, torch.float32)
    ys = comm.empty(n * P, torch.float32)
    src = make_inputs(P, n * P, torch.float32)
    for x, s in zip(xs, src):
        x.copy_(s)
    exp = ref_reduce(src, "sum")
    prog = comm.program("allreduce", "radix_batch", n * P, 2, 1, 0, True, True)
    assert prog.work_elems == 0
    chb.all_reduce(comm, xs, out=ys, algo="radix_batch", k=2, b=1)
    for r in range(P):
        check(ys[r], exp, torch.float32, P)
    # in place on symmetric buffers goes through the staged lowering
    chb.all_reduce(comm, xs, out=xs, algo="radix_batch", k=2, b=2)
    for r in range(P):
        check(xs[r], exp, torch.float32, P)
    comm.check()


def test_auto_choice_and_reference_signatures(comms):
    P = 8
    comm = comms(P)
    # lengths that the ranks divide and lengths that they do not (the tuned table may name a schedule that slices
    # the vector into P parts for the former only)
    for n in (8, 4096, 1 << 18, 1, 2, 3, 13):
        ins = make_inputs(P, n, torch.float32)
        exp = ref_reduce(ins, "sum")
        outs = chb.all_reduce(comm, ins)
        for r in range(P):
            check(outs[r], exp, torch.float32, P)
    n = 64
    send = make_inputs(P, n * P, torch.int32)
    recv = [torch.zeros(n * P, dtype=torch.int32, device="cuda") for _ in range(P)]
    assert chb.all_reduce_radix_batch(send, recv, n * P, "sum", comm, 2, 4) == 0
    assert torch.equal(recv[3], ref_reduce(send, "sum").to(torch.int32))
    out = [torch.zeros(n, dtype=torch.int32, device="cuda") for _ in range(P)]
    assert chb.reduce_scatter_radix_batch(send, out, n, "sum", comm, 2, 2) == 0
    assert torch.equal(out[2], ref_reduce(send, "sum").to(torch.int32)[2 * n:3 * n])
    small = [s[:n].contiguous() for s in send]
    assert chb.allgather_radix_batch(small, n, recv, comm, 4, 8) == 0
    assert torch.equal(recv[7], torch.cat(small))
    # wrong group size and wrong count come back as error codes, like MPI_ERR_*
    assert chb.all_reduce_radix_batch(send, recv, n * P, "sum", comm, 2, 3) != 0
    assert chb.all_reduce_radix_batch(send, recv, n * P - 1, "sum", comm, 2, 2) != 0
    comm.check()


def test_barrier(comms):
    comm = comms(8)
    for _ in range(3):
        comm.barrier()
    comm.check()
    assert comm.status(0)["code"] == 0


def test_round_trace(comms):
    P = 8
    comm = comms(P)
    comm.enable_trace(32)
    ins = make_inputs(P, P * 4096, torch.float32)
    prog = comm.program("allreduce", "radix_batch", P * 4096, 2, 4)
    chb.all_reduce(comm, ins, algo="radix_batch:pull", k=2, b=4)
    for r in (0, 5):
        tr = comm.read_trace(prog.nrounds, r)
        assert len(tr) == prog.nrounds
        assert all(e >= s for s, e in tr), tr
        assert all(tr[i + 1][0] >= tr[i][1] - 1e-3 for i in range(len(tr) - 1)), tr   # rounds are ordered
        assert tr[-1][1] > 0                                                          # and were really stamped
    # the push form stamps its levels too (first thread of the rank: start of the level, end of its own share)
    prog_ll = comm.program("allreduce", "radix_batch", P * 4096, 2, 4, in_symmetric=True, out_symmetric=True)
    chb.all_reduce(comm, ins, algo="radix_batch:ll", k=2, b=4)
    for r in (0, 5):
        tr = comm.read_trace(prog_ll.nrounds, r)
        assert all(e >= s for s, e in tr) and tr[-1][1] > 0, tr
        assert all(tr[i + 1][0] >= tr[i][0] for i in range(len(tr) - 1)), tr
    comm.enable_trace(0)
    chb.all_reduce(comm, ins, algo="radix_batch", k=2, b=4)
    comm.check()


def test_cuda_graph_replay(comms):
    """Epochs and sequence numbers live in device memory, so a captured collective can be replayed."""
    P = 4
    comm = comms(P)
    n = 2048
    xs = comm.empty(n * P, torch.float32)
    ys = comm.empty(n * P, torch.float32)
    zs = comm.empty(n * P, torch.float32)
    src = make_inputs(P, n * P, torch.float32, seed=9)
    for x, s_ in zip(xs, src):
        x.copy_(s_)
    # warm up outside of capture (program upload, caches)
    chb.all_reduce(comm, xs, out=ys, algo="radix_batch", k=2, b=2)
    chb.all_reduce(comm, xs, out=zs, algo="ll")
    torch.cuda.synchronize()
    st = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(st):
        with torch.cuda.graph(g, stream=st):
            chb.all_reduce(comm, xs, out=ys, algo="radix_batch", k=2, b=2, stream=st)
            chb.all_reduce(comm, ys, out=zs, algo="ll", scale=0.5, stream=st)
    for it in range(4):
        for x, s_ in zip(xs, src):
            x.copy_(s_ * (it + 1))
        torch.cuda.synchronize()
        g.replay()
        torch.cuda.synchronize()
        exp = ref_reduce(src, "sum") * (it + 1)
        for r in range(P):
            check(ys[r], exp, torch.float32, P)
            check(zs[r], exp * P * 0.5, torch.float32, P * P)
    # the communicator keeps working eagerly after replays
    chb.all_reduce(comm, xs, out=ys, algo="radix_batch", k=2, b=2)
    comm.check()


def test_in_place_flagged_line_kernels(comms):
    P = 8
    comm = comms(P)
    for algo in ("ll", "ll2"):
        for n in (5, 4096):
            src = make_inputs(P, n * P, torch.float32, seed=n)
            bufs = [s_.clone() for s_ in src]
            exp = ref_reduce(src, "sum")
            chb.all_reduce(comm, bufs, out=bufs, algo=algo)
            for r in range(P):
                check(bufs[r], exp, torch.float32, P)
    comm.check()


@pytest.mark.parametrize("P", [2, 4, 8])
def test_bulk_copy_allgather(comms, P):
    """Allgather through the bulk-copy engine (shared-memory ring, mbarriers)."""
    comm = comms(P)
    for dtype, n in ((torch.float32, 4), (torch.float32, 2052), (torch.bfloat16, 8 * 3001), (torch.float32, (1 << 20) + 12)):
        xs = comm.empty(n, dtype)
        src = make_inputs(P, n, dtype, seed=n)
        for x, s_ in zip(xs, src):
            x.copy_(s_)
        outs = chb.all_gather(comm, xs, algo="bulk")
        cat = torch.cat(src)
        for r in range(P):
            assert torch.equal(outs[r], cat)
        for nctas in (1, 7):
            outs = chb.all_gather(comm, xs, algo="bulk", nctas=nctas)
            assert torch.equal(outs[P - 1], cat)
    # inputs outside the symmetric heap fall back to a step program
    loose = make_inputs(P, 1024, torch.float32)
    outs = chb.all_gather(comm, loose, algo="bulk")
    assert torch.equal(outs[0], torch.cat(loose))
    comm.check()


def test_single_rank_world_is_a_local_copy(cuda):
    """P = 1: every collective degenerates to a copy; large aligned ones take the lean copy kernel,
    the rest the interpreter; both keep the communicator's launch counter."""
    comm = Communicator.emulated(1, scratch_bytes=1 << 20, user_bytes=(16 << 20) + 4096)
    before = comm.status()["launches"]
    calls = 0
    for n in ((1 << 20) + 4, (1 << 20) + 3, 1 << 18, 5):
        for dtype in (torch.float32, torch.bfloat16):
            x = torch.randn(n, device="cuda").to(dtype)
            for fn in (chb.all_reduce, chb.reduce_scatter, chb.all_gather):
                y = fn(comm, x)
                calls += 1
                assert torch.equal(y, x), (n, dtype, fn.__name__)
            y = chb.all_reduce(comm, x, scale=0.5)
            calls += 1
            assert torch.allclose(y.float(), x.float() * 0.5, rtol=1e-2)
    xs, ys = comm.empty(1 << 21, torch.float32), comm.empty(1 << 21, torch.float32)
    xs.copy_(torch.randn(1 << 21, device="cuda"))
    chb.all_reduce(comm, xs, out=ys)
    calls += 1
    assert torch.equal(xs, ys)
    assert comm.status()["launches"] - before == calls
    comm.check()
    comm.close()


def test_program_cache_starts_over_when_full(cuda):
    """More distinct message sizes than the per-communicator program cache holds: the cache
    (host programs and their device copies) is dropped and refilled without disturbing results."""
    comm = Communicator.emulated(2, scratch_bytes=1 << 20, user_bytes=1 << 20)
    base = make_inputs(2, 1200, torch.int32)
    for n in range(1, 1101):
        ins = [t[:n] for t in base]
        outs = chb.all_reduce(comm, ins, algo="recursive_doubling")
        if n % 97 == 0 or n > 1090:
            assert torch.equal(outs[0], ins[0] + ins[1]) and torch.equal(outs[1], outs[0])
    comm.check()
    comm.close()


def test_host_buffer_allreduce_pipeline(cuda):
    """Pinned host -> device -> allreduce -> pinned host in chunks on three streams (world of one rank)."""
    from configurable_hierarchical_allreduce_algorithms_b200.ops.host import HostAllReduce

    comm = Communicator.emulated(1, scratch_bytes=1 << 20, user_bytes=8 << 20)
    pipe = HostAllReduce(comm, torch.float32, chunk_elems=1 << 16, depth=2)
    for n in (5, 1 << 16, (7 << 15) + 3):          # less than a chunk, exactly one, several with a ragged tail
        hx = torch.randn(n).pin_memory()
        hy = pipe(hx, scale=2.0)
        torch.cuda.current_stream().synchronize()
        assert torch.equal(hy, hx * 2.0)
        hy2 = torch.empty(n).pin_memory()
        assert chb.all_reduce_host(comm, hx, hy2, chunk_elems=1 << 15, depth=3) is hy2
        torch.cuda.synchronize()
        assert torch.equal(hy2, hx)
    assert pipe.h2d_bytes == pipe.d2h_bytes == 4 * (5 + (1 << 16) + (7 << 15) + 3)
    hx = torch.randn((5 << 15) + 1).pin_memory()
    a, g = pipe.reduce_scatter(hx), pipe.all_gather(hx)
    torch.cuda.synchronize()
    assert torch.equal(a, hx) and torch.equal(g, hx)       # one rank: both are the identity
    comm.check()
    comm.close()


@pytest.mark.parametrize("P,b,k", [(8, 4, 2), (8, 2, 3), (6, 3, 2), (4, 1, 2)])
def test_stand_alone_phases_chain_on_the_gpu(comms, P, b, k):
    """intra reduce-scatter -> lane reduce -> scatter equals the reduce-scatter; gather -> lane allgather ->
    Bruck allgather equals the allgather (the layouts between the phases are the reference's)."""
    from configurable_hierarchical_allreduce_algorithms_b200.ops.collectives import phase

    comm = comms(P)
    n = 1000
    xs = make_inputs(P, P * n, torch.int32, seed=3)
    total = torch.stack(xs).sum(0)
    y = phase(comm, "intra_reduce_scatter_radix_batch", xs, n, k=k, b=b)
    y = phase(comm, "inter_reduce_linear", y, n, k=k, b=b)
    y = phase(comm, "intra_scatter_radix_batch", y, n, k=k, b=b)
    for r in range(P):
        assert torch.equal(y[r], total[r * n:(r + 1) * n])
    blocks = [x[:n].contiguous() for x in xs]
    g = phase(comm, "intra_gather_k_nomial", blocks, n, k=k, b=b)
    g = phase(comm, "inter_allgather_linear", g, n, k=k, b=b)
    g = phase(comm, "intra_allgather_k_brucks", g, n * b, k=k, b=b)
    for r in range(P):
        assert torch.equal(g[r], torch.cat(blocks))
    comm.check()


def test_alltoallv_c_entry_point_in_a_world_of_one(cuda):
    """tuna2_algorithm through its exported symbol: count exchange on the device, packed-layout checks, error codes."""
    import ctypes as C
    from configurable_hierarchical_allreduce_algorithms_b200 import _native as NN

    comm = Communicator.emulated(1, scratch_bytes=1 << 20, user_bytes=1 << 20)
    L = C.CDLL(str(NN._LIB_PATH))
    vp, i32, ip = C.c_void_p, C.c_int, C.POINTER(C.c_int)
    L.chb_set_stream.argtypes = [vp]
    L.chb_set_stream(torch.cuda.current_stream().cuda_stream)
    L.tuna2_algorithm.argtypes = [i32, i32, vp, ip, ip, i32, vp, ip, ip, i32, vp]
    x = torch.arange(1000, device="cuda", dtype=torch.int32)
    y = torch.zeros(1000, device="cuda", dtype=torch.int32)
    one, zero = (C.c_int * 1)(1000), (C.c_int * 1)(0)
    assert L.tuna2_algorithm(2, 1, x.data_ptr(), one, zero, NN.I32, y.data_ptr(), one, zero, NN.I32, comm.handle) == 0
    torch.cuda.synchronize()
    assert torch.equal(x, y)
    bad = (C.c_int * 1)(8)
    assert L.tuna2_algorithm(2, 1, x.data_ptr(), one, bad, NN.I32, y.data_ptr(), one, zero, NN.I32, comm.handle) == NN.ERR_UNSUPPORTED
    assert L.tuna2_algorithm(2, 1, x.data_ptr(), one, zero, NN.I32, y.data_ptr(), one, zero, NN.F32, comm.handle) == NN.ERR_UNSUPPORTED
    wrong = (C.c_int * 1)(999)
    assert L.tuna2_algorithm(2, 1, x.data_ptr(), one, zero, NN.I32, y.data_ptr(), wrong, zero, NN.I32, comm.handle) == NN.ERR_COUNT
    comm.check()
    comm.close()


# ---------------------------------------------------------------- execution modes of step programs
MODE_CASES = [("radix_batch", 2, 1), ("radix_batch", 2, 2), ("radix_batch", 4, 4), ("radix_batch", 8, 8),
              ("radix_batch", 3, 4), ("recursive_doubling", 2, 1), ("reduce_scatter_allgather", 2, 1),
              ("ring", 2, 1), ("recursive_multiplying", 3, 1), ("semi_radix_batch", 2, 2)]


@pytest.mark.parametrize("mode", ["ll", "pull"])
@pytest.mark.parametrize("algo,k,b", MODE_CASES)
def test_allreduce_program_modes(comms, algo, k, b, mode):
    """Every schedule gives the same sums whether readers pull or owners push flagged lines."""
    P = 8
    comm = comms(P)
    for dtype, n in ((torch.float32, 8 * 1024), (torch.bfloat16, 8 * 33), (torch.int32, 8 * 3), (torch.float32, 8),
                     (torch.float64, 8 * 5), (torch.float16, 8 * 129)):
        ins = make_inputs(P, n, dtype, seed=n)
        exp = ref_reduce(ins, "sum")
        outs = chb.all_reduce(comm, ins, algo=f"{algo}:{mode}", k=k, b=b)
        for r in range(P):
            check(outs[r], exp, dtype, P)
    # scale is applied exactly once, in place works, back-to-back launches alternate the inbox halves
    ins = make_inputs(P, 8 * 100, torch.float32, seed=5)
    exp = ref_reduce(ins, "sum")
    for _ in range(5):
        outs = chb.all_reduce(comm, ins, algo=f"{algo}:{mode}", k=k, b=b, scale=0.5)
    for r in range(P):
        check(outs[r], exp * 0.5, torch.float32, P)
    bufs = [x.clone() for x in ins]
    chb.all_reduce(comm, bufs, out=bufs, algo=f"{algo}:{mode}", k=k, b=b)
    for r in range(P):
        check(bufs[r], exp, torch.float32, P)
    comm.check()


@pytest.mark.parametrize("mode", ["ll", "pull"])
@pytest.mark.parametrize("P", [2, 3, 4, 6, 8])
def test_rs_ag_program_modes(comms, P, mode):
    comm = comms(P)
    for b in [d for d in (1, 2, 3, 4, 8) if P % d == 0]:
        for k in (2, 3):
            for dtype, n in ((torch.float32, 1), (torch.float32, 31), (torch.bfloat16, 127), (torch.int64, 5), (torch.float32, 2048)):
                ins = make_inputs(P, n * P, dtype, seed=n + b)
                exp = ref_reduce(ins, "sum")
                outs = chb.reduce_scatter(comm, ins, algo=f"radix_batch:{mode}", k=k, b=b)
                for r in range(P):
                    check(outs[r], exp[r * n:(r + 1) * n], dtype, P)
                blocks = [x[:n].contiguous() for x in ins]
                outs = chb.all_gather(comm, blocks, algo=f"radix_batch:{mode}", k=k, b=b)
                cat = torch.cat(blocks)
                for r in range(P):
                    assert torch.equal(outs[r], cat)
    # max / min through the flagged lines as well
    ins = make_inputs(P, 64 * P, torch.float32, seed=9)
    for op in ("max", "min"):
        outs = chb.all_reduce(comm, ins, op=op, algo=f"radix_batch:{mode}", k=2, b=1)
        for r in range(P):
            check(outs[r], ref_reduce(ins, op), torch.float32, P)
    comm.check()


def test_ll_mode_refuses_what_does_not_fit(comms):
    P = 4
    comm = comms(P)
    n = (comm.ll_max_bytes * P) // 4 * 2           # twice what the inbox holds
    ins = make_inputs(P, n, torch.float32)
    with pytest.raises(chb.CollectiveError):
        chb.all_reduce(comm, ins, algo="radix_batch:ll", k=2, b=1)
    # without a pinned mode the same call falls back to the pull interpreter
    outs = chb.all_reduce(comm, ins, algo="radix_batch", k=2, b=1)
    check(outs[0], ref_reduce(ins, "sum"), torch.float32, P)
    comm.check()


@pytest.mark.parametrize("k,b", [(2, 1), (2, 2), (4, 4), (2, 8)])
def test_tile_scheduler_large_steps(comms, k, b):
    """Steps of several MiB are cut into tiles dealt over the CTAs; odd lengths leave ragged last tiles
    and unaligned tails, a sliced view shifts every pointer off the 32-byte grid."""
    P = 8
    comm = comms(P)
    for dtype, n in ((torch.float32, (1 << 19) + 24), (torch.bfloat16, (1 << 20) + 8 * 5)):
        n = n // P * P
        ins = make_inputs(P, n, dtype, seed=k + b)
        exp = ref_reduce(ins, "sum")
        for nctas in (3, 16):
            outs = chb.all_reduce(comm, ins, algo="radix_batch:pull", k=k, b=b, nctas=nctas)
            for r in range(P):
                check(outs[r], exp, dtype, P)
        m = n // P
        outs = chb.reduce_scatter(comm, ins, algo="radix_batch:pull", k=k, b=b, nctas=8)
        for r in range(P):
            check(outs[r], exp[r * m:(r + 1) * m], dtype, P)
        blocks = [x[:m + 0].contiguous() for x in ins]
        outs = chb.all_gather(comm, blocks, algo="radix_batch:pull", k=k, b=b, nctas=8)
        for r in range(P):
            assert torch.equal(outs[r], torch.cat(blocks))
    # pointers 4 bytes off the vector grid: the scalar path of the same tiles
    big = make_inputs(P, (1 << 18) + P, torch.float32, seed=3)
    ins = [x[1:1 + (1 << 18)] for x in big]
    outs = chb.all_reduce(comm, [x.contiguous() for x in ins], algo="radix_batch:pull", k=k, b=b, nctas=4)
    check(outs[P - 1], ref_reduce(ins, "sum"), torch.float32, P)
    comm.check()


def test_schedule_tables_in_global_memory(cuda):
    """Both program kernels keep their rank's schedule tables in shared memory when they fit; the other path (tables
    read from global memory, what a very long schedule gets) is chosen per process, so it runs in a child."""
    import os
    import subprocess
    import sys
    code = r"""
import torch
import configurable_hierarchical_allreduce_algorithms_b200 as chb
from configurable_hierarchical_allreduce_algorithms_b200.parallel.comm import Communicator
P, n = 8, 8 * 1031
comm = Communicator.emulated(P, scratch_bytes=8 << 20, user_bytes=1 << 20)
g = torch.Generator(device="cuda").manual_seed(5)
ins = [torch.randint(-50, 50, (n,), generator=g, device="cuda", dtype=torch.int32) for _ in range(P)]
exp = torch.stack(ins).sum(0)
for algo, k, b in (("radix_batch:pull", 2, 1), ("radix_batch:pull", 2, 4), ("radix_batch:ll", 2, 1), ("radix_batch:ll", 4, 2),
                   ("ring:pull", 2, 1), ("recursive_doubling:ll", 2, 1)):
    outs = chb.all_reduce(comm, ins, algo=algo, k=k, b=b)
    torch.cuda.synchronize()
    comm.check()
    assert all(torch.equal(o, exp) for o in outs), algo
outs = chb.all_gather(comm, [x[:1031].contiguous() for x in ins], algo="radix_batch:ll", k=2, b=2)
assert all(torch.equal(o, torch.cat([x[:1031] for x in ins])) for o in outs)
comm.close()
print("tables in global memory: ok")
"""
    env = dict(os.environ, CHB_TABLES_IN_SMEM="0")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, env=env,
                       cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode == 0 and "tables in global memory: ok" in r.stdout, r.stdout + r.stderr
