"""Schedule compiler: every generator against naive sum / concat on the host simulator.

Mirrors the reference's self-checking benchmark rows (is_correct column,
testing/custom_implementations/work_dir/all_gather/main.cpp:16-24,54-55) and
its per-file debug mains with counts {1, 3, 16, 31}
(testing/mpich_implementations/reduce_scatter/reduce_scatter_pairwise.cpp:91-159).
"""
import numpy as np
import pytest

from configurable_hierarchical_allreduce_algorithms_b200.parallel.program import (
    Program, ProgramError, list_algorithms)


def pattern(P, n, dt=np.int32, seed=7):
    # (seed*31 + r*1009 + i) mod 97
    return [((seed * 31 + r * 1009 + np.arange(n)) % 97).astype(dt) for r in range(P)]


def expected(coll, ins, P, n, aux=0, op="sum"):
    red = {"sum": np.add, "max": np.maximum, "min": np.minimum}[op]
    if coll in ("allreduce", "reduce_scatter"):
        tot = ins[0].copy()
        for x in ins[1:]:
            tot = red(tot, x)
        if coll == "allreduce":
            return [tot] * P
        return [tot[r * n:(r + 1) * n] for r in range(P)]
    if coll == "allgather":
        return [np.concatenate(ins)] * P
    if coll == "alltoall":
        return [np.concatenate([ins[s][r * n:(r + 1) * n] for s in range(P)]) for r in range(P)]
    if coll == "gather":
        return [np.concatenate(ins) if r == aux else None for r in range(P)]
    raise AssertionError(coll)


def run_case(coll, algo, P, n, k, b, aux=0, sym=(False, False), dt=np.int32, op="sum", in_place=False):
    count = n * P if coll == "allreduce" else n
    p = Program(coll, algo, P, count, k, b, aux, sym[0], sym[1], in_place)
    p.verify()
    ins = pattern(P, p.in_elems, dt)
    exp = expected(coll, ins, P, n, aux, op)
    for seed in (0, 1):
        outs = p.simulate(ins, op=op, seed=seed)
        for r in range(P):
            if exp[r] is not None:
                np.testing.assert_array_equal(outs[r], exp[r], err_msg=f"{coll}/{algo} P={P} n={n} k={k} b={b} rank {r}")
    return p


def divisors(P):
    return [b for b in range(1, P + 1) if P % b == 0]


@pytest.mark.parametrize("coll", ["allgather", "reduce_scatter", "allreduce"])
@pytest.mark.parametrize("P", [1, 2, 3, 4, 6, 8, 9, 12, 16])
def test_radix_batch_grid(coll, P):
    for b in divisors(P):
        for k in (2, 3, 4, 5, 7, 8, 16):
            for n in (1, 3):
                run_case(coll, "radix_batch", P, n, k, b)
    run_case(coll, "radix_batch", P, 31, 2, divisors(P)[-1], sym=(True, True))


@pytest.mark.parametrize("P", [24, 32, 64])
def test_radix_batch_many_ranks(P):
    # the regime the reference targets: many groups, G >= b, partial last stage
    for b in (4, 8):
        if P % b:
            continue
        for k in (2, 4, 7):
            for coll in ("allgather", "reduce_scatter", "allreduce"):
                run_case(coll, "radix_batch", P, 2, k, b)


def test_radix_batch_rejects_bad_group_size():
    for coll in ("allgather", "reduce_scatter", "allreduce"):
        with pytest.raises(ProgramError, match="divide"):
            Program(coll, "radix_batch", 6, 12, 2, 4)
    with pytest.raises(ProgramError, match="multiple"):
        Program("allreduce", "radix_batch", 4, 10, 2, 2)


def test_message_counts_match_reference_probe():
    # P = 8 allreduce: 112 / 56 / 22-28 / 14-15 messages for b = 1 / 2 / 4 / 8 and
    # 2 (P-1) N elements moved, except (k=4, b=8) which moves 7 % more
    N = 8 * 64
    exp = {(2, 1): 112, (2, 2): 56, (2, 4): 22, (4, 4): 28, (2, 8): 14, (4, 8): 15}
    for (k, b), msgs in exp.items():
        p = Program("allreduce", "radix_batch", 8, N, k, b, 0, True, True)
        assert p.remote_msgs == msgs, (k, b, p.remote_msgs)
        assert p.remote_elems == (2 * 7 * N if (k, b) != (4, 8) else 2 * 7 * N * 15 // 14), (k, b)


BASELINES = [(c, a) for c in ("allreduce", "reduce_scatter", "allgather", "alltoall") for a in list_algorithms(c)
             if a != "radix_batch"]


@pytest.mark.parametrize("coll,algo", BASELINES)
def test_baselines(coll, algo):
    for P in (1, 2, 3, 4, 5, 6, 7, 8, 12):
        ks = (2,) if algo in ("ring", "recursive_doubling", "pairwise", "recursive_halving", "linear",
                              "reduce_scatter_allgather") else (2, 3, 4, 8)
        bs = (1, 2, 3, P) if algo in ("radix_block", "tuna", "custom", "inter_reduce_exchange_bcast") else (1,)
        if algo == "semi_radix_batch":
            bs = divisors(P)
        for k in ks:
            for b in bs:
                for n in (1, 3, 16):
                    try:
                        run_case(coll, algo, P, n, k, b)
                    except ProgramError as e:
                        assert "power-of-two" in str(e), e


def test_gather_knomial():
    for P in (1, 2, 5, 8):
        for root in (0, P - 1):
            for k in (2, 3, 8):
                run_case("gather", "k_nomial", P, 3, k, 1, aux=root)


@pytest.mark.parametrize("dt,op", [(np.float64, "sum"), (np.float64, "max"), (np.int32, "max"), (np.int32, "min"),
                                   (np.float32, "sum"), (np.int64, "sum")])
def test_dtypes_and_ops(dt, op):
    # INT/SUM, DOUBLE/MAX ... x counts {1, 3, 16, 31}, like the reference's debug mains
    for n in (1, 3, 16, 31):
        for coll, algo in (("allreduce", "radix_batch"), ("reduce_scatter", "radix_batch"),
                           ("reduce_scatter", "pairwise"), ("allreduce", "recursive_doubling"),
                           ("reduce_scatter", "radix")):
            run_case(coll, algo, 6, n, 3, 3 if algo == "radix_batch" else 1, dt=dt, op=op)


def test_in_place_lowering():
    for coll, algo, b in (("allreduce", "radix_batch", 2), ("allreduce", "ring", 1), ("reduce_scatter", "radix_batch", 4)):
        p = run_case(coll, algo, 8, 5, 2, b, in_place=True)
        # no step may read the caller's input after the staging copy
        ops, srcs, *_ = p.tables()
        staged = [o for o in ops if any(s[1] == 0 for s in srcs[o[6]:o[6] + o[7]])]
        assert all(o[2] == 2 for o in staged)


def test_symmetric_buffers_need_no_staging():
    p = Program("allreduce", "radix_batch", 8, 8 * 128, 2, 1, 0, True, True)
    assert p.work_elems == 0 and p.nrounds == 3     # entry round (owners announce their inputs), reduce, broadcast
    q = Program("allreduce", "radix_batch", 8, 8 * 128, 2, 1, 0, False, False)
    assert q.work_elems > 0 and q.nrounds > p.nrounds


def test_config1_cpu_plumbing_single_process():
    # 4 ranks, k=2, b=1, int32, 1024 elements per rank, values (seed*31 + r*1009 + i) mod 97
    run_case("allreduce", "radix_batch", 4, 1024, 2, 1)
    run_case("reduce_scatter", "radix_batch", 4, 1024, 2, 1)
    run_case("allgather", "radix_batch", 4, 1024, 2, 1)


def test_phases_as_standalone_collectives():
    # intra_<algo>: inside every group of b consecutive ranks; inter_<algo>: along every lane of stride b
    P, b, n = 12, 4, 3
    G = P // b
    ins = [(np.arange(n) + 100 * r).astype(np.int32) for r in range(P)]
    o = Program("allgather", "intra_k_brucks", P, n, 3, b)
    o.verify()
    out = o.simulate(ins)
    for r in range(P):
        g = r // b
        np.testing.assert_array_equal(out[r], np.concatenate(ins[g * b:(g + 1) * b]))
    o = Program("allgather", "inter_linear", P, n, 2, b)
    o.verify()
    out = o.simulate(ins)
    for r in range(P):
        np.testing.assert_array_equal(out[r], np.concatenate([ins[q] for q in range(r % b, P, b)]))
    ins = [(np.arange(n * G) + 7 * r).astype(np.int32) for r in range(P)]
    out = Program("reduce_scatter", "inter_pairwise", P, n, 2, b).simulate(ins)
    for r in range(P):
        tot = sum(ins[q] for q in range(r % b, P, b))
        np.testing.assert_array_equal(out[r], tot[(r // b) * n:(r // b + 1) * n])
    ins = [(np.arange(n * b) + 7 * r).astype(np.int32) for r in range(P)]
    out = Program("reduce_scatter", "intra_radix", P, n, 3, b).simulate(ins)
    for r in range(P):
        tot = sum(ins[(r // b) * b:(r // b + 1) * b])
        np.testing.assert_array_equal(out[r], tot[(r % b) * n:(r % b + 1) * n])


def test_alltoallv_store_and_forward():
    rng = np.random.default_rng(0)
    for P in (1, 2, 5, 8):
        counts = rng.integers(0, 6, size=(P, P))
        for r, b in ((2, 1), (3, 2), (8, 8)):
            p = Program.alltoallv(counts, r, b)
            p.verify()
            ins = []
            for s in range(P):
                x = np.full(p.in_elems, -1, np.int64)
                off = 0
                for d in range(P):
                    x[off:off + counts[s, d]] = 1000 * s + 10 * d + np.arange(counts[s, d])
                    off += counts[s, d]
                ins.append(x)
            outs = p.simulate(ins)
            for d in range(P):
                off = 0
                for s in range(P):
                    exp = 1000 * s + 10 * d + np.arange(counts[s, d])
                    np.testing.assert_array_equal(outs[d][off:off + counts[s, d]], exp)
                    off += counts[s, d]


def test_threaded_host_executor_matches_simulator():
    # real concurrency: one thread per rank, release / acquire on round counters
    rng = np.random.default_rng(1)
    for coll, algo, k, b in (("allreduce", "radix_batch", 2, 4), ("allreduce", "recursive_doubling", 2, 1),
                             ("reduce_scatter", "radix_batch", 3, 2), ("allgather", "radix_batch", 2, 8),
                             ("allreduce", "ring", 2, 1), ("reduce_scatter", "radix_block", 2, 2)):
        P, n = 8, 257
        p = Program(coll, algo, P, n * P if coll == "allreduce" else n, k, b)
        ins = [rng.integers(0, 100, p.in_elems).astype(np.int64) for _ in range(P)]
        ref = p.simulate(ins)
        for _ in range(3):
            got, sec = p.run_threads(ins, iters=2)
            assert sec > 0
            for a, e in zip(got, ref):
                np.testing.assert_array_equal(a, e)
