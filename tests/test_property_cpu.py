"""Randomised shapes: any registered algorithm, any rank count up to 24, any radix, any group size that
divides the ranks, ragged element counts, every way of lowering (private, peer-visible or aliased caller
buffers), random interleavings - the simulated result is the definition
of the collective and the schedule has no unsynchronised hazard."""
import numpy as np
from hypothesis import HealthCheck, given, settings, strategies as st

from configurable_hierarchical_allreduce_algorithms_b200 import Program, ProgramError, list_algorithms

COLLS = ["allreduce", "reduce_scatter", "allgather"]


@st.composite
def cases(draw):
    coll = draw(st.sampled_from(COLLS))
    algo = draw(st.sampled_from(list_algorithms(coll)))
    P = draw(st.integers(1, 24))
    b = draw(st.sampled_from([d for d in range(1, P + 1) if P % d == 0]))
    k = draw(st.integers(2, 9))
    n = draw(st.integers(1, 7))
    op = draw(st.sampled_from(["sum", "max", "min"]))
    seed = draw(st.integers(0, 2 ** 31))
    lowering = draw(st.sampled_from(["private", "symmetric", "in_symmetric", "out_symmetric", "in_place"]))
    return coll, algo, P, k, b, n, op, seed, lowering


@settings(max_examples=500, deadline=None, suppress_health_check=list(HealthCheck))
@given(cases())
def test_random_shapes(case):
    coll, algo, P, k, b, n, op, seed, lowering = case
    flags = dict(in_symmetric=lowering in ("symmetric", "in_symmetric"), out_symmetric=lowering in ("symmetric", "out_symmetric"),
                 in_place=lowering == "in_place")
    count = n * P if coll == "allreduce" else n
    aux = 0
    if algo == "inter_reduce_exchange_bcast":
        aux = b                                     # ranks per node
    try:
        p = Program(coll, algo, P, count, k=k, b=b, aux=aux, **flags)
    except ProgramError as e:
        # a documented precondition (power-of-two ranks for recursive doubling allgather, ...), never a crash
        assert any(w in str(e) for w in ("power", "divide", "multiple", "must", "needs", "radix", "ranks")), str(e)
        return
    p.verify()
    rng = np.random.default_rng(seed)
    ins = [rng.integers(-40, 40, p.in_elems).astype(np.int64) for _ in range(P)]
    outs = p.simulate(ins, op=op, seed=seed, alias=lowering == "in_place")      # in place: one buffer per rank
    if coll == "allgather":
        exp = [np.concatenate(ins)] * P
    else:
        red = {"sum": np.sum, "max": np.max, "min": np.min}[op](np.stack(ins), axis=0)
        exp = [red] * P if coll == "allreduce" else [red[r * n:(r + 1) * n] for r in range(P)]
    for r in range(P):
        np.testing.assert_array_equal(outs[r], exp[r], err_msg=f"{case} rank {r}")
    if seed % 4 == 0 and lowering != "in_place":      # a quarter of the cases also under real concurrency (one thread per rank)
        outs, _ = p.run_threads(ins, op=op)
        for r in range(P):
            np.testing.assert_array_equal(outs[r], exp[r], err_msg=f"{case} rank {r} (threads)")


@st.composite
def push_cases(draw):
    coll = draw(st.sampled_from(COLLS + ["alltoall"]))
    algo = draw(st.sampled_from(list_algorithms(coll)))
    P = draw(st.integers(2, 16))
    b = draw(st.sampled_from([d for d in range(1, P + 1) if P % d == 0]))
    k = draw(st.integers(2, 9))
    n = draw(st.integers(1, 9))
    dt = draw(st.sampled_from([np.uint8, np.int32, np.int64]))
    threads = draw(st.sampled_from([1, 2, 3, 7, 32]))
    seed = draw(st.integers(0, 2 ** 31))
    in_place = draw(st.booleans()) and coll in ("allreduce",)
    return coll, algo, P, k, b, n, dt, threads, seed, in_place


@settings(max_examples=300, deadline=None, suppress_health_check=list(HealthCheck))
@given(push_cases())
def test_random_shapes_push_form(case):
    """The flagged-line (push) form of the same programs, executed line by line on the host under random thread
    interleavings: inbox slots, forwards, partial last lines (1-, 4- and 8-byte elements) and the barriers that
    the plan kept must give the definition of the collective."""
    coll, algo, P, k, b, n, dt, threads, seed, in_place = case
    count = n * P if coll == "allreduce" else n
    aux = b if algo == "inter_reduce_exchange_bcast" else 0
    try:
        p = Program(coll, algo, P, count, k=k, b=b, aux=aux, in_symmetric=True, out_symmetric=True, in_place=in_place)
    except ProgramError:
        return
    rng = np.random.default_rng(seed)
    ins = [rng.integers(0, 30, p.in_elems).astype(dt) for _ in range(P)]
    outs = p.simulate_ll(ins, seed=seed, threads=threads)
    if coll == "allgather":
        exp = [np.concatenate(ins)] * P
    elif coll == "alltoall":
        exp = [np.concatenate([ins[s][r * n:(r + 1) * n] for s in range(P)]) for r in range(P)]
    else:
        red = np.stack(ins).sum(axis=0, dtype=dt)
        exp = [red] * P if coll == "allreduce" else [red[r * n:(r + 1) * n] for r in range(P)]
    for r in range(P):
        np.testing.assert_array_equal(outs[r], exp[r], err_msg=f"{case} rank {r}")
