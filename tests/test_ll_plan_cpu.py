"""Host half of the flagged-line (push) execution of step programs: which messages are forwarded line by line
from the previous round's steps, and where a rank-local barrier is still needed (csrc/kernels/llprog.cu)."""
import pytest

from configurable_hierarchical_allreduce_algorithms_b200 import Program


def _prog(coll, algo, P, count, k=2, b=1, in_place=False):
    return Program(coll, algo, P, count, k, b, in_symmetric=True, out_symmetric=True, in_place=in_place)


def test_flat_two_round_allreduce_needs_no_barrier_and_forwards_the_whole_broadcast():
    P, n = 8, 1024
    info = _prog("allreduce", "radix_batch", P, n * P, 2, 1).ll_info(4)
    # reduce round: every rank pushes P-1 chunks; broadcast round: all P * (P-1) messages are forwarded by the reducers
    assert info["levels"] == 3                         # entry round (empty in this mode), reduce, broadcast
    assert info["pushed"] == P * (P - 1) and info["forwarded"] == P * (P - 1)
    assert info["barriers"] == 0
    assert info["inbox_lines"] == 2 * (P - 1) * n * 4 // 8


def test_one_round_collectives_are_one_push_phase():
    P, n = 4, 100
    for coll in ("allgather", "reduce_scatter"):
        info = _prog(coll, "radix_batch", P, n, 2, 1).ll_info(2)
        assert info["pushed"] == P * (P - 1) and info["forwarded"] == 0 and info["barriers"] == 0


@pytest.mark.parametrize("k,b", [(2, 2), (2, 4), (4, 4), (8, 8)])
def test_hierarchical_shapes_forward_and_keep_only_the_barriers_that_order_something(k, b):
    P, n = 8, 64
    prog = _prog("allreduce", "radix_batch", P, n * P, k, b)
    info = prog.ll_info(4)
    total = info["pushed"] + info["forwarded"]
    assert total == prog.remote_msgs                     # every remote source is a message, pushed or forwarded
    assert info["forwarded"] > 0
    assert info["barriers"] < P * (info["levels"] - 1)   # fewer than one per rank and round boundary


def test_in_place_form_reads_the_staged_copy_and_therefore_keeps_a_barrier():
    P, n = 4, 256
    a = _prog("allreduce", "radix_batch", P, n * P, 2, 1).ll_info(4)
    b = _prog("allreduce", "radix_batch", P, n * P, 2, 1, in_place=True).ll_info(4)
    assert a["barriers"] == 0 and b["barriers"] > 0


def test_element_size_scales_the_lines():
    P, n = 4, 1000
    prog = _prog("allreduce", "recursive_doubling", P, n, 2, 1)
    assert prog.ll_info(8)["inbox_lines"] == 2 * prog.ll_info(4)["inbox_lines"]
    assert prog.ll_info(2)["inbox_lines"] * 4 == prog.ll_info(8)["inbox_lines"]


# ---- the push form executed on the host, line by line (csrc/sched/ll_plan.cc: simulate_ll) ----
import numpy as np  # noqa: E402

from configurable_hierarchical_allreduce_algorithms_b200.parallel.program import ProgramError, list_algorithms  # noqa: E402


def _pattern(P, n, dt, seed=5):
    return [((seed * 31 + r * 1009 + np.arange(n) * 7) % 97).astype(dt) for r in range(P)]


def _expected(coll, ins, P, n):
    if coll == "allgather":
        return [np.concatenate(ins)] * P
    if coll == "alltoall":
        return [np.concatenate([ins[s][r * n:(r + 1) * n] for s in range(P)]) for r in range(P)]
    tot = ins[0].copy()
    for x in ins[1:]:
        tot = tot + x
    return [tot] * P if coll == "allreduce" else [tot[r * n:(r + 1) * n] for r in range(P)]


def _check(coll, algo, P, n, k, b, dt=np.int32, threads=5, seeds=(0, 1, 2)):
    count = n * P if coll == "allreduce" else n
    prog = _prog(coll, algo, P, count, k, b)
    ins = _pattern(P, prog.in_elems, dt)
    exp = _expected(coll, ins, P, n)
    for seed in seeds:
        outs = prog.simulate_ll(ins, seed=seed, threads=threads)
        for r in range(P):
            np.testing.assert_array_equal(outs[r], exp[r], err_msg=f"{coll}/{algo} P={P} n={n} k={k} b={b} rank {r} seed {seed}")
    return prog


@pytest.mark.parametrize("coll", ["allreduce", "reduce_scatter", "allgather"])
@pytest.mark.parametrize("P", [2, 3, 4, 6, 8, 12])
def test_radix_batch_push_form_on_the_host(coll, P):
    """Every (k, b) shape: inbox slots, pushes, line-level forwards and the barriers that were kept give the sum / the
    concatenation under random interleavings of the ranks' threads.  Odd counts leave partial last lines."""
    for b in [d for d in range(1, P + 1) if P % d == 0]:
        for k in (2, 3, 4, 8):
            for n in (1, 5, 16):
                _check(coll, "radix_batch", P, n, k, b)


@pytest.mark.parametrize("coll", ["allreduce", "reduce_scatter", "allgather", "alltoall"])
def test_every_algorithm_push_form_on_the_host(coll):
    ran = 0
    for algo in list_algorithms(coll):
        for P in (2, 4, 5, 8):
            for k, b in ((2, 1), (4, 2)):
                if P % b:
                    continue
                try:
                    _check(coll, algo, P, 7, k, b, seeds=(0, 3))
                    ran += 1
                except ProgramError:
                    pass     # shape not defined for this algorithm (e.g. a power-of-two baseline at P = 5)
    assert ran > (10 if coll != "alltoall" else 3)


@pytest.mark.parametrize("dt", [np.uint8, np.int64, np.float64, np.float32])
def test_push_form_element_sizes(dt):
    """1-, 4- and 8-byte elements: 8, 2 and 1 elements per line, forwards at offsets that are whole lines only."""
    for P, k, b in ((4, 2, 2), (8, 2, 1), (8, 8, 8), (6, 3, 2)):
        _check("allreduce", "radix_batch", P, 3, k, b, dt=dt)
        _check("allreduce", "radix_batch", P, 8, k, b, dt=dt)


def test_push_form_matches_the_pull_form_bit_for_bit_on_floats():
    """Both forms add in the program's order, so floats that do not add exactly agree to the last bit."""
    P, n = 8, 33
    rng = np.random.default_rng(3)
    ins = [rng.standard_normal(n * P).astype(np.float32) for _ in range(P)]
    for k, b in ((2, 1), (2, 4), (4, 2), (8, 8)):
        prog = _prog("allreduce", "radix_batch", P, n * P, k, b)
        pull = prog.simulate(ins, seed=1)
        push = prog.simulate_ll(ins, seed=2, threads=7)
        for r in range(P):
            assert pull[r].tobytes() == push[r].tobytes()


def test_one_thread_per_rank_and_many():
    for threads in (1, 2, 64):
        _check("allreduce", "radix_batch", 8, 16, 2, 2, threads=threads, seeds=(0,))


def test_staged_program_is_refused():
    prog = Program("allreduce", "radix_batch", 4, 64, 2, 1)      # lowered with staging copies
    with pytest.raises(RuntimeError, match="staging"):
        prog.simulate_ll(_pattern(4, 64, np.int32))


def test_the_simulator_notices_a_plan_without_its_barriers():
    """The in-place form reads a staged copy of its input, so it keeps barriers; with the barriers ignored, threads
    that own different lines in consecutive rounds read the copy before it is complete."""
    P, n = 4, 64
    prog = _prog("allreduce", "radix_batch", P, n * P, 2, 1, in_place=True)
    assert prog.ll_info(4)["barriers"] > 0
    ins = _pattern(P, prog.in_elems, np.int32)
    exp = _expected("allreduce", ins, P, n)
    wrong = 0
    for threads in (7, 64):
        for seed in range(6):
            outs = prog.simulate_ll(ins, seed=seed, threads=threads)
            assert all((outs[r] == exp[r]).all() for r in range(P))
            outs = prog.simulate_ll(ins, seed=seed, threads=threads, fault=1)
            wrong += any((outs[r] != exp[r]).any() for r in range(P))
    assert wrong > 0


def test_the_simulator_notices_a_message_that_nobody_sends():
    P, n = 8, 16
    prog = _prog("allreduce", "radix_batch", P, n * P, 2, 1)
    with pytest.raises(RuntimeError, match=r"deadlock: rank \d+ level \d+ waits for line \d+ from rank \d+"):
        prog.simulate_ll(_pattern(P, prog.in_elems, np.int32), fault=2)


@pytest.mark.parametrize("coll", ["allreduce", "reduce_scatter", "allgather", "alltoall"])
def test_back_to_back_launches_share_two_inbox_halves(coll):
    """Five launches in a row, every rank going on as soon as its own previous launch has returned and the inbox
    halves alternating by launch parity: in these collectives nobody can get two launches ahead of a rank that
    still has to read a line, so no line is ever overwritten unread."""
    for algo in list_algorithms(coll):
        for P, k, b in ((2, 2, 1), (4, 2, 2), (8, 2, 1), (8, 8, 8)):
            try:
                prog = _prog(coll, algo, P, 5 * P if coll == "allreduce" else 5, k, b)
            except ProgramError:
                continue
            ins = _pattern(P, prog.in_elems, np.int32)
            exp = _expected(coll, ins, P, 5)
            for seed in (0, 1, 2):
                outs = prog.simulate_ll(ins, seed=seed, threads=3, launches=5)
                for r in range(P):
                    np.testing.assert_array_equal(outs[r], exp[r])


def test_a_gather_would_overwrite_unread_lines():
    """Why the executor refuses collectives such as gather: a leaf only sends, so it runs launches ahead of its
    parent, and its third launch writes into the half that still holds the unread line of its first."""
    prog = _prog("gather", "k_nomial", 8, 6, 2, 1)
    ins = _pattern(8, prog.in_elems, np.int32)
    prog.simulate_ll(ins, seed=0, threads=2, launches=1)       # one launch alone is fine
    hazards = 0
    for seed in range(10):
        try:
            prog.simulate_ll(ins, seed=seed, threads=2, launches=6)
        except RuntimeError as e:
            assert "meets an unread line" in str(e)
            hazards += 1
    assert hazards > 0


def test_a_ranks_own_table_entries_are_small():
    """The executor keeps them in shared memory up to 40 KiB: every schedule of the sweeps is far below that."""
    for coll, algo, P, k, b in (("allreduce", "radix_batch", 8, 2, 1), ("allreduce", "radix_batch", 8, 2, 4), ("allreduce", "ring", 16, 2, 1),
                                ("allgather", "radix_batch", 16, 2, 4), ("alltoall", "tuna", 8, 2, 2)):
        info = _prog(coll, algo, P, P * 64 if coll == "allreduce" else 64, k, b).ll_info(4)
        assert 0 < info["rank_table_bytes"] < (8 << 10), (coll, algo, P, info)
