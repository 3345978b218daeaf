"""Entry handshake of programs whose caller input is pulled directly by peers.

With one rank per GPU a reader may be ahead of the owner of a peer-visible input: whatever produces that
input (an upload, a backward kernel) is ordered on the OWNER's stream only.  The lowering therefore makes
every such read wait for the owner's round 0.  The simulator and the threaded executor model the hazard
directly: an input that peers pull holds poison until its owner starts, so a schedule without the
handshake returns poisoned sums (checked by hand once: both fail without it).
"""
import numpy as np
import pytest

from configurable_hierarchical_allreduce_algorithms_b200 import Program, list_algorithms

ALGOS = [("allreduce", a) for a in ("radix_batch", "recursive_doubling", "ring", "reduce_scatter_allgather",
                                    "recursive_exchange", "semi_radix_batch")] + \
        [("reduce_scatter", a) for a in ("radix_batch", "pairwise", "recursive_halving")] + \
        [("allgather", a) for a in ("radix_batch", "k_brucks", "ring")]


def _io(coll, P, n, rng):
    if coll == "allgather":
        ins = [rng.integers(-50, 50, n).astype(np.int32) for _ in range(P)]
        exp = [np.concatenate(ins)] * P
        return ins, exp, n
    ins = [rng.integers(-50, 50, n * P).astype(np.int32) for _ in range(P)]
    tot = sum(ins)
    if coll == "allreduce":
        return ins, [tot] * P, n * P
    return ins, [tot[r * n:(r + 1) * n] for r in range(P)], n


@pytest.mark.parametrize("coll,algo", ALGOS)
@pytest.mark.parametrize("P", [2, 4, 6])
def test_peers_wait_for_the_owner_of_a_pulled_input(coll, algo, P):
    rng = np.random.default_rng(P)
    for b in (1, 2):
        ins, exp, count = _io(coll, P, 24, rng)
        prog = Program(coll, algo, P, count, 2, b, in_symmetric=True, out_symmetric=True)
        prog.verify()
        ops, srcs, waits, _, signals = prog.tables()
        if prog.reads_peer_in:
            # every rank whose input is pulled announces its entry in round 0
            owners = set()
            for o in ops:
                rank, _, _, _, _, _, sb, ns = (int(v) for v in o)
                for p_, buf, _ in srcs[sb:sb + ns]:
                    if int(p_) != rank and int(buf) == 0:
                        owners.add(int(p_))
                        # and the reader never sits in round 0
                        assert int(o[1]) >= 1
            announced = {int(s[0]) for s in signals if int(s[1]) == 0}
            assert owners <= announced
        for seed in range(4):
            outs = prog.simulate([x.copy() for x in ins], seed=seed)
            for r in range(P):
                assert np.array_equal(outs[r], exp[r]), (coll, algo, P, b, seed, r)
        for late in (0, P - 1):
            outs, _ = prog.run_threads([x.copy() for x in ins], late_rank=late, delay_ms=15)
            for r in range(P):
                assert np.array_equal(outs[r], exp[r]), (coll, algo, P, b, "late", late, r)


def test_staged_and_in_place_programs_need_no_entry_round():
    # inputs that peers cannot see are staged by their owner (a step of the owner): same number of rounds as before
    p_private = Program("allreduce", "radix_batch", 4, 64, 2, 1)
    p_direct = Program("allreduce", "radix_batch", 4, 64, 2, 1, in_symmetric=True, out_symmetric=True)
    assert p_direct.nrounds == 3 and p_private.nrounds == 4   # entry + reduce + broadcast / stage + reduce + stage + broadcast
    p_alias = Program("allreduce", "radix_batch", 4, 64, 2, 1, in_symmetric=True, out_symmetric=True, in_place=True)
    p_alias.verify()
    assert not any(int(buf) == 0 and int(peer) != int(o[0])
                   for o in p_alias.tables()[0]
                   for peer, buf, _ in p_alias.tables()[1][int(o[6]):int(o[6]) + int(o[7])])


def test_all_listed_algorithms_verify_with_direct_inputs():
    for coll in ("allreduce", "reduce_scatter", "allgather"):
        for algo in list_algorithms(coll):
            for P in (3, 8):
                for b in (1, 2, 4):
                    if P % b:
                        continue
                    try:
                        prog = Program(coll, algo, P, 8 * P if coll == "allreduce" else 8, 2, b,
                                       in_symmetric=True, out_symmetric=True)
                    except ValueError:
                        continue
                    prog.verify()
