"""The stand-alone phases of the hierarchical collectives (the reference tests them one function at a
time: all_gather_0_3_beta.cpp:36,141,377; intra_reduce_scatter_radix.cpp:208; inter_linear_reduce.cpp:11;
intra_scatter_radix_batch.cpp:11).  Each phase against its definition, and the chains
gather -> lane allgather -> Bruck allgather  and  intra reduce-scatter -> lane reduce -> scatter
against the full allgather / reduce-scatter, which pins the buffer layouts between the phases."""
import numpy as np
import pytest

from configurable_hierarchical_allreduce_algorithms_b200 import Program, list_algorithms

GRID = [(P, b, k) for P in (1, 2, 4, 6, 8, 12, 16, 18) for b in range(1, P + 1) if P % b == 0 for k in (2, 3, 4)
        if not (P > 12 and k == 4)]
POISON = -17


def rnd(P, n, seed):
    r = np.random.default_rng(seed)
    return [r.integers(-50, 50, n).astype(np.int32) for _ in range(P)]


def run(name, P, c, k, b, ins, seed=0):
    p = Program("phase", name, P, c, k=k, b=b)
    p.verify()
    assert p.in_elems == ins[0].size
    return p.simulate(ins, seed=seed)


def test_phase_names_are_listed():
    assert set(list_algorithms("phase")) == {"intra_gather_k_nomial", "inter_allgather_linear", "intra_allgather_k_brucks",
                                             "intra_reduce_scatter_radix_batch", "inter_reduce_linear", "intra_scatter_radix_batch"}
    with pytest.raises(Exception):
        Program("phase", "intra_gather_k_nomial", 6, 4, k=2, b=4)       # b must divide P
    with pytest.raises(Exception):
        Program("phase", "no_such_phase", 4, 4, k=2, b=2)


@pytest.mark.parametrize("P,b,k", GRID)
def test_allgather_phases_and_their_chain(P, b, k):
    c, G = 3, P // b
    T = -(-G // b)
    chunk = b * c
    x = rnd(P, c, 1)
    # 1. gather to the rotating root
    g1 = run("intra_gather_k_nomial", P, c, k, b, x)
    for grp in range(G):
        root = grp * b + grp % b
        assert np.array_equal(g1[root], np.concatenate([x[grp * b + s] for s in range(b)]))
    # 2. lane allgather of the roots' chunks (non-roots hold poison: nobody may read them)
    g2 = run("inter_allgather_linear", P, c, k, b, g1, seed=3)
    for r in range(P):
        q, l = divmod(r, b)
        for s in range(T):
            d = s * b + l
            if d < G:
                assert np.array_equal(g2[r][s * chunk:(s + 1) * chunk], g1[d * b + l])
    # 3. Bruck allgather of the stages: the full allgather, in rank order
    g3 = run("intra_allgather_k_brucks", P, chunk, k, b, g2, seed=5)
    full = np.concatenate(x)
    for r in range(P):
        assert np.array_equal(g3[r], full), (r,)


@pytest.mark.parametrize("P,b,k", GRID)
def test_reduce_scatter_phases_and_their_chain(P, b, k):
    n, G = 3, P // b
    T = -(-G // b)
    chunk = b * n
    x = rnd(P, P * n, 2)
    total = np.sum(x, axis=0)
    # 4. reduce-scatter of the chunks inside every group
    r4 = run("intra_reduce_scatter_radix_batch", P, n, k, b, x)
    for r in range(P):
        grp, slot = divmod(r, b)
        for s in range(T):
            d = s * b + slot
            if d < G:
                exp = np.sum([x[grp * b + j][d * chunk:(d + 1) * chunk] for j in range(b)], axis=0)
                assert np.array_equal(r4[r][s * chunk:(s + 1) * chunk], exp)
    # 5. lane reduce onto the lane roots
    r5 = run("inter_reduce_linear", P, n, k, b, r4, seed=4)
    for d in range(G):
        root = d * b + d % b
        assert np.array_equal(r5[root], total[d * chunk:(d + 1) * chunk])
    # 6. scatter from the roots: the full reduce-scatter
    r6 = run("intra_scatter_radix_batch", P, n, k, b, r5, seed=6)
    for r in range(P):
        assert np.array_equal(r6[r], total[r * n:(r + 1) * n]), (r,)


def test_phases_run_on_host_threads():
    P, b, k, n = 8, 4, 2, 5
    x = rnd(P, P * n, 9)
    p = Program("phase", "intra_reduce_scatter_radix_batch", P, n, k=k, b=b)
    outs, _ = p.run_threads(x)
    assert np.array_equal(outs[0][:b * n], np.sum([xi[:b * n] for xi in x[:b]], axis=0))
