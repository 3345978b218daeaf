"""Same inputs through the reference's own sources (built unmodified against
the thread-per-rank MPI shim, baseline/build_reference.py) and through this
library's schedules: results must be identical for integers."""
import subprocess
from pathlib import Path

import numpy as np
import pytest

from configurable_hierarchical_allreduce_algorithms_b200.parallel.program import Program

ROOT = Path(__file__).resolve().parent.parent
EXE = ROOT / "baseline" / "_ref" / "ref_driver"


@pytest.fixture(scope="module")
def ref_driver():
    if not EXE.exists():
        import sys
        sys.path.insert(0, str(ROOT))
        from baseline import build_reference
        if not (build_reference.REF / "testing").exists():
            pytest.skip("reference sources are not available on this machine")
        build_reference.build()
    return EXE


def reference_result(exe, coll, P, k, b, n, seed):
    r = subprocess.run([str(exe), "check", coll, str(P), str(k), str(b), str(n), str(seed)],
                       capture_output=True, text=True, timeout=120)
    vals = [int(v) for v in r.stdout.split()]
    assert vals[0] == 0, "the reference itself failed (timeout / bad destination / truncation)"
    per = {"ag": n * P, "rs": n, "ar": n * P, "semi": n * P}[coll]
    return [np.array(vals[1 + i * per:1 + (i + 1) * per], dtype=np.int32) for i in range(P)]


@pytest.mark.parametrize("P,b", [(4, 1), (4, 2), (8, 2), (8, 4), (8, 8), (12, 3), (16, 4), (18, 3)])
def test_same_results_as_reference(ref_driver, P, b):
    seed, n = 5, 3
    for k in (2, 3, 4, 7):
        for short, coll in (("ag", "allgather"), ("rs", "reduce_scatter"), ("ar", "allreduce")):
            ref = reference_result(ref_driver, short, P, k, b, n, seed)
            count = n * P if coll == "allreduce" else n
            prog = Program(coll, "radix_batch", P, count, k, b)
            ins = [((seed * 31 + r * 1009 + np.arange(prog.in_elems)) % 97).astype(np.int32) for r in range(P)]
            ours = prog.simulate(ins)
            for r in range(P):
                np.testing.assert_array_equal(ours[r], ref[r], err_msg=f"{coll} P={P} k={k} b={b} rank {r}")


PHASE_EXE = ROOT / "baseline" / "_ref" / "ref_phase_driver"
PHASES = ["intra_gather_k_nomial", "inter_allgather_linear", "intra_allgather_k_brucks",
          "intra_reduce_scatter_radix_batch", "inter_reduce_linear", "intra_scatter_radix_batch"]


@pytest.fixture(scope="module")
def ref_phase_driver(ref_driver):
    if not PHASE_EXE.exists():
        from baseline import build_reference
        if not (build_reference.REF / "testing").exists():
            pytest.skip("reference sources are not available on this machine")
        build_reference.build_phases()
    return PHASE_EXE


def reference_phase(exe, phase, P, k, b, c, seed, nout):
    r = subprocess.run([str(exe), phase, str(P), str(k), str(b), str(c), str(seed)], capture_output=True, text=True, timeout=120)
    vals = [int(v) for v in r.stdout.split()]
    assert vals and vals[0] == 0, f"the reference's {phase} itself failed for P={P} k={k} b={b}"
    return [np.array(vals[1 + i * nout:1 + (i + 1) * nout], dtype=np.int32) for i in range(P)]


@pytest.mark.parametrize("P,b", [(4, 2), (8, 2), (8, 4), (9, 3), (12, 2), (12, 3), (16, 4), (18, 3), (6, 6), (4, 1), (10, 2), (15, 3),
                                 (20, 4), (14, 2), (24, 4), (21, 3)])
def test_stand_alone_phases_match_the_reference(ref_phase_driver, P, b):
    """Each phase function of the reference (built unmodified) against the program of the same name: every entry
    the reference defines must be identical, and entries it leaves alone must be left alone here too."""
    seed, c = 3, 2
    for k in (2, 3, 4):
        for phase in PHASES:
            prog = Program("phase", phase, P, c, k, b)
            ref = reference_phase(ref_phase_driver, phase, P, k, b, c, seed, prog.out_elems)
            ins = [((seed * 31 + r * 1009 + np.arange(prog.in_elems) * 7) % 97).astype(np.int32) for r in range(P)]
            ours = prog.simulate(ins)
            for r in range(P):
                np.testing.assert_array_equal(ours[r], ref[r], err_msg=f"{phase} P={P} k={k} b={b} rank {r}")


MPICH_EXE = ROOT / "baseline" / "_ref" / "ref_mpich_driver"
MPICH = {  # reference entry point -> (collective, algorithm here, takes a radix)
    "ar_recursive_doubling": ("allreduce", "recursive_doubling", False),
    "ar_ring": ("allreduce", "ring", False),
    "ar_reduce_scatter_allgather": ("allreduce", "reduce_scatter_allgather", False),
    "ar_recursive_multiplying": ("allreduce", "recursive_multiplying", True),
    "ar_k_reduce_scatter_allgather": ("allreduce", "k_reduce_scatter_allgather", True),
    "ar_recursive_exchange": ("allreduce", "recursive_exchange", True),
    "ar_smp": ("allreduce", "inter_reduce_exchange_bcast", False),          # built with 2 ranks per node
    "rs_rec_halving": ("reduce_scatter", "recursive_halving", False),
    "rs_rec_doubling": ("reduce_scatter", "recursive_doubling", False),
    "rs_pairwise": ("reduce_scatter", "pairwise", False),
    "rs_radix": ("reduce_scatter", "radix", True),
}


@pytest.fixture(scope="module")
def ref_mpich_driver(ref_driver):
    if not MPICH_EXE.exists():
        from baseline import build_reference
        if not (build_reference.REF / "testing").exists():
            pytest.skip("reference sources are not available on this machine")
        build_reference.build_mpich()
    return MPICH_EXE


@pytest.mark.parametrize("name", sorted(MPICH))
def test_mpich_style_baselines_match_the_reference(ref_mpich_driver, name):
    """The reference's MPICH-style baselines (built unmodified) and the programs of the same algorithms:
    identical results, also where the number of ranks is not a power of the radix, and for the reference's
    in-place form."""
    coll, algo, has_k = MPICH[name]
    seed, n = 3, 3
    for P in (2, 3, 4, 5, 6, 7, 8, 12):
        nout = n * P if coll == "allreduce" else n
        ins = [((seed * 31 + q * 1009 + np.arange(n * P) * 7) % 97).astype(np.int32) for q in range(P)]
        if name == "ar_smp" and P % 2:
            continue                                   # whole nodes of two ranks
        for k in ((2, 3, 4) if has_k else (2,)):
            ours = Program(coll, algo, P, n * P if coll == "allreduce" else n, k, 1, aux=2 if name == "ar_smp" else 0).simulate(ins)
            for mode in ([], ["inplace"]) if name != "ar_smp" else ([],):
                r = subprocess.run([str(ref_mpich_driver), name, str(P), str(k), str(n), str(seed)] + mode,
                                   capture_output=True, text=True, timeout=120)
                vals = [int(v) for v in r.stdout.split()]
                assert vals and vals[0] == 0, f"the reference's {name} itself failed for P={P} k={k} {mode}"
                for q in range(P):
                    np.testing.assert_array_equal(ours[q], np.array(vals[1 + q * nout:1 + (q + 1) * nout], dtype=np.int32),
                                                  err_msg=f"{name} P={P} k={k} {mode} rank {q}")


def _ref_earlier(exe, name, P, k, n, seed, extra, nout):
    r = subprocess.run([str(exe), name, str(P), str(k), str(n), str(seed)] + ([str(extra)] if extra is not None else []),
                       capture_output=True, text=True, timeout=30)
    vals = [int(v) for v in r.stdout.split()]
    assert vals and vals[0] == 0, f"the reference's {name} itself failed for P={P} k={k} extra={extra}"
    return [np.array(vals[1 + q * nout:1 + (q + 1) * nout], dtype=np.int32) for q in range(P)]


def test_earlier_variants_match_the_reference(ref_mpich_driver):
    """The earlier variants the reference keeps in its tree, built unmodified: the store-and-forward
    reduce-scatter (radix r <= P - 2, batch b), the flat radix-k Bruck allgather, the flat k-nomial gather, the k-nomial
    reduce-scatter (on the shapes where the reference's own copy works: P a power of k) and the
    all-to-all-v with ragged counts."""
    seed, n = 5, 3
    pat = lambda q, m: ((seed * 31 + q * 1009 + np.arange(m) * 7) % 97).astype(np.int32)
    for P in (2, 3, 4, 5, 6, 8, 9, 12):
        full = [pat(q, n * P) for q in range(P)]
        for r_ in (2, 3, 4):
            if r_ > P - 2:
                continue                      # the reference's copy does not terminate once the radix reaches P - 1
            for batch in (1, 2, P):
                ours = Program("reduce_scatter", "radix_block", P, n, r_, batch).simulate(full)
                ref = _ref_earlier(ref_mpich_driver, "rs_radix_block", P, r_, n, seed, batch, n)
                for q in range(P):
                    np.testing.assert_array_equal(ours[q], ref[q], err_msg=f"radix_block P={P} r={r_} b={batch} rank {q}")
        for k in (2, 3):
            if P not in {2: (2, 4, 8), 3: (3, 9)}[k]:
                continue      # elsewhere the reference's copy returns another rank's block (P=3, k=2) or an error code
            ours = Program("reduce_scatter", "k_nomial", P, n, k, 1).simulate(full)
            ref = _ref_earlier(ref_mpich_driver, "rs_k_nomial", P, k, n, seed, None, n)
            for q in range(P):
                np.testing.assert_array_equal(ours[q], ref[q], err_msg=f"k_nomial P={P} k={k} rank {q}")
        blocks = [pat(q, n) for q in range(P)]
        for k in (2, 3, 4):
            ours = Program("allgather", "k_brucks", P, n, k, 1).simulate(blocks)
            ref = _ref_earlier(ref_mpich_driver, "ag_k_brucks", P, k, n, seed, None, n * P)
            for q in range(P):
                np.testing.assert_array_equal(ours[q], ref[q], err_msg=f"k_brucks P={P} k={k} rank {q}")
            ours = Program("gather", "k_nomial", P, n, k, 1, aux=0).simulate(blocks)
            ref = _ref_earlier(ref_mpich_driver, "gather_k_nomial", P, k, n, seed, None, n * P)
            np.testing.assert_array_equal(ours[0], ref[0], err_msg=f"gather_k_nomial P={P} k={k}")
        # all-to-all-v: rank s sends n + (s + 2 d) % 3 elements to rank d
        cnt = lambda s_, d_: n + (s_ + 2 * d_) % 3
        counts = [[cnt(s_, d_) for d_ in range(P)] for s_ in range(P)]
        nin = max(sum(row) for row in counts)
        nout = max(sum(counts[s_][d_] for s_ in range(P)) for d_ in range(P))
        for r_, batch in ((2, 1), (3, 2)):
            if P < 3:
                continue
            prog = Program.alltoallv(counts, r=r_, b=batch)
            ours = prog.simulate([pat(q, prog.in_elems) for q in range(P)])
            ref = _ref_earlier(ref_mpich_driver, "a2av_tuna2", P, r_, n, seed, batch, nout)
            assert prog.in_elems == nin
            for q in range(P):
                m = sum(counts[s_][q] for s_ in range(P))
                np.testing.assert_array_equal(ours[q][:m], ref[q][:m], err_msg=f"alltoallv P={P} r={r_} b={batch} rank {q}")


@pytest.mark.parametrize("P,b", [(4, 2), (8, 2), (8, 4), (8, 8), (6, 3), (12, 3), (12, 2), (16, 4)])
def test_semi_custom_and_custom_allreduce_match_the_reference(ref_driver, P, b):
    """all_reduce_semi_radix_batch (recursive-halving reduce-scatter + hierarchical allgather,
    all_reduce_semi_custom_0_1.cpp:159-193) and the earlier custom allreduce (store-and-forward reduce-scatter +
    hierarchical allgather, all_reduce_custom_0_2.cpp:49-663), both built unmodified."""
    seed, n = 5, 2
    custom_exe = ROOT / "baseline" / "_ref" / "ref_custom_driver"
    if not custom_exe.exists():
        from baseline import build_reference
        build_reference.build_custom()
    ins = [((seed * 31 + r * 1009 + np.arange(n * P)) % 97).astype(np.int32) for r in range(P)]
    for k in (2, 3):
        ref = reference_result(ref_driver, "semi", P, k, b, n, seed)
        ours = Program("allreduce", "semi_radix_batch", P, n * P, k, b).simulate(ins)
        for r in range(P):
            np.testing.assert_array_equal(ours[r], ref[r], err_msg=f"semi P={P} k={k} b={b} rank {r}")
        if k <= P - 2:       # the store-and-forward half of the reference does not terminate with a radix of P - 1 or more
            out = subprocess.run([str(custom_exe), str(P), str(k), str(b), str(n), str(seed)], capture_output=True, text=True, timeout=30)
            vals = [int(v) for v in out.stdout.split()]
            assert vals and vals[0] == 0, f"the reference's custom allreduce failed for P={P} r={k} b={b}"
            ours = Program("allreduce", "custom", P, n * P, k, b).simulate(ins)
            for r in range(P):
                np.testing.assert_array_equal(ours[r], np.array(vals[1 + r * n * P:1 + (r + 1) * n * P], dtype=np.int32),
                                              err_msg=f"custom P={P} r={k} b={b} rank {r}")


@pytest.mark.parametrize("P,b", [(4, 1), (4, 2), (8, 2), (8, 4), (8, 8), (12, 3), (16, 4), (18, 3), (6, 6), (9, 3), (10, 2), (12, 2)])
def test_float_results_are_bit_identical_to_the_reference(ref_driver, P, b):
    """float32 inputs that do not add exactly: the bits of a sum depend on the order of the additions.  The pull
    programs combine their sources in the order in which the reference receives and reduces them, so the results
    agree bit for bit (reduce-scatter, allreduce and the semi-custom allreduce)."""
    seed, n = 5, 3
    pat = lambda q: (((seed * 31 + q * 1009 + np.arange(n * P)) % 97).astype(np.float32) / np.float32(7.0)
                     + np.float32(q) * np.float32(0.37)).astype(np.float32)
    ins = [pat(q) for q in range(P)]
    exact = np.sum(np.stack(ins).astype(np.float64), axis=0)
    for k in (2, 3, 4):
        for short, coll, algo in (("rs", "reduce_scatter", "radix_batch"), ("ar", "allreduce", "radix_batch"),
                                  ("semi", "allreduce", "semi_radix_batch")):
            r = subprocess.run([str(ref_driver), "checkf", short, str(P), str(k), str(b), str(n), str(seed)],
                               capture_output=True, text=True, timeout=120)
            vals = [int(v) for v in r.stdout.split()]
            assert vals and vals[0] == 0
            per = n if short == "rs" else n * P
            ours = Program(coll, algo, P, per, k, b).simulate(ins)
            for q in range(P):
                ref = np.array(vals[1 + q * per:1 + (q + 1) * per], dtype=np.uint32)
                np.testing.assert_array_equal(ours[q].view(np.uint32), ref, err_msg=f"{coll}/{algo} P={P} k={k} b={b} rank {q}")
    # the test has teeth: another order of the same additions changes bits for these inputs
    flipped = np.sum(np.stack(ins[::-1]), axis=0, dtype=np.float32)
    forward = ins[0].copy()
    for x in ins[1:]:
        forward = forward + x
    backward = ins[-1].copy()
    for x in ins[-2::-1]:
        backward = backward + x
    assert np.allclose(forward, exact, rtol=1e-5) and flipped.shape == forward.shape
    if P >= 8:
        assert not np.array_equal(forward.view(np.uint32), backward.view(np.uint32))


@pytest.mark.parametrize("name", sorted(n for n in MPICH if n != "ar_smp"))
def test_mpich_style_baselines_are_bit_identical_on_floats(ref_mpich_driver, name):
    """float32 inputs that do not add exactly: every MPICH-style baseline adds in the reference's order (phases,
    neighbour order, fold order, block boundaries), so the sums agree bit for bit.  The SMP allreduce is left out:
    its order is that of the MPI library's own MPI_Reduce / MPI_Allreduce, which MPI does not define."""
    coll, algo, has_k = MPICH[name]
    seed, n = 3, 3
    for P in (2, 3, 4, 5, 6, 7, 8, 12):
        nout = n * P if coll == "allreduce" else n
        ins = [(((seed * 31 + q * 1009 + np.arange(n * P) * 7) % 97).astype(np.float32) / np.float32(7.0)
                + np.float32(q) * np.float32(0.37)).astype(np.float32) for q in range(P)]
        for k in ((2, 3, 4) if has_k else (2,)):
            r = subprocess.run([str(ref_mpich_driver), name, str(P), str(k), str(n), str(seed), "float"],
                               capture_output=True, text=True, timeout=120)
            vals = [int(v) for v in r.stdout.split()]
            assert vals and vals[0] == 0
            ours = Program(coll, algo, P, n * P if coll == "allreduce" else n, k, 1).simulate(ins)
            for q in range(P):
                np.testing.assert_array_equal(ours[q].view(np.uint32), np.array(vals[1 + q * nout:1 + (q + 1) * nout], dtype=np.uint32),
                                              err_msg=f"{name} P={P} k={k} rank {q}")
