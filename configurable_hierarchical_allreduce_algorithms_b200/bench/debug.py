"""Self-checking debug run of one algorithm on the host simulator, the
counterpart of the reference's per-file ``main()`` under ``-DDEBUG_MODE``
(built by ``make debug-<impl>``, testing/Makefile:130-134; e.g. closed-form
expectation ``sum_r (r + 0.1 i)`` and sizes {1, 100, 1000} in
testing/mpich_implementations/all_reduce/allreduce_recursive_doubling.cpp:105-257,
``k`` in 2..9 with a table in allreduce_recursive_multiplying.cpp:222-333).

    python -m configurable_hierarchical_allreduce_algorithms_b200.bench.debug <collective> <algorithm> [P=8] [b=1] [dump=1]

Prints, per (k, count): rounds, messages, elements moved, scratch elements and PASS / FAIL;
``dump=1`` also prints every rank's steps of the last program (rank-ordered, like the
reference's before / after buffer dumps).  Exit code 1 if anything fails.
"""
from __future__ import annotations

import sys

import numpy as np

from ..parallel.program import Program, ProgramError


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if len(argv) < 2:
        raise SystemExit(__doc__)
    coll, algo = argv[0], argv[1]
    opt = {"P": 8, "b": 1, "dump": 0}
    for a in argv[2:]:
        k, v = a.split("=")
        opt[k] = int(v)
    P, b = opt["P"], opt["b"]
    bad = 0
    print(f"{coll}/{algo}  P={P} b={b}")
    print(f"{'k':>3} {'count':>6} {'rounds':>6} {'msgs':>6} {'elems moved':>12} {'scratch':>8}  result")
    last = None
    for k in range(2, 10):
        for n in (1, 100, 1000):
            count = n * P if coll == "allreduce" else n
            try:
                p = Program(coll, algo, P, count, k, b)
            except ProgramError as e:
                print(f"{k:>3} {n:>6}  not applicable: {e}")
                continue
            p.verify()
            ins = [(r + 0.1 * np.arange(p.in_elems)).astype(np.float64) for r in range(P)]
            outs = p.simulate(ins)
            tot = sum(ins)
            if coll == "allreduce":
                ok = all(np.allclose(o, tot) for o in outs)          # closed form: sum_r (r + 0.1 i)
            elif coll == "reduce_scatter":
                ok = all(np.allclose(outs[r], tot[r * n:(r + 1) * n]) for r in range(P))
            elif coll == "allgather":
                ok = all(np.array_equal(o, np.concatenate(ins)) for o in outs)
            elif coll == "alltoall":
                ok = all(np.array_equal(outs[r], np.concatenate([ins[s][r * n:(r + 1) * n] for s in range(P)])) for r in range(P))
            else:
                ok = np.array_equal(outs[0], np.concatenate(ins))
            bad += not ok
            last = p
            print(f"{k:>3} {n:>6} {p.nrounds:>6} {p.remote_msgs:>6} {p.remote_elems:>12} {p.work_elems:>8}  {'PASS' if ok else 'FAIL'}")
    if opt["dump"] and last is not None:
        names = {0: "IN", 1: "OUT", 2: "WORK"}
        for r in range(P):
            print(f"-- rank {r}")
            for s in last.steps(r):
                srcs = " + ".join(f"{names[bf]}@{pr}[{off}]" for pr, bf, off in s.srcs)
                print(f"   round {s.round}: {names[s.dst_buf]}[{s.dst_off}:{s.dst_off + s.count}] {'+=' if s.acc else '='} {srcs}")
    print("ALL PASS" if not bad else f"{bad} FAILED")
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
