"""Median-winner-per-cell tuning table (host logic only)."""
import json

import pytest

from configurable_hierarchical_allreduce_algorithms_b200.utils import autotune


class FakeComm:
    P, device, nlocal = 8, 0, 1
    ll_max_bytes, ll2_max_bytes, has_multicast = 1 << 20, 4 << 20, True


def _samples():
    out = []
    for nbytes, best in ((1024, "ll"), (1 << 20, "ll2"), (1 << 26, "nvls")):
        for algo, t in (("ll", 3.0), ("ll2", 2.0), ("nvls", 4.0), ("radix_batch", 5.0)):
            for rep in range(3):
                out.append({"coll": "allreduce", "dtype": "fp32", "bytes": nbytes, "algo": algo, "k": 2, "b": 1,
                            "nctas": 0, "time_s": (1.0 if algo == best else t) + 0.01 * rep, "is_correct": 1})
    return out


def test_winners_and_table(tmp_path, monkeypatch):
    w = autotune.winners(_samples())
    assert w[("allreduce", "fp32", 1024)][0][0] == "ll"
    assert w[("allreduce", "fp32", 1 << 26)][0][0] == "nvls"
    table = autotune.build_table(_samples(), "cpu", 8)
    rows = table["cpu|8|allreduce|fp32"]
    assert [r[1] for r in rows] == ["ll", "ll2", "nvls"] and rows[-1][0] == 1 << 62
    path = tmp_path / "t.json"
    autotune.save_table(table, path)
    assert json.loads(path.read_text()) == table
    monkeypatch.setenv("CHB_TUNE_TABLE", str(path))
    autotune.reload()
    import torch
    c = autotune.choose(FakeComm(), "allreduce", 2000, torch.float32, True)
    assert c.algo == "ll2"                      # first row whose max_bytes covers the size
    assert autotune.choose(FakeComm(), "allreduce", 1 << 28, torch.float32, True).algo == "nvls"
    # a multicast winner falls back to the heuristic when the buffers are not symmetric
    assert autotune.choose(FakeComm(), "allreduce", 1 << 28, torch.float32, False).algo != "nvls"
    monkeypatch.setenv("CHB_ALGO", "ring")
    assert autotune.choose(FakeComm(), "allreduce", 64, torch.float32, True).algo == "ring"
    monkeypatch.delenv("CHB_ALGO")
    monkeypatch.delenv("CHB_TUNE_TABLE")
    autotune.reload()


def test_incorrect_rows_are_refused():
    bad = _samples()
    bad[0]["is_correct"] = 0
    with pytest.raises(ValueError, match="incorrect"):
        autotune.winners(bad)


def test_tuner_candidates_cover_the_kernel_families():
    """Every cell's candidate list names only runnable configurations and offers each kernel family where it applies."""
    from configurable_hierarchical_allreduce_algorithms_b200.bench import tune

    class Comm:
        ll_max_bytes, ll2_max_bytes, has_multicast = 1 << 20, 4 << 20, True

    for P in (2, 4, 8):
        for coll in ("allreduce", "reduce_scatter", "allgather"):
            for nbytes in (8, 1 << 10, 1 << 16, 1 << 20, 1 << 24, 1 << 30):
                total = nbytes * (P if coll != "allreduce" else 1)
                cands = tune.candidates(coll, P, nbytes, Comm, total)
                assert cands and len(set(cands)) == len(cands)
                for name, k, b, nctas in cands:
                    assert k >= 2 and P % b == 0 and nctas >= 0
                    algo, _, mode = name.partition(":")              # "<program>:ll" / "<program>:pull" pin the execution mode
                    assert mode in ("", "ll", "pull") and (not mode or algo in {"radix_batch", "recursive_doubling", "reduce_scatter_allgather"})
                    assert mode != "ll" or total <= 4 << 20
                    assert algo in {"ll", "ll2", "radix_batch", "nvls", "nvls1", "bulk", "recursive_doubling", "reduce_scatter_allgather"}
                    assert algo != "ll2" or coll == "allreduce"
                    assert algo != "bulk" or (coll == "allgather" and nbytes >= 1 << 20)
                algos = {c[0].partition(":")[0] for c in cands}
                assert "radix_batch" in algos
                # the k in {2, 4, 8} x b in {1, 2, 4} grid is there, as distinct programs
                shapes = {(k, b) for a, k, b, _ in cands if a.startswith("radix_batch")}
                assert shapes == set(tune.grid_cells(P)) and (2, 1) in shapes
                for k in (2, 4, 8):
                    for b in (1, 2, 4):
                        if b <= P and P % b == 0:
                            assert tune.canonical(k, b) in shapes
                assert ("ll" in algos) == (nbytes <= Comm.ll_max_bytes)
                if nbytes >= 1 << 24:
                    assert "nvls" in algos and ("bulk" in algos) == (coll == "allgather")
    Comm.has_multicast = False
    assert all(c[0] not in ("nvls", "nvls1") for c in tune.candidates("allreduce", 8, 1 << 24, Comm))


def test_markdown_summary_of_a_sweep(tmp_path):
    from configurable_hierarchical_allreduce_algorithms_b200.bench import tune

    class Comm:
        ll_max_bytes, ll2_max_bytes, has_multicast = 1 << 20, 4 << 20, True

    rows = []
    for sz in (32768, 1 << 24):
        for (a, k, b, c) in tune.candidates("allreduce", 8, sz, Comm, sz):
            rows.append([f"allreduce_{a}", k, b, 8, sz // 32, 1e-5 * (1 + k + b), 1, "fp32", "sum", sz, 0, 0, 0, 8, c])
        rows.append(["allreduce_radix_batch:pull", 4, 4, 8, sz // 32, 1e-9, 0, "fp32", "sum", sz, 0, 0, 0, 8, 64])   # wrong result: never wins
        for name in ("nccl", "nccl_ring", "nccl_tree"):
            rows.append([f"allreduce_{name}", 0, 0, 8, sz // 32, 3e-5, 1, "fp32", "sum", sz, 0, 0, 0, 8, 0])
    out = tmp_path / "s.md"
    tune.write_markdown(str(out), rows, 8, "NVIDIA B200", "-m x.tune --iters 3")
    text = out.read_text()
    assert "## allreduce, fp32" in text and "k=2 b=1" in text and "WRONG" in text and "| 32768 |" in text
    assert "0.00x" not in text.split("Best time")[0].splitlines()[-2]


def _recorded_samples():
    """Candidate medians recorded by ``bench/tune.py`` on 8 x B200 (fp32 rows of one sweep)."""
    import csv
    from pathlib import Path

    path = Path(__file__).resolve().parent / "data" / "tune_samples_8xB200_fp32.csv"
    out = []
    with open(path) as f:
        for r in csv.DictReader(f):
            name = r["algorithm_name"]
            coll = next(c for c in ("allreduce", "reduce_scatter", "allgather") if name.startswith(c + "_"))
            algo = name[len(coll) + 1:]
            if algo.startswith("nccl") or algo == "fp8wire":
                continue                                   # the library baseline and the lossy format are never candidates
            P, total = int(r["nprocs"]), int(r["bytes"])
            out.append({"coll": coll, "dtype": r["dtype"], "bytes": total if coll == "allreduce" else total // P,
                        "algo": algo, "k": int(r["k"]), "b": int(r["b"]), "nctas": int(r["nctas"]),
                        "time_s": float(r["time"]), "is_correct": int(r["is_correct"])})
    return out


def test_tuned_choice_is_within_five_percent_of_the_exhaustive_best_on_recorded_samples(tmp_path, monkeypatch):
    """The table built from a recorded sweep answers, for every measured cell, a candidate whose recorded time is
    within 5 % of the fastest candidate of that cell (merging neighbouring cells with the same winner and the
    lookup by ``max_bytes`` must not lose anything)."""
    import torch

    samples = _recorded_samples()
    assert len(samples) > 300 and all(s["is_correct"] == 1 for s in samples)
    table = autotune.build_table(samples, "NVIDIA B200", 8)
    path = tmp_path / "t.json"
    autotune.save_table(table, path, merge=False)
    monkeypatch.setenv("CHB_TUNE_TABLE", str(path))
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "get_device_name", lambda *_: "NVIDIA B200")
    autotune.reload()
    cells = {}
    for s in samples:
        cells.setdefault((s["coll"], s["bytes"]), {})[(s["algo"], s["k"], s["b"], s["nctas"])] = s["time_s"]
    worst = 0.0
    for (coll, nbytes), cands in cells.items():
        c = autotune.choose(FakeComm(), coll, nbytes, torch.float32, True)
        got = cands[(c.algo, c.k, c.b, c.nctas)]
        best = min(cands.values())
        worst = max(worst, got / best)
        assert got <= 1.05 * best, (coll, nbytes, c, got, best)
    # sizes between two measured cells take the next cell's winner: judged on a sweep with every other size held out
    sizes = {coll: sorted({b for (c, b) in cells if c == coll}) for coll in ("allreduce", "reduce_scatter", "allgather")}
    held = {(coll, b) for coll, bs in sizes.items() for b in bs[1::2]}
    table2 = autotune.build_table([s for s in samples if (s["coll"], s["bytes"]) not in held], "NVIDIA B200", 8)
    autotune.save_table(table2, path, merge=False)
    autotune.reload()
    ratios = []
    for (coll, nbytes) in sorted(held):
        c = autotune.choose(FakeComm(), coll, nbytes, torch.float32, True)
        cands = cells[(coll, nbytes)]
        key = (c.algo, c.k, c.b, c.nctas)
        if key not in cands:                                # e.g. a CTA count that was not offered at this size
            same = [t for (a, k, b, _), t in cands.items() if (a, k, b) == key[:3]]
            if not same:
                continue
            got = min(same)
        else:
            got = cands[key]
        ratios.append(got / min(cands.values()))
    assert ratios and sorted(ratios)[len(ratios) // 2] <= 1.25, ratios      # the median held-out cell stays close
    monkeypatch.delenv("CHB_TUNE_TABLE")
    autotune.reload()
