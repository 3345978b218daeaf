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
                cands = tune.candidates(coll, P, nbytes, Comm)
                assert cands and len(set(cands)) == len(cands)
                for algo, k, b, nctas in cands:
                    assert k >= 2 and P % b == 0 and nctas >= 0
                    assert algo in {"ll", "ll2", "radix_batch", "nvls", "nvls1", "bulk", "recursive_doubling"}
                    assert algo != "ll2" or coll == "allreduce"
                    assert algo != "bulk" or (coll == "allgather" and nbytes >= 1 << 20)
                algos = {c[0] for c in cands}
                assert "radix_batch" in algos
                assert ("ll" in algos) == (nbytes <= Comm.ll_max_bytes)
                if nbytes >= 1 << 24:
                    assert "nvls" in algos and ("bulk" in algos) == (coll == "allgather")
    Comm.has_multicast = False
    assert all(c[0] not in ("nvls", "nvls1") for c in tune.candidates("allreduce", 8, 1 << 24, Comm))
