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
