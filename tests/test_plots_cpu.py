"""The analysis scripts on a synthetic CSV (every kind, every statistic) and on the reference's own published
result files, which use the same schema (testing/plots/*/results_*_final.csv)."""
import os
from pathlib import Path

import numpy as np
import pandas as pd
import pytest

from configurable_hierarchical_allreduce_algorithms_b200.bench import plots

REF_PLOTS = Path(os.environ.get("CHB_REFERENCE_DIR", Path(__file__).resolve().parents[2] / "reference")) / "testing" / "plots"


def _synthetic(path):
    rng = np.random.default_rng(0)
    rows = []
    for nprocs in (4, 8):
        for n in (1, 64, 4096):
            for rep in range(5):
                for k in (2, 3, 4):
                    t = 1e-5 * (1 + 0.1 * k) * (1 + n / 4096) * (1 + 0.01 * rng.random())
                    rows.append(("all_reduce_radix_batch", k, 4, nprocs, n, t if k != 3 else t * 0.5, 1))
                rows.append(("allreduce_ring", 0, 0, nprocs, n, 3e-5 * (1 + n / 4096), 1))
                rows.append(("MPICH_allreduce", 0, 0, nprocs, n, 2e-5 * (1 + n / 4096), 1))
    pd.DataFrame(rows, columns=["algorithm_name", "k", "b", "nprocs", "send_count", "time", "is_correct"]).to_csv(path, index=False)


def test_every_analysis_on_a_synthetic_file(tmp_path):
    csv = tmp_path / "r.csv"
    _synthetic(csv)
    w = plots.winners_table(plots.load(str(csv)))
    assert len(w) == 6 and (w.winner == "all_reduce_radix_batch (k=3)").all()       # k = 3 was made twice as fast
    assert ((w.speedup > 2.5) & (w.speedup < 4.5)).all()                            # library time / winner time
    for stat in ("median", "mean", "min"):
        outs = [plots.median_best(str(csv), str(tmp_path), stat), plots.radix(str(csv), str(tmp_path), stat),
                plots.winners(str(csv), str(tmp_path), stat)] + plots.per_algo(str(csv), str(tmp_path), stat)
        for o in outs:
            assert Path(o).exists() and Path(o).stat().st_size > 0
    if plots.plt is None:       # markdown fallbacks carry the numbers themselves
        txt = Path(plots.radix(str(csv), str(tmp_path))).read_text()
        assert "| 1 | 3 |" in txt and "best k" in txt
    plots.main(["winners", str(csv), "--outdir", str(tmp_path / "cli")])
    assert any((tmp_path / "cli").iterdir())


@pytest.mark.parametrize("rel", ["reduce_scatter/results_polaris_final.csv", "all_gather/results_aurora_64_final.csv",
                                 "all_reduce/results_custom_polaris.csv"])
def test_reference_result_files_load_and_rank(tmp_path, rel):
    """A user's existing result files work unchanged: winners per (nprocs, send_count) with the library baseline's name
    recognised, so the speed-up column is filled."""
    path = REF_PLOTS / rel
    if not path.exists():
        pytest.skip("the reference's result files are not available on this machine")
    df = plots.load(str(path))
    w = plots.winners_table(df)
    assert len(w) > 10 and w.speedup.notna().mean() > 0.9
    assert w.winner.str.contains("radix_batch|standard|MPICH|reduce_scatter|allgather|all_reduce").all()
    out = plots.median_best(str(path), str(tmp_path))
    assert Path(out).exists()


def test_tuner_samples_through_the_winner_analysis(tmp_path):
    """The tuner's CSV (all collectives in one file, NCCL rows named <collective>_nccl[_ring|_tree], a CTA count per
    candidate) goes through the same analysis: one collective at a time, the speed-up against NCCL's default."""
    from configurable_hierarchical_allreduce_algorithms_b200.bench import plots
    src = Path(__file__).parent / "data" / "tune_samples_8xB200_fp32.csv"
    try:
        plots.main(["median_best", str(src), "--coll", "allreduce", "--outdir", str(tmp_path)])
    finally:
        plots.FILTER.update(coll="", dtype="")
    outs = list(tmp_path.glob("median_best_*"))
    assert len(outs) == 1
    if outs[0].suffix == ".md":
        text = outs[0].read_text()
        rows = [l for l in text.splitlines() if l.startswith("| 8 |")]
        assert len(rows) >= 8 and all("allreduce_" in r and "nccl" not in r.split("|")[3] for r in rows)
        assert all(r.strip().endswith("x |") and "nan" not in r for r in rows)
