"""The benchmark driver under gloo: argv grammar, CSV schema, resume by append,
and the plot scripts' refusal of incorrect rows."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import pandas as pd
import pytest

ROOT = Path(__file__).resolve().parent.parent
MOD = "configurable_hierarchical_allreduce_algorithms_b200.bench.driver"


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run(args, cwd):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "4", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), "-m", MOD] + args
    env = dict(os.environ, PYTHONPATH=str(ROOT), CUDA_VISIBLE_DEVICES="")
    r = subprocess.run(cmd, cwd=cwd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]


@pytest.mark.timeout(900)
def test_driver_writes_reference_schema_and_appends(tmp_path):
    out = tmp_path / "r.csv"
    common = ["b=2", "base=4", "reps=2", "backend=gloo", f"out={out}", "algos=radix_batch,ring,recursive_doubling"]
    _run(["2", "--overwrite"] + common, tmp_path)
    df = pd.read_csv(out)
    assert list(df.columns[:7]) == ["algorithm_name", "k", "b", "nprocs", "send_count", "time", "is_correct"]
    assert (df.is_correct == 1).all() and (df.nprocs == 4).all()
    assert set(df.send_count) == {4, 8}
    assert {"all_reduce_radix_batch", "allreduce_ring", "allreduce_recursive_doubling", "MPICH_allreduce"} <= set(df.algorithm_name)
    n1 = len(df)
    _run(["1", "coll=allgather"] + common[:-1] + ["algos=radix_batch,k_brucks"], tmp_path)   # appended, no second header
    df2 = pd.read_csv(out)
    assert len(df2) > n1 and "allgather_standard" in set(df2.algorithm_name)
    # plots: winner grid from the same file, and refusal of incorrect rows
    from configurable_hierarchical_allreduce_algorithms_b200.bench import plots
    png = plots.median_best(str(out), outdir=str(tmp_path))
    assert Path(png).exists()
    bad = df2.copy()
    bad.loc[0, "is_correct"] = 0
    badp = tmp_path / "bad.csv"
    bad.to_csv(badp, index=False)
    with pytest.raises(SystemExit):
        plots.median_best(str(badp), outdir=str(tmp_path))
