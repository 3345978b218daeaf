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


@pytest.mark.timeout(900)
def test_driver_two_levels_and_launcher(tmp_path):
    """4 gloo ranks as 2 boxes of 2: the swept algorithm inside a box, a ring program along the lanes;
    and the launcher's command lines for the three environments."""
    out = tmp_path / "two.csv"
    for coll in ("allreduce", "reduce_scatter", "allgather"):
        _run(["2", "base=8", "reps=2", "backend=gloo", f"out={out}", "local_size=2", "inter_algo=ring", f"coll={coll}",
              "algos=radix_batch,ring,reduce_scatter_allgather"], tmp_path)
    df = pd.read_csv(out)
    assert (df.is_correct == 1).all() and (df.nprocs == 4).all() and (df.b[df.algorithm_name.str.contains("radix_batch")] == 2).all()
    assert {"all_reduce_radix_batch", "allreduce_ring", "reduce_scatter_ring", "allgather_radix_batch"} <= set(df.algorithm_name)
    assert "allreduce_reduce_scatter_allgather" not in set(df.algorithm_name)      # cannot serve as a level's reduce-scatter: skipped
    _run(["1", "base=8", "reps=1", "backend=gloo", f"out={out}", "local_size=2", "inter_algo=library"], tmp_path)
    assert (pd.read_csv(out).is_correct == 1).all()

    from configurable_hierarchical_allreduce_algorithms_b200.bench import launch
    cmd = launch.build_command("LOCAL", 2, 2, 0, "127.0.0.1:29577", ["3", "b=2"])
    assert "--nproc-per-node=4" in cmd and "backend=gloo" in cmd and "num_nodes=2" in cmd and "b=2" in cmd
    cmd = launch.build_command("MULTINODE", 8, 2, 1, "node0:29500", ["3", "backend=gpu"])
    assert "--nnodes=2" in cmd and "--node-rank=1" in cmd and cmd.count("backend=gpu") == 1 and "node0" in cmd
    cmd = launch.build_command("B200", 8, 1, 0, "127.0.0.1:29500", ["3"])
    assert "--nproc-per-node=8" in cmd and "backend=gpu" in cmd
    with pytest.raises(SystemExit):
        launch.build_command("MOON", 1, 1, 0, "127.0.0.1:1", [])
    assert launch.main(["--env", "LOCAL", "--ranks-per-node", "2", "--dry-run", "--", "2", "b=2"]) == 0
