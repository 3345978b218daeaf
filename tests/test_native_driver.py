"""The native launcher + benchmark driver (`bin/chb_bench`, no Python and no MPI in its call path):
argument grammar on CPU, an emulated world on one GPU, forked one-rank-per-GPU processes on several."""
import subprocess
from pathlib import Path

import pandas as pd
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
EXE = ROOT / "configurable_hierarchical_allreduce_algorithms_b200" / "bin" / "chb_bench"
COLS = ["algorithm_name", "k", "b", "nprocs", "send_count", "time", "is_correct"]


@pytest.fixture(scope="module")
def exe():
    from configurable_hierarchical_allreduce_algorithms_b200 import _build
    _build.build()
    assert EXE.exists()
    return str(EXE)


def test_argument_grammar(exe, tmp_path):
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 2 and "usage" in r.stderr
    r = subprocess.run([exe, "2", "bogus=1"], capture_output=True, text=True)
    assert r.returncode == 2 and "Unknown parameter: bogus=1" in r.stderr
    r = subprocess.run([exe, "2", "coll=broadcast"], capture_output=True, text=True)
    assert r.returncode == 2
    r = subprocess.run([exe, "2", "emulate=4", "b=3"], capture_output=True, text=True)
    assert r.returncode == 2 and "divide" in r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("coll,dtype,op", [("allreduce", "int32", "sum"), ("allreduce", "bf16", "max"),
                                           ("reduce_scatter", "fp32", "sum"), ("allgather", "fp64", "sum")])
def test_emulated_world(exe, tmp_path, cuda, coll, dtype, op):
    out = tmp_path / "r.csv"
    args = [exe, "3", "--overwrite", "emulate=4", "b=2", "base=1000", f"coll={coll}", f"dtype={dtype}", f"op={op}", "reps=2", f"out={out}"]
    r = subprocess.run(args, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    df = pd.read_csv(out)
    assert list(df.columns[:7]) == COLS
    assert (df.is_correct == 1).all() and (df.nprocs == 4).all() and set(df.send_count) == {1000, 2000, 4000}
    assert len(set(df.algorithm_name)) >= 3
    n1 = len(df)
    r = subprocess.run(args[:2] + args[3:] + ["symmetric=1", "algos=radix_batch,ll"], capture_output=True, text=True, timeout=300)   # appends
    assert r.returncode == 0, r.stdout + r.stderr
    df2 = pd.read_csv(out)
    assert len(df2) > n1 and (df2.is_correct == 1).all()


@pytest.mark.multigpu
@pytest.mark.parametrize("coll", ["allreduce", "reduce_scatter", "allgather"])
def test_forked_ranks_one_per_gpu(exe, tmp_path, coll):
    from conftest import gpus_for_test
    n = gpus_for_test(4)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    n = 2 if n < 4 else 4
    out = tmp_path / "r.csv"
    r = subprocess.run([exe, "3", "--overwrite", f"ngpus={n}", f"b={n}", "base=4096", f"coll={coll}", "dtype=fp32", "reps=3",
                        "symmetric=1", f"out={out}"], capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout + r.stderr
    df = pd.read_csv(out)
    assert (df.is_correct == 1).all() and (df.nprocs == n).all()
    names = set(df.algorithm_name)
    assert any("radix_batch" in x for x in names)
    assert names & {"MPICH_allreduce", "reduce_scatter_standard", "allgather_standard"}, names     # the NCCL row
    # the launcher's heaps come from the native virtual-memory allocator with a multicast alias where the devices have
    # one: the in-switch kernels then run from this binary too (skipped, with a message, where there is no alias)
    out2 = tmp_path / "nvls.csv"
    r = subprocess.run([exe, "2", "--overwrite", f"ngpus={n}", f"b={n}", "base=4096", f"coll={coll}", "dtype=fp32", "reps=3",
                        "symmetric=1", "algos=nvls,radix_batch", f"out={out2}"], capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout + r.stderr
    df2 = pd.read_csv(out2)
    assert (df2.is_correct == 1).all()
    if "skipped" not in r.stderr:
        assert any("nvls" in x for x in set(df2.algorithm_name)), set(df2.algorithm_name)


LINKBW = EXE.with_name("chb_linkbw")


def test_linkbw_arguments(exe):
    r = subprocess.run([str(LINKBW), "0"], capture_output=True, text=True)
    assert r.returncode == 2 and "usage" in r.stderr
    r = subprocess.run([str(LINKBW), "8", "1"], capture_output=True, text=True)
    assert r.returncode == 2


@pytest.mark.gpu
def test_linkbw_runs(exe, cuda):
    """Two GPUs: one CSV row per (width, mode, directions, CTAs) with positive rates, and pulling from the peer is not
    faster than copying locally.  One GPU: it says what it needs and leaves."""
    r = subprocess.run([str(LINKBW), "64", "2"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    if torch.cuda.device_count() < 2:
        assert "needs two GPUs" in r.stdout
        return
    if "cannot access" in r.stdout:
        return
    import io
    df = pd.read_csv(io.StringIO(r.stdout))
    assert len(df) == 2 * 3 * 2 * 4 and (df.GBps_gpu0 > 0).all()
    pull = df[(df["mode"] == "pull (read peer)") & (df.directions == "both")].GBps_gpu0.max()
    local = df[(df["mode"] == "local copy") & (df.directions == "both")].GBps_gpu0.max()
    assert pull < local
