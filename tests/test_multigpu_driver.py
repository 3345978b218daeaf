"""The benchmark driver on GPUs with registered (symmetric) buffers, so that the kernel-level
algorithms (flagged lines, NVLS, bulk copies) run under its self-check.  Needs >= 2 GPUs."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import pandas as pd
import pytest
import torch

pytestmark = pytest.mark.multigpu
ROOT = Path(__file__).resolve().parent.parent
MOD = "configurable_hierarchical_allreduce_algorithms_b200.bench.driver"


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.timeout(600)
@pytest.mark.parametrize("coll,algos", [("allgather", "radix_batch,bulk,ll,nvls"), ("allreduce", "radix_batch,ll,ll2,nvls,ring"),
                                        ("reduce_scatter", "radix_batch,ll,nvls,pairwise")])
def test_driver_on_symmetric_buffers(tmp_path, coll, algos):
    from conftest import gpus_for_test
    n = gpus_for_test(4)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    n = 2 if n < 4 else 4
    out = tmp_path / "r.csv"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n), "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), "-m", MOD, "3", "--overwrite", "base=4096", "dtype=fp32",
           f"coll={coll}", f"algos={algos}", "reps=3", "symmetric=1", f"out={out}", f"b={n}"]
    env = dict(os.environ, PYTHONPATH=str(ROOT))
    r = subprocess.run(cmd, cwd=tmp_path, env=env, capture_output=True, text=True, timeout=500)
    assert r.returncode == 0, r.stderr[-3000:]
    df = pd.read_csv(out)
    assert (df.is_correct == 1).all(), df[df.is_correct != 1]
    names = set(df.algorithm_name)
    for a in algos.split(","):
        if a != "nvls":      # needs a multicast alias, skipped by the driver where there is none
            assert any(a in x for x in names), (a, names)


@pytest.mark.timeout(600)
def test_driver_two_levels_on_gpus(tmp_path):
    """Boxes of L GPUs (L = 1 with two GPUs, 2 with four): kernels inside a box, NCCL or a ring program along the lanes."""
    from conftest import gpus_for_test
    n = gpus_for_test(4)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    n = 2 if n < 4 else 4
    out = tmp_path / "two.csv"
    for inter in ("library", "ring"):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n), "--master-addr",
               "127.0.0.1", "--master-port", str(_free_port()), "-m", MOD, "2", "base=4096", "dtype=fp32", "coll=allreduce",
               "algos=radix_batch,ring", "reps=2", f"local_size={n // 2}", f"inter_algo={inter}", f"out={out}"]
        r = subprocess.run(cmd, cwd=tmp_path, env=dict(os.environ, PYTHONPATH=str(ROOT)), capture_output=True, text=True, timeout=500)
        assert r.returncode == 0, r.stderr[-3000:]
    df = pd.read_csv(out)
    assert (df.is_correct == 1).all() and (df.nprocs == n).all() and len(df) >= 16
