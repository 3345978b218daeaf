"""The C ABI from a plain C program (no Python in the call path)."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "configurable_hierarchical_allreduce_algorithms_b200"


def _build(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    exe = tmp_path / "c_abi_example"
    cmd = [nvcc, "-x", "c", str(ROOT / "tests" / "native" / "c_abi_example.c"), "-I", str(PKG / "csrc" / "api"),
           "-L", str(PKG), "-lchb", "-Xlinker", f"-rpath={PKG}", "-o", str(exe)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    return exe


def test_c_example_compiles_against_the_headers(tmp_path):
    from configurable_hierarchical_allreduce_algorithms_b200 import _native
    _native.lib()                      # builds libchb.so if needed
    _build(tmp_path)


@pytest.mark.gpu
def test_c_example_runs(tmp_path, cuda):
    exe = _build(tmp_path)
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "C ABI OK" in r.stdout, r.stdout + r.stderr


def test_native_bootstrap_rendezvous(tmp_path):
    """Forked C ranks meet through the shared-memory bootstrap; a missing rank ends in a timeout, not a hang."""
    from configurable_hierarchical_allreduce_algorithms_b200 import _native
    _native.lib()
    cc = shutil.which("gcc") or "gcc"
    exe = tmp_path / "bootstrap_test"
    cmd = [cc, str(ROOT / "tests" / "native" / "bootstrap_test.c"), "-I", str(PKG / "csrc" / "boot"),
           "-L", str(PKG), "-lchb", f"-Wl,-rpath,{PKG}", "-o", str(exe)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "BOOTSTRAP OK" in r.stdout, r.stdout + r.stderr


def _build_ranks_example(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    exe = tmp_path / "native_ranks_example"
    cmd = [nvcc, "-x", "c", str(ROOT / "tests" / "native" / "native_ranks_example.c"), "-I", str(PKG / "csrc" / "api"),
           "-I", str(PKG / "csrc" / "boot"), "-L", str(PKG), "-lchb", "-Xlinker", f"-rpath={PKG}", "-o", str(exe)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    return exe


def test_native_ranks_example_compiles(tmp_path):
    """Launcher + bootstrap + cudaIpc communicator + reference-signature call from plain C: the headers fit together."""
    from configurable_hierarchical_allreduce_algorithms_b200 import _native
    _native.lib()
    _build_ranks_example(tmp_path)


@pytest.mark.multigpu
def test_native_ranks_example_runs(tmp_path):
    import torch
    from conftest import gpus_for_test
    n = gpus_for_test(4)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    exe = _build_ranks_example(tmp_path)
    r = subprocess.run([str(exe), str(min(n, 4))], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "NATIVE RANKS OK" in r.stdout, r.stdout + r.stderr
