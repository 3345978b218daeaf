"""The checked build (-DCHB_CHECK_BOUNDS: in-kernel range test of every step) must keep compiling for sm_100a."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "configurable_hierarchical_allreduce_algorithms_b200" / "csrc"


@pytest.mark.timeout(900)
def test_interpreter_compiles_with_bounds_checks(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        pytest.skip("no nvcc")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
           "-DCHB_CHECK_BOUNDS", "-Xcompiler", "-fPIC", "-Xptxas", "-v", "-I", str(CSRC), "-c",
           str(CSRC / "kernels" / "interp.cu"), "-o", str(tmp_path / "interp_checked.o")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    assert "ST_OUT_OF_RANGE" in (CSRC / "kernels" / "common.cuh").read_text()
