"""`python setup.py build_ext --inplace` is the documented way to build the native library in the tree."""
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_setup_py_builds_in_place():
    r = subprocess.run([sys.executable, "setup.py", "-q", "build_ext", "--inplace"], cwd=ROOT, capture_output=True, text=True, timeout=1800)
    assert r.returncode == 0, r.stderr[-2000:]
    lib = ROOT / "configurable_hierarchical_allreduce_algorithms_b200" / "libchb.so"
    assert lib.exists() and str(lib) in r.stdout
