"""Host half of the native code under the compiler's sanitizers.

The schedule compiler (IR, generators, lowering, verifier, simulator) and the
threaded executor are built from source together with
``tests/native/sanitize_host.cc`` and run over every registered algorithm:
once with AddressSanitizer + UndefinedBehaviorSanitizer, once (threaded
executor only) with ThreadSanitizer.  The reference has no sanitizer runs
(plain ``mpicxx -O2``, testing/Makefile:26-41); this stands in for the device
tools that cannot be used on the kernels.
"""
from __future__ import annotations

import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
CSRC = ROOT / "configurable_hierarchical_allreduce_algorithms_b200" / "csrc"
DRIVER = ROOT / "tests" / "native" / "sanitize_host.cc"
CXX = shutil.which("g++")


def _build(tmp_path, name, flags):
    exe = tmp_path / name
    probe = tmp_path / "probe.cc"
    probe.write_text("int main(){return 0;}\n")
    if subprocess.run([CXX, *flags, str(probe), "-o", str(tmp_path / "probe")], capture_output=True).returncode != 0:
        pytest.skip(f"{' '.join(flags)} is not available with this compiler")
    srcs = sorted(str(p) for p in (CSRC / "sched").glob("*.cc"))
    r = subprocess.run([CXX, "-std=c++17", "-O1", "-g", *flags, "-I", str(CSRC), str(DRIVER), *srcs, "-o", str(exe), "-lpthread"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-4000:]
    return exe


@pytest.mark.skipif(CXX is None, reason="no g++")
def test_schedule_compiler_under_asan_ubsan(tmp_path):
    exe = _build(tmp_path, "san_au", ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"])
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, (r.stdout[-2000:], r.stderr[-4000:])
    assert "0 failures" in r.stdout


@pytest.mark.skipif(CXX is None, reason="no g++")
def test_threaded_executor_under_tsan(tmp_path):
    exe = _build(tmp_path, "san_t", ["-fsanitize=thread"])
    r = subprocess.run([str(exe), "threads-only"], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, (r.stdout[-2000:], r.stderr[-4000:])
    assert "0 failures" in r.stdout and "ThreadSanitizer" not in r.stderr


@pytest.mark.skipif(CXX is None, reason="no g++")
def test_bootstrap_under_asan_ubsan(tmp_path):
    """The shared-memory rendezvous (forked ranks, barriers, blob exchange, a rank that never arrives) with
    AddressSanitizer + UndefinedBehaviorSanitizer in every process."""
    flags = ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"]
    probe = tmp_path / "probe.cc"
    probe.write_text("int main(){return 0;}\n")
    if subprocess.run([CXX, *flags, str(probe), "-o", str(tmp_path / "probe")], capture_output=True).returncode != 0:
        pytest.skip("sanitizers are not available with this compiler")
    obj = tmp_path / "bootstrap_test.o"
    r = subprocess.run([shutil.which("gcc") or "gcc", "-O1", "-g", *flags, "-I", str(CSRC / "boot"), "-c",
                        str(ROOT / "tests" / "native" / "bootstrap_test.c"), "-o", str(obj)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    exe = tmp_path / "bootstrap_san"
    r = subprocess.run([CXX, "-std=c++17", "-O1", "-g", *flags, "-I", str(CSRC), str(obj), str(CSRC / "boot" / "bootstrap.cc"), str(CSRC / "boot" / "fdpass.cc"),
                        "-o", str(exe), "-lpthread", "-lrt"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "BOOTSTRAP OK" in r.stdout, (r.stdout[-1000:], r.stderr[-3000:])
    assert "Sanitizer" not in r.stderr
