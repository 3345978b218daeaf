"""In-tree build of the native library (``libchb.so``).

Host sources (``csrc/**/*.cc``) are compiled with g++, device sources
(``csrc/**/*.cu``) with nvcc for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a -lineinfo``); everything is linked
into one shared object next to this file, so a snapshot of the source tree
carries the built library with it.  Objects are rebuilt when their source or
any header under ``csrc/`` is newer.

Run ``python -m configurable_hierarchical_allreduce_algorithms_b200._build`` to
build by hand; ``build(verbose=True)`` prints the ptxas resource usage.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "build" / "obj"
LIB = HERE / "libchb.so"
TOOLS = CSRC / "tools"              # stand-alone programs linked against the library
BIN = HERE / "bin"

NVCC = os.environ.get("CHB_NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
CXX = os.environ.get("CXX") or shutil.which("g++") or "g++"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]
if os.environ.get("CHB_CHECK_BOUNDS") == "1":   # checked build: in-kernel range test of every step
    NVCC_FLAGS.append("-DCHB_CHECK_BOUNDS")
CXX_FLAGS = ["-O2", "-fPIC", "-std=c++17", "-Wall", "-Wno-sign-compare"]


def _sources():
    cc = sorted(p for p in CSRC.rglob("*.cc") if TOOLS not in p.parents)
    cu = sorted(p for p in CSRC.rglob("*.cu") if TOOLS not in p.parents)
    return cc, cu


def _newest_header() -> float:
    t = 0.0
    for pat in ("*.h", "*.cuh", "*.hpp"):
        for h in CSRC.rglob(pat):
            t = max(t, h.stat().st_mtime)
    return t


def _obj_for(src: Path) -> Path:
    rel = src.relative_to(CSRC)
    return OBJ / ("__".join(rel.parts) + ".o")


def _compile(src: Path, obj: Path, verbose: bool) -> str:
    if src.suffix == ".cu":
        cmd = [NVCC, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    else:
        cuda_inc = str(Path(NVCC).resolve().parent.parent / "include")
        cmd = [CXX, *CXX_FLAGS, "-I", str(CSRC), "-I", cuda_inc, "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    return r.stderr if verbose else ""


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile what is out of date and link ``libchb.so``; returns its path."""
    cc, cu = _sources()
    OBJ.mkdir(parents=True, exist_ok=True)
    hdr_t = _newest_header()
    todo, objs = [], []
    for src in cc + cu:
        obj = _obj_for(src)
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_t):
            todo.append((src, obj))
    logs = []
    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            futs = {ex.submit(_compile, s, o, verbose): s for s, o in todo}
            for f in cf.as_completed(futs):
                out = f.result()
                if out:
                    logs.append(f"== {futs[f].name}\n{out}")
    need_link = bool(todo) or not LIB.exists() or any(o.stat().st_mtime > LIB.stat().st_mtime for o in objs)
    if need_link:
        # linked next to its final place and renamed into it: a process that loads the library (or a copy of the
        # tree taken) while a build is running sees the old file or the new one, never a half-written one
        tmp = LIB.with_name(LIB.name + ".tmp")
        if cu:
            cmd = [NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(tmp),
                   *map(str, objs), "-lpthread"]
        else:
            cmd = [CXX, "-shared", "-o", str(tmp), *map(str, objs), "-lpthread"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, LIB)
    if cu:
        _build_tools(hdr_t, force)
    if verbose and logs:
        print("\n".join(logs))
    return LIB


def _build_tools(hdr_t: float, force: bool) -> None:
    """``bin/<name>`` from every ``csrc/tools/<name>.cu`` (run-path relative, so the tree can be moved)."""
    BIN.mkdir(exist_ok=True)
    for src in sorted(TOOLS.glob("*.cu")):
        exe = BIN / src.stem
        if not force and exe.exists() and exe.stat().st_mtime >= max(src.stat().st_mtime, hdr_t, LIB.stat().st_mtime):
            continue
        tmp = exe.with_name(exe.name + ".tmp")
        cmd = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-I", str(CSRC),
               str(src), "-o", str(tmp), "-L", str(HERE), "-lchb", "-ldl", "-Xlinker", "-rpath=$ORIGIN/.."]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"tool build failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, exe)


if __name__ == "__main__":
    p = build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print(p)
