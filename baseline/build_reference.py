"""Build the reference's own allreduce / reduce-scatter / allgather sources,
unmodified, against the thread-per-rank MPI shim in ``baseline/shim``.

The reference is plain MPI C++ without a Python package, so the prescribed
``pip install --target baseline/_ref`` has nothing to install; this script is
the replacement: it copies the three source files into ``baseline/_ref/src``
(git-ignored) and links them with the shim into ``baseline/_ref/ref_driver``.
Run it once where the reference tree is mounted; the binary travels with the
snapshot.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
# reference tree: argv[1], $CHB_REFERENCE_DIR, or a "reference" directory next to this repository
REF = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(
    os.environ.get("CHB_REFERENCE_DIR", HERE.parent.parent / "reference"))
W = REF / "testing" / "custom_implementations" / "work_dir"
SOURCES = [W / "all_gather" / "all_gather_radix_batch_1_0.cpp",
           W / "reduce_scatter" / "reduce_scatter_radix_batch.cpp",
           W / "all_reduce" / "all_reduce_radix_batch.cpp",
           W / "all_reduce" / "all_reduce_semi_custom_0_1.cpp"]
CUSTOM = W / "all_reduce" / "all_reduce_custom_0_2.cpp"    # defines its own all_reduce_radix_batch: a binary of its own
# the stand-alone phase functions live in files of their own; the allgather ones come with a test main and an
# older allgather_radix_batch, so they go into a second binary (renamed by -D, the sources stay untouched)
PHASE_SOURCES = [W / "reduce_scatter" / "intra_reduce_scatter_radix.cpp",
                 W / "reduce_scatter" / "inter_linear_reduce.cpp",
                 W / "reduce_scatter" / "intra_scatter_radix_batch.cpp"]
AG_BETA = W / "all_gather" / "outdated_versions" / "all_gather_0_3_beta.cpp"
M = REF / "testing" / "mpich_implementations"
# the MPICH-style baselines (the SMP allreduce fixes its node size at compile time: built with RANKS_PER_NODE=2)
MPICH_SOURCES = [M / "all_reduce" / f for f in (
    "allreduce_recursive_doubling.cpp", "allreduce_ring.cpp", "allreduce_reduce_scatter_allgather.cpp",
    "allreduce_recursive_multiplying.cpp", "allreduce_k_reduce_scatter_allgather.cpp", "allreduce_recexch.cpp",
    "allreduce_inter_reduce_exchange_bcast.cpp")] + [
    M / "reduce_scatter" / f for f in ("reduce_scatter_recursive_halving.cpp", "reduce_scatter_pairwise.cpp",
                                       "reduce_scatter_radix.cpp", "reduce_scatter_recursive_doubling.cpp")]
# earlier variants kept in the reference tree; three of them come with a test main, renamed by -D
EARLIER = {W / "reduce_scatter" / "tuna_based_outdated" / "reduce_scatter_radix_block_0_1.cpp": None,
           W / "reduce_scatter" / "tuna_based_outdated" / "reduce_scatter_k_nomial.cpp": "k_nomial_test_main",
           W / "reduce_scatter" / "debug" / "tuna.cpp": "tuna_test_main",
           W / "all_gather" / "outdated_versions" / "all_gather_0_1_alpha.cpp": "ag_alpha_test_main"}


def build() -> Path:
    out = HERE / "_ref"
    src = out / "src"
    src.mkdir(parents=True, exist_ok=True)
    copied = []
    for s in SOURCES:
        d = src / s.name
        shutil.copyfile(s, d)
        copied.append(str(d))
    exe = out / "ref_driver"
    cmd = ["g++", "-O3", "-std=c++17", "-w", "-pthread", "-I", str(HERE / "shim"),
           str(HERE / "shim" / "ref_driver.cpp"), str(HERE / "shim" / "shim.cpp"), *copied, "-o", str(exe)]
    subprocess.run(cmd, check=True)
    build_phases()
    build_mpich()
    build_custom()
    return exe


def build_custom() -> Path:
    out = HERE / "_ref"
    src = out / "src"
    d = src / CUSTOM.name
    shutil.copyfile(CUSTOM, d)
    exe = out / "ref_custom_driver"
    subprocess.run(["g++", "-O2", "-std=c++17", "-w", "-pthread", "-I", str(HERE / "shim"),
                    str(HERE / "shim" / "ref_custom_driver.cpp"), str(HERE / "shim" / "shim.cpp"), str(d), "-o", str(exe)],
                   check=True)
    return exe


def build_mpich() -> Path:
    out = HERE / "_ref"
    src = out / "src" / "mpich"
    src.mkdir(parents=True, exist_ok=True)
    for h in (M / "all_reduce" / "common.hpp", M / "reduce_scatter" / "reduce_scatter.hpp"):
        shutil.copyfile(h, src / h.name)
    objs = []
    for s, rename in [(m, None) for m in MPICH_SOURCES] + list(EARLIER.items()):
        d = src / s.name
        shutil.copyfile(s, d)
        o = d.with_suffix(".o")
        subprocess.run(["g++", "-O2", "-std=c++17", "-w", "-pthread", "-I", str(HERE / "shim"), "-I", str(src),
                        "-DRANKS_PER_NODE=2", *([f"-Dmain={rename}"] if rename else []), "-c", str(d), "-o", str(o)], check=True)
        objs.append(str(o))
    exe = out / "ref_mpich_driver"
    subprocess.run(["g++", "-O2", "-std=c++17", "-w", "-pthread", "-I", str(HERE / "shim"),
                    str(HERE / "shim" / "ref_mpich_driver.cpp"), str(HERE / "shim" / "shim.cpp"), *objs, "-o", str(exe)],
                   check=True)
    return exe


def build_phases() -> Path:
    out = HERE / "_ref"
    src = out / "src"
    src.mkdir(parents=True, exist_ok=True)
    objs = []
    for s in PHASE_SOURCES + [AG_BETA]:
        d = src / s.name
        shutil.copyfile(s, d)
        o = d.with_suffix(".o")
        extra = ["-Dmain=reference_test_main"] if s == AG_BETA else []
        subprocess.run(["g++", "-O2", "-std=c++17", "-w", "-pthread", "-I", str(HERE / "shim"), *extra, "-c", str(d),
                        "-o", str(o)], check=True)
        objs.append(str(o))
    exe = out / "ref_phase_driver"
    subprocess.run(["g++", "-O2", "-std=c++17", "-w", "-pthread", "-I", str(HERE / "shim"),
                    str(HERE / "shim" / "ref_phase_driver.cpp"), str(HERE / "shim" / "shim.cpp"), *objs, "-o", str(exe)],
                   check=True)
    return exe


if __name__ == "__main__":
    print(build())
