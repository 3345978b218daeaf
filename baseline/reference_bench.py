"""Reference arm of bench.py: the reference's own ``all_reduce_radix_batch``
(unmodified source, ``baseline/_ref/src``) on the host CPUs, N ranks as
threads over the MPI shim in ``baseline/shim`` — the image has no MPI.  Same
metric and configuration as the main arm: sum allreduce of ``--bytes`` fp32
per rank, ``k = 2, b = 1`` (the flat setting, which is the reference's best
large-message shape), value = N * bytes / time.
"""
from __future__ import annotations

import json
import os
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
EXE = HERE / "_ref" / "ref_driver"


def _unavailable(why: str) -> dict:
    return {"impl": "reference", "unavailable": why}


def run(args) -> dict | None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None   # the N ranks are threads of rank 0's process
    N = max(1, int(os.environ.get("WORLD_SIZE", args.gpus)))
    if not EXE.exists():
        try:
            from . import build_reference
            build_reference.build()
        except Exception as e:  # noqa: BLE001
            return _unavailable(f"reference sources not built and not buildable here: {e!r}"[:200])
    S = int(args.bytes)
    try:
        import psutil
        need = 6 * S * N
        if psutil.virtual_memory().available < need:
            return _unavailable(f"host memory: {need >> 30} GiB needed for {N} thread ranks of {S >> 20} MiB")
    except ImportError:
        pass
    # the CPU code needs seconds per GiB-sized step: a handful of steps is enough for a stable mean
    K, W = max(1, min(int(args.steps), 5)), 1
    try:
        r = subprocess.run([str(EXE), "time", "ar", str(N), "2", "1", str(S), str(K), str(W)],
                           capture_output=True, text=True, timeout=3000)
    except subprocess.TimeoutExpired:
        return _unavailable("reference run exceeded 3000 s")
    line = [l for l in r.stdout.splitlines() if l.startswith("{")]
    if r.returncode != 0 or not line:
        return _unavailable(f"reference driver failed rc={r.returncode}: {r.stderr[-150:]}")
    d = json.loads(line[-1])
    ms = d["ms_per_step"]
    # the same collective with this library's schedule on host threads (one thread per rank, same machine):
    # a CPU-to-CPU comparison that does not involve the GPUs at all
    host_ms = None
    try:
        import numpy as np
        import sys
        sys.path.insert(0, str(HERE.parent))
        from configurable_hierarchical_allreduce_algorithms_b200.parallel.program import Program
        n = S // 4 // N * N
        prog = Program("allreduce", "radix_batch", N, n, 2, 1)
        ins = [np.full(n, float(r), np.float32) for r in range(N)]
        _, sec = prog.run_threads(ins, iters=2)
        host_ms = sec * 1e3
    except Exception:  # noqa: BLE001 - optional extra
        host_ms = None
    algbw = S / (ms * 1e-3) / 1e9
    return {
        "impl": "reference", "metric": "allreduce_sum_fp32_aggregate_algbw_GBps", "value": algbw * N, "unit": "GB/s",
        "n_gpus": N, "steps": K, "warmup": W, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp32", "data": "synthetic", "is_correct": bool(d["is_correct"]),
        "algbw_GBps": algbw, "busbw_GBps": algbw * 2 * (N - 1) / N,
        "config": {"model": "allreduce sum fp32", "bytes_per_gpu": S, "parallelism": f"{N} CPU thread ranks",
                   "algorithm": "all_reduce_radix_batch k=2 b=1",
                   "transport": "thread-per-rank MPI shim on the host CPUs (no MPI installation on the image)",
                   "timing": "host clock, Barrier; t0; call; Barrier; t1 as in the reference's drivers"},
        "gpu_launches": 0,
        "this_library_same_schedule_on_host_threads_ms": host_ms,
    }
