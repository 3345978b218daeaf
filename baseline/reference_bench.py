"""Reference arm of bench.py: the reference's own ``all_reduce_radix_batch``
(unmodified source, ``baseline/_ref/src``) on the host CPUs, N ranks as
threads over the MPI stand-in of ``baseline/shim`` (the image has no MPI).  Same
metric, configuration, step and warm-up counts as the main arm: sum allreduce
of ``--bytes`` fp32 per rank, ``k = 2, b = 1`` (the flat setting, the
reference's best large-message shape), value = N * bytes / time.

The reference's buffers are host arrays, so its timed call
(testing/custom_implementations/work_dir/all_reduce/main.cpp:55-66: Barrier; t0;
call; Barrier; t1) already is an end-to-end number: host buffer in, host buffer
out, no device on the path.  It is therefore reported both as ``value`` and as
``e2e`` (with zero bytes over PCIe).

Nothing of this repository's library is imported or loaded here: the process
runs ``baseline/_ref/ref_driver`` and parses its one line of output.
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


def run(args, config: dict, metric: str) -> dict | None:
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
    K, W = max(1, int(args.steps)), max(int(args.warmup), 3)      # the same counts as the main arm
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
    algbw = S / (ms * 1e-3) / 1e9
    return {
        "impl": "reference", "metric": metric, "value": algbw * N, "unit": "GB/s",
        "n_gpus": N, "steps": K, "warmup": W, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp32", "data": "synthetic", "is_correct": bool(d["is_correct"]),
        "algbw_GBps": algbw, "busbw_GBps": algbw * 2 * (N - 1) / N,
        "config": config,
        "arm": {"algorithm": "all_reduce_radix_batch k=2 b=1 (unmodified reference source)",
                "ranks": f"{N} CPU thread ranks",
                "transport": "thread-per-rank MPI stand-in on the host CPUs (no MPI installation on the image); "
                             "large messages are copied once, by the receiver",
                "timing": "host clock, Barrier; t0; call; Barrier; t1 as in the reference's drivers"},
        "gpu_launches": 0,
        "e2e": {"value": algbw * N, "unit": "GB/s", "ms_per_step": ms, "steps": K,
                "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "note": "the reference's buffers are host buffers: its timed call is host in, host out"},
    }
