"""Per-message-size choice of (algorithm, k, b, CTAs).

The reference tunes offline: its drivers sweep ``k`` (and ``b`` across job
scripts) and its plotters pick the median winner per ``(nprocs, send_count)``
cell (testing/plots/all_reduce/median_best_plotter.py:29-56).  Here the same
"median winner per cell" rule is applied to measured device times and the
result is kept in a JSON table keyed by ``(gpu, P, collective, dtype)`` that
:func:`choose` consults at call time; without a table a size heuristic is used.

Table format::

    {"NVIDIA B200|8|allreduce|fp32": [[max_bytes, algo, k, b, nctas], ...]}   # ascending max_bytes
"""
from __future__ import annotations

import json
import os
import statistics
from dataclasses import dataclass
from pathlib import Path

import torch

DEFAULT_TABLE = Path(__file__).resolve().parent / "tuned_b200.json"
_tables: dict | None = None


@dataclass(frozen=True)
class Choice:
    algo: str
    k: int = 2
    b: int = 1
    nctas: int = 0


def _load() -> dict:
    global _tables
    if _tables is None:
        path = Path(os.environ.get("CHB_TUNE_TABLE", DEFAULT_TABLE))
        try:
            _tables = json.loads(path.read_text())
        except (OSError, ValueError):
            _tables = {}
    return _tables


def reload(path: str | None = None) -> None:
    global _tables
    _tables = None
    if path:
        os.environ["CHB_TUNE_TABLE"] = path


def _key(comm, coll: str, dtype) -> str:
    name = torch.cuda.get_device_name(comm.device) if torch.cuda.is_available() else "cpu"
    short = {"torch.float32": "fp32", "torch.bfloat16": "bf16", "torch.float16": "fp16"}
    return f"{name}|{comm.P}|{coll}|{short.get(str(dtype), str(dtype).replace('torch.', ''))}"


def heuristic(comm, coll: str, payload_bytes: int, symmetric: bool) -> Choice:
    """Fallback rule: one-shot flagged lines while latency-bound, then the
    flat two-phase schedule (b = 1), NVLS when a multicast alias exists."""
    forced = os.environ.get("CHB_ALGO")
    if forced:
        return Choice(forced, int(os.environ.get("CHB_K", 2)), int(os.environ.get("CHB_B", 1)), 0)
    ll_cut = min(comm.ll_max_bytes, 64 << 10 if coll == "allreduce" else 128 << 10)
    if comm.P > 1 and payload_bytes <= ll_cut:
        return Choice("ll")
    if comm.P > 2 and coll == "allreduce" and payload_bytes <= min(comm.ll2_max_bytes, 2 << 20):
        return Choice("ll2")
    if comm.has_multicast and symmetric and comm.nlocal == 1 and coll in ("allreduce", "reduce_scatter", "allgather"):
        return Choice("nvls")
    return Choice("radix_batch", 2, 1, 0)


def choose(comm, coll: str, payload_bytes: int, dtype, symmetric: bool) -> Choice:
    rows = _load().get(_key(comm, coll, dtype))
    if rows and not os.environ.get("CHB_ALGO"):
        for max_bytes, algo, k, b, nctas in rows:
            if payload_bytes <= max_bytes:
                if algo == "nvls" and not (comm.has_multicast and symmetric):
                    break
                return Choice(algo, int(k), int(b), int(nctas))
    return heuristic(comm, coll, payload_bytes, symmetric)


def winners(samples: list[dict]) -> dict:
    """Median winner per (collective, dtype, bytes) cell.

    ``samples``: dicts with keys coll, dtype, bytes, algo, k, b, nctas, time_s, is_correct.
    Rows with ``is_correct != 1`` poison their cell exactly as the reference's
    plotters refuse incorrect data (median_best_plotter.py:15-20): they raise.
    """
    bad = [s for s in samples if int(s.get("is_correct", 1)) != 1]
    if bad:
        raise ValueError(f"{len(bad)} incorrect samples, refusing to tune from them (first: {bad[0]})")
    cells: dict = {}
    for s in samples:
        cells.setdefault((s["coll"], s["dtype"], int(s["bytes"])), {}).setdefault(
            (s["algo"], int(s["k"]), int(s["b"]), int(s.get("nctas", 0))), []).append(float(s["time_s"]))
    out = {}
    for cell, cands in cells.items():
        med = {c: statistics.median(v) for c, v in cands.items()}
        best = min(med, key=med.get)
        out[cell] = (best, med[best], med)
    return out


def build_table(samples: list[dict], gpu: str, P: int) -> dict:
    """Collapse per-cell winners into ascending ``max_bytes`` rows per (collective, dtype)."""
    table: dict = {}
    w = winners(samples)
    for (coll, dtype, nbytes) in sorted(w, key=lambda c: (c[0], c[1], c[2])):
        (algo, k, b, nctas), _, _ = w[(coll, dtype, nbytes)]
        rows = table.setdefault(f"{gpu}|{P}|{coll}|{dtype}", [])
        if rows and rows[-1][1:] == [algo, k, b, nctas]:
            rows[-1][0] = nbytes
        else:
            rows.append([nbytes, algo, k, b, nctas])
    for rows in table.values():
        rows[-1][0] = 1 << 62
    return table


def save_table(table: dict, path: str | os.PathLike = DEFAULT_TABLE, merge: bool = True) -> None:
    path = Path(path)
    cur = {}
    if merge and path.exists():
        try:
            cur = json.loads(path.read_text())
        except ValueError:
            cur = {}
    cur.update(table)
    path.write_text(json.dumps(cur, indent=1, sort_keys=True))
    reload()
