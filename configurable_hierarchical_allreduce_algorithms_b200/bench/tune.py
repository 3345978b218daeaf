"""Measured autotuning: sweep (algorithm, k, b, CTAs) per collective and message
size, keep the median winner per cell, write the table ``utils/autotune.py``
consults at call time.

    torchrun --nproc-per-node N -m configurable_hierarchical_allreduce_algorithms_b200.bench.tune \
        [--sizes 8,1024,...] [--dtypes fp32,bf16] [--iters 20] [--out table.json] [--csv samples.csv]

The reference tunes the same way, offline: its drivers sweep ``k`` for a fixed
``b`` and its plotters pick the median winner per ``(nprocs, send_count)``
(testing/custom_implementations/work_dir/all_gather/main.cpp:186-190,
testing/plots/all_reduce/median_best_plotter.py:29-56).  NCCL is timed next to
every cell as the bar to beat.  Times are CUDA-event device times, max over ranks.
"""
from __future__ import annotations

import argparse
import csv
import json
import os
import statistics
import sys

import torch
import torch.distributed as dist

from .. import all_gather, all_reduce, reduce_scatter
from ..parallel.comm import CollectiveError, Communicator
from ..utils import autotune

DT = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


def canonical(k: int, b: int) -> tuple[int, int]:
    """(k, b) cells that compile to the same program share one measurement: without groups (b = 1) the radix
    plays no part, and a radix above the group size behaves like the group size (one phase either way)."""
    return (2, 1) if b <= 1 else (min(k, b), b)


def grid_cells(P: int) -> list[tuple[int, int]]:
    """The k in {2, 4, 8} x b in {1, 2, 4} grid (plus b = P), as distinct programs."""
    return sorted({canonical(k, b) for b in (1, 2, 4, P) if b <= P and P % b == 0 for k in (2, 4, 8)})


def candidates(coll: str, P: int, nbytes: int, comm, total: int | None = None) -> list[tuple]:
    """(algo, k, b, nctas) tuples worth timing for this cell.  ``nbytes``: payload per rank pair (the size
    the tuned table is keyed by); ``total``: bytes of the whole vector."""
    total = total if total is not None else nbytes
    out = []
    if nbytes <= comm.ll_max_bytes:
        out.append(("ll", 2, 1, 0))
    if coll == "allreduce" and P > 1 and 64 <= nbytes <= comm.ll2_max_bytes:
        out.append(("ll2", 2, 1, 0))
        if nbytes >= (1 << 20):
            out.append(("ll2", 2, 1, 64))
    for k, b in grid_cells(P):
        flat = b == 1
        if total <= (4 << 20):                       # owners push flagged lines: one traversal per round
            out.append(("radix_batch:ll", k, b, 0))
            if flat and total >= (1 << 20):          # the default stops at 64 CTAs
                out.append(("radix_batch:ll", k, b, 128))
        if total <= (64 << 10):                      # readers pull: the persistent interpreter
            out.append(("radix_batch:pull", k, b, 1))
        elif total <= (4 << 20):
            out += [("radix_batch:pull", k, b, n) for n in ((8, 32) if flat else (16,))]
        else:
            out += [("radix_batch:pull", k, b, n) for n in ((32, 64, 128) if flat else (64,))]
    if comm.has_multicast and nbytes % 16 == 0 and nbytes >= 16 * P:
        for n in ((1, 4, 16) if nbytes <= (1 << 20) else (8, 16, 32, 64)):
            out.append(("nvls", 2, 1, n))
            if coll == "allreduce" and nbytes <= (4 << 20):
                out.append(("nvls1", 2, 1, n))
    if coll == "allgather" and nbytes % 16 == 0 and nbytes >= (1 << 20):
        for n in (64, 128):
            out.append(("bulk", 2, 1, n))
    if coll == "allreduce":                          # the reference's MPICH-style baselines as programs on the GPU
        for a in ("recursive_doubling", "reduce_scatter_allgather"):
            if total <= (4 << 20):
                out.append((a + ":ll", 2, 1, 0))
            else:
                out.append((a + ":pull", 2, 1, 64))
    return out


def time_call(fn, iters: int, world: int) -> float:
    """Median device time (ms) of `iters` individually timed calls, max over ranks."""
    ts = []
    for _ in range(iters):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        torch.cuda._sleep(200_000)  # ~0.1 ms of device work: the call is enqueued behind it
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    t = torch.tensor(ts, device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return statistics.median(t.tolist())


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="8,256,4096,32768,262144,1048576,8388608,67108864,268435456")
    ap.add_argument("--dtypes", default="fp32,bf16")
    ap.add_argument("--colls", default="allreduce,reduce_scatter,allgather")
    ap.add_argument("--iters", type=int, default=15)
    ap.add_argument("--out", default=str(autotune.DEFAULT_TABLE))
    ap.add_argument("--csv", default="")
    ap.add_argument("--no-save", action="store_true")
    ap.add_argument("--no-nccl-algos", action="store_true", help="skip the NCCL ring / tree rows")
    ap.add_argument("--md", default="", help="write a markdown summary (winners, the (k, b) grid, NCCL) to this file")
    args = ap.parse_args(argv)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    lr = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(lr)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=torch.device("cuda", lr))
    sizes = [int(s) for s in args.sizes.split(",") if s]
    smax = max(sizes)
    comm = Communicator.from_process_group(scratch_bytes=2 * smax + (32 << 20), user_bytes=2 * smax + (64 << 20))
    P = comm.P
    nccl_groups = {}
    if world > 1 and not args.no_nccl_algos:
        for name in ("Ring", "Tree"):                  # NCCL pinned to one algorithm: read when a group's communicator is set up
            try:
                os.environ["NCCL_ALGO"] = name
                grp = dist.new_group(ranks=list(range(world)), backend="nccl")
                dist.all_reduce(torch.ones(8, device="cuda"), group=grp)
                torch.cuda.synchronize()
                nccl_groups[name.lower()] = grp
            except Exception as e:  # noqa: BLE001
                if rank == 0:
                    print(f"# NCCL_ALGO={name}: {e!r}"[:200], flush=True)
            finally:
                os.environ.pop("NCCL_ALGO", None)
    xb = comm.empty(smax, torch.uint8)
    yb = comm.empty(smax, torch.uint8)
    xb.copy_(torch.randint(0, 60, (smax,), device="cuda", dtype=torch.uint8))
    gpu = torch.cuda.get_device_name(lr)
    samples, rows = [], []
    for dname in args.dtypes.split(","):
        dtype = DT[dname]
        esz = torch.empty((), dtype=dtype).element_size()
        x, y = xb.view(dtype), yb.view(dtype)
        for coll in args.colls.split(","):
            for sz in sizes:
                # sz = total vector bytes (allreduce) or P * block bytes (reduce-scatter / allgather)
                n = max(1, sz // esz // P)
                if coll == "allreduce":
                    xin, yout, payload = x[:n * P], y[:n * P], n * P * esz
                    call = lambda a, k, b, c: all_reduce(comm, xin, out=yout, algo=a, k=k, b=b, nctas=c)
                    ref = lambda: dist.all_reduce(yout)
                    ref_g = lambda g_: dist.all_reduce(yout, group=g_)
                    factor = 2 * (P - 1) / P
                elif coll == "reduce_scatter":
                    xin, yout, payload = x[:n * P], y[:n], n * esz
                    call = lambda a, k, b, c: reduce_scatter(comm, xin, out=yout, algo=a, k=k, b=b, nctas=c)
                    ref = lambda: dist.reduce_scatter_tensor(yout, xin)
                    ref_g = lambda g_: dist.reduce_scatter_tensor(yout, xin, group=g_)
                    factor = (P - 1) / P
                else:
                    xin, yout, payload = x[:n], y[:n * P], n * esz
                    call = lambda a, k, b, c: all_gather(comm, xin, out=yout, algo=a, k=k, b=b, nctas=c)
                    ref = lambda: dist.all_gather_into_tensor(yout, xin)
                    ref_g = lambda g_: dist.all_gather_into_tensor(yout, xin, group=g_)
                    factor = (P - 1) / P
                total = n * P * esz
                expected = None
                if total <= (64 << 20):                    # NCCL's result for this cell, kept for the checks below
                    if coll == "allreduce":
                        expected = xin.clone()
                        dist.all_reduce(expected)
                    elif coll == "reduce_scatter":
                        expected = torch.empty_like(yout)
                        dist.reduce_scatter_tensor(expected, xin)
                    else:
                        expected = torch.empty_like(yout)
                        dist.all_gather_into_tensor(expected, xin)
                for _ in range(3):
                    ref()
                t_nccl = time_call(ref, args.iters, world)
                best = None
                for gname, grp in nccl_groups.items():
                    if gname == "tree" and coll != "allreduce":
                        continue                           # NCCL has no tree form of reduce-scatter / allgather
                    for _ in range(3):
                        ref_g(grp)
                    tg = time_call(lambda: ref_g(grp), args.iters, world)
                    rows.append([f"{coll}_nccl_{gname}", 0, 0, P, n, tg * 1e-3, 1, dname, "sum", total,
                                 total / (tg * 1e-3) / 1e9, total / (tg * 1e-3) / 1e9 * factor, tg * 1e3, P, 0])
                for (a, k, b, c) in candidates(coll, P, payload, comm, total):
                    try:
                        for _ in range(2):
                            call(a, k, b, c)
                        ok = 1
                        if expected is not None:           # the candidate's output against NCCL's, all ranks
                            tol = (1e-5 if dname == "fp32" else 2e-2) * P
                            flag = torch.tensor([1 if torch.allclose(yout.float(), expected.float(), rtol=tol, atol=1e-30) else 0], device="cuda")
                            if world > 1:
                                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                            ok = int(flag.item())
                        t = time_call(lambda: call(a, k, b, c), args.iters, world)
                        comm.check()
                        if not ok:
                            if rank == 0:
                                print(f"# WRONG RESULT {coll} {a} k={k} b={b} ctas={c} {dname} {total} B", flush=True)
                            rows.append([f"{coll}_{a}", k, b, P, n, t * 1e-3, 0, dname, "sum", total, 0, 0, t * 1e3, P, c])
                            continue
                    except CollectiveError as e:
                        if rank == 0:
                            print(f"# skip {coll} {a} k={k} b={b}: {e}", flush=True)
                        continue
                    samples.append({"coll": coll, "dtype": dname, "bytes": payload, "algo": a, "k": k, "b": b,
                                    "nctas": c, "time_s": t * 1e-3, "is_correct": 1})
                    rows.append([f"{coll}_{a}", k, b, P, n, t * 1e-3, 1, dname, "sum", total,
                                 total / (t * 1e-3) / 1e9, total / (t * 1e-3) / 1e9 * factor, t * 1e3, P, c])
                    if best is None or t < best[0]:
                        best = (t, a, k, b, c)
                if coll == "reduce_scatter" and n % 128 == 0 and dname in ("fp32", "bf16"):
                    # lossy wire format: reported next to the exact candidates, never chosen by the table
                    from ..ops import fused
                    try:
                        for _ in range(2):
                            fused.reduce_scatter_fp8(comm, xin, out=yout)
                        t8 = time_call(lambda: fused.reduce_scatter_fp8(comm, xin, out=yout), args.iters, world)
                        comm.check()
                        rows.append([f"{coll}_fp8wire", 0, 0, P, n, t8 * 1e-3, 1, dname, "sum", total,
                                     total / (t8 * 1e-3) / 1e9, total / (t8 * 1e-3) / 1e9 * factor, t8 * 1e3, P, 0])
                        if rank == 0:
                            print(f"{'  fp8 wire':14s} {dname} {total:>11d} B  {t8 * 1e3:9.1f} us", flush=True)
                    except CollectiveError as e:
                        if rank == 0:
                            print(f"# skip fp8 wire: {e}", flush=True)
                rows.append([f"{coll}_nccl", 0, 0, P, n, t_nccl * 1e-3, 1, dname, "sum", total,
                             total / (t_nccl * 1e-3) / 1e9, total / (t_nccl * 1e-3) / 1e9 * factor, t_nccl * 1e3, P, 0])
                if rank == 0 and best:
                    print(f"{coll:14s} {dname} {total:>11d} B  best {best[1]:>18s} k={best[2]} b={best[3]} ctas={best[4]:<3d}"
                          f" {best[0] * 1e3:9.1f} us  busbw {total / (best[0] * 1e-3) / 1e9 * factor:7.1f} GB/s |"
                          f" nccl {t_nccl * 1e3:9.1f} us  {total / (t_nccl * 1e-3) / 1e9 * factor:7.1f} GB/s"
                          f"  x{t_nccl / best[0]:.2f}", flush=True)
    if rank == 0:
        if args.csv:
            with open(args.csv, "w", newline="") as f:
                w = csv.writer(f)
                w.writerow(["algorithm_name", "k", "b", "nprocs", "send_count", "time", "is_correct", "dtype", "op",
                            "bytes", "algbw_GBs", "busbw_GBs", "p50_us", "ngpus", "nctas"])
                w.writerows(rows)
        if args.md:
            write_markdown(args.md, rows, P, gpu, " ".join(sys.argv if argv is None else ["tune"] + list(argv)))
        table = autotune.build_table(samples, gpu, P)
        if not args.no_save:
            autotune.save_table(table, args.out)
        print(json.dumps(table))
    comm.close()
    dist.destroy_process_group()


def write_markdown(path: str, rows: list, P: int, gpu: str, cmdline: str) -> None:
    """Winners per cell, the best time of every (k, b) shape of the hierarchical algorithm, and NCCL (its default
    and pinned to ring / tree), from the rows of one sweep."""
    import collections

    cells = collections.OrderedDict()
    for r in rows:
        name, k, b, _, _, t, ok, dname, _, total = r[:10]
        ctas = r[14] if len(r) > 14 else 0
        coll = next(c for c in ("allreduce", "reduce_scatter", "allgather") if name.startswith(c))
        cells.setdefault((coll, dname, int(total)), []).append((name[len(coll) + 1:], int(k), int(b), int(ctas), float(t) * 1e6, int(ok)))
    L = [f"# Sweep on {P} x {gpu}: median device time per call (us), max over ranks", "",
         "Made by (from the repository root, on the GPUs named above):", "", "```",
         f"python -m torch.distributed.run --nnodes=1 --nproc-per-node {P} --master-addr 127.0.0.1 -m "
         f"configurable_hierarchical_allreduce_algorithms_b200.bench.tune {cmdline.split('tune', 1)[-1].strip()}", "```", "",
         "Size = bytes of the whole vector (allreduce) or of all P blocks (reduce-scatter, allgather).  `rb` = the hierarchical",
         "radix-k / group-b program (`radix_batch`), `:ll` = owners push flagged lines, `:pull` = readers pull (persistent",
         "interpreter).  Cells of the k x b grid that compile to the same program are measured once: b = 1 ignores k, and a radix",
         "above the group size equals the group size.  A row with a wrong result is listed as WRONG and never wins.", ""]
    for coll in ("allreduce", "reduce_scatter", "allgather"):
        for dname in sorted({c[1] for c in cells}):
            sizes = sorted({c[2] for c in cells if c[0] == coll and c[1] == dname})
            if not sizes:
                continue
            shapes = sorted({(k, b) for (c, d, _), v in cells.items() if c == coll and d == dname for (a, k, b, _, _, _) in v if a.startswith("radix_batch")})
            L += [f"## {coll}, {dname}", "",
                  "| size | best of this library | us | best rb cell | us | NCCL | ring | tree | best / NCCL | best rb / NCCL |",
                  "|---|---|---|---|---|---|---|---|---|---|"]
            for sz in sizes:
                v = cells[(coll, dname, sz)]
                ours = [x for x in v if not x[0].startswith("nccl") and x[0] != "fp8wire" and x[5] == 1]
                rb = [x for x in ours if x[0].startswith("radix_batch")]
                nc = {x[0]: x[4] for x in v if x[0].startswith("nccl")}
                if not ours or "nccl" not in nc:
                    continue
                bo, br = min(ours, key=lambda x: x[4]), (min(rb, key=lambda x: x[4]) if rb else None)
                fmt = lambda x: f"{x[0]} k={x[1]} b={x[2]} ctas={x[3]}"
                L.append(f"| {sz} | {fmt(bo)} | {bo[4]:.1f} | {fmt(br) if br else '-'} | {br[4] if br else 0:.1f} | {nc['nccl']:.1f} | "
                         f"{nc.get('nccl_ring', 0):.1f} | {nc.get('nccl_tree', 0):.1f} | {nc['nccl'] / bo[4]:.2f}x | "
                         f"{(nc['nccl'] / br[4]) if br else 0:.2f}x |")
            L += ["", "Best time (us) of every (k, b) shape over its execution modes and CTA counts:", "",
                  "| size | " + " | ".join(f"k={k} b={b}" for k, b in shapes) + " | recursive doubling | Rabenseifner |",
                  "|---|" + "---|" * (len(shapes) + 2)]
            for sz in sizes:
                v = cells[(coll, dname, sz)]
                def best(pred):
                    xs = [x[4] for x in v if pred(x) and x[5] == 1]
                    bad = any(pred(x) and x[5] != 1 for x in v)
                    return (f"{min(xs):.1f}" if xs else "-") + (" (WRONG rows)" if bad else "")
                L.append(f"| {sz} | " + " | ".join(best(lambda x, k=k, b=b: x[0].startswith("radix_batch") and (x[1], x[2]) == (k, b)) for k, b in shapes)
                         + f" | {best(lambda x: x[0].startswith('recursive_doubling'))} | {best(lambda x: x[0].startswith('reduce_scatter_allgather'))} |")
            L.append("")
    with open(path, "w") as f:
        f.write("\n".join(L) + "\n")


if __name__ == "__main__":
    main(sys.argv[1:])
