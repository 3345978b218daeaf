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


def candidates(coll: str, P: int, nbytes: int, comm) -> list[tuple]:
    """(algo, k, b, nctas) tuples worth timing for this cell."""
    out = []
    if nbytes <= comm.ll_max_bytes:
        out.append(("ll", 2, 1, 0))
    if coll == "allreduce" and P > 1 and 64 <= nbytes <= comm.ll2_max_bytes:
        out.append(("ll2", 2, 1, 0))
        if nbytes >= (1 << 20):
            out.append(("ll2", 2, 1, 64))
    divs = [b for b in (1, 2, 4, 8) if P % b == 0 and b <= P]
    for b in divs:
        ks = sorted({2, 4, max(2, b)}) if b > 2 else [2]
        for k in ks:
            if nbytes <= (256 << 10):
                out.append(("radix_batch", k, b, 1))
                out.append(("radix_batch", k, b, 4))
            elif nbytes <= (4 << 20):
                for n in (4, 16, 32):
                    out.append(("radix_batch", k, b, n))
            else:
                for n in (32, 64, 128):
                    out.append(("radix_batch", k, b, n))
    if comm.has_multicast and nbytes % 16 == 0 and nbytes >= 16 * P:
        for n in ((1, 4, 16) if nbytes <= (1 << 20) else (8, 16, 24, 32, 64)):
            out.append(("nvls", 2, 1, n))
            if coll == "allreduce" and nbytes <= (4 << 20):
                out.append(("nvls1", 2, 1, n))
    if coll == "allgather" and nbytes % 16 == 0 and nbytes >= (1 << 20):
        for n in (64, 128):
            out.append(("bulk", 2, 1, n))
    if coll == "allreduce" and nbytes <= (4 << 20):
        out += [("recursive_doubling", 2, 1, 1 if nbytes <= (1 << 20) else 16)]
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
    args = ap.parse_args(argv)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    lr = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(lr)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=torch.device("cuda", lr))
    sizes = [int(s) for s in args.sizes.split(",") if s]
    smax = max(sizes)
    comm = Communicator.from_process_group(scratch_bytes=smax + (32 << 20), user_bytes=2 * smax + (64 << 20))
    P = comm.P
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
                    factor = 2 * (P - 1) / P
                elif coll == "reduce_scatter":
                    xin, yout, payload = x[:n * P], y[:n], n * esz
                    call = lambda a, k, b, c: reduce_scatter(comm, xin, out=yout, algo=a, k=k, b=b, nctas=c)
                    ref = lambda: dist.reduce_scatter_tensor(yout, xin)
                    factor = (P - 1) / P
                else:
                    xin, yout, payload = x[:n], y[:n * P], n * esz
                    call = lambda a, k, b, c: all_gather(comm, xin, out=yout, algo=a, k=k, b=b, nctas=c)
                    ref = lambda: dist.all_gather_into_tensor(yout, xin)
                    factor = (P - 1) / P
                total = n * P * esz
                for _ in range(3):
                    ref()
                t_nccl = time_call(ref, args.iters, world)
                best = None
                for (a, k, b, c) in candidates(coll, P, payload, comm):
                    try:
                        for _ in range(2):
                            call(a, k, b, c)
                        t = time_call(lambda: call(a, k, b, c), args.iters, world)
                        comm.check()
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
        table = autotune.build_table(samples, gpu, P)
        if not args.no_save:
            autotune.save_table(table, args.out)
        print(json.dumps(table))
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1:])
