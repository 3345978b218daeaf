#!/usr/bin/env python
"""Headline benchmark: allreduce (sum, fp32) bandwidth and latency on N B200s.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N ...            # the reference's own CPU code

One "step" is one allreduce of ``--bytes`` per GPU (default 1 GiB, larger than
the 126 MB L2, so no flush is needed between steps).  The headline ``value`` is
the whole-job algorithm bandwidth N * bytes / time in GB/s (weak scaling: the
per-GPU vector is fixed as N grows); the bus bandwidth (x 2(N-1)/N), the p50
latency / bus bandwidth per message size for allreduce, reduce-scatter and
allgather, and NCCL's numbers for the same sizes measured in the same process
are reported next to it.  Times are CUDA-event times on the launching stream,
max over ranks.  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.idx = device_index
        self.rows = []
        self._stop = threading.Event()
        self._t = None

    def _loop(self):
        # NVML (read-only queries) samples every 2 ms, so that a timed region of a few ms still holds samples;
        # nvidia-smi is the fallback
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = None
            try:
                import torch
                uuid = str(torch.cuda.get_device_properties(self.idx).uuid)
            except Exception:  # noqa: BLE001
                pass
            h = None
            if uuid:
                try:
                    h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
                except Exception:  # noqa: BLE001
                    h = None
            if h is None:
                h = pynvml.nvmlDeviceGetHandleByIndex(self.idx)
            mx = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            bits = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}
            while not self._stop.is_set():
                sm = pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
                try:
                    rs = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
                except Exception:  # noqa: BLE001
                    rs = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                row = [str(self.idx), str(sm), str(mx), "", "", time.perf_counter()]
                ts = row.pop()
                row += ["Active" if rs & bits[n] else "Not Active"
                        for n in ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")]
                self.rows.append(row + [ts])
                self._stop.wait(0.002)
            return
        except Exception:  # noqa: BLE001
            pass
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                      "-i", str(self.idx)], capture_output=True, text=True, timeout=5).stdout
                for line in out.strip().splitlines():
                    self.rows.append([c.strip() for c in line.split(",")][:9] + [time.perf_counter()])
            except Exception:  # noqa: BLE001
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._t = threading.Thread(target=self._loop, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def mark(self, t0: float, t1: float):
        """Timed region [t0, t1] (perf_counter): summary() prefers the samples inside it."""
        self.window = (t0, t1)

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = self.rows
        w = getattr(self, "window", None)
        where = "timed region"
        if w:
            inside = [r for r in rows if w[0] <= r[-1] <= w[1]]
            if inside:
                rows = inside
            else:   # region shorter than the sampling period: the samples taken under the preceding warm-up load
                rows = [r for r in rows if r[-1] <= w[1]][-20:] or rows
                where = "warm-up immediately before the timed region (region shorter than one sampling period)"
        for r in rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[5:9]):
                if str(v).lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "sampled_during": where}


# ----------------------------------------------------------------------------- helpers
def device_time_ms(fn, steps, stream_sync, barrier):
    """Time `steps` back-to-back calls of fn with CUDA events; returns total ms on this rank."""
    import torch

    barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    barrier()
    return e0.elapsed_time(e1)


def per_call_ms(fn, iters, flush, barrier):
    """Individually timed calls with an L2 flush (untimed) before each; returns list of ms."""
    import torch

    out = []
    for _ in range(iters):
        barrier()
        torch.cuda.synchronize()
        # the flush runs on the stream while the host enqueues the collective behind
        # it, so the interval between the two events is device time, not launch latency
        flush()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1))
    return out


METRIC = "allreduce_sum_fp32_aggregate_algbw_GBps"


def headline_config(N: int, S: int) -> dict:
    """What is measured, identical for both arms (what differs between them goes under "arm")."""
    return {"model": "allreduce sum fp32 (config 2 of the sweep: 8 B - 1 GiB)", "bytes_per_gpu": S,
            "global_batch": None, "seq_len": None, "parallelism": f"{N} ranks",
            "l2": "inputs larger than L2 for the headline; explicit 256 MiB L2 flush before every timed call in the sweep"}


def emulated_rows(W: int, K: int) -> list:
    """Allreduce of eight emulated ranks on the current GPU: every rank's kernel runs in one cooperative launch.
    Per row: the schedule, the bytes per rank, microseconds per call (CUDA events, L2 flushed before every timed
    call) and the comparison with an fp64 sum of the inputs."""
    import torch

    import configurable_hierarchical_allreduce_algorithms_b200 as chb
    from configurable_hierarchical_allreduce_algorithms_b200.parallel.comm import Communicator

    P = 8
    comm = Communicator.emulated(P, ll_bytes=1 << 20, scratch_bytes=72 << 20, user_bytes=1 << 20)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    rows = []
    try:
        for nbytes in (32 << 10, 1 << 20, 16 << 20):
            n = nbytes // 4
            g = torch.Generator(device="cuda").manual_seed(77)
            ins = [torch.rand(n, generator=g, device="cuda") * 2 - 1 for _ in range(P)]
            exp = torch.stack([t.double() for t in ins]).sum(0)
            cands = [("radix_batch:pull", 2, 1), ("radix_batch:pull", 4, 2), ("radix_batch:pull", 8, 8)]
            if nbytes <= (1 << 20):
                cands += [("radix_batch:ll", 2, 1), ("radix_batch:ll", 8, 8), ("ll" if nbytes <= (64 << 10) else "ll2", 2, 1)]
            for algo, k, b in cands:
                row = {"algo": algo, "k": k, "b": b, "bytes_per_rank": nbytes, "dtype": "fp32"}
                rows.append(row)
                try:
                    outs = chb.all_reduce(comm, ins, algo=algo, k=k, b=b)
                    torch.cuda.synchronize()
                    comm.check()
                except Exception as e:  # noqa: BLE001 - e.g. messages larger than the inbox: say so and go on
                    row["skipped"] = repr(e)[:120]
                    comm.clear_error()
                    continue
                err = max(float((o.double() - exp).abs().max()) for o in outs)
                for _ in range(W):
                    chb.all_reduce(comm, ins, algo=algo, k=k, b=b)
                ts = []
                for _ in range(K):
                    flush.fill_(1)
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    chb.all_reduce(comm, ins, algo=algo, k=k, b=b)
                    e1.record()
                    torch.cuda.synchronize()
                    ts.append(e0.elapsed_time(e1) * 1e3)
                comm.check()
                row.update({"us_p50": statistics.median(ts), "is_correct": err <= 1e-4 * P, "max_abs_err": err})
    finally:
        comm.close()
    return rows


def reference_arm(args):
    from baseline import reference_bench

    N = max(1, int(os.environ.get("WORLD_SIZE", args.gpus)))
    out = reference_bench.run(args, headline_config(N, int(args.bytes)), METRIC)
    if out is not None:
        print(json.dumps(out), flush=True)


def roofline(N: int, S: int, kernel: str, ms_per_step: float, peaks: dict) -> dict:
    """Bytes one GPU must put on NVLink for an allreduce of S bytes, over the link rate.
    Pull / push two-shot: 2 (N-1)/N S per direction.  In-switch (multimem) two-shot: the switch reads every
    GPU's copy of a slice and writes the result to every GPU, S (1 + 1/N) per direction per GPU.
    N = 1: a local copy, 2 S at the measured HBM copy bandwidth."""
    if N == 1:
        bw = peaks.get("hbm_gbs", 6650.0) * 1e9
        ideal = 2 * S / bw * 1e3
        return {"model": "local copy, 2 S bytes at the measured HBM copy bandwidth", "ideal_ms": ideal,
                "frac_of_measured": ideal / ms_per_step}
    if kernel.startswith("nvls"):
        nbytes, model = S * (1 + 1 / N), "in-switch two-shot: S (1 + 1/N) bytes per direction per GPU"
    else:
        nbytes, model = 2 * (N - 1) / N * S, "peer two-shot: 2 (N-1)/N S bytes per direction per GPU"
    i900, i770 = nbytes / 900e9 * 1e3, nbytes / 770e9 * 1e3
    return {"model": model, "bytes_per_direction": nbytes, "ideal_ms_at_900_nominal": i900, "frac_of_900_nominal": i900 / ms_per_step,
            "ideal_ms_at_770_measured": i770, "frac_of_770_measured": i770 / ms_per_step}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-emulated", action="store_true", help="skip the emulated 8-rank table of the 1-GPU run")
    ap.add_argument("--bytes", type=int, default=1 << 30, help="allreduce vector bytes per GPU (headline)")
    ap.add_argument("--sweep", default=",".join(str(8 * 4 ** i) for i in range(14)) + ",1073741824",
                    help="comma separated message sizes in bytes for the latency / bandwidth table ('' = none); "
                         "default 8 B ... 512 MiB in powers of 4, and 1 GiB")
    ap.add_argument("--sweep-iters", type=int, default=7)
    ap.add_argument("--grid", default="32768,1048576,16777216,1073741824",
                    help="sizes of the (k, b) grid / NCCL ring, tree / reference-algorithm table ('' = none)")
    ap.add_argument("--rows-out", default="", help="also write sweep and grid rows to this JSON file")
    ap.add_argument("--no-nccl", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    # cores and memory node nearest this rank's GPU, before any pinned buffer is allocated
    from configurable_hierarchical_allreduce_algorithms_b200.utils import affinity, autotune
    host_binding = affinity.bind_to_gpu(local_rank)

    import configurable_hierarchical_allreduce_algorithms_b200 as chb
    from configurable_hierarchical_allreduce_algorithms_b200.parallel.comm import CollectiveError, Communicator

    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    N = world
    W = max(args.warmup, 3)
    K = args.steps
    S = args.bytes
    nelem = S // 4

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def all_ranks_ok(ok: bool) -> bool:
        if world == 1:
            return bool(ok)
        t = torch.tensor([1 if ok else 0], device="cuda", dtype=torch.int32)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item())

    heap_user = 2 * S + (64 << 20) + (0 if args.no_e2e else (8 * (32 << 20) + (1 << 20)))   # + the host pipeline's chunks
    if world > 1:
        # scratch: the hierarchical shapes (b > 1) and the full-vector baselines keep up to two vectors of temporaries
        comm = Communicator.from_process_group(scratch_bytes=2 * S + (32 << 20), user_bytes=heap_user)
    else:
        comm = Communicator.emulated(1, scratch_bytes=1 << 20, user_bytes=heap_user)

    def unl(x):  # emulated single-rank world hands out lists
        return x[0] if isinstance(x, list) else x

    x = unl(comm.empty(nelem, torch.float32))
    y = unl(comm.empty(nelem, torch.float32))
    g = torch.Generator(device="cuda").manual_seed(1234 + rank)
    x.copy_(torch.rand(nelem, generator=g, device="cuda") * 2 - 1)

    def step():
        chb.all_reduce(comm, x, out=y)

    # ---- correctness of the timed call (against NCCL when there are peers, else identity)
    step()
    torch.cuda.synchronize()
    comm.check()
    ref = x.clone()
    if world > 1:
        dist.all_reduce(ref)
    err = float((y - ref).abs().max())
    tol = 1e-4 * N if world > 1 else 0.0
    correct = all_ranks_ok(err <= tol)
    headline_kernel = autotune.choose(comm, "allreduce", S, torch.float32, True)

    with ClockSampler(local_rank) as cs:
        for _ in range(W):
            step()
        torch.cuda.synchronize()
        t_end = time.perf_counter() + 2.0
        while not cs.rows and time.perf_counter() < t_end:     # sampler start-up (no collectives here:
            time.sleep(0.01)                                   # every rank must issue the same number of calls)
        for _ in range(max(W, 50)):                            # load right before the timed region
            step()
        l0 = comm.launches
        tw0 = time.perf_counter()
        ms = device_time_ms(step, K, None, barrier)
        cs.mark(tw0, time.perf_counter())
    launches = comm.launches - l0
    ms = max_over_ranks(ms)
    comm.check()
    ms_per_step = ms / K
    algbw = S / (ms_per_step * 1e-3) / 1e9
    value = algbw * N
    busbw = algbw * (2 * (N - 1) / N)
    clocks = cs.summary()

    # ---- NCCL on the same buffers: its default choice, and ring / tree pinned through NCCL_ALGO on groups of their own
    nccl = None
    nccl_groups = {}
    if world > 1 and not args.no_nccl:
        z = x.clone()
        for _ in range(W):
            dist.all_reduce(z)
        t = max_over_ranks(device_time_ms(lambda: dist.all_reduce(z), K, None, barrier)) / K
        nccl = {"ms_per_step": t, "algbw_GBps": S / (t * 1e-3) / 1e9, "busbw_GBps": S / (t * 1e-3) / 1e9 * 2 * (N - 1) / N}
        del z
        for name in ("Ring", "Tree"):
            try:
                os.environ["NCCL_ALGO"] = name          # read when the group's communicator is set up
                grp = dist.new_group(ranks=list(range(world)), backend="nccl")
                w1 = torch.ones(8, device="cuda")
                dist.all_reduce(w1, group=grp)           # the communicator exists before the variable goes away
                torch.cuda.synchronize()
                nccl_groups[name.lower()] = grp
            except Exception as e:  # noqa: BLE001 - an optional comparison row
                nccl_groups[name.lower()] = None
                if rank == 0:
                    print(f"# NCCL_ALGO={name}: {e!r}"[:200], file=sys.stderr)
            finally:
                os.environ.pop("NCCL_ALGO", None)

    # ---- end to end through the public API: pinned host -> device, allreduce, device -> host
    e2e = None
    if not args.no_e2e:
        hx = torch.empty(nelem, dtype=torch.float32).pin_memory()
        hx.copy_(x.cpu())
        hy = torch.empty(nelem, dtype=torch.float32).pin_memory()

        from configurable_hierarchical_allreduce_algorithms_b200.ops.host import HostAllReduce

        # the public host-buffer call: chunks flow pinned host -> device -> allreduce -> pinned host on three
        # streams, so upload and download (different copy engines, full-duplex PCIe) overlap
        pipe = HostAllReduce(comm, torch.float32, chunk_elems=8 << 20, depth=4)

        def e2e_step():
            pipe(hx, hy)
            torch.cuda.current_stream().synchronize()

        def timed(fn, reps):
            barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            barrier()
            return max_over_ranks(e0.elapsed_time(e1)) / reps, (time.perf_counter() - t0) * 1e3 / reps

        ke = max(3, min(K, 10))
        for _ in range(3):
            e2e_step()
        tms, wall = timed(e2e_step, ke)
        e2e_ok = all_ranks_ok(bool(torch.equal(hy, y.cpu())))       # the whole vector against the device result
        # what the host side of this box allows with every rank copying at once: upload alone, download alone, both
        # together (no collective), and the chunked collective alone; the pipeline cannot beat the slowest of them
        s_up, s_dn = torch.cuda.Stream(), torch.cuda.Stream()
        ch = 8 << 20

        def copies(up: bool, down: bool):
            cur = torch.cuda.current_stream()
            s_up.wait_stream(cur)
            s_dn.wait_stream(cur)
            for a in range(0, nelem, ch):
                e = min(nelem, a + ch)
                if up:
                    with torch.cuda.stream(s_up):
                        x[a:e].copy_(hx[a:e], non_blocking=True)
                if down:
                    with torch.cuda.stream(s_dn):
                        hy[a:e].copy_(y[a:e], non_blocking=True)
            cur.wait_stream(s_up)
            cur.wait_stream(s_dn)
            cur.synchronize()

        def coll_only():
            for a in range(0, nelem, ch):
                e = min(nelem, a + ch)
                chb.all_reduce(comm, x[a:e], out=y[a:e])
            torch.cuda.current_stream().synchronize()

        x_keep = x.clone()
        stages = {}
        for name, fn in (("upload_only", lambda: copies(True, False)), ("download_only", lambda: copies(False, True)),
                         ("upload_and_download", lambda: copies(True, True)), ("collective_only", coll_only)):
            fn()
            stages[name + "_ms"] = timed(fn, 3)[0]
        x.copy_(x_keep)
        step()                                                   # y holds the reduced vector again
        torch.cuda.synchronize()
        del x_keep
        floor_ms = max(stages["upload_and_download_ms"], stages["collective_only_ms"])
        e2e = {"value": N * S / (tms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": tms, "steps": ke,
               "h2d_bytes_per_step": S, "d2h_bytes_per_step": S, "wall_ms_per_step": wall, "is_correct": e2e_ok,
               "checked": "whole output vector against the device-side result, all ranks",
               "api": "HostAllReduce: 32 MiB chunks, upload / allreduce / download pipelined on three streams",
               "stages": stages, "host_binding": host_binding,
               "host_ceiling_GBps": N * S / (floor_ms * 1e-3) / 1e9,
               "frac_of_host_ceiling": floor_ms / tms,
               "ceiling_note": "ceiling = N * bytes / max(all ranks uploading and downloading at once, chunked collective alone)"}
        del hx, hy

    # ---- latency / bandwidth table: algo="auto" against NCCL's default, three collectives, fp32 and bf16
    sweep = []
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    flush = lambda: flush_buf.fill_(1)

    def close_enough(a, b, dtype):
        tol_ = (1e-5 if dtype == torch.float32 else 2e-2) * max(N, 1)
        return bool(torch.allclose(a.float(), b.float(), rtol=tol_, atol=tol_))

    scratch_ref = torch.empty(min(nelem, 1 << 26), dtype=torch.float32, device="cuda") if args.sweep else None   # NCCL's output for the checks

    def run_sweep(dtype, dname):
        for sz in [int(s) for s in args.sweep.split(",") if s]:
            if sz > S:
                continue
            esz = 4 if dtype == torch.float32 else 2
            ne = max(1, sz // esz)
            ne_rs = max(1, ne // max(N, 1))
            xf, yf = x.view(dtype), y.view(dtype)     # slices below may be longer than ne for tiny sizes
            xv, yv = xf[:ne], yf[:ne]
            row = {"bytes": ne * esz, "dtype": dname}
            rf = scratch_ref.view(dtype)
            cases = {
                "allreduce": (lambda: chb.all_reduce(comm, xv, out=yv),
                              (lambda: dist.all_reduce(yv)) if world > 1 else None, 2 * (N - 1) / N, ne * esz,
                              (lambda: (rf[:ne].copy_(xv), dist.all_reduce(rf[:ne]) if world > 1 else None, (yv, rf[:ne]))[-1])),
                "reduce_scatter": (lambda: chb.reduce_scatter(comm, xf[:ne_rs * N], out=yf[:ne_rs]),
                                   (lambda: dist.reduce_scatter_tensor(yf[:ne_rs], xf[:ne_rs * N])) if world > 1 else None,
                                   (N - 1) / N, ne_rs * N * esz,
                                   (lambda: (dist.reduce_scatter_tensor(rf[:ne_rs], xf[:ne_rs * N]) if world > 1
                                             else rf[:ne_rs].copy_(xf[:ne_rs]), (yf[:ne_rs], rf[:ne_rs]))[-1])),
                "allgather": (lambda: chb.all_gather(comm, xf[:ne_rs], out=yf[:ne_rs * N]),
                              (lambda: dist.all_gather_into_tensor(yf[:ne_rs * N], xf[:ne_rs])) if world > 1 else None,
                              (N - 1) / N, ne_rs * N * esz,
                              (lambda: (dist.all_gather_into_tensor(rf[:ne_rs * N], xf[:ne_rs]) if world > 1
                                        else rf[:ne_rs].copy_(xf[:ne_rs]), (yf[:ne_rs * N], rf[:ne_rs * N]))[-1])),
            }
            for name, (ours, theirs, factor, total_bytes, checker) in cases.items():
                # about 20 ms of back-to-back calls first (the same count on every rank): after the small
                # sizes of the sweep the links and clocks need more than three calls to be back at speed
                n_warm = min(100, max(3, int(20e-3 / (20e-6 + total_bytes / 2e11))))
                try:
                    ours()
                except CollectiveError as e:
                    # an argument the library refuses (the same answer on every rank, before anything is launched):
                    # the cell says so and the table goes on
                    row[name] = {"skipped": str(e)[:160]}
                    comm.clear_error()
                    continue
                for _ in range(n_warm):
                    ours()
                t = [max_over_ranks(v) for v in per_call_ms(ours, args.sweep_iters, flush, barrier)]
                p50 = statistics.median(t)
                row[name] = {"p50_us": p50 * 1e3, "busbw_GBps": total_bytes / (p50 * 1e-3) / 1e9 * factor}
                if total_bytes <= scratch_ref.numel() * 4:
                    ours()
                    got, want = checker()
                    torch.cuda.synchronize()
                    row[name]["is_correct"] = all_ranks_ok(close_enough(got, want, dtype))
                if theirs is not None and not args.no_nccl:
                    for _ in range(n_warm):
                        theirs()
                    t = [max_over_ranks(v) for v in per_call_ms(theirs, args.sweep_iters, flush, barrier)]
                    p50n = statistics.median(t)
                    row[name]["nccl_p50_us"] = p50n * 1e3
                    row[name]["nccl_busbw_GBps"] = total_bytes / (p50n * 1e-3) / 1e9 * factor
                    row[name]["vs_nccl"] = p50n / p50
            sweep.append(row)
        comm.check()

    if args.sweep:
        run_sweep(torch.float32, "fp32")

    # ---- the (k, b) grid of the hierarchical allreduce, the MPICH-style reference algorithms as programs on the
    # GPU, and NCCL pinned to ring / tree: fp32 sum allreduce, p50 of individually timed calls, checked against NCCL
    grid = []
    if args.grid and world > 1:
        refbuf = torch.empty(nelem, dtype=torch.float32, device="cuda")
        for sz in [int(s) for s in args.grid.split(",") if s]:
            if sz > S:
                continue
            ne = max(N, sz // 4 // N * N)
            xv, yv = x[:ne], y[:ne]
            refbuf[:ne].copy_(xv)
            dist.all_reduce(refbuf[:ne])
            iters = 5 if sz >= (256 << 20) else args.sweep_iters
            # the same amount of back-to-back warm-up calls as in the sweep: the first calls after an idle spell are slow
            n_warm = min(100, max(3, int(20e-3 / (20e-6 + ne * 4 / 2e11))))
            cands = [("radix_batch", k, b) for b in (1, 2, 4) if N % b == 0 and b <= N for k in (2, 4, 8)]
            cands += [("recursive_doubling", 2, 1), ("reduce_scatter_allgather", 2, 1), ("ring", 2, 1)]
            for algo, k, b in cands:
                rec = {"bytes": ne * 4, "algo": algo, "k": k, "b": b}
                try:
                    fn = lambda: chb.all_reduce(comm, xv, out=yv, algo=algo, k=k, b=b)
                    yv.zero_()
                    for _ in range(n_warm):
                        fn()
                    torch.cuda.synchronize()
                    comm.check()
                    rec["is_correct"] = all_ranks_ok(close_enough(yv, refbuf[:ne], torch.float32))
                    t = [max_over_ranks(v) for v in per_call_ms(fn, iters, flush, barrier)]
                    p50 = statistics.median(t)
                    rec.update(p50_us=p50 * 1e3, busbw_GBps=ne * 4 / (p50 * 1e-3) / 1e9 * 2 * (N - 1) / N)
                except CollectiveError as e:
                    rec["skipped"] = str(e)[:120]
                    comm.clear_error()
                grid.append(rec)
            if not args.no_nccl:
                for name, grp in [("nccl_default", None)] + [("nccl_" + n_, g_) for n_, g_ in nccl_groups.items()]:
                    if name != "nccl_default" and grp is None:
                        grid.append({"bytes": ne * 4, "algo": name, "skipped": "group could not be created"})
                        continue
                    fn = (lambda: dist.all_reduce(yv, group=grp)) if grp is not None else (lambda: dist.all_reduce(yv))
                    for _ in range(n_warm):
                        fn()
                    t = [max_over_ranks(v) for v in per_call_ms(fn, iters, flush, barrier)]
                    p50 = statistics.median(t)
                    grid.append({"bytes": ne * 4, "algo": name, "p50_us": p50 * 1e3,
                                 "busbw_GBps": ne * 4 / (p50 * 1e-3) / 1e9 * 2 * (N - 1) / N})
        del refbuf
        comm.check()

    # ---- launch-free latency: 20 back-to-back allreduces captured in one CUDA graph (small sizes only)
    graph_lat = []
    if args.sweep and not args.no_graph:
        try:
            for sz in (8, 1024, 32768):
                ne = max(1, sz // 4)
                xv, yv = x[:ne], y[:ne]
                row = {"bytes": ne * 4, "dtype": "fp32", "calls_per_graph": 20}
                for name, fn in (("ours", lambda: chb.all_reduce(comm, xv, out=yv, stream=gs)),
                                 ("nccl", (lambda: dist.all_reduce(yv)) if world > 1 and not args.no_nccl else None)):
                    if fn is None:
                        continue
                    gs = torch.cuda.Stream()
                    with torch.cuda.stream(gs):
                        for _ in range(3):
                            fn()
                    torch.cuda.synchronize()
                    barrier()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.stream(gs):
                        with torch.cuda.graph(g, stream=gs):
                            for _ in range(20):
                                fn()
                    ts = []
                    for _ in range(7):
                        barrier()
                        torch.cuda.synchronize()
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record()
                        g.replay()
                        e1.record()
                        torch.cuda.synchronize()
                        ts.append(max_over_ranks(e0.elapsed_time(e1)) / 20)
                    row[name + "_us_per_call"] = statistics.median(ts) * 1e3
                    del g
                graph_lat.append(row)
            comm.check()
        except Exception as e:  # noqa: BLE001 - an optional table must not cost the headline
            graph_lat = [{"error": repr(e)[:200]}]

    # ---- the same table on bf16 data: the input buffer is refilled with bf16 values first (an fp32 vector seen as
    # bf16 would be full of NaN and huge values), which is why this comes after everything that wants the fp32 input
    if args.sweep:
        g = torch.Generator(device="cuda").manual_seed(4321 + rank)
        xb = x.view(torch.bfloat16)
        half = xb.numel() // 2
        for lo in (0, half):                                   # in two pieces: no second full-size temporary
            xb[lo:lo + half].copy_((torch.rand(half, generator=g, device="cuda") * 2 - 1).to(torch.bfloat16))
        run_sweep(torch.bfloat16, "bf16")
        sweep.sort(key=lambda r: (r["bytes"], r["dtype"] != "fp32"))
    scratch_ref = None

    # ---- one GPU has no peers, so the headline above is a copy.  To show the collective kernels themselves on this
    # GPU too, eight ranks are emulated on it (one cooperative launch runs all ranks; "peer" reads and pushes go
    # through this GPU's memory instead of NVLink): the hierarchical program in both execution modes and the
    # flagged-line kernels, checked against an fp64 sum.  These rows say nothing about NVLink.
    emulated = []
    if world == 1 and args.sweep and not args.no_emulated:
        try:
            emulated = emulated_rows(max(3, W), max(5, min(K, 20)))
        except Exception as e:  # noqa: BLE001 - an optional table must not cost the headline
            emulated = [{"error": repr(e)[:200]}]

    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except (OSError, ValueError):
            pass
        rf = roofline(N, S, headline_kernel.algo, ms_per_step, peaks)
        if args.rows_out:
            try:
                with open(args.rows_out, "w") as f:
                    json.dump({"n_gpus": N, "sweep": sweep, "grid": grid, "graph_replay_latency": graph_lat}, f)
            except OSError:
                pass
        out = {
            "metric": METRIC,
            "value": value, "unit": "GB/s", "n_gpus": N, "steps": K, "warmup": W, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
            "impl": "ours",
            "busbw_GBps": busbw, "algbw_GBps": algbw,
            "config": headline_config(N, S),
            "arm": {"ranks": f"{N} ranks, one per GPU", "backend": comm.backend, "nvls": comm.has_multicast,
                    "headline_kernel": f"{headline_kernel.algo} k={headline_kernel.k} b={headline_kernel.b}"},
            "roofline": rf,
            "roofline_frac": rf.get("frac_of_770_measured", rf.get("frac_of_measured")),
            "is_correct": bool(correct), "max_abs_err": err,
            "clocks": clocks, "gpu_launches": launches, "e2e": e2e, "nccl": nccl,
            "grid": grid, "sweep": sweep, "graph_replay_latency": graph_lat,
        }
        if emulated:
            out["emulated_8_ranks_on_one_gpu"] = emulated
        print(json.dumps(out), flush=True)
    comm.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
