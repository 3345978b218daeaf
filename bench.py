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


def reference_arm(args):
    from baseline import reference_bench

    out = reference_bench.run(args)
    if out is not None:
        print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--bytes", type=int, default=1 << 30, help="allreduce vector bytes per GPU (headline)")
    ap.add_argument("--sweep", default="8,512,32768,1048576,33554432,268435456",
                    help="comma separated message sizes in bytes for the latency / bandwidth table ('' = none)")
    ap.add_argument("--sweep-iters", type=int, default=10)
    ap.add_argument("--no-nccl", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    import configurable_hierarchical_allreduce_algorithms_b200 as chb
    from configurable_hierarchical_allreduce_algorithms_b200.parallel.comm import Communicator

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
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

    heap_user = 2 * S + (64 << 20) + (0 if args.no_e2e else (6 * (64 << 20) + (1 << 20)))   # + the host pipeline's chunks
    if world > 1:
        comm = Communicator.from_process_group(scratch_bytes=max(64 << 20, S + (16 << 20)) if N > 1 else 1 << 20,
                                               user_bytes=heap_user)
    else:
        comm = Communicator.emulated(1, scratch_bytes=1 << 20, user_bytes=heap_user)

    def unl(x):  # emulated single-rank world hands out lists
        return x[0] if isinstance(x, list) else x

    x = unl(comm.empty(nelem, torch.float32))
    y = unl(comm.empty(nelem, torch.float32))
    g = torch.Generator(device="cuda").manual_seed(1234 + rank)
    x.copy_(torch.rand(nelem, generator=g, device="cuda") * 2 - 1)
    wrap = lambda t: t  # one local rank per process: tensors, not lists

    def step():
        chb.all_reduce(comm, wrap(x), out=wrap(y))

    # ---- correctness of the timed call (against NCCL when there are peers, else identity)
    step()
    torch.cuda.synchronize()
    comm.check()
    if world > 1:
        ref = x.clone()
        dist.all_reduce(ref)
        err = float((y - ref).abs().max())
        tol = 1e-4 * N
    else:
        err = float((y - x).abs().max())
        tol = 0.0
    correct = err <= tol

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

    # ---- NCCL on the same buffers
    nccl = None
    if world > 1 and not args.no_nccl:
        z = x.clone()
        for _ in range(W):
            dist.all_reduce(z)
        t = max_over_ranks(device_time_ms(lambda: dist.all_reduce(z), K, None, barrier)) / K
        nccl = {"ms_per_step": t, "algbw_GBps": S / (t * 1e-3) / 1e9, "busbw_GBps": S / (t * 1e-3) / 1e9 * 2 * (N - 1) / N}
        del z

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

        ke = max(3, min(K, 10))
        for _ in range(3):
            e2e_step()
        barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(ke):
            e2e_step()
        e1.record()
        torch.cuda.synchronize()
        barrier()
        tms = max_over_ranks(e0.elapsed_time(e1)) / ke
        wall = (time.perf_counter() - t0) * 1e3 / ke
        probe = slice(nelem - (1 << 20), nelem)      # the last chunk's tail: wrong only if the pipeline lost a chunk
        e2e_ok = bool(torch.equal(hy[probe], y[probe].cpu()))
        e2e = {"value": N * S / (tms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": tms, "steps": ke,
               "h2d_bytes_per_step": S, "d2h_bytes_per_step": S, "wall_ms_per_step": wall, "is_correct": e2e_ok,
               "api": "HostAllReduce: 32 MiB chunks, upload / allreduce / download pipelined on three streams"}
        del hx, hy

    # ---- latency / bandwidth table
    sweep = []
    if args.sweep:
        flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        flush = lambda: flush_buf.fill_(1)
        for sz in [int(s) for s in args.sweep.split(",") if s]:
            if sz > S:
                continue
            for dtype, dname in ((torch.float32, "fp32"), (torch.bfloat16, "bf16")):
                esz = 4 if dtype == torch.float32 else 2
                ne = max(1, sz // esz)
                ne_rs = max(1, ne // max(N, 1))
                xf, yf = x.view(dtype), y.view(dtype)     # slices below may be longer than ne for tiny sizes
                xv, yv = xf[:ne], yf[:ne]
                row = {"bytes": ne * esz, "dtype": dname}
                cases = {
                    "allreduce": (lambda: chb.all_reduce(comm, wrap(xv), out=wrap(yv)),
                                  (lambda: dist.all_reduce(yv)) if world > 1 else None, 2 * (N - 1) / N, ne * esz),
                    "reduce_scatter": (lambda: chb.reduce_scatter(comm, wrap(xf[:ne_rs * N]), out=wrap(yf[:ne_rs])),
                                       (lambda: dist.reduce_scatter_tensor(yf[:ne_rs], xf[:ne_rs * N])) if world > 1 else None,
                                       (N - 1) / N, ne_rs * N * esz),
                    "allgather": (lambda: chb.all_gather(comm, wrap(xf[:ne_rs]), out=wrap(yf[:ne_rs * N])),
                                  (lambda: dist.all_gather_into_tensor(yf[:ne_rs * N], xf[:ne_rs])) if world > 1 else None,
                                  (N - 1) / N, ne_rs * N * esz),
                }
                for name, (ours, theirs, factor, total_bytes) in cases.items():
                    # about 30 ms of back-to-back calls first (the same count on every rank): after the small
                    # sizes of the sweep the links and clocks need more than three calls to be back at speed
                    n_warm = min(200, max(3, int(30e-3 / (20e-6 + total_bytes / 2e11))))
                    for _ in range(n_warm):
                        ours()
                    t = [max_over_ranks(v) for v in per_call_ms(ours, args.sweep_iters, flush, barrier)]
                    p50 = statistics.median(t)
                    row[name] = {"p50_us": p50 * 1e3, "busbw_GBps": total_bytes / (p50 * 1e-3) / 1e9 * factor}
                    if theirs is not None and not args.no_nccl:
                        for _ in range(n_warm):
                            theirs()
                        t = [max_over_ranks(v) for v in per_call_ms(theirs, args.sweep_iters, flush, barrier)]
                        p50n = statistics.median(t)
                        row[name]["nccl_p50_us"] = p50n * 1e3
                        row[name]["nccl_busbw_GBps"] = total_bytes / (p50n * 1e-3) / 1e9 * factor
                sweep.append(row)
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


    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except (OSError, ValueError):
            pass
        # roofline: bytes that must cross NVLink per GPU / measured peer bandwidth (770 GB/s per direction),
        # or for one GPU the local copy at the measured HBM copy bandwidth
        if N > 1:
            ideal_ms = (2 * (N - 1) / N * S) / 770e9 * 1e3
        else:
            ideal_ms = (2 * S) / (peaks.get("hbm_gbs", 6650.0) * 1e9) * 1e3
        out = {
            "metric": "allreduce_sum_fp32_aggregate_algbw_GBps",
            "value": value, "unit": "GB/s", "n_gpus": N, "steps": K, "warmup": W, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
            "impl": "ours",
            "config": {"model": "allreduce sum fp32 (config 2 of the sweep: 8 B - 1 GiB)", "bytes_per_gpu": S,
                       "global_batch": None, "seq_len": None, "parallelism": f"{N} ranks, one per GPU",
                       "backend": comm.backend, "nvls": comm.has_multicast,
                       "l2": "inputs larger than L2 for the headline; explicit 256 MiB L2 flush before every timed call in the sweep"},
            "algbw_GBps": algbw, "busbw_GBps": busbw, "roofline_frac": ideal_ms / ms_per_step,
            "roofline_note": "of measured (770 GB/s NVLink per direction; HBM copy from MEASURED_PEAKS.json at N=1)",
            "is_correct": bool(correct), "max_abs_err": err,
            "clocks": clocks, "gpu_launches": launches, "e2e": e2e, "nccl": nccl, "sweep": sweep,
            "graph_replay_latency": graph_lat,
        }
        print(json.dumps(out), flush=True)
    comm.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
