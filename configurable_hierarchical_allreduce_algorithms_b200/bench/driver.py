"""Benchmark driver with the reference's command line and CSV schema.

    torchrun --nproc-per-node N -m configurable_hierarchical_allreduce_algorithms_b200.bench.driver \
        <n_iter> [--overwrite] [b=<group>] [base=<elements>] [num_nodes=<n>] [radix_increment=<step>]
        [coll=allreduce|reduce_scatter|allgather] [dtype=int32|fp32|bf16|fp64] [op=sum|max|min]
        [algos=radix_batch,ring,...] [reps=50] [backend=gpu|gloo] [out=<file.csv>] [symmetric=1]
        [local_size=<ranks per box>] [inter_algo=ring|library|...]

Like the reference's drivers (testing/custom_implementations/work_dir/all_reduce/main.cpp:111-199,
.../all_gather/main.cpp:109-201, .../reduce_scatter/main.cpp:169-264, testing/main.cpp:146-220):
message sizes double ``n_iter`` times starting from ``base`` elements per rank, the radix sweeps
``k = 2 .. b-1`` in steps of ``radix_increment`` for the hierarchical algorithm, every repetition is
checked against the library collective (``MPI_Allreduce`` there, NCCL / gloo here) and written as one
CSV row ``algorithm_name,k,b,nprocs,send_count,time,is_correct`` (the same columns, followed by
``dtype,op,bytes,algbw_GBs,busbw_GBs,ngpus,p50_us,roofline_frac``: the last two are per configuration, the
median over its repetitions and the share of the NVLink roofline that median reaches).  An existing file
is appended to unless ``--overwrite`` is given, and rows are flushed configuration by configuration, so an
interrupted sweep resumes where it stopped.
Correctness is AND-reduced and time MAX-reduced over ranks, as in the reference's reduce-scatter
driver (main.cpp:79-83).  ``symmetric=1`` places input and output in the peer-visible heap (registered
buffers: nothing is staged, and the kernel-level algorithms ``ll``, ``ll2``, ``nvls``, ``bulk`` can be
named in ``algos``).  ``local_size=L`` (implied when torchrun reports fewer local than global ranks, i.e.
several machines) runs every collective on two physical levels: the swept algorithm inside each box of
``L`` ranks, ``inter_algo`` along the lanes across boxes (``library`` = NCCL / gloo's own collective,
anything else a step program over host copies).  Time is device time (CUDA events) on GPUs and wall time under gloo.
"""
from __future__ import annotations

import os
import sys
import time

import torch
import torch.distributed as dist

DT = {"int32": torch.int32, "fp32": torch.float32, "bf16": torch.bfloat16, "fp64": torch.float64, "fp16": torch.float16}
HEADER = "algorithm_name,k,b,nprocs,send_count,time,is_correct,dtype,op,bytes,algbw_GBs,busbw_GBs,ngpus,p50_us,roofline_frac"
BASELINES = {
    "allreduce": ["recursive_doubling", "ring", "reduce_scatter_allgather", "k_reduce_scatter_allgather",
                  "recursive_multiplying", "recursive_exchange"],
    "reduce_scatter": ["recursive_halving", "recursive_doubling", "pairwise", "radix"],
    "allgather": ["k_brucks", "ring"],
}
VENDOR = {"allreduce": "MPICH_allreduce", "reduce_scatter": "reduce_scatter_standard", "allgather": "allgather_standard"}
K_ALGOS = {"radix_batch", "k_reduce_scatter_allgather", "recursive_multiplying", "recursive_exchange", "radix",
           "k_brucks", "semi_radix_batch", "custom", "radix_block"}


def parse(argv):
    if not argv or not argv[0].lstrip("-").isdigit():
        raise SystemExit(__doc__)
    o = {"n_iter": int(argv[0]), "overwrite": False, "b": 0, "base": 1, "num_nodes": 1, "radix_increment": 1,
         "coll": "allreduce", "dtype": "int32", "op": "sum", "algos": "", "reps": 50, "backend": "", "out": "",
         "symmetric": 0, "local_size": 0, "inter_algo": "ring"}
    for a in argv[1:]:
        if a == "--overwrite":
            o["overwrite"] = True
        elif "=" in a and a.split("=", 1)[0] in o:
            k, v = a.split("=", 1)
            o[k] = type(o[k])(v) if not isinstance(o[k], bool) else v.lower() in ("1", "true")
        else:
            raise SystemExit(f"Unknown parameter: {a}")
    return o


def make_input(rank, n_in, dtype, device):
    # the reference's deterministic ramps (rank*count + i), folded to stay exact in every dtype
    i = torch.arange(n_in, device=device, dtype=torch.int64)
    return ((rank * 1009 + i * 31 + 7) % 97).to(dtype)


def main(argv=None):
    o = parse(list(sys.argv[1:] if argv is None else argv))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    lr = int(os.environ.get("LOCAL_RANK", "0"))
    backend = o["backend"] or ("gpu" if torch.cuda.is_available() else "gloo")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29540")
    if backend == "gpu":
        torch.cuda.set_device(lr)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", lr))
        device = torch.device("cuda", lr)
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        device = torch.device("cpu")
    P = world
    coll, dtype, op = o["coll"], DT[o["dtype"]], o["op"]
    b = o["b"] or P
    if P % b:
        raise SystemExit(f"b={b} must divide the number of ranks ({P})")
    esz = torch.empty((), dtype=dtype).element_size()
    max_n = o["base"] << max(0, o["n_iter"] - 1)
    comm = None
    from ..parallel import hierarchy as H
    L = o["local_size"] or int(os.environ.get("LOCAL_WORLD_SIZE", P))
    if L >= P or L < 1 or P % L:
        L = 0                                               # one box: a single level
    intra_group = inter_group = inter_prog_group = None
    if L:
        intra_group, inter_group = H.split_world(L)
        inter_prog_group = inter_group
        if backend == "gpu" and o["inter_algo"] != "library":
            _, inter_prog_group = H.split_world(L, backend="gloo")   # step programs on host copies need a CPU group
        if not o["b"] or L % b:
            b = L                                           # the group size of the swept algorithm lives inside a box
        o["symmetric"] = 0                                  # the levels exchange intermediate tensors of their own
    PL = L or P                                             # ranks of the level the swept algorithm runs on
    if backend == "gpu":
        from ..parallel.comm import Communicator
        total = max_n * P * esz
        comm = Communicator.from_process_group(group=intra_group, scratch_bytes=4 * total + (32 << 20),
                                               user_bytes=(64 << 20) + (2 * total + 4096 if o["symmetric"] else 0))
    sym_in = sym_out = None
    if comm is not None and o["symmetric"]:
        # registered buffers: input and output live in the peer-visible heap, so nothing is staged
        sym_in = comm.empty(max_n * (1 if coll == "allgather" else P), dtype)
        sym_out = comm.empty(max_n * (1 if coll == "reduce_scatter" else P), dtype)
    from .. import all_gather, all_reduce, reduce_scatter
    from ..parallel.comm import CollectiveError
    from ..parallel.program import ProgramError
    from ..parallel import gloo_exec

    def two_level(algo, k, gb):
        """The swept algorithm inside a box, inter_algo along the lanes."""
        intra = H.DeviceLevel(comm, algo, k, gb) if backend == "gpu" else H.GlooLevel(intra_group, algo, k, gb)
        if o["inter_algo"] == "library":
            inter = H.LibraryLevel(inter_group)
        else:
            inter = H.GlooLevel(inter_prog_group, o["inter_algo"], 2, 1)
        return H.TwoLevel(intra, inter)

    path = o["out"] or f"results{P}_{o['num_nodes']}_{b}.csv"
    csv = None
    if rank == 0:
        fresh = o["overwrite"] or not os.path.exists(path)
        csv = open(path, "w" if fresh else "a")
        if fresh:
            csv.write(HEADER + "\n")
    redop = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}[op]
    algos = [a for a in o["algos"].split(",") if a] or (["radix_batch", "ring"] if L else ["radix_batch"] + BASELINES[coll])

    def run_one(name, algo, k, bb, n, x, ref):
        """`reps` timed, checked repetitions of one configuration."""
        send_count = n
        kk, gb = (k or 2), (bb or 1)       # the CSV keeps 0 for "not applicable", the generators need valid values
        rows = []                          # one row per repetition; written together once their median is known
        for _ in range(o["reps"]):
            if backend == "gpu":
                dist.barrier()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                out = None
                if sym_out is not None:
                    out = sym_out[:n * (1 if coll == "reduce_scatter" else P)]
                try:
                    if algo == "vendor":
                        y = vendor(x)
                    elif L:
                        lvl = two_level(algo, kk, gb)
                        y = lvl.all_reduce(x, op) if coll == "allreduce" else (
                            lvl.reduce_scatter(x, op) if coll == "reduce_scatter" else lvl.all_gather(x))
                    elif coll == "allreduce":
                        y = all_reduce(comm, x, out=out, op=op, algo=algo, k=kk, b=gb)
                    elif coll == "reduce_scatter":
                        y = reduce_scatter(comm, x, out=out, op=op, algo=algo, k=kk, b=gb)
                    else:
                        y = all_gather(comm, x, out=out, algo=algo, k=kk, b=gb)
                except (CollectiveError, ProgramError) as e:
                    # a capability this communicator lacks (no multicast alias, message too large for the
                    # flagged-line inbox ...): the same on every rank, so all of them skip the configuration
                    if rank == 0:
                        print(f"skipped {name} k={k} b={bb} count={n}: {e}", file=sys.stderr, flush=True)
                    return
                e1.record()
                torch.cuda.synchronize()
                t = e0.elapsed_time(e1) * 1e-3
            else:
                dist.barrier()
                t0 = time.perf_counter()
                try:
                    if algo == "vendor":
                        y = vendor(x)
                    elif L:
                        lvl = two_level(algo, kk, gb)
                        y = lvl.all_reduce(x, op) if coll == "allreduce" else (
                            lvl.reduce_scatter(x, op) if coll == "reduce_scatter" else lvl.all_gather(x))
                    else:
                        count = n * P if coll == "allreduce" else n
                        y = gloo_exec.run_collective(coll, algo, x, count, kk, gb, op=op)
                except ProgramError as e:     # e.g. an allreduce-only algorithm asked to serve as a level's reduce-scatter
                    if rank == 0:
                        print(f"skipped {name} k={k} b={bb} count={n}: {e}", file=sys.stderr, flush=True)
                    return
                dist.barrier()
                t = time.perf_counter() - t0
            ok = torch.equal(y, ref) if not dtype.is_floating_point else bool(
                torch.allclose(y.double(), ref.double(), rtol=1e-5 if dtype != torch.bfloat16 else 2e-2, atol=1e-5 * P))
            flag = torch.tensor([1 if ok else 0, 0], device=device, dtype=torch.float64)
            tt = torch.tensor([t], device=device, dtype=torch.float64)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            if rank == 0:
                t = float(tt.item())
                total = n * P * esz
                factor = 2 * (P - 1) / P if coll == "allreduce" else (P - 1) / P
                rows.append((t, f"{name},{k},{bb},{P},{send_count},{t:.9f},{int(flag[0].item())},{o['dtype']},{op},{total},"
                                f"{total / t / 1e9:.4f},{total / t / 1e9 * factor:.4f},{P if backend == 'gpu' else 0}"))
        if rank == 0 and rows:
            # p50 of the configuration, and the share of the NVLink roofline it reaches: the bytes one GPU must
            # move per direction (bus-bandwidth factor times the vector) over the measured 770 GB/s peer rate
            p50 = sorted(t for t, _ in rows)[len(rows) // 2]
            total = n * P * esz
            factor = 2 * (P - 1) / P if coll == "allreduce" else (P - 1) / P
            frac = (total * factor / 770e9) / p50 if backend == "gpu" and P > 1 else 0.0
            for _, line in rows:
                csv.write(f"{line},{p50 * 1e6:.3f},{frac:.4f}\n")
            csv.flush()

    def vendor(x):
        if coll == "allreduce":
            y = x.clone()
            dist.all_reduce(y, op=redop)
            return y
        if coll == "reduce_scatter":
            if backend == "gpu":
                y = torch.empty(x.numel() // P, dtype=x.dtype, device=device)
                dist.reduce_scatter_tensor(y, x, op=redop)
                return y
            y = x.clone()
            dist.all_reduce(y, op=redop)
            n = x.numel() // P
            return y[rank * n:(rank + 1) * n].clone()
        parts = [torch.empty_like(x) for _ in range(P)]
        dist.all_gather(parts, x)
        return torch.cat(parts)

    for i in range(o["n_iter"]):
        n = o["base"] << i                                   # elements per rank
        n_in = n if coll == "allgather" else n * P
        x = make_input(rank, n_in, dtype, device)
        if sym_in is not None:
            sym_in[:n_in].copy_(x)
            x = sym_in[:n_in]
        ref = vendor(x)
        for algo in algos:
            name = f"{coll}_{algo}" if algo != "radix_batch" else {"allreduce": "all_reduce_radix_batch", "reduce_scatter": "reduce_scatter_radix_batch", "allgather": "allgather_radix_batch"}[coll]
            if algo in K_ALGOS:
                hi = max(3, b) if algo == "radix_batch" else max(3, PL)
                for k in range(2, hi, max(1, o["radix_increment"])):
                    run_one(name, algo, k, b if algo in ("radix_batch", "semi_radix_batch", "custom", "radix_block") else 0, n, x, ref)
            else:
                run_one(name, algo, 0, 0, n, x, ref)
        run_one(VENDOR[coll], "vendor", 0, 0, n, x, ref)
    if csv:
        csv.close()
    if comm:
        comm.check()
        comm.close()
    dist.barrier()                    # nobody tears its transport down while a peer is still in the last collective
    dist.destroy_process_group()
    return path


if __name__ == "__main__":
    main()
    if not torch.cuda.is_available():
        # CPU ranks leave without the interpreter's teardown: on a busy machine gloo's helper threads can still be
        # alive when static destructors run, which ends a rank that has already written everything with SIGABRT.
        # GPU ranks take the normal way out, so that mapped peer memory is released in order.
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
