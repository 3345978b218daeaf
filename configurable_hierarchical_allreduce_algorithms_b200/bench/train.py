"""Training-step benchmarks for the two model configurations:

    torchrun --nproc-per-node N -m configurable_hierarchical_allreduce_algorithms_b200.bench.train --mode dp
        GPT-2-medium shaped decoder (24 layers, d_model 1024, 16 heads, vocab 50257, seq 1024, micro-batch 8 per
        GPU, bf16 parameters, fp32 gradients in 25 MB buckets): bucketed allreduce with fused 1/P scale,
        overlapped with backward.  Reports tokens/s and exposed communication time per step.
    ... --mode zero
        Llama style 1.3B decoder (24 layers, d_model 2048, 16 heads, SwiGLU 5504, seq 2048, bf16): gradient
        reduce-scatter fused with the sharded AdamW update, parameter allgather with the radix-batch kernels.

``--impl nccl`` runs the same step with torch.distributed collectives for comparison.
Random-init weights, random token ids.  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch
import torch.distributed as dist

from ..models.gpt import GPT, GPTConfig
from ..parallel.comm import Communicator
from ..parallel.ddp import DataParallel, FusedMasterAdamW, MasterAdamW
from ..parallel.zero import ShardedAdamW


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="dp", choices=["dp", "zero"])
    ap.add_argument("--impl", default="ours", choices=["ours", "nccl", "torchddp"])
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--micro-batch", type=int, default=0)
    ap.add_argument("--tiny", action="store_true", help="small model for smoke tests")
    ap.add_argument("--algo", default="auto")
    ap.add_argument("--k", type=int, default=2)
    ap.add_argument("--b", type=int, default=1)
    ap.add_argument("--comm-ctas", type=int, default=0, help="dp: CTAs of each bucket's allreduce kernel (0 = its own choice)")
    ap.add_argument("--out", default="", help="append the JSON line to this file as well")
    args = ap.parse_args(argv)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    lr_ = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(lr_)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", lr_))
    torch.manual_seed(0)
    if args.mode == "dp":
        cfg = GPTConfig.tiny("gpt2") if args.tiny else GPTConfig.gpt2_medium()
        mb = args.micro_batch or (2 if args.tiny else 8)
    else:
        cfg = GPTConfig.tiny("llama") if args.tiny else GPTConfig.llama_1p3b()
        mb = args.micro_batch or (2 if args.tiny else 4)
    model = GPT(cfg).cuda().to(torch.bfloat16)
    nparam = model.num_params()
    ours = args.impl == "ours"
    comm = None
    if ours:
        need = nparam * (8 if args.mode == "dp" else 6) + (256 << 20)
        comm = (Communicator.from_process_group(user_bytes=need, scratch_bytes=256 << 20) if world > 1
                else Communicator.emulated(1, user_bytes=need, scratch_bytes=1 << 20))
    torch_ddp = None
    if args.impl == "torchddp":
        # the stock data-parallel path: bf16 gradients, 25 MB buckets, NCCL allreduce overlapped by torch
        assert args.mode == "dp"
        torch_ddp = (torch.nn.parallel.DistributedDataParallel(model, device_ids=[lr_], bucket_cap_mb=25)
                     if world > 1 else model)
        topt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
        ddp, opt = None, None
    elif args.mode == "dp":
        ddp = DataParallel(model, comm=comm if ours else None, algo=args.algo, k=args.k, b=args.b, comm_ctas=args.comm_ctas)
        if not ours:
            ddp.cuda = False     # library collectives on CUDA tensors through torch.distributed
        opt = FusedMasterAdamW(ddp) if ours else MasterAdamW(ddp)
    else:
        opt = ShardedAdamW(model, comm=comm if ours else None, ag_algo=args.algo, ag_k=args.k, ag_b=args.b)
        ddp = None
    T = cfg.seq_len
    host_tokens = torch.randint(0, cfg.vocab, (args.steps + args.warmup, mb, T)).pin_memory()
    dev_tokens = torch.empty(mb, T, dtype=torch.long, device="cuda")
    loss_host = torch.zeros(1).pin_memory()

    def step(i):
        dev_tokens.copy_(host_tokens[i], non_blocking=True)          # this step's inputs from pinned host memory
        if torch_ddp is not None:
            topt.zero_grad(set_to_none=True)
            loss = torch_ddp(dev_tokens, dev_tokens)
            loss.backward()
            topt.step()
            loss_host.copy_(loss.detach().float().reshape(1), non_blocking=True)
            return loss
        (ddp or opt).zero_grad()
        loss = (ddp or model)(dev_tokens, dev_tokens)
        loss.backward()
        if ddp is not None:
            ddp.finish()
        opt.step()
        loss_host.copy_(loss.detach().float().reshape(1), non_blocking=True)   # the step's result back to the host
        return loss

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    l0 = comm.launches if comm else 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    exposed = []
    t0 = time.perf_counter()
    e0.record()
    for i in range(args.steps):
        step(args.warmup + i)
        if ddp is not None and ours and i == args.steps - 1:
            torch.cuda.synchronize()
            exposed.append(ddp.exposed_comm_ms())
    e1.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    ms = e0.elapsed_time(e1)
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / args.steps
    if comm:
        comm.check()
    out = None
    if rank == 0:
        out = {
            "metric": "tokens_per_s", "value": world * mb * T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "mode": args.mode, "impl": args.impl, "ms_per_step": ms, "steps": args.steps, "warmup": args.warmup,
            "loss": float(loss_host.item()), "params": nparam, "micro_batch": mb, "seq_len": T, "dtype": "bf16",
            "exposed_comm_ms": exposed[-1] if exposed else None,
            "collective_launches": (comm.launches - l0) if comm else None,
            "h2d_bytes_per_step": mb * T * 8, "d2h_bytes_per_step": 4, "wall_ms_per_step": wall * 1e3 / args.steps,
            "algo": args.algo, "k": args.k, "b": args.b, "comm_ctas": args.comm_ctas, "data": "synthetic"}
        if args.mode == "zero" and ours:
            out["param_allgather"] = "%s k=%d b=%d" % opt.ag_choice()
        print(json.dumps(out), flush=True)
        if args.out:
            with open(args.out, "a") as f:
                f.write(json.dumps(out) + "\n")
    if comm:
        comm.close()
    if world > 1:
        dist.destroy_process_group()
    return out


if __name__ == "__main__":
    main()
