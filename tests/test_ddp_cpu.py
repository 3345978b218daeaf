"""Bucketing / hook logic of the data-parallel wrapper on CPU: two gloo ranks
with half the batch each must produce the gradients (and, after one optimizer
step, the parameters) of one process running the whole batch."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from configurable_hierarchical_allreduce_algorithms_b200.models.gpt import GPT, GPTConfig
from configurable_hierarchical_allreduce_algorithms_b200.parallel.ddp import DataParallel, MasterAdamW


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _data():
    g = torch.Generator().manual_seed(0)
    return torch.randint(0, 257, (4, 32), generator=g)


def _worker(rank, P, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=P)
    torch.manual_seed(1)
    model = GPT(GPTConfig.tiny("gpt2"))
    ddp = DataParallel(model, comm=None, bucket_bytes=64 << 10)
    assert len(ddp.buckets) > 1
    opt = MasterAdamW(ddp, lr=1e-2)
    x = _data()[rank * 2:(rank + 1) * 2]
    ddp.zero_grad()
    with ddp.no_sync():                      # accumulate one micro-batch without reducing
        (ddp(x[:1], x[:1]) * 0.5).backward()
    (ddp(x[1:], x[1:]) * 0.5).backward()
    ddp.finish()
    grads = {n: p.reduced_grad.clone().numpy() for n, p in model.named_parameters()}
    opt.step()
    if rank == 0:
        q.put((grads, {n: p.detach().clone().numpy() for n, p in model.named_parameters()}))   # plain arrays: no shared-memory handles
    dist.barrier()                    # nobody tears its transport down while a peer is still communicating
    dist.destroy_process_group()
    os._exit(0)                       # skip the interpreter's teardown: helper threads of the transport may still be alive


def test_two_ranks_match_single_process():
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    grads, params = q.get()
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    torch.manual_seed(1)
    ref = GPT(GPTConfig.tiny("gpt2"))
    x = _data()
    loss = sum(ref(x[i:i + 1], x[i:i + 1]) for i in range(4)) / 4
    loss.backward()
    for n, p in ref.named_parameters():
        torch.testing.assert_close(torch.from_numpy(grads[n]), p.grad, rtol=1e-4, atol=1e-6)
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    opt.step()
    for n, p in ref.named_parameters():
        torch.testing.assert_close(torch.from_numpy(params[n]), p.detach(), rtol=1e-4, atol=1e-5)
