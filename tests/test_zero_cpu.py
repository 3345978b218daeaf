"""Sharded optimizer step on CPU (gloo fallback): two ranks must end up with
the parameters of one process running AdamW on the whole batch."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from configurable_hierarchical_allreduce_algorithms_b200.models.gpt import GPT, GPTConfig
from configurable_hierarchical_allreduce_algorithms_b200.parallel.zero import ShardedAdamW


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _data():
    return torch.randint(0, 257, (4, 32), generator=torch.Generator().manual_seed(0))


def _worker(rank, P, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=P)
    torch.manual_seed(1)
    model = GPT(GPTConfig.tiny("llama"))
    opt = ShardedAdamW(model, comm=None, lr=1e-2)
    x = _data()[rank * 2:(rank + 1) * 2]
    for _ in range(2):
        opt.zero_grad()
        model(x, x).backward()
        opt.step()
    if rank == 1:
        q.put({n: p.detach().clone().numpy() for n, p in model.named_parameters()})
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
    params = q.get()
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    torch.manual_seed(1)
    ref = GPT(GPTConfig.tiny("llama"))
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    x = _data()
    for _ in range(2):
        opt.zero_grad()
        ((ref(x[:2], x[:2]) + ref(x[2:], x[2:])) / 2).backward()
        opt.step()
    for n, p in ref.named_parameters():
        torch.testing.assert_close(torch.from_numpy(params[n]), p.detach(), rtol=2e-4, atol=2e-5)
