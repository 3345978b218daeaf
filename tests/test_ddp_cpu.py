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


class _TwoHeads(torch.nn.Module):
    """A layer that only gets a gradient when ``use_b`` is set."""

    def __init__(self):
        super().__init__()
        self.a = torch.nn.Linear(8, 8)
        self.b = torch.nn.Linear(8, 8)

    def forward(self, x, use_b):
        y = self.a(x)
        return (y + self.b(x)).sum() if use_b else y.sum()


def test_several_micro_batches_inside_one_no_sync_block_all_count():
    # single process, world of one: the wrapper's accumulation must equal plain autograd accumulation
    torch.manual_seed(3)
    m, ref = _TwoHeads(), _TwoHeads()
    ref.load_state_dict(m.state_dict())
    ddp = DataParallel(m, comm=None, bucket_bytes=1 << 8)
    xs = [torch.randn(2, 8) for _ in range(4)]
    ddp.zero_grad()
    with ddp.no_sync():
        for x in xs[:3]:                      # three backward passes in ONE context
            ddp(x, True).backward()
    ddp(xs[3], True).backward()
    ddp.finish()
    for x in xs:
        ref(x, True).backward()
    for (n, p), (_, q) in zip(m.named_parameters(), ref.named_parameters()):
        torch.testing.assert_close(p.reduced_grad, q.grad, rtol=1e-5, atol=1e-6, msg=n)


def test_parameter_without_gradient_contributes_zero_not_last_steps_values():
    torch.manual_seed(4)
    m, ref = _TwoHeads(), _TwoHeads()
    ref.load_state_dict(m.state_dict())
    ddp = DataParallel(m, comm=None, bucket_bytes=1 << 8)
    x = torch.randn(2, 8)
    ddp.zero_grad()
    ddp(x, True).backward()                   # step 1: every parameter gets a gradient
    ddp.finish()
    ddp.zero_grad()
    ddp(x, False).backward()                  # step 2: head b is unused
    ddp.finish()
    ref(x, False).backward()
    for (n, p), (_, q) in zip(m.named_parameters(), ref.named_parameters()):
        exp = q.grad if q.grad is not None else torch.zeros_like(q)
        torch.testing.assert_close(p.reduced_grad, exp, rtol=1e-5, atol=1e-6, msg=n)
    # and accumulation across a pass in which b is unused keeps b's earlier contribution
    ddp.zero_grad()
    with ddp.no_sync():
        ddp(x, True).backward()
        ddp(x, False).backward()
    ddp(x, False).backward()
    ddp.finish()
    ref.zero_grad()
    ref(x, True).backward(); ref(x, False).backward(); ref(x, False).backward()
    for (n, p), (_, q) in zip(m.named_parameters(), ref.named_parameters()):
        torch.testing.assert_close(p.reduced_grad, q.grad, rtol=1e-5, atol=1e-6, msg=n)
