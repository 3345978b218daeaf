"""Checkpoint / resume of the optimizer states (single process, host fallback):
training 2 + 2 steps with a save / load in between equals training 4 steps."""
import io

import torch

from configurable_hierarchical_allreduce_algorithms_b200.models.gpt import GPT, GPTConfig
from configurable_hierarchical_allreduce_algorithms_b200.parallel.ddp import DataParallel, MasterAdamW
from configurable_hierarchical_allreduce_algorithms_b200.parallel.zero import ShardedAdamW


def _data():
    return torch.randint(0, 257, (2, 32), generator=torch.Generator().manual_seed(0))


def _train(model, opt, steps, ddp=None):
    x = _data()
    for _ in range(steps):
        (ddp or opt).zero_grad()
        (ddp or model)(x, x).backward()
        if ddp:
            ddp.finish()
        opt.step()


def _roundtrip(sd):
    buf = io.BytesIO()
    torch.save(sd, buf)
    buf.seek(0)
    return torch.load(buf, weights_only=False)


def test_sharded_adamw_resume():
    torch.manual_seed(1)
    a = GPT(GPTConfig.tiny("llama"))
    oa = ShardedAdamW(a, comm=None, lr=1e-2)
    _train(a, oa, 4)
    torch.manual_seed(1)
    b = GPT(GPTConfig.tiny("llama"))
    ob = ShardedAdamW(b, comm=None, lr=1e-2)
    _train(b, ob, 2)
    sd = _roundtrip(ob.state_dict())
    torch.manual_seed(1)
    c = GPT(GPTConfig.tiny("llama"))
    oc = ShardedAdamW(c, comm=None, lr=1e-2)
    oc.load_state_dict(sd)
    oc.sync_params()
    _train(c, oc, 2)
    for (n, p), (_, q) in zip(a.named_parameters(), c.named_parameters()):
        torch.testing.assert_close(p, q, rtol=1e-6, atol=1e-7, msg=n)


def test_master_adamw_resume():
    torch.manual_seed(1)
    a = GPT(GPTConfig.tiny("gpt2"))
    da = DataParallel(a, comm=None, bucket_bytes=64 << 10)
    oa = MasterAdamW(da, lr=1e-2)
    _train(a, oa, 4, da)
    torch.manual_seed(1)
    b = GPT(GPTConfig.tiny("gpt2"))
    db = DataParallel(b, comm=None, bucket_bytes=64 << 10)
    ob = MasterAdamW(db, lr=1e-2)
    _train(b, ob, 2, db)
    sd = _roundtrip(ob.state_dict())
    torch.manual_seed(7)                      # different init: everything must come from the checkpoint
    c = GPT(GPTConfig.tiny("gpt2"))
    dc = DataParallel(c, comm=None, bucket_bytes=64 << 10)
    oc = MasterAdamW(dc, lr=1e-2)
    oc.load_state_dict(sd)
    _train(c, oc, 2, dc)
    for (n, p), (_, q) in zip(a.named_parameters(), c.named_parameters()):
        torch.testing.assert_close(p, q, rtol=1e-6, atol=1e-7, msg=n)
