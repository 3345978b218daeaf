"""ZeRO-style sharded optimizer step.

All parameters live in one flat bf16 buffer and all gradients in one flat fp32
buffer, both in symmetric memory.  ``step()`` is two launches:

1. ``reduce_scatter_adam`` — rank r pulls shard r of every rank's gradient
   buffer (or has the switch sum it), applies AdamW to its fp32 master shard
   and writes the updated bf16 shard into the parameter buffer
   (``csrc/kernels/fused_adam.cu``);
2. an allgather of the parameter buffer with the configurable radix-batch
   schedule (or NVLS / the tuned choice).

The reference provides the two primitives only
(reduce_scatter_radix_batch.cpp:200, all_gather_radix_batch_1_0.cpp:37).
With ``comm=None`` the same step runs over ``torch.distributed`` (gloo) with
plain tensor math: the host-level fallback used by the CPU tests.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import collectives, fused


class ShardedAdamW:
    def __init__(self, module: torch.nn.Module, comm=None, lr=3e-4, betas=(0.9, 0.95), eps=1e-8,
                 weight_decay=0.1, ag_algo: str = "auto", ag_k: int = 2, ag_b: int = 1, group=None):
        self.module, self.comm, self.group = module, comm, group
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.ag_algo, self.ag_k, self.ag_b = ag_algo, ag_k, ag_b
        self.P = comm.P if comm is not None else (dist.get_world_size(group) if dist.is_initialized() else 1)
        self.rank = comm.rank if comm is not None else (dist.get_rank(group) if dist.is_initialized() else 0)
        self.params = [p for p in module.parameters() if p.requires_grad]
        dev = self.params[0].device
        offs, total = [], 0
        for p in self.params:
            offs.append(total)
            total += (p.numel() + 7) // 8 * 8          # 16-byte aligned bf16 slots
        unit = 64 * self.P
        total = (total + unit - 1) // unit * unit
        self.n = total // self.P
        self.total = total
        if comm is not None:
            self.grad_flat = comm.empty(total, torch.float32)
            self.param_flat = comm.empty(total, torch.bfloat16)
        else:
            self.grad_flat = torch.zeros(total, device=dev)
            self.param_flat = torch.zeros(total, dtype=self.params[0].dtype, device=dev)
        self.grad_flat.zero_()
        self.param_flat.zero_()
        self._off = dict(zip(self.params, offs))
        self._queued = []                  # (parameter, gradient) pairs not yet moved into the flat buffer
        self._fresh = set()                # parameters whose next gradient overwrites its slot (after zero_grad)
        for p, off in zip(self.params, offs):
            self.param_flat[off:off + p.numel()].copy_(p.detach().reshape(-1))
            p.data = self.param_flat[off:off + p.numel()].view_as(p)     # the model now lives in the flat buffer
            p.main_grad = self.grad_flat[off:off + p.numel()].view_as(p)
            p.register_post_accumulate_grad_hook(self._hook)
        lo = self.rank * self.n
        self.master = self.param_flat[lo:lo + self.n].float().clone()
        self.exp_avg = torch.zeros(self.n, device=dev)
        self.exp_avg_sq = torch.zeros(self.n, device=dev)
        self.t = 0

    _FLUSH_AT = 48                         # gradients per fill kernel (one launch's table)

    def _hook(self, p):
        # queued, then moved in groups by one multi-tensor kernel (bf16 -> fp32, overwrite or accumulate)
        self._queued.append((p, p.grad))
        p.grad = None
        if len(self._queued) >= self._FLUSH_AT:
            self._flush()

    def _flush(self):
        if not self._queued:
            return
        if self.comm is not None and self.grad_flat.is_cuda:
            fused.bucket_fill(self.grad_flat, [(g, self._off[p], p in self._fresh) for p, g in self._queued])
        else:
            for p, g in self._queued:
                if p in self._fresh:
                    p.main_grad.copy_(g)
                else:
                    p.main_grad.add_(g)
        for p, _ in self._queued:
            self._fresh.discard(p)
        self._queued = []

    def zero_grad(self):
        """Start a new accumulation without touching memory: the first gradient of every parameter
        overwrites its slot; slots that receive none are cleared when the step is taken."""
        self._flush()
        self._fresh = set(self.params)

    def ag_choice(self):
        """(algorithm, k, b) the parameter allgather runs with: the pinned one, or what the tuned table
        answers for this shard size."""
        if self.comm is None:
            return ("library", 0, 0)
        if self.ag_algo != "auto":
            return (self.ag_algo, self.ag_k, self.ag_b)
        from ..utils import autotune
        c = autotune.choose(self.comm, "allgather", self.n * self.param_flat.element_size(), self.param_flat.dtype, True)
        return (c.algo, c.k, c.b)

    @torch.no_grad()
    def step(self, stream=None):
        self.t += 1
        self._flush()
        for p in self._fresh:              # no gradient since zero_grad: the slot still holds the previous step's values
            p.main_grad.zero_()
        self._fresh = set()
        lo = self.rank * self.n
        shard = self.param_flat[lo:lo + self.n]
        if self.comm is not None:
            fused.reduce_scatter_adam(self.comm, self.grad_flat, self.master, self.exp_avg, self.exp_avg_sq, shard,
                                      lr=self.lr, betas=self.betas, eps=self.eps, weight_decay=self.wd, step=self.t,
                                      grad_scale=1.0 / self.P, stream=stream)
            collectives.all_gather(self.comm, shard, out=self.param_flat, algo=self.ag_algo, k=self.ag_k,
                                   b=self.ag_b, stream=stream)
            return
        # host-level fallback: same arithmetic with library collectives
        if self.P > 1 and self.grad_flat.is_cuda:
            g = torch.empty(self.n, device=self.grad_flat.device)
            dist.reduce_scatter_tensor(g, self.grad_flat, group=self.group)
            g = g / self.P
        else:
            g = self.grad_flat.clone()
            if self.P > 1:
                dist.all_reduce(g, group=self.group)      # gloo has no reduce-scatter
            g = g[lo:lo + self.n] / self.P
        b1, b2 = self.betas
        self.exp_avg.mul_(b1).add_(g, alpha=1 - b1)
        self.exp_avg_sq.mul_(b2).addcmul_(g, g, value=1 - b2)
        mhat = self.exp_avg / (1 - b1 ** self.t)
        vhat = self.exp_avg_sq / (1 - b2 ** self.t)
        self.master.sub_(self.lr * (mhat / (vhat.sqrt() + self.eps) + self.wd * self.master))
        shard.copy_(self.master)
        if self.P > 1 and shard.is_cuda:
            dist.all_gather_into_tensor(self.param_flat, shard.clone(), group=self.group)
        elif self.P > 1:
            parts = [torch.empty_like(shard) for _ in range(self.P)]
            dist.all_gather(parts, shard.clone(), group=self.group)
            self.param_flat.copy_(torch.cat(parts))

    # ------------------------------------------------------------------ checkpoint / resume
    def state_dict(self) -> dict:
        """This rank's shard of the optimizer state (save one file per rank with ``torch.save``)."""
        return {"rank": self.rank, "world": self.P, "n": self.n, "step": self.t,
                "master": self.master.detach().cpu().clone(), "exp_avg": self.exp_avg.detach().cpu().clone(),
                "exp_avg_sq": self.exp_avg_sq.detach().cpu().clone(),
                "hyper": {"lr": self.lr, "betas": self.betas, "eps": self.eps, "weight_decay": self.wd}}

    @torch.no_grad()
    def load_state_dict(self, sd: dict) -> None:
        """Restore a shard saved by :meth:`state_dict` with the same world size; the bf16 parameter
        shard is rebuilt from the fp32 master (call ``step``-free ``sync_params`` afterwards)."""
        if sd["world"] != self.P or sd["rank"] != self.rank or sd["n"] != self.n:
            raise ValueError("optimizer shard was saved for a different rank / world size / model")
        self.t = int(sd["step"])
        self.master.copy_(sd["master"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        lo = self.rank * self.n
        self.param_flat[lo:lo + self.n].copy_(self.master)

    @torch.no_grad()
    def sync_params(self, stream=None) -> None:
        """Allgather the parameter shards (after ``load_state_dict``)."""
        lo = self.rank * self.n
        shard = self.param_flat[lo:lo + self.n]
        if self.comm is not None:
            collectives.all_gather(self.comm, shard, out=self.param_flat, algo=self.ag_algo, k=self.ag_k,
                                   b=self.ag_b, stream=stream)
        elif self.P > 1:
            parts = [torch.empty_like(shard) for _ in range(self.P)]
            dist.all_gather(parts, shard.clone(), group=self.group)
            self.param_flat.copy_(torch.cat(parts))
