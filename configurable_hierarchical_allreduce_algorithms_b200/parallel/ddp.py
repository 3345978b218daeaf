"""Data-parallel gradient path: fp32 gradient buckets in symmetric memory,
allreduce with the 1/P scale fused into the kernel, launched per bucket on a
side stream as soon as the bucket's last gradient has been accumulated, so the
communication overlaps the rest of backward.

The reference stops at the allreduce primitive
(testing/custom_implementations/work_dir/all_reduce/all_reduce_radix_batch.cpp:202);
this module is the data-parallel use of it.

With ``comm=None`` the buckets are ordinary tensors and the reduction goes
through ``torch.distributed`` (gloo on CPU): the host-level fallback, used by
the CPU tests of the bucketing logic.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import collectives


class _Bucket:
    def __init__(self, index, numel, acc, red):
        self.index, self.numel = index, numel
        self.acc, self.red = acc, red        # accumulate buffer, reduced result
        self.params = []
        self.pending = 0
        self.ready_event = None
        self.fresh = set()                   # parameters whose next gradient overwrites their slot (after zero_grad)
        self.queued = []                     # (parameter, gradient) pairs not yet moved into the bucket


class DataParallel:
    def __init__(self, module: torch.nn.Module, comm=None, bucket_bytes: int = 25 << 20, overlap: bool = True,
                 algo: str = "auto", k: int = 2, b: int = 1, group=None, comm_ctas: int = 0):
        """``comm_ctas``: CTAs of each bucket's allreduce kernel (0 = the kernel's own choice).  A small number
        leaves the SMs and HBM bandwidth to the backward kernels it overlaps with."""
        self.module, self.comm, self.group = module, comm, group
        self.algo, self.k, self.b, self.overlap, self.comm_ctas = algo, k, b, overlap, comm_ctas
        self.world = comm.P if comm is not None else (dist.get_world_size(group) if dist.is_initialized() else 1)
        self.cuda = comm is not None
        self.side = torch.cuda.Stream() if self.cuda else None
        self.require_sync = True
        self.buckets: list[_Bucket] = []
        self._where = {}
        params = [p for p in module.parameters() if p.requires_grad]
        cap = max(1, bucket_bytes // 4)
        groups, cur, cur_n = [], [], 0
        for p in reversed(params):           # gradients become ready roughly in reverse order
            if cur and cur_n + p.numel() > cap:
                groups.append(cur)
                cur, cur_n = [], 0
            cur.append(p)
            cur_n += p.numel()
        if cur:
            groups.append(cur)
        for gi, ps in enumerate(groups):
            n = sum((p.numel() + 3) // 4 * 4 for p in ps)       # 16-byte aligned slots
            if self.cuda:
                acc, red = comm.empty(n, torch.float32), comm.empty(n, torch.float32)
                acc.zero_()
            else:
                dev = ps[0].device
                acc, red = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
            bk = _Bucket(gi, n, acc, red)
            off = 0
            for p in ps:
                self._where[p] = (bk, off)
                p.main_grad = bk.acc[off:off + p.numel()].view_as(p)
                p.reduced_grad = bk.red[off:off + p.numel()].view_as(p)
                bk.params.append(p)
                off += (p.numel() + 3) // 4 * 4
                p.register_post_accumulate_grad_hook(self._hook)
            bk.pending = len(ps)
            self.buckets.append(bk)
        self.stats = {"launched": 0}
        self._ev_bwd_end = self._ev_comm_end = None

    # ------------------------------------------------------------------ hooks
    def _hook(self, p):
        bk, _ = self._where[p]
        # the gradient is only queued here; the whole bucket is filled by ONE kernel when its last
        # gradient has arrived (bf16 / fp16 / fp32 -> fp32, overwrite or accumulate per parameter)
        bk.queued.append((p, p.grad))
        p.grad = None
        bk.pending -= 1
        if bk.pending == 0:
            self._fill(bk)
            if self.require_sync:
                self._reduce(bk)

    def _fill(self, bk: _Bucket):
        """Move the queued gradients into the bucket: fresh slots are overwritten (first micro-batch after
        ``zero_grad``, so the bucket needs no zero fill), the others accumulate in fp32."""
        if not bk.queued:
            return
        if self.cuda:
            from ..ops import fused
            fused.bucket_fill(bk.acc, [(g, self._where[p][1], p in bk.fresh) for p, g in bk.queued])
        else:
            for p, g in bk.queued:
                if p in bk.fresh:
                    p.main_grad.copy_(g)
                else:
                    p.main_grad.add_(g)
        for p, _ in bk.queued:
            bk.fresh.discard(p)
        bk.queued = []

    def _reduce(self, bk: _Bucket):
        scale = 1.0 / self.world
        self.stats["launched"] += 1
        if not self.cuda:
            bk.red.copy_(bk.acc)
            if self.world > 1:
                dist.all_reduce(bk.red, group=self.group)
            bk.red.mul_(scale)
            return
        if self.overlap:
            ev = torch.cuda.Event()
            ev.record()
            self.side.wait_event(ev)
            stream = self.side
        else:
            stream = None
        collectives.all_reduce(self.comm, bk.acc, out=bk.red, algo=self.algo, k=self.k, b=self.b, scale=scale,
                               nctas=self.comm_ctas, stream=stream)

    # ------------------------------------------------------------------ step protocol
    def forward(self, *a, **kw):
        return self.module(*a, **kw)

    __call__ = forward

    def finish(self):
        """Call after backward: waits for the bucket reductions and re-arms the hooks."""
        for bk in self.buckets:
            if bk.pending != 0:
                # some parameters received no gradient in this pass: take what arrived, and a slot that
                # is still fresh holds the previous step's values, so it counts as zero
                self._fill(bk)
                if self.require_sync:
                    for p in list(bk.fresh):
                        p.main_grad.zero_()
                    bk.fresh.clear()
                    self._reduce(bk)
        if self.cuda:
            self._ev_bwd_end = torch.cuda.Event(enable_timing=True)
            self._ev_bwd_end.record()
            if self.overlap:
                self._ev_comm_end = torch.cuda.Event(enable_timing=True)
                self._ev_comm_end.record(self.side)
                torch.cuda.current_stream().wait_stream(self.side)
        for bk in self.buckets:
            bk.pending = len(bk.params)

    def exposed_comm_ms(self) -> float:
        """Communication time not hidden behind backward in the last step (after a synchronize)."""
        if not (self.cuda and self.overlap and self._ev_comm_end is not None):
            return 0.0
        return max(0.0, self._ev_bwd_end.elapsed_time(self._ev_comm_end))

    def zero_grad(self):
        """Start a new accumulation: the first gradient written to a slot replaces its content."""
        for bk in self.buckets:
            bk.fresh = set(bk.params)

    def no_sync(self):
        """Context manager for gradient accumulation: bucket reductions are skipped; every backward pass
        inside still accumulates into the buckets (any number of micro-batches per context)."""
        ddp = self

        class _Ctx:
            def __enter__(self):
                ddp.require_sync = False

            def __exit__(self, *a):
                ddp.require_sync = True
                for bk in ddp.buckets:
                    ddp._fill(bk)                  # a pass that left some parameters without a gradient
                    bk.pending = len(bk.params)

        return _Ctx()

    def grads(self):
        return [(p, p.reduced_grad) for bk in self.buckets for p in bk.params]


class FusedMasterAdamW:
    """Same update as :class:`MasterAdamW` in one kernel per bucket: reduced fp32
    gradient -> AdamW on the fp32 master -> bf16 parameters, which are re-homed in
    one flat bf16 buffer per bucket (``csrc/kernels/fused_adam.cu``).  CUDA, bf16 parameters."""

    def __init__(self, ddp: DataParallel, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1):
        from ..ops import fused
        self._fused = fused
        self.ddp, self.lr, self.betas, self.eps, self.wd, self.t = ddp, lr, betas, eps, weight_decay, 0
        self.state = []
        for bk in ddp.buckets:
            flat_p = torch.zeros(bk.numel, dtype=torch.bfloat16, device=bk.red.device)
            master = torch.zeros_like(bk.red)
            off = 0
            for p in bk.params:
                assert p.dtype == torch.bfloat16, "the fused optimizer keeps bf16 parameters"
                flat_p[off:off + p.numel()].copy_(p.detach().reshape(-1))
                master[off:off + p.numel()].copy_(p.detach().reshape(-1).float())
                p.data = flat_p[off:off + p.numel()].view_as(p)
                off += (p.numel() + 3) // 4 * 4
            self.state.append((bk, flat_p, master, torch.zeros_like(master), torch.zeros_like(master)))

    @torch.no_grad()
    def step(self):
        self.t += 1
        for bk, flat_p, master, m, v in self.state:
            self._fused.adam_flat(bk.red, master, m, v, flat_p, lr=self.lr, betas=self.betas, eps=self.eps,
                                  weight_decay=self.wd, step=self.t)

    def state_dict(self) -> dict:
        return {"step": self.t, "buckets": [(ms.cpu().clone(), m.cpu().clone(), v.cpu().clone())
                                            for _, _, ms, m, v in self.state]}

    @torch.no_grad()
    def load_state_dict(self, sd: dict) -> None:
        self.t = int(sd["step"])
        for (_, flat_p, master, m, v), (sm, s1, s2) in zip(self.state, sd["buckets"]):
            master.copy_(sm)
            m.copy_(s1)
            v.copy_(s2)
            flat_p.copy_(master)


class MasterAdamW:
    """AdamW on fp32 master copies fed by the reduced fp32 gradients of a
    :class:`DataParallel`; the (bf16) model parameters are refreshed from the
    masters after every step.  One flat fp32 parameter per bucket, so the
    update is a handful of fused kernels whatever the number of layers."""

    def __init__(self, ddp: DataParallel, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1):
        self.ddp = ddp
        self.masters = []
        for bk in ddp.buckets:
            flat = torch.zeros_like(bk.red)
            off = 0
            for p in bk.params:
                flat[off:off + p.numel()].copy_(p.detach().reshape(-1).float())
                off += (p.numel() + 3) // 4 * 4
            flat = torch.nn.Parameter(flat)
            flat.grad = bk.red
            self.masters.append(flat)
        fused = ddp.cuda
        self.opt = torch.optim.AdamW(self.masters, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                     **({"fused": True} if fused else {}))

    @torch.no_grad()
    def step(self):
        self.opt.step()
        if not hasattr(self, "_dst"):
            self._dst, self._src = [], []
            for bk, flat in zip(self.ddp.buckets, self.masters):
                off = 0
                for p in bk.params:
                    self._dst.append(p)
                    self._src.append(flat[off:off + p.numel()].view_as(p))
                    off += (p.numel() + 3) // 4 * 4
        torch._foreach_copy_(self._dst, self._src)

    # ------------------------------------------------------------------ checkpoint / resume
    def state_dict(self) -> dict:
        return {"opt": self.opt.state_dict(), "masters": [m.detach().cpu().clone() for m in self.masters]}

    @torch.no_grad()
    def load_state_dict(self, sd: dict) -> None:
        for m, saved in zip(self.masters, sd["masters"]):
            m.copy_(saved)
        self.opt.load_state_dict(sd["opt"])
        for bk, flat in zip(self.ddp.buckets, self.masters):
            flat.grad = bk.red
            off = 0
            for p in bk.params:
                p.copy_(flat[off:off + p.numel()].view_as(p))
                off += (p.numel() + 3) // 4 * 4
