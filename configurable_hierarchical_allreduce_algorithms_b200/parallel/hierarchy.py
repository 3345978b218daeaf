"""Two physical levels: several NVSwitch domains (boxes) joined by a host network.

Inside one box every collective is a single kernel over peer memory
(:class:`DeviceLevel`).  Across boxes the ranks with the same local index form
a *lane*, exactly the inter-group lanes of the reference's hierarchical
algorithms with ``b`` = ranks per box
(testing/custom_implementations/work_dir/all_reduce/all_reduce_radix_batch.cpp:489-573 for the
lane phase, :247-480 for the intra-group phase): lane traffic goes through
``torch.distributed`` - its own collectives (:class:`LibraryLevel`: NCCL between GPUs of
different boxes, gloo between hosts) or any step program replayed with
two-sided messages (:class:`GlooLevel`, which is how the reference runs every phase).

:class:`TwoLevel` composes one level of each kind::

    allreduce       = intra reduce-scatter -> lane allreduce      -> intra allgather
    reduce-scatter  = intra reduce-scatter of the lane-major view -> lane reduce-scatter
    allgather       = lane allgather       -> intra allgather     -> group-major view

Global rank ``r`` lives in box ``r // L`` with local index ``r % L`` (``L`` ranks per box),
the reference's ``node_id = rank / b`` and ``node_rank = rank % b``
(testing/custom_implementations/work_dir/all_gather/all_gather_radix_batch_1_0.cpp:45-48).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

_RED = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}


def split_world(local_size: int, backend: str | None = None):
    """Create the box group and the lane group of the calling rank.

    Every rank of the default group must call this (``dist.new_group`` is
    collective).  Returns ``(intra_group, inter_group)``.
    """
    world, rank = dist.get_world_size(), dist.get_rank()
    if local_size < 1 or world % local_size:
        raise ValueError(f"ranks per box ({local_size}) must divide the number of ranks ({world})")
    boxes = world // local_size
    intra = inter = None
    for g in range(boxes):
        grp = dist.new_group(list(range(g * local_size, (g + 1) * local_size)), backend=backend)
        if rank // local_size == g:
            intra = grp
    for l in range(local_size):
        grp = dist.new_group(list(range(l, world, local_size)), backend=backend)
        if rank % local_size == l:
            inter = grp
    return intra, inter


class LibraryLevel:
    """One level run by ``torch.distributed``'s own collectives on the tensors' device."""

    def __init__(self, group=None):
        self.group = group if group is not None else dist.group.WORLD
        self.P = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)

    def all_reduce(self, x: torch.Tensor, op: str = "sum") -> torch.Tensor:
        y = x.clone()
        if self.P > 1:
            dist.all_reduce(y, op=_RED[op], group=self.group)
        return y

    def reduce_scatter(self, x: torch.Tensor, op: str = "sum") -> torch.Tensor:
        n = x.numel() // self.P
        if self.P == 1:
            return x.clone()
        if x.is_cuda:
            y = torch.empty(n, dtype=x.dtype, device=x.device)
            dist.reduce_scatter_tensor(y, x.contiguous(), op=_RED[op], group=self.group)
            return y
        y = self.all_reduce(x, op)     # gloo has no reduce-scatter
        return y[self.rank * n:(self.rank + 1) * n].clone()

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        if self.P == 1:
            return x.clone()
        y = torch.empty(x.numel() * self.P, dtype=x.dtype, device=x.device)
        if x.is_cuda:
            dist.all_gather_into_tensor(y, x.contiguous(), group=self.group)
        else:
            dist.all_gather(list(y.view(self.P, -1).unbind(0)), x.contiguous(), group=self.group)
        return y


class GlooLevel:
    """One level run as a step program over two-sided messages between CPU copies.

    Device tensors are staged through host memory, which is what an inter-box
    lane without GPU-direct networking does anyway.
    """

    def __init__(self, group=None, algo: str = "radix_batch", k: int = 2, b: int = 1):
        self.group = group if group is not None else dist.group.WORLD
        self.P = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.algo, self.k, self.b = algo, k, b

    def _run(self, coll, x, count, op="sum"):
        from . import gloo_exec

        if self.P == 1:
            return x.clone()
        host = x.detach().to("cpu").contiguous()
        y = gloo_exec.run_collective(coll, self.algo, host, count, self.k, self.b, op=op, group=self.group)
        return y.to(x.device)

    def all_reduce(self, x, op="sum"):
        n = x.numel()
        pad = (-n) % self.P        # the hierarchical allreduce wants a multiple of the number of ranks
        if pad:
            x = torch.cat([x, x.new_zeros(pad)])
        return self._run("allreduce", x, x.numel(), op)[:n]

    def reduce_scatter(self, x, op="sum"):
        return self._run("reduce_scatter", x, x.numel() // self.P, op)

    def all_gather(self, x):
        return self._run("allgather", x, x.numel())


class DeviceLevel:
    """One level run by the GPU kernels of a :class:`~.comm.Communicator` (one rank per process)."""

    def __init__(self, comm, algo: str = "auto", k: int = 2, b: int = 1):
        self.comm = comm
        self.P, self.rank = comm.P, comm.rank
        self.algo, self.k, self.b = algo, k, b

    def all_reduce(self, x, op="sum"):
        from ..ops import collectives as ops

        return ops.all_reduce(self.comm, x, op=op, algo=self.algo, k=self.k, b=self.b)

    def reduce_scatter(self, x, op="sum"):
        from ..ops import collectives as ops

        return ops.reduce_scatter(self.comm, x, op=op, algo=self.algo, k=self.k, b=self.b)

    def all_gather(self, x):
        from ..ops import collectives as ops

        return ops.all_gather(self.comm, x, algo=self.algo, k=self.k, b=self.b)


class TwoLevel:
    """Collectives over ``boxes x ranks-per-box`` ranks from an intra-box and a lane level.

    ``intra`` and ``inter`` are any of :class:`DeviceLevel`, :class:`LibraryLevel`,
    :class:`GlooLevel` (anything with ``P``, ``rank``, ``all_reduce``, ``reduce_scatter``,
    ``all_gather``).  Block order of reduce-scatter inputs and allgather outputs is by
    global rank ``box * L + local``.
    """

    def __init__(self, intra, inter):
        self.intra, self.inter = intra, inter
        self.L, self.G = intra.P, inter.P
        self.P = self.L * self.G
        self.rank = inter.rank * self.L + intra.rank

    def all_reduce(self, x: torch.Tensor, op: str = "sum") -> torch.Tensor:
        shape, x = x.shape, x.contiguous().view(-1)
        n = x.numel()
        pad = (-n) % self.L
        if pad:
            x = torch.cat([x, x.new_zeros(pad)])
        part = self.intra.reduce_scatter(x, op)        # my slice, reduced over my box
        part = self.inter.all_reduce(part, op)         # ... and over the boxes
        return self.intra.all_gather(part)[:n].view(shape)

    def reduce_scatter(self, x: torch.Tensor, op: str = "sum") -> torch.Tensor:
        x = x.contiguous().view(-1)
        if x.numel() % self.P:
            raise ValueError("reduce-scatter input must hold one block per rank")
        n = x.numel() // self.P
        # lane-major view: the blocks for local index l of every box become contiguous
        y = x.view(self.G, self.L, n).transpose(0, 1).contiguous().view(-1)
        part = self.intra.reduce_scatter(y, op)        # [G, n]: partial sums for (every box, my local index)
        return self.inter.reduce_scatter(part, op)     # [n]: block of (my box, my local index)

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        x = x.contiguous().view(-1)
        n = x.numel()
        lane = self.inter.all_gather(x)                # [G, n]: my local index in every box
        full = self.intra.all_gather(lane)             # [L, G, n]
        return full.view(self.L, self.G, n).transpose(0, 1).contiguous().view(-1)
