"""Execute a step program with one process per rank over ``torch.distributed``
point-to-point messages (gloo on CPU tensors).

This is the host-side level of the hierarchy and the CPU plumbing path: the
same schedule that the GPU interpreter runs is replayed with two-sided
messages, which is how the reference runs everything
(``MPI_Isend / MPI_Irecv / MPI_Waitall / MPI_Reduce_local``, e.g.
testing/custom_implementations/work_dir/all_reduce/all_reduce_radix_batch.cpp:353-364).

A pull step ``dst = src_0 op src_1 ...`` executed by rank r in round t turns,
for every remote source, into a send posted by the owning peer at the start of
*its* round t and a receive posted by r; message matching replaces the device
flags.  Within a pair, messages are matched by an explicit running tag.
"""
from __future__ import annotations

from collections import defaultdict

import torch
import torch.distributed as dist

from .program import BUF_IN, BUF_OUT, BUF_WORK, Program

_REDUCE = {
    "sum": lambda a, b: a.add_(b),
    "max": lambda a, b: torch.maximum(a, b, out=a),
    "min": lambda a, b: torch.minimum(a, b, out=a),
    "prod": lambda a, b: a.mul_(b),
}


class GlooExecutor:
    def __init__(self, prog: Program, group=None):
        self.prog = prog
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        assert dist.get_world_size(self.group) == prog.P, "program compiled for a different world size"
        ops, srcs, *_ = prog.tables()
        # per round: my steps, and what I have to serve to peers
        self.my_steps = defaultdict(list)     # round -> [(op_index, op_row, [(peer, buf, off)])]
        self.serve = defaultdict(list)        # round -> [(dst_rank, buf, off, count, tag_key)]
        for i, o in enumerate(ops):
            rank, rnd, _, _, count, _, sb, ns = (int(v) for v in o)
            ss = [(int(p), int(b), int(f)) for p, b, f in srcs[sb:sb + ns]]
            if rank == self.rank:
                self.my_steps[rnd].append((i, o, ss))
            else:
                for j, (p, b, f) in enumerate(ss):
                    if p == self.rank:
                        self.serve[rnd].append((rank, b, f, count, (i, j)))
        self.nrounds = prog.nrounds

    def _glob(self, r: int) -> int:
        return dist.get_global_rank(self.group, r) if self.group is not dist.group.WORLD else r

    def run(self, x: torch.Tensor, out: torch.Tensor | None = None, op: str = "sum") -> torch.Tensor:
        p = self.prog
        x = x.contiguous().view(-1)
        assert x.numel() == p.in_elems
        if out is None:
            out = torch.empty(p.out_elems, dtype=x.dtype)
        work = torch.empty(max(p.work_elems, 1), dtype=x.dtype)
        bufs = {BUF_IN: x, BUF_OUT: out.view(-1), BUF_WORK: work}
        red = _REDUCE[op]
        tags = defaultdict(int)  # (src, dst) -> running tag, advanced identically on both sides
        for t in range(self.nrounds):
            reqs, recvd = [], {}
            # both sides enumerate messages in (op index, source index) order
            sends = sorted(self.serve.get(t, []), key=lambda s: s[4])
            for (dst, b, f, count, _key) in sends:
                tag = tags[(self.rank, dst)]
                tags[(self.rank, dst)] += 1
                reqs.append(dist.isend(bufs[b][f:f + count], self._glob(dst), group=self.group, tag=tag))
            for (i, o, ss) in self.my_steps.get(t, []):
                count = int(o[4])
                for j, (peer, b, f) in enumerate(ss):
                    if peer != self.rank:
                        tmp = torch.empty(count, dtype=x.dtype)
                        tag = tags[(peer, self.rank)]
                        tags[(peer, self.rank)] += 1
                        reqs.append(dist.irecv(tmp, self._glob(peer), group=self.group, tag=tag))
                        recvd[(i, j)] = tmp
            for r in reqs:
                r.wait()
            for (i, o, ss) in self.my_steps.get(t, []):
                _, _, dbuf, doff, count, acc = (int(v) for v in o[:6])
                dst = bufs[dbuf][doff:doff + count]
                parts = [recvd[(i, j)] if peer != self.rank else bufs[b][f:f + count]
                         for j, (peer, b, f) in enumerate(ss)]
                if acc:
                    val = dst
                    rest = parts
                else:
                    val = parts[0].clone()
                    rest = parts[1:]
                for q in rest:
                    red(val, q)
                if not acc:
                    dst.copy_(val)
        return out


_EXECUTORS: dict = {}     # (program, group) -> executor with its per-round send / receive lists already built


def run_collective(coll: str, algo: str, x: torch.Tensor, count: int, k: int = 2, b: int = 1, aux: int = 0,
                   op: str = "sum", group=None) -> torch.Tensor:
    """Compile (cached per process) and execute one collective on CPU tensors."""
    from .program import cached_program

    P = dist.get_world_size(group if group is not None else dist.group.WORLD)
    prog = cached_program(coll, algo, P, count, k, b, aux, False, False)
    key = (id(prog), id(group))         # both objects stay alive (program cache / caller's group), so ids are stable
    ex = _EXECUTORS.get(key)
    if ex is None:
        if len(_EXECUTORS) > 256:
            _EXECUTORS.clear()
        ex = _EXECUTORS[key] = GlooExecutor(prog, group)
    return ex.run(x, op=op)
