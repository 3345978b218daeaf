"""Collectives on host buffers, the memory space the reference works in
(its ``sendbuf`` / ``recvbuf`` are host arrays handed to MPI, e.g.
testing/custom_implementations/work_dir/all_reduce/main.cpp:43-76).

The vector is cut into chunks that flow through three stages on three streams:
pinned host -> device copy, the collective on registered (peer-visible) device
buffers, device -> pinned host copy.  The two copy directions use different copy
engines and PCIe is full duplex, so a long vector costs about one direction's
transfer time instead of the sum of upload, collective and download.
"""
from __future__ import annotations

import torch

from ..parallel.comm import Communicator
from . import collectives as ops


class HostAllReduce:
    """Reusable pipeline for allreduces of pinned host tensors of one dtype.

    ``chunk_elems`` elements per chunk, ``depth`` chunks in flight (device memory:
    ``2 * depth * chunk`` from the communicator's registered region).  One rank per
    process (or a world of one rank).
    """

    def __init__(self, comm: Communicator, dtype=torch.float32, chunk_elems: int = 16 << 20, depth: int = 3):
        if comm.nlocal != 1:
            raise ValueError("host pipelines need one rank per process")
        self.comm, self.dtype, self.chunk, self.depth = comm, dtype, int(chunk_elems), int(depth)
        self.xin = [comm.empty(self.chunk, dtype) for _ in range(depth)]
        self.yout = [comm.empty(self.chunk, dtype) for _ in range(depth)]
        self.s_in, self.s_out = torch.cuda.Stream(), torch.cuda.Stream()
        self.h2d = [torch.cuda.Event() for _ in range(depth)]
        self.done = [torch.cuda.Event() for _ in range(depth)]
        self.d2h = [torch.cuda.Event() for _ in range(depth)]
        self.h2d_bytes = self.d2h_bytes = 0

    def __call__(self, hx: torch.Tensor, hy: torch.Tensor | None = None, op: str = "sum", scale: float = 1.0,
                 algo: str = "auto", k: int = 2, b: int = 1) -> torch.Tensor:
        """hy = scale * allreduce(hx); both pinned host tensors.  Returns hy once every copy has been
        enqueued: synchronise the current stream before reading it."""
        if hx.is_cuda or hx.dtype != self.dtype:
            raise ValueError("input must be a host tensor of the pipeline's dtype")
        if hy is None:
            hy = torch.empty_like(hx).pin_memory()
        hx1, hy1 = hx.view(-1), hy.view(-1)
        n = hx1.numel()
        main = torch.cuda.current_stream()
        self.s_in.wait_stream(main)          # earlier work of the caller that produced hx / reads hy
        self.s_out.wait_stream(main)
        nchunks = (n + self.chunk - 1) // self.chunk
        for c in range(nchunks):
            a, e = c * self.chunk, min(n, (c + 1) * self.chunk)
            m, slot = e - a, c % self.depth
            if c >= self.depth:
                self.s_in.wait_event(self.done[slot])      # the collective has consumed this input slot
            with torch.cuda.stream(self.s_in):
                self.xin[slot][:m].copy_(hx1[a:e], non_blocking=True)
                self.h2d[slot].record(self.s_in)
            main.wait_event(self.h2d[slot])
            if c >= self.depth:
                main.wait_event(self.d2h[slot])            # the download has drained this output slot
            ops.all_reduce(self.comm, self.xin[slot][:m], out=self.yout[slot][:m], op=op, scale=scale, algo=algo, k=k, b=b)
            self.done[slot].record(main)
            self.s_out.wait_event(self.done[slot])
            with torch.cuda.stream(self.s_out):
                hy1[a:e].copy_(self.yout[slot][:m], non_blocking=True)
                self.d2h[slot].record(self.s_out)
        main.wait_stream(self.s_out)
        main.wait_stream(self.s_in)
        self.h2d_bytes += n * hx.element_size()
        self.d2h_bytes += n * hx.element_size()
        return hy


def all_reduce_host(comm: Communicator, hx: torch.Tensor, hy: torch.Tensor | None = None, op: str = "sum",
                    scale: float = 1.0, chunk_elems: int = 16 << 20, depth: int = 3, **kw) -> torch.Tensor:
    """One-off form of :class:`HostAllReduce`; the pipeline is cached on the communicator per
    (dtype, chunk, depth) so repeated calls reuse its device buffers."""
    cache = comm.__dict__.setdefault("_host_pipelines", {})
    key = (hx.dtype, int(chunk_elems), int(depth))
    pipe = cache.get(key)
    if pipe is None:
        pipe = cache[key] = HostAllReduce(comm, hx.dtype, chunk_elems, depth)
    return pipe(hx, hy, op=op, scale=scale, **kw)
