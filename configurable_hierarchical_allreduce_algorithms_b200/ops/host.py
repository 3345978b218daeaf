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
    """Reusable pipeline for collectives on pinned host tensors of one dtype (allreduce by call,
    :meth:`reduce_scatter` and :meth:`all_gather` as methods).

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

        def upload(slot, a, e):
            self.xin[slot][:e - a].copy_(hx1[a:e], non_blocking=True)

        def collective(slot, m):
            ops.all_reduce(self.comm, self.xin[slot][:m], out=self.yout[slot][:m], op=op, scale=scale, algo=algo, k=k, b=b)

        def download(slot, a, e):
            hy1[a:e].copy_(self.yout[slot][:e - a], non_blocking=True)

        self._pipeline(n, self.chunk, upload, collective, download)
        self.h2d_bytes += n * hx.element_size()
        self.d2h_bytes += n * hx.element_size()
        return hy

    def _pipeline(self, n, m_max, upload, collective, download):
        """Chunks [a, e) of at most m_max elements through upload (side stream), collective (current
        stream) and download (other side stream); a slot is reused only when its previous user is done."""
        main = torch.cuda.current_stream()
        self.s_in.wait_stream(main)          # earlier work of the caller that produced the input / reads the output
        self.s_out.wait_stream(main)
        for c in range((n + m_max - 1) // m_max):
            a, e = c * m_max, min(n, (c + 1) * m_max)
            slot = c % self.depth
            if c >= self.depth:
                self.s_in.wait_event(self.done[slot])      # the collective has consumed this input slot
            with torch.cuda.stream(self.s_in):
                upload(slot, a, e)
                self.h2d[slot].record(self.s_in)
            main.wait_event(self.h2d[slot])
            if c >= self.depth:
                main.wait_event(self.d2h[slot])            # the download has drained this output slot
            collective(slot, e - a)
            self.done[slot].record(main)
            self.s_out.wait_event(self.done[slot])
            with torch.cuda.stream(self.s_out):
                download(slot, a, e)
                self.d2h[slot].record(self.s_out)
        main.wait_stream(self.s_out)
        main.wait_stream(self.s_in)

    # ---- the other two collectives: block structure kept by 2-D copies
    def reduce_scatter(self, hx: torch.Tensor, hy: torch.Tensor | None = None, op: str = "sum", scale: float = 1.0,
                       algo: str = "auto", k: int = 2, b: int = 1) -> torch.Tensor:
        """hx: P blocks of n elements (pinned host); hy: this rank's reduced block of n elements."""
        P = self.comm.P
        n = hx.numel() // P
        if hx.numel() != n * P or n == 0:
            raise ValueError("reduce-scatter input must hold one non-empty block per rank")
        if hy is None:
            hy = torch.empty(n, dtype=hx.dtype).pin_memory()
        hx2, hy1 = hx.view(P, n), hy.view(-1)
        m_max = self.chunk // P
        if m_max < 1:
            raise ValueError("chunk smaller than one element per rank")

        def upload(slot, a, e):
            self.xin[slot][:P * (e - a)].view(P, e - a).copy_(hx2[:, a:e], non_blocking=True)

        def collective(slot, m):
            ops.reduce_scatter(self.comm, self.xin[slot][:P * m], out=self.yout[slot][:m], op=op, scale=scale, algo=algo, k=k, b=b)

        def download(slot, a, e):
            hy1[a:e].copy_(self.yout[slot][:e - a], non_blocking=True)

        self._pipeline(n, m_max, upload, collective, download)
        self.h2d_bytes += hx.numel() * hx.element_size()
        self.d2h_bytes += n * hx.element_size()
        return hy

    def all_gather(self, hx: torch.Tensor, hy: torch.Tensor | None = None, algo: str = "auto", k: int = 2,
                   b: int = 1) -> torch.Tensor:
        """hx: this rank's n elements (pinned host); hy: the P blocks in rank order."""
        P = self.comm.P
        n = hx.numel()
        if n == 0:
            raise ValueError("allgather input must not be empty")
        if hy is None:
            hy = torch.empty(n * P, dtype=hx.dtype).pin_memory()
        hx1, hy2 = hx.view(-1), hy.view(P, n)
        m_max = self.chunk // P
        if m_max < 1:
            raise ValueError("chunk smaller than one element per rank")

        def upload(slot, a, e):
            self.xin[slot][:e - a].copy_(hx1[a:e], non_blocking=True)

        def collective(slot, m):
            ops.all_gather(self.comm, self.xin[slot][:m], out=self.yout[slot][:P * m], algo=algo, k=k, b=b)

        def download(slot, a, e):
            hy2[:, a:e].copy_(self.yout[slot][:P * (e - a)].view(P, e - a), non_blocking=True)

        self._pipeline(n, m_max, upload, collective, download)
        self.h2d_bytes += n * hx.element_size()
        self.d2h_bytes += n * P * hx.element_size()
        return hy


def all_reduce_host(comm: Communicator, hx: torch.Tensor, hy: torch.Tensor | None = None, op: str = "sum",
                    scale: float = 1.0, chunk_elems: int = 16 << 20, depth: int = 3, **kw) -> torch.Tensor:
    """One-off form of :class:`HostAllReduce`; the pipeline is cached on the communicator per
    (dtype, chunk, depth) so repeated calls reuse its device buffers."""
    cache = comm._host_pipelines
    key = (hx.dtype, int(chunk_elems), int(depth))
    pipe = cache.get(key)
    if pipe is None:
        pipe = cache[key] = HostAllReduce(comm, hx.dtype, chunk_elems, depth)
    return pipe(hx, hy, op=op, scale=scale, **kw)
