"""Tensor-level collectives: all_reduce, reduce_scatter, all_gather, all_to_all.

Every function takes a :class:`~..parallel.comm.Communicator` and either one
tensor (one rank per process) or a list of P tensors (emulated world), and an
``algo``:

``"auto"``
    pick by message size: the flagged-line one-shot kernel for latency-bound
    sizes, the NVLS ``multimem`` kernels for large symmetric buffers when the
    communicator has a multicast alias, the hierarchical radix-batch program
    with the tuned ``(k, b)`` otherwise (see ``utils/autotune.py``).
``"ll"``, ``"nvls"``
    force those kernels.
any name from ``list_algorithms(coll)``
    run that step program (``k`` / ``b`` as in the reference signatures:
    ``k`` = radix inside a group, ``b`` = group size;
    testing/custom_implementations/work_dir/all_reduce/all_reduce_radix_batch.cpp:202-204).

``scale`` multiplies the reduced values exactly once (fused into the kernel).
All launches are asynchronous on the current (or given) stream.
"""
from __future__ import annotations

import torch

import ctypes as C

from ..parallel.comm import Communicator, CollectiveError, DTYPES, OPS, _stream_ptr
from ..parallel.program import ProgramError
from ..utils import autotune
from .. import _native as N

LL_AR, LL_RS, LL_AG = 0, 1, 2


def _as_list(comm: Communicator, x):
    return [x] if isinstance(x, torch.Tensor) else list(x)


def _ret(comm: Communicator, xs):
    return xs if comm.nlocal > 1 else xs[0]


def _alloc_like(comm, ins, numel):
    return [torch.empty(numel, dtype=t.dtype, device=t.device) for t in ins]


def _ll_ok(comm, ins, outs, payload_bytes):
    if payload_bytes > comm.ll_max_bytes:
        return False
    return all((t.data_ptr() % 8) == 0 for t in ins + outs)


# kernels and programs that take an allreduce of any length; every other schedule cuts the vector into P slices
_ANY_COUNT = ("ll", "ll2", "nvls", "nvls1", "recursive_doubling", "ring", "k_reduce_scatter_allgather",
              "recursive_multiplying", "recursive_exchange", "inter_reduce_exchange_bcast")


def any_count(coll: str, algo: str, k: int, b: int, count: int, P: int, ll_ok: bool, payload_bytes: int = 0):
    """The tuned table and the fallback rule are made from vectors whose length is a multiple of the number of
    ranks.  An allreduce of any other length keeps the choice only if that kernel takes any length; otherwise it
    runs on the one-shot line kernel up to 256 KiB (if the message fits its inbox), as recursive doubling
    (whole-vector exchanges, few rounds) up to 1 MiB and as the ring (bandwidth-optimal, ragged chunks) above."""
    if coll != "allreduce" or P <= 1 or count % P == 0 or algo.split(":")[0] in _ANY_COUNT:
        return algo, k, b
    if ll_ok and payload_bytes <= (256 << 10):      # one-shot: every rank sends the whole vector to every peer
        return "ll", 2, 1
    return ("recursive_doubling", 2, 1) if payload_bytes <= (1 << 20) else ("ring", 2, 1)


_COLL = {"allreduce": 0, "reduce_scatter": 1, "allgather": 2, "alltoall": 3, "gather": 4, "phase": 5}
_ALGO_BYTES: dict = {}
_NVTX = __import__("os").environ.get("CHB_NVTX", "0") == "1"   # NVTX range around every launch


def _run(comm: Communicator, coll: str, ins, outs, count: int, op, algo, k, b, aux, scale, nctas, stream,
         payload_bytes: int, ll_mode: int):
    """Pick the kernel and enqueue it with a single native call."""
    auto = algo == "auto"
    if auto:
        sym = comm.is_symmetric(ins[0]) and comm.is_symmetric(outs[0])
        key = (coll, payload_bytes, ins[0].dtype, sym)
        choice = comm._choices.get(key)
        if choice is None:
            choice = autotune.choose(comm, coll, payload_bytes, ins[0].dtype, sym)
            comm._choices[key] = choice
        algo, k, b = choice.algo, choice.k, choice.b
        if nctas == 0:
            nctas = choice.nctas
        if algo == "ll" and not _ll_ok(comm, ins, outs, payload_bytes):
            algo, k, b = "radix_batch", 2, 1
        elif algo == "ll2" and not (payload_bytes <= comm.ll2_max_bytes and _ll_ok(comm, ins, outs, 0)):
            algo, k, b = "radix_batch", 2, 1
        elif algo.startswith("nvls") and not (comm.has_multicast and sym and comm.nlocal == 1
                                              and payload_bytes % 16 == 0):
            algo, k, b = "radix_batch", 2, 1
        if coll == "allreduce" and count % comm.P:
            algo, k, b = any_count(coll, algo, k, b, count, comm.P, _ll_ok(comm, ins, outs, payload_bytes), payload_bytes)
    if algo == "bulk" and not (coll == "allgather" and payload_bytes % 16 == 0 and comm.is_symmetric(ins[0])
                               and all(t.data_ptr() % 16 == 0 for t in ins + outs)):
        algo, k, b = "radix_batch", 2, 1      # the bulk-copy engine needs 16-byte granularity and a peer-visible input
    if coll == "alltoall" and algo == "radix_batch":
        algo = "tuna"
    ab = _ALGO_BYTES.get(algo)
    if ab is None:
        ab = _ALGO_BYTES[algo] = algo.encode()
    n = len(ins)
    if _NVTX:
        torch.cuda.nvtx.range_push(f"chb.{coll}.{algo}[{payload_bytes}B]")
    rc = N.lib().chb_collective(comm._h, _COLL[coll], ab, k, b, aux, DTYPES[ins[0].dtype], OPS[op],
                                (C.c_void_p * n)(*[t.data_ptr() for t in ins]),
                                (C.c_void_p * n)(*[t.data_ptr() for t in outs]),
                                count, scale, nctas, _stream_ptr(stream))
    if rc == N.ERR_COUNT and auto and algo.endswith(":ll"):
        # the tuned row was measured with a larger flagged-line inbox than this communicator has: same program, pulled
        ab = (algo[:-3] + ":pull").encode()
        rc = N.lib().chb_collective(comm._h, _COLL[coll], ab, k, b, aux, DTYPES[ins[0].dtype], OPS[op],
                                    (C.c_void_p * n)(*[t.data_ptr() for t in ins]),
                                    (C.c_void_p * n)(*[t.data_ptr() for t in outs]),
                                    count, scale, nctas, _stream_ptr(stream))
    if _NVTX:
        torch.cuda.nvtx.range_pop()
    if rc:
        comm._err(rc)
    comm.launches += 1


def all_reduce(comm: Communicator, x, out=None, op: str = "sum", algo: str = "auto", k: int = 2, b: int = 1,
               aux: int = 0, scale: float = 1.0, nctas: int = 0, stream=None):
    """out[i] = scale * (x_0[i] op x_1[i] op ... op x_{P-1}[i]) on every rank."""
    ins = _as_list(comm, x)
    n = ins[0].numel()
    outs = _as_list(comm, out) if out is not None else _alloc_like(comm, ins, n)
    _run(comm, "allreduce", ins, outs, n, op, algo, k, b, aux, scale, nctas, stream, n * ins[0].element_size(), LL_AR)
    return _ret(comm, outs)


def reduce_scatter(comm: Communicator, x, out=None, op: str = "sum", algo: str = "auto", k: int = 2, b: int = 1,
                   aux: int = 0, scale: float = 1.0, nctas: int = 0, stream=None):
    """x holds P blocks of n elements; rank r receives the reduction of block r."""
    ins = _as_list(comm, x)
    total = ins[0].numel()
    if total % comm.P:
        raise CollectiveError(N.ERR_COUNT, "reduce_scatter input length must be a multiple of the number of ranks")
    n = total // comm.P
    outs = _as_list(comm, out) if out is not None else _alloc_like(comm, ins, n)
    _run(comm, "reduce_scatter", ins, outs, n, op, algo, k, b, aux, scale, nctas, stream, n * ins[0].element_size(), LL_RS)
    return _ret(comm, outs)


def all_gather(comm: Communicator, x, out=None, algo: str = "auto", k: int = 2, b: int = 1, aux: int = 0,
               nctas: int = 0, stream=None):
    """Every rank contributes n elements; out holds the P blocks in rank order."""
    ins = _as_list(comm, x)
    n = ins[0].numel()
    outs = _as_list(comm, out) if out is not None else _alloc_like(comm, ins, n * comm.P)
    _run(comm, "allgather", ins, outs, n, "sum", algo, k, b, aux, 1.0, nctas, stream, n * ins[0].element_size(), LL_AG)
    return _ret(comm, outs)


def all_to_all(comm: Communicator, x, out=None, algo: str = "tuna", k: int = 2, b: int = 1, nctas: int = 0, stream=None):
    """Block s of rank r's output is block r of rank s's input (equal block sizes)."""
    ins = _as_list(comm, x)
    total = ins[0].numel()
    if total % comm.P:
        raise CollectiveError(N.ERR_COUNT, "all_to_all input length must be a multiple of the number of ranks")
    n = total // comm.P
    outs = _as_list(comm, out) if out is not None else _alloc_like(comm, ins, total)
    if algo == "auto":
        algo = "linear"
    _run(comm, "alltoall", ins, outs, n, "sum", algo, k, b, 0, 1.0, nctas, stream, 1 << 62, LL_AG)
    return _ret(comm, outs)


def gather(comm: Communicator, x, root: int = 0, out=None, k: int = 2, nctas: int = 0, stream=None):
    """k-nomial gather of one block per rank to ``root`` (other ranks' out is scratch)."""
    ins = _as_list(comm, x)
    n = ins[0].numel()
    outs = _as_list(comm, out) if out is not None else _alloc_like(comm, ins, n * comm.P)
    _run(comm, "gather", ins, outs, n, "sum", "k_nomial", k, 1, root, 1.0, nctas, stream, 1 << 62, LL_AG)
    return _ret(comm, outs)


def phase(comm: Communicator, name: str, x, count: int, k: int = 2, b: int = 1, op: str = "sum", out=None,
          nctas: int = 0, stream=None):
    """One phase of the hierarchical collectives as a call of its own (``name``: see
    ``list_algorithms("phase")``), with the buffer layouts of the reference's stand-alone phase
    functions (testing/custom_implementations/work_dir/reduce_scatter/intra_reduce_scatter_radix.cpp:208,
    inter_linear_reduce.cpp:11, intra_scatter_radix_batch.cpp:11,
    all_gather/outdated_versions/all_gather_0_3_beta.cpp:36,141,377).  Output entries that the phase does
    not define (non-root ranks, missing stages) are left as they were."""
    from ..parallel.program import cached_program

    prog = cached_program("phase", name, comm.P, count, k, b)
    ins = _as_list(comm, x)
    if ins[0].numel() != prog.in_elems:
        raise ValueError(f"{name}: input must hold {prog.in_elems} elements")
    outs = _as_list(comm, out) if out is not None else _alloc_like(comm, ins, prog.out_elems)
    _run(comm, "phase", ins, outs, count, op, name, k, b, 0, 1.0, nctas, stream, 1 << 62, LL_AG)
    return _ret(comm, outs)


# ---- reference call signatures (count-based, explicit output) ---------------------------
def allgather_radix_batch(sendbuf, sendcount: int, recvbuf, comm: Communicator, k: int, b: int, stream=None) -> int:
    """Counterpart of ``allgather_radix_batch(sendbuf, sendcount, datatype, recvbuf, comm, k, b)``
    (testing/custom_implementations/work_dir/all_gather/all_gather_radix_batch_1_0.cpp:37);
    the datatype comes from the tensors.  Returns 0 or an error code."""
    return _guard(lambda: all_gather(comm, _narrow(sendbuf, sendcount), _narrow(recvbuf, sendcount * comm.P),
                                     algo="radix_batch", k=k, b=b, stream=stream))


def reduce_scatter_radix_batch(sendbuf, recvbuf, recvcount: int, op: str, comm: Communicator, k: int, b: int,
                               stream=None) -> int:
    """Counterpart of ``reduce_scatter_radix_batch(sendbuf, recvbuf, recvcount, datatype, op, comm, k, b)``
    (testing/custom_implementations/work_dir/reduce_scatter/reduce_scatter_radix_batch.cpp:200-202).
    ``sendbuf=None`` means in place (input taken from ``recvbuf``, which then holds P*recvcount elements)."""
    if sendbuf is None:
        return _guard(lambda: _rs_in_place(comm, recvbuf, recvcount, op, k, b, stream))
    return _guard(lambda: reduce_scatter(comm, _narrow(sendbuf, recvcount * comm.P), _narrow(recvbuf, recvcount),
                                         op=op, algo="radix_batch", k=k, b=b, stream=stream))


def all_reduce_radix_batch(sendbuf, recvbuf, count: int, op: str, comm: Communicator, k: int, b: int, stream=None) -> int:
    """Counterpart of ``all_reduce_radix_batch(sendbuf, recvbuf, count, datatype, op, comm, k, b)``
    (testing/custom_implementations/work_dir/all_reduce/all_reduce_radix_batch.cpp:202-204).
    ``sendbuf=None`` means in place.  ``count`` must be a multiple of the number of ranks."""
    src = recvbuf if sendbuf is None else sendbuf
    return _guard(lambda: all_reduce(comm, _narrow(src, count), _narrow(recvbuf, count), op=op,
                                     algo="radix_batch", k=k, b=b, stream=stream))


def _rs_in_place(comm, recvbuf, recvcount, op, k, b, stream):
    bufs = _as_list(comm, recvbuf)
    tmp = [t[: recvcount * comm.P].clone() for t in bufs]
    reduce_scatter(comm, _ret(comm, tmp), _narrow(recvbuf, recvcount), op=op, algo="radix_batch", k=k, b=b, stream=stream)


def _narrow(x, n):
    if isinstance(x, torch.Tensor):
        return x.view(-1)[:n]
    return [t.view(-1)[:n] for t in x]


def _guard(fn) -> int:
    try:
        fn()
        return N.SUCCESS
    except ProgramError as e:
        msg = str(e)
        return N.ERR_COUNT if "count" in msg else N.ERR_ARG
    except CollectiveError as e:
        return e.code
