"""Communicator: the symmetric heaps of P ranks plus the kernels that run on them.

Two flavours share every code path below the constructor:

* ``Communicator.emulated(P)`` — all P ranks live on ONE GPU (P slices of one
  allocation, one cooperative launch executes every rank).  Used by the
  single-GPU tests and for developing schedules without a multi-GPU box.
* ``Communicator.from_process_group(group)`` — one rank per process / GPU over
  NVLink; heaps are exchanged either as cudaIpc handles (``backend="ipc"``,
  native) or through ``torch.distributed._symmetric_memory``
  (``backend="symm_mem"``), which also yields the NVLS multicast alias used by
  the ``multimem`` kernels.

The reference has no counterpart of this object: its "communicator" is an
``MPI_Comm`` and all buffers are host memory
(testing/custom_implementations/work_dir/all_gather/all_gather_radix_batch_1_0.cpp:37-64).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Sequence

import torch

from .. import _native as N
from .program import Program, cached_program

vp, i32, i64, u64, f32 = C.c_void_p, C.c_int, C.c_int64, C.c_uint64, C.c_float
N.optional("chb_heap_bytes", C.c_size_t, [i32, C.c_size_t, C.c_size_t, C.c_size_t])
N.optional("chb_comm_create", vp, [i32, i32, i32, C.POINTER(vp), vp, C.c_size_t, C.c_size_t, C.c_size_t, C.c_char_p, i32])
N.optional("chb_comm_destroy", None, [vp])
N.optional("chb_comm_last_error", C.c_char_p, [vp])
N.optional("chb_comm_set_timeout_us", i32, [vp, u64])
N.optional("chb_comm_info", i32, [vp, C.POINTER(i64), i32])
N.optional("chb_comm_user_ptr", vp, [vp, i32])
N.optional("chb_comm_scratch_ptr", vp, [vp, i32])
N.optional("chb_barrier", i32, [vp, u64, vp])
N.optional("chb_comm_status", i32, [vp, i32, C.POINTER(u64), vp])
N.optional("chb_comm_clear_error", i32, [vp, vp])
N.optional("chb_comm_trace_enable", i32, [vp, i32])
N.optional("chb_comm_trace_read", i32, [vp, i32, C.POINTER(u64), i32, vp])
N.optional("chb_ipc_alloc", i32, [C.c_size_t, C.POINTER(vp), vp])
N.optional("chb_ipc_open", i32, [vp, C.POINTER(vp)])
N.optional("chb_ipc_close", i32, [vp])
N.optional("chb_dev_alloc", i32, [C.c_size_t, C.POINTER(vp)])
N.optional("chb_dev_free", i32, [vp])
N.optional("chb_program_prepare", i32, [vp, vp])
N.optional("chb_program_release", None, [vp, vp])
N.optional("chb_run_program", i32, [vp, vp, i32, i32, C.POINTER(vp), C.POINTER(vp), f32, i32, vp])
N.optional("chb_run_program_ll", i32, [vp, vp, i32, i32, C.POINTER(vp), C.POINTER(vp), f32, i32, vp])
N.optional("chb_program_ll_lines", C.c_longlong, [vp, i32])
N.optional("chb_ll_max_bytes", C.c_longlong, [vp])
N.optional("chb_ll_collective", i32, [vp, i32, i32, i32, C.POINTER(vp), C.POINTER(vp), C.c_longlong, f32, i32, vp])
N.optional("chb_collective", i32, [vp, i32, C.c_char_p, i32, i32, i32, i32, i32, C.POINTER(vp), C.POINTER(vp), i64, f32, i32, vp])
N.optional("chb_bootstrap_create", i32, [C.c_char_p, i32, i32, i32, C.POINTER(vp)])
N.optional("chb_bootstrap_barrier", i32, [vp])
N.optional("chb_bootstrap_destroy", None, [vp])
N.optional("chb_comm_create_ipc", vp, [vp, C.c_size_t, C.c_size_t, C.c_size_t, C.c_char_p, i32])
N.optional("chb_comm_create_vmm", vp, [vp, C.c_size_t, C.c_size_t, C.c_size_t, i32, C.POINTER(i32), C.c_char_p, i32])
N.optional("chb_nvls_collective", i32, [vp, i32, i32, vp, vp, C.c_longlong, f32, i32, vp])

DTYPES = {
    torch.float32: N.F32, torch.bfloat16: N.BF16, torch.float16: N.F16, torch.int32: N.I32,
    torch.float64: N.F64, torch.int64: N.I64, torch.uint8: N.U8,
}
OPS = {"sum": N.SUM, "max": N.MAX, "min": N.MIN, "prod": N.PROD}
STATUS_NAMES = {
    0: "ok", 1: "timeout waiting for a peer to leave the previous collective",
    2: "timeout waiting for a peer's round", 3: "timeout waiting for peers to finish reading",
    4: "timeout at the rank-local barrier", 5: "timeout waiting for a flagged line",
    6: "timeout in barrier", 7: "a step addressed memory outside its buffer (checked build)",
}


class CollectiveError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"{N.ERR_NAMES.get(code, code)}: {msg}")
        self.code = code


class _CudaBuf:
    """Minimal ``__cuda_array_interface__`` holder to wrap a raw device pointer."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2,
        }


def _stream_ptr(stream=None) -> int:
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


class Communicator:
    def __init__(self):
        raise TypeError("use Communicator.emulated(...) or Communicator.from_process_group(...)")

    # ------------------------------------------------------------------ construction
    @classmethod
    def _new(cls):
        self = object.__new__(cls)
        self._h = None
        self._keep = []          # objects that own memory the native side points into
        self._ipc_opened = []
        self._own_heap_ptr = None
        self._user_off = 0
        self._programs = {}
        self._choices = {}       # (collective, bytes, dtype, symmetric) -> autotune.Choice
        self._user_ranges = []
        self._host_pipelines = {}  # (dtype, chunk, depth) -> ops.host.HostAllReduce
        self.group = None
        return self

    @classmethod
    def emulated(cls, P: int, device: int | None = None, ll_bytes: int = 256 << 10,
                 scratch_bytes: int = 64 << 20, user_bytes: int = 16 << 20, timeout_us: int = 2_000_000):
        """All P ranks on one GPU; collectives take / return lists of P tensors."""
        L = N.lib()
        if not hasattr(L, "chb_comm_create"):
            raise N.NativeLibraryMissing("libchb.so was built without its CUDA half")
        self = cls._new()
        dev = torch.cuda.current_device() if device is None else device
        torch.cuda.set_device(dev)
        heap_bytes = int(L.chb_heap_bytes(P, ll_bytes, scratch_bytes, user_bytes))
        heap = torch.zeros(P * heap_bytes, dtype=torch.uint8, device=f"cuda:{dev}")
        self._keep.append(heap)
        ptrs = (vp * P)(*[heap.data_ptr() + p * heap_bytes for p in range(P)])
        self._finish(0, P, P, ptrs, 0, ll_bytes, scratch_bytes, user_bytes, dev, timeout_us)
        self.backend = "emulated"
        return self

    @classmethod
    def from_process_group(cls, group=None, backend: str | None = None, ll_bytes: int = 4 << 20,
                           scratch_bytes: int = 256 << 20, user_bytes: int = 64 << 20,
                           timeout_us: int = 10_000_000):
        """One rank per process.  ``backend``: "symm_mem" (VMM + NVLS multicast via
        torch's symmetric memory), "ipc" (native cudaIpc handles) or None = try
        symm_mem, fall back to ipc.  Env CHB_BACKEND overrides."""
        import torch.distributed as dist

        L = N.lib()
        if not hasattr(L, "chb_comm_create"):
            raise N.NativeLibraryMissing("libchb.so was built without its CUDA half")
        self = cls._new()
        group = group if group is not None else dist.group.WORLD
        self.group = group
        P, rank = dist.get_world_size(group), dist.get_rank(group)
        dev = torch.cuda.current_device()
        backend = os.environ.get("CHB_BACKEND", backend or "auto")
        heap_bytes = int(L.chb_heap_bytes(P, ll_bytes, scratch_bytes, user_bytes))
        ptrs, mc = None, 0
        if P == 1:
            heap = torch.zeros(heap_bytes, dtype=torch.uint8, device=f"cuda:{dev}")
            self._keep.append(heap)
            ptrs, backend = [heap.data_ptr()], "local"
        elif backend in ("auto", "symm_mem"):
            err = None
            try:
                ptrs, mc = self._heap_symm_mem(group, heap_bytes, dev)
            except Exception as e:  # noqa: BLE001 - any failure means "not available here"
                err, ptrs = e, None
            # every rank must end up on the same backend: agree before going on
            oks = [None] * P
            dist.all_gather_object(oks, err is None, group=group)
            if all(oks):
                backend = "symm_mem"
                mcs = [None] * P
                dist.all_gather_object(mcs, bool(mc), group=group)
                if not all(mcs):
                    mc = 0            # multicast must be usable on all ranks or on none
            else:
                if backend == "symm_mem":
                    raise err if err is not None else RuntimeError("symmetric-memory rendezvous failed on a peer")
                self._symm_mem_error = repr(err)
                ptrs, mc = None, 0
        if ptrs is None:
            ptrs = self._heap_ipc(group, heap_bytes, rank, P)
            backend = "ipc"
        self.backend = backend
        arr = (vp * P)(*ptrs)
        self._finish(rank, P, 1, arr, mc, ll_bytes, scratch_bytes, user_bytes, dev, timeout_us)
        torch.cuda.synchronize()
        dist.barrier(group)  # nobody signals into a heap before every rank has set up
        return self

    @classmethod
    def from_shared_memory(cls, name: str, rank: int, world: int, ll_bytes: int = 4 << 20,
                           scratch_bytes: int = 256 << 20, user_bytes: int = 64 << 20,
                           timeout_us: int = 10_000_000, rendezvous_timeout_ms: int = 60_000,
                           heap: str = "auto", multicast: bool = True):
        """One rank per process without ``torch.distributed``: the ranks of one box meet through the
        native shared-memory bootstrap (``name`` = "/something", the same on every rank, unique per job).
        ``heap="vmm"``: heaps from CUDA's virtual-memory allocator, shared as file descriptors, with an NVLink
        multicast alias when ``multicast`` and every device has one (the ``multimem`` kernels then run);
        ``heap="ipc"``: cudaIpc handles; ``"auto"``: vmm, else ipc.  The path the native launcher uses."""
        L = N.lib()
        if not hasattr(L, "chb_comm_create_ipc"):
            raise N.NativeLibraryMissing("libchb.so was built without its CUDA half")
        self = cls._new()
        dev = torch.cuda.current_device()
        torch.cuda.init()
        torch.zeros(1, device=f"cuda:{dev}")          # the primary context exists before the native side allocates
        boot = vp()
        rc = L.chb_bootstrap_create(name.encode(), rank, world, rendezvous_timeout_ms, C.byref(boot))
        if rc:
            raise CollectiveError(rc, f"rendezvous '{name}' of {world} ranks failed")
        self._boot = boot
        err = C.create_string_buffer(256)
        h = None
        self.backend = "ipc-native"
        if heap in ("auto", "vmm") and os.environ.get("CHB_VMM", "1") != "0":
            code = i32(0)
            want_mc = 1 if (multicast and os.environ.get("CHB_NVLS", "1") != "0") else 0
            h = L.chb_comm_create_vmm(boot, ll_bytes, scratch_bytes, user_bytes, want_mc, C.byref(code), err, len(err))
            if h:
                self.backend = "vmm-native"
            elif heap == "vmm" or code.value != N.ERR_UNSUPPORTED:
                L.chb_bootstrap_destroy(boot)
                self._boot = None
                raise CollectiveError(code.value or N.ERR_OTHER, err.value.decode())
        if not h:
            h = L.chb_comm_create_ipc(boot, ll_bytes, scratch_bytes, user_bytes, err, len(err))
        if not h:
            L.chb_bootstrap_destroy(boot)
            self._boot = None
            raise CollectiveError(N.ERR_OTHER, err.value.decode())
        self._adopt(h, world, rank, 1, dev, timeout_us)
        return self

    def _heap_symm_mem(self, group, heap_bytes, dev):
        import torch.distributed._symmetric_memory as symm_mem

        name = group.group_name if hasattr(group, "group_name") else group
        try:
            symm_mem.enable_symm_mem_for_group(name)
        except Exception:  # noqa: BLE001 - newer torch enables every group implicitly
            pass
        t = symm_mem.empty(heap_bytes, dtype=torch.uint8, device=f"cuda:{dev}")
        t.zero_()
        torch.cuda.synchronize()
        hdl = symm_mem.rendezvous(t, name)
        self._keep += [t, hdl]
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        mc = 0
        if os.environ.get("CHB_NVLS", "1") != "0":
            try:
                mc = int(hdl.multicast_ptr or 0)
            except Exception:  # noqa: BLE001
                mc = 0
        return ptrs, mc

    def _heap_ipc(self, group, heap_bytes, rank, P):
        import torch.distributed as dist

        L = N.lib()
        ptr = vp()
        handle = (C.c_char * 64)()
        rc = L.chb_ipc_alloc(heap_bytes, C.byref(ptr), handle)
        if rc:
            raise CollectiveError(rc, "cudaIpc allocation of the symmetric heap failed")
        self._own_heap_ptr = ptr.value
        handles = [None] * P
        dist.all_gather_object(handles, bytes(handle), group=group)
        ptrs = []
        for p in range(P):
            if p == rank:
                ptrs.append(ptr.value)
            else:
                q = vp()
                h = (C.c_char * 64).from_buffer_copy(handles[p])
                rc = L.chb_ipc_open(h, C.byref(q))
                if rc:
                    raise CollectiveError(rc, f"cannot open the heap of rank {p} (no peer access?)")
                self._ipc_opened.append(q.value)
                ptrs.append(q.value)
        return ptrs

    def _finish(self, rank, P, nlocal, ptrs, mc, ll_bytes, scratch_bytes, user_bytes, dev, timeout_us):
        L = N.lib()
        err = C.create_string_buffer(256)
        h = L.chb_comm_create(rank, P, nlocal, ptrs, mc or None, ll_bytes, scratch_bytes, user_bytes, err, len(err))
        if not h:
            raise CollectiveError(N.ERR_ARG, err.value.decode())
        self._adopt(h, P, rank, nlocal, dev, timeout_us)

    def _adopt(self, h, P, rank, nlocal, dev, timeout_us):
        L = N.lib()
        self._h = h
        self.P, self.rank, self.nlocal, self.device = P, rank, nlocal, dev
        info = (i64 * 11)()
        L.chb_comm_info(h, info, 11)
        self.scratch_bytes, self.user_bytes, self.heap_bytes = int(info[5]), int(info[6]), int(info[7])
        self.ll_max_bytes, self.sm_count, self.has_multicast = int(info[8]), int(info[9]), bool(info[10])
        self.ll2_max_bytes = (self.ll_max_bytes // 16) * 8 * P   # two-shot flagged lines: half a slot per slice
        self.set_timeout_us(int(os.environ.get("CHB_TIMEOUT_US", timeout_us)))
        self.launches = 0   # kernels launched by this communicator (all local ranks count as one)

    def close(self):
        if self._h:
            L = N.lib()
            torch.cuda.synchronize()
            self._host_pipelines = {}                    # their buffers live in the heap that goes away below
            if getattr(self, "_boot", None):
                L.chb_bootstrap_barrier(self._boot)      # nobody frees a heap that a peer may still read
            L.chb_comm_destroy(self._h)
            self._h = None
            for q in self._ipc_opened:
                L.chb_ipc_close(q)
            self._ipc_opened = []
            if self._own_heap_ptr:
                L.chb_dev_free(self._own_heap_ptr)
                self._own_heap_ptr = None
            if getattr(self, "_boot", None):
                L.chb_bootstrap_destroy(self._boot)
                self._boot = None
            self._keep = []

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass

    # ------------------------------------------------------------------ helpers
    @property
    def handle(self):
        return self._h

    def set_timeout_us(self, us: int):
        self.timeout_us = us
        N.lib().chb_comm_set_timeout_us(self._h, us)

    def _err(self, rc: int):
        if rc:
            raise CollectiveError(rc, N.lib().chb_comm_last_error(self._h).decode())

    def empty(self, numel: int, dtype=torch.float32) -> list[torch.Tensor] | torch.Tensor:
        """Allocate a peer-visible tensor from the user region of the symmetric
        heap (bump allocator, never freed; same call order on every rank)."""
        esz = torch.empty((), dtype=dtype).element_size()
        nbytes = (numel * esz + 255) // 256 * 256
        if self._user_off + nbytes > self.user_bytes:
            raise MemoryError("symmetric user region exhausted; create the communicator with a larger user_bytes")
        outs = []
        for l in range(self.nlocal):
            base = N.lib().chb_comm_user_ptr(self._h, l)
            t = torch.as_tensor(_CudaBuf(base + self._user_off, numel * esz), device=f"cuda:{self.device}")
            outs.append(t.view(dtype))
        self._user_off += nbytes
        self._keep.append(outs)
        return outs if self.nlocal > 1 else outs[0]

    def is_symmetric(self, t: torch.Tensor) -> bool:
        """True if the tensor lives in the peer-visible user region of a local rank."""
        if not self._user_ranges:
            for l in range(self.nlocal):
                base = N.lib().chb_comm_user_ptr(self._h, l)
                self._user_ranges.append((base, base + self.user_bytes))
        p = t.data_ptr()
        for lo, hi in self._user_ranges:
            if lo <= p < hi:
                return True
        return False

    def _lists(self, x):
        if isinstance(x, torch.Tensor):
            assert self.nlocal == 1, "an emulated communicator takes one tensor per rank"
            return [x]
        assert len(x) == self.nlocal
        return list(x)

    def _ptrs(self, ts: Sequence[torch.Tensor]):
        return (vp * len(ts))(*[t.data_ptr() for t in ts])

    # ------------------------------------------------------------------ status
    def barrier(self, timeout_us: int = 0, stream=None):
        self._err(N.lib().chb_barrier(self._h, timeout_us, _stream_ptr(stream)))
        self.launches += 1

    def status(self, local_index: int = 0, stream=None) -> dict:
        """Synchronise the stream and read the control block of a local rank."""
        st = (u64 * 8)()
        rc = N.lib().chb_comm_status(self._h, local_index, st, _stream_ptr(stream))
        to_i = lambda v: v - (1 << 64) if v >= (1 << 63) else v
        d = {"rc": rc, "code": int(st[0]), "what": STATUS_NAMES.get(int(st[0]), "?"), "rank": int(st[1]),
             "round": to_i(int(st[2])), "peer": to_i(int(st[3])), "expected": int(st[4]), "seen": int(st[5]),
             "launches": int(st[6]), "epoch": int(st[7])}
        return d

    def check(self, stream=None):
        """Raise :class:`CollectiveError` if any local rank recorded an expired wait."""
        for l in range(self.nlocal):
            d = self.status(l, stream)
            if d["rc"] == N.ERR_TIMEOUT:
                raise CollectiveError(N.ERR_TIMEOUT, f"rank {d['rank']}: {d['what']} (round {d['round']}, peer {d['peer']}, "
                                                      f"expected {d['expected']}, seen {d['seen']})")
            if d["rc"]:
                self._err(d["rc"])

    def enable_trace(self, rounds: int = 64):
        """Record per-round device timestamps of program launches (0 switches it off)."""
        self._err(N.lib().chb_comm_trace_enable(self._h, rounds))
        self._trace_rounds = rounds

    def read_trace(self, nrounds: int, local_index: int = 0, stream=None) -> list[tuple[float, float]]:
        """(start_us, end_us) of every round of the last program launch, relative to the first round's start."""
        n = min(nrounds, getattr(self, "_trace_rounds", 0))
        buf = (u64 * (2 * n))()
        self._err(N.lib().chb_comm_trace_read(self._h, local_index, buf, n, _stream_ptr(stream)))
        t0 = buf[0] if n else 0
        return [((buf[2 * i] - t0) / 1e3, (buf[2 * i + 1] - t0) / 1e3) for i in range(n)]

    def clear_error(self, stream=None):
        self._err(N.lib().chb_comm_clear_error(self._h, _stream_ptr(stream)))

    # ------------------------------------------------------------------ launchers
    def program(self, coll: str, algo: str, count: int, k: int = 2, b: int = 1, aux: int = 0,
                in_symmetric: bool = False, out_symmetric: bool = False, in_place: bool = False) -> Program:
        return cached_program(coll, algo, self.P, count, k, b, aux, in_symmetric, out_symmetric, in_place)

    def run_program(self, prog: Program, ins, outs, op: str = "sum", scale: float = 1.0, nctas: int = 0, stream=None,
                    mode: str = "pull"):
        """Launch a compiled program.  ``mode="pull"``: the persistent interpreter (readers pull over
        NVLink, rounds separated by flags); ``mode="ll"``: owners push flagged lines into the readers'
        inboxes (one traversal per round; the program must be lowered with ``in_symmetric`` and
        ``out_symmetric``, and fit the inbox)."""
        ins, outs = self._lists(ins), self._lists(outs)
        dt = DTYPES[ins[0].dtype]
        for t in ins:
            assert t.is_contiguous() and t.numel() >= prog.in_elems and t.dtype == ins[0].dtype
        for t in outs:
            assert t.is_contiguous() and t.numel() >= prog.out_elems and t.dtype == ins[0].dtype
        fn = N.lib().chb_run_program_ll if mode == "ll" else N.lib().chb_run_program
        rc = fn(self._h, prog.handle, dt, OPS[op], self._ptrs(ins), self._ptrs(outs), scale, nctas, _stream_ptr(stream))
        self._err(rc)
        self.launches += 1

    def run_ll(self, mode: int, ins, outs, count: int, op: str = "sum", scale: float = 1.0, nctas: int = 0, stream=None):
        ins, outs = self._lists(ins), self._lists(outs)
        dt = DTYPES[ins[0].dtype]
        rc = N.lib().chb_ll_collective(self._h, mode, dt, OPS[op], self._ptrs(ins), self._ptrs(outs), count,
                                       scale, nctas, _stream_ptr(stream))
        self._err(rc)
        self.launches += 1
