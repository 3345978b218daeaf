"""Python view of a compiled step program (``csrc/sched/program.h``).

A program is the schedule of one collective algorithm for a fixed
``(collective, algorithm, P, k, b, count)``: per rank and per round a list of
pull steps ``dst = [dst op] src_0 op src_1 ...`` plus the cross-rank waits and
signals that order them.  The same object feeds

* :meth:`Program.simulate` — all ranks on host buffers in one process,
* :class:`..parallel.gloo_exec.GlooExecutor` — one process per rank, CPU tensors,
* the persistent GPU interpreter kernel (``csrc/kernels/interp.cu``).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from functools import lru_cache

import numpy as np

from .. import _native as N

BUF_IN, BUF_OUT, BUF_WORK = 0, 1, 2

_NP_DTYPES = {
    N.F32: np.float32, N.F64: np.float64, N.I32: np.int32, N.I64: np.int64, N.U8: np.uint8,
}
_DT_FROM_NP = {np.dtype(v): k for k, v in _NP_DTYPES.items()}
_OPS = {"sum": N.SUM, "max": N.MAX, "min": N.MIN, "prod": N.PROD}

COLLECTIVES = ("allreduce", "reduce_scatter", "allgather", "alltoall", "gather")


class ProgramError(ValueError):
    """The requested algorithm cannot be built for these parameters."""


def list_algorithms(coll: str) -> list[str]:
    buf = C.create_string_buffer(1024)
    N.lib().chb_list_algorithms(coll.encode(), buf, len(buf))
    s = buf.value.decode()
    return s.split(",") if s else []


@dataclass(frozen=True)
class Step:
    rank: int
    round: int
    dst_buf: int
    dst_off: int
    count: int
    acc: bool
    srcs: tuple  # of (peer, buf, off)


class Program:
    def __init__(self, coll: str, algo: str, P: int, count: int, k: int = 2, b: int = 1, aux: int = 0,
                 in_symmetric: bool = False, out_symmetric: bool = False, in_place: bool = False):
        L = N.lib()
        err = C.create_string_buffer(512)
        h = L.chb_program_create(coll.encode(), algo.encode(), P, k, b, count, aux,
                                 int(in_symmetric) | (2 if in_place else 0), int(out_symmetric), err, len(err))
        if not h:
            raise ProgramError(err.value.decode() or "program creation failed")
        self._h = h
        self.coll, self.algo, self.k, self.b, self.count, self.aux = coll, algo, k, b, count, aux
        info = (C.c_int64 * 32)()
        L.chb_program_info(h, info, 32)
        (self.P, self.nrounds, self.in_elems, self.out_elems, self.work_elems, self.nops,
         self.remote_msgs, self.remote_elems, self.max_rank_remote_elems, self.local_elems,
         self.max_nsrc, rpi, rpo, self.nsrcs, self.nwaits, self.nexit_waits, self.nsignals) = [int(x) for x in info[:17]]
        self.reads_peer_in, self.reads_peer_out = bool(rpi), bool(rpo)
        self.in_symmetric, self.out_symmetric, self.in_place = in_symmetric, out_symmetric, in_place
        self.name = L.chb_program_name(h).decode()
        self._tables = None

    @classmethod
    def alltoallv(cls, counts, r: int = 2, b: int = 1) -> "Program":
        """All-to-all-v program; ``counts[s][d]`` = elements rank s sends to rank d."""
        counts = np.ascontiguousarray(counts, dtype=np.int64)
        P = counts.shape[0]
        assert counts.shape == (P, P)
        L = N.lib()
        err = C.create_string_buffer(512)
        h = L.chb_program_create_alltoallv(P, r, b, counts.ctypes.data_as(C.POINTER(C.c_int64)), err, len(err))
        if not h:
            raise ProgramError(err.value.decode() or "program creation failed")
        self = cls.__new__(cls)
        self._h = h
        self.coll, self.algo, self.k, self.b, self.count, self.aux = "alltoallv", "tuna", r, b, 0, 0
        info = (C.c_int64 * 32)()
        L.chb_program_info(h, info, 32)
        (self.P, self.nrounds, self.in_elems, self.out_elems, self.work_elems, self.nops,
         self.remote_msgs, self.remote_elems, self.max_rank_remote_elems, self.local_elems,
         self.max_nsrc, rpi, rpo, self.nsrcs, self.nwaits, self.nexit_waits, self.nsignals) = [int(x) for x in info[:17]]
        self.reads_peer_in, self.reads_peer_out = bool(rpi), bool(rpo)
        self.in_symmetric = self.out_symmetric = self.in_place = False
        self.name = L.chb_program_name(h).decode()
        self._tables = None
        return self

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                N.lib().chb_program_destroy(self._h)
                self._h = None
        except Exception:
            pass

    @property
    def handle(self):
        return self._h

    # ------------------------------------------------------------------ tables
    def tables(self):
        """(ops[NOPS,8], srcs[NSRCS,3], waits[NWAITS,4], exit_waits[*,3], signals[*,3]) as int64 arrays."""
        if self._tables is None:
            ops = np.zeros((self.nops, 8), np.int64)
            srcs = np.zeros((self.nsrcs, 3), np.int64)
            waits = np.zeros((self.nwaits, 4), np.int64)
            ex = np.zeros((self.nexit_waits, 3), np.int64)
            sig = np.zeros((self.nsignals, 3), np.int64)
            p = lambda a: a.ctypes.data_as(C.c_void_p)
            N.lib().chb_program_export(self._h, p(ops), p(srcs), p(waits), p(ex), p(sig))
            self._tables = (ops, srcs, waits, ex, sig)
        return self._tables

    def steps(self, rank: int | None = None) -> list[Step]:
        ops, srcs, *_ = self.tables()
        out = []
        for o in ops:
            if rank is not None and o[0] != rank:
                continue
            s = tuple((int(p), int(b), int(f)) for p, b, f in srcs[o[6]:o[6] + o[7]])
            out.append(Step(int(o[0]), int(o[1]), int(o[2]), int(o[3]), int(o[4]), bool(o[5]), s))
        return out

    # ------------------------------------------------------------------ checks
    def verify(self) -> int:
        err = C.create_string_buffer(2048)
        bad = N.lib().chb_program_verify(self._h, err, len(err))
        if bad:
            raise AssertionError(f"{self.name}: {bad} unsynchronised hazards: {err.value.decode()}")
        return 0

    def simulate(self, inputs: list[np.ndarray], op: str = "sum", seed: int = 0, alias: bool = False) -> list[np.ndarray]:
        """Run all P ranks on host arrays; returns the P output arrays.  ``alias=True`` hands every rank ONE
        buffer as both input and output (the in-place form; the program must have been created with
        ``in_place=True``)."""
        assert len(inputs) == self.P
        dt = inputs[0].dtype
        code = _DT_FROM_NP[np.dtype(dt)]
        ins = [np.ascontiguousarray(x, dtype=dt) for x in inputs]
        for x in ins:
            assert x.size == self.in_elems, (x.size, self.in_elems)
        if alias:
            assert self.in_place, "aliased buffers need a program lowered with in_place=True"
            bufs = [np.full(max(self.in_elems, self.out_elems), 239 if np.dtype(dt).kind == "u" else -17, dtype=dt) for _ in range(self.P)]
            for b_, x in zip(bufs, ins):
                b_[:x.size] = x
            ins, outs = bufs, bufs
        else:
            # outputs start poisoned so that positions the program never writes stand out
            outs = [np.full(self.out_elems, 239 if np.dtype(dt).kind == "u" else -17, dtype=dt) for _ in range(self.P)]
        ip = (C.c_void_p * self.P)(*[x.ctypes.data for x in ins])
        opp = (C.c_void_p * self.P)(*[x.ctypes.data for x in outs])
        err = C.create_string_buffer(512)
        rc = N.lib().chb_program_simulate(self._h, code, _OPS[op], ip, opp, seed, err, len(err))
        if rc:
            raise RuntimeError(f"simulate({self.name}) failed: {err.value.decode()}")
        return [o[:self.out_elems] for o in outs]

    def simulate_ll(self, inputs: list[np.ndarray], op: str = "sum", seed: int = 0, threads: int = 5,
                    fault: int = 0, launches: int = 1) -> list[np.ndarray]:
        """Run the push (flagged-line) form of this program on host arrays, line by line, the way the GPU executor
        does: ``threads`` virtual threads per rank, advanced in a random order drawn from ``seed``; only the plan's
        own messages, forwards and barriers order them.  The program must have been lowered with
        ``in_symmetric=True, out_symmetric=True`` (the push form has no staging copies).  ``fault`` injects a defect
        into the plan to test the simulator itself: 1 ignores the plan's barriers, 2 drops one forward per step.
        ``launches`` runs the program that often back to back, every rank going on as soon as its own previous launch
        has returned; a rank that gets two launches ahead of a reader of its lines is reported."""
        assert len(inputs) == self.P
        dt = inputs[0].dtype
        code = _DT_FROM_NP[np.dtype(dt)]
        ins = [np.ascontiguousarray(x, dtype=dt) for x in inputs]
        for x in ins:
            assert x.size == self.in_elems, (x.size, self.in_elems)
        poison = 239 if np.dtype(dt).kind == "u" else -17
        outs = [np.full(self.out_elems, poison, dtype=dt) for _ in range(self.P)]
        ip = (C.c_void_p * self.P)(*[x.ctypes.data for x in ins])
        opp = (C.c_void_p * self.P)(*[x.ctypes.data for x in outs])
        err = C.create_string_buffer(512)
        rc = N.lib().chb_program_simulate_ll(self._h, code, _OPS[op], ip, opp, seed, threads, fault, launches, err, len(err))
        if rc:
            raise RuntimeError(f"simulate_ll({self.name}) failed: {err.value.decode()}")
        return outs

    def ll_info(self, elem_bytes: int = 4) -> dict:
        """Shape of the flagged-line (push) form of this program: rounds, messages pushed per round's push phase,
        messages forwarded line by line from the previous round's steps, rank-local barriers (all ranks), lines in
        the fullest inbox and in the busiest (rank, round), bytes of the largest rank's own table entries (kept in shared
        memory by the executor up to 40 KiB)."""
        L = N.lib()
        v = (C.c_longlong * 7)()
        rc = L.chb_program_ll_info(self._h, elem_bytes, v, 7)
        if rc:
            raise RuntimeError(f"ll_info failed with code {rc}")
        return dict(zip(("levels", "pushed", "forwarded", "barriers", "inbox_lines", "busiest_level_lines", "rank_table_bytes"),
                        [int(x) for x in v]))

    def run_threads(self, inputs: list[np.ndarray], op: str = "sum", iters: int = 1,
                    late_rank: int | None = None, delay_ms: int = 20):
        """Run all P ranks as concurrent host threads; returns (outputs, mean seconds per repetition).

        With ``late_rank`` the run is done once, that rank's thread starts ``delay_ms`` late and its input
        holds poison until then: a schedule that lets a peer pull an input before its owner has entered
        the collective returns poisoned sums."""
        dt = inputs[0].dtype
        code = _DT_FROM_NP[np.dtype(dt)]
        ins = [np.ascontiguousarray(x, dtype=dt) for x in inputs]
        outs = [np.full(self.out_elems, -17, dtype=dt) for _ in range(self.P)]
        ip = (C.c_void_p * self.P)(*[x.ctypes.data for x in ins])
        opp = (C.c_void_p * self.P)(*[x.ctypes.data for x in outs])
        sec = C.c_double(0.0)
        if late_rank is not None:
            rc = N.lib().chb_program_run_threads_late(self._h, code, _OPS[op], ip, opp, late_rank, delay_ms)
        else:
            rc = N.lib().chb_program_run_threads(self._h, code, _OPS[op], ip, opp, iters, C.byref(sec))
        if rc:
            raise RuntimeError(f"run_threads({self.name}) failed with code {rc}")
        return outs, sec.value


@lru_cache(maxsize=512)
def cached_program(coll: str, algo: str, P: int, count: int, k: int = 2, b: int = 1, aux: int = 0,
                   in_symmetric: bool = False, out_symmetric: bool = False, in_place: bool = False) -> Program:
    return Program(coll, algo, P, count, k, b, aux, in_symmetric, out_symmetric, in_place)
