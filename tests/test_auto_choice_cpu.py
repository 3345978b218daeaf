"""What `algo="auto"` does with an allreduce whose length is not a multiple of the number of ranks: the tuned
table is made from divisible lengths and may name a schedule that cuts the vector into P slices."""
import json
from pathlib import Path
from types import SimpleNamespace

import pytest
import torch

from configurable_hierarchical_allreduce_algorithms_b200.ops.collectives import _ANY_COUNT, any_count
from configurable_hierarchical_allreduce_algorithms_b200.parallel.program import Program, ProgramError
from configurable_hierarchical_allreduce_algorithms_b200.utils import autotune

TABLE = Path(autotune.__file__).with_name("tuned_b200.json")


def test_divisible_lengths_keep_the_tuned_choice():
    assert any_count("allreduce", "radix_batch:ll", 8, 8, 16, 8, True, 64) == ("radix_batch:ll", 8, 8)
    assert any_count("reduce_scatter", "radix_batch:ll", 2, 1, 3, 8, True, 12) == ("radix_batch:ll", 2, 1)
    assert any_count("allreduce", "radix_batch", 2, 1, 7, 1, False, 28) == ("radix_batch", 2, 1)


def test_other_lengths_fall_back_to_kernels_that_take_any_length():
    assert any_count("allreduce", "radix_batch:ll", 8, 8, 2, 8, True, 8) == ("ll", 2, 1)
    assert any_count("allreduce", "radix_batch:pull", 2, 1, (1 << 16) + 1, 8, False, 4 * ((1 << 16) + 1)) == ("recursive_doubling", 2, 1)
    assert any_count("allreduce", "radix_batch", 2, 1, (1 << 22) + 3, 4, False, 4 * ((1 << 22) + 3)) == ("ring", 2, 1)
    for algo in ("ll", "ll2", "nvls", "recursive_doubling:pull", "ring:ll"):
        assert any_count("allreduce", algo, 2, 1, 13, 8, False, 52)[0] == algo


def test_the_any_length_list_is_true():
    """Every program named there compiles for lengths that no rank count divides; the sliced ones refuse."""
    for algo in _ANY_COUNT:
        if algo in ("ll", "ll2", "nvls", "nvls1"):
            continue
        for P, count in ((4, 2), (8, 13), (6, 7), (3, 1)):
            Program("allreduce", algo, P, count, 2, 1, aux=1 if algo == "inter_reduce_exchange_bcast" else 0)
    with pytest.raises(ProgramError):
        Program("allreduce", "radix_batch", 8, 2, 8, 8)


def test_every_row_of_the_committed_table_survives_small_odd_lengths():
    """The case that bit: a tuned row `radix_batch:ll` for allreduce up to 16 or 32 bytes met an 8-byte vector on 4
    and 8 ranks.  Walk every allreduce row of the table with lengths 1, 2, 3, ... elements."""
    table = json.loads(TABLE.read_text())
    seen = 0
    for key, rows in table.items():
        gpu, P, coll, dt = key.split("|")
        if coll != "allreduce":
            continue
        P = int(P)
        esz = 4 if dt == "fp32" else 2
        for count in (1, 2, 3, 5, 8, 13, 1000, 4097):
            payload = count * esz
            algo, k, b = next(((a, k_, b_) for mx, a, k_, b_, _ in rows if payload <= mx), ("radix_batch", 2, 1))
            algo, k, b = any_count(coll, algo, k, b, count, P, payload <= (256 << 10), payload)
            base = algo.split(":")[0]
            if base in ("ll", "ll2", "nvls", "nvls1"):
                continue
            Program("allreduce", base, P, count, k, b)        # must compile for this length
            seen += 1
    assert seen > 0


class _FakeLib:
    """Stands in for libchb.so: records what `_run` asks for and refuses what the real library would refuse for
    its length (a sliced schedule on a vector that P does not divide)."""

    def __init__(self, P, real):
        self.P, self.calls, self._real = P, [], real

    def __getattr__(self, name):          # everything else (the schedule compiler) is the real library
        return getattr(self._real, name)

    def chb_collective(self, h, coll, algo, k, b, aux, dtype, op, ins, outs, count, scale, nctas, stream):
        name = algo.decode()
        base = name.split(":")[0]
        self.calls.append((coll, name, k, b, count))
        if base in ("ll", "ll2", "nvls", "nvls1", "bulk"):
            return 0
        try:
            Program(["allreduce", "reduce_scatter", "allgather"][coll], base, self.P, count, k, b)
        except ProgramError:
            return 4        # what the library answers for a bad count
        return 0


@pytest.mark.parametrize("multicast", [True, False])
@pytest.mark.parametrize("P", [2, 4, 8])
def test_the_sizes_of_the_benchmark_sweep_reach_a_kernel_that_takes_them(P, multicast, monkeypatch):
    """`bench.py` sweeps allreduce / reduce-scatter / allgather from 8 bytes up with `algo="auto"` on symmetric
    buffers.  With the committed table for P ranks, every call must name a kernel or a program that accepts the
    length (the first sweep size is two fp32 elements, fewer than the ranks), with and without a multicast alias (without
    one the in-switch rows of the table give way to the fallback rule)."""
    from configurable_hierarchical_allreduce_algorithms_b200 import _native as N
    from configurable_hierarchical_allreduce_algorithms_b200.ops import collectives as ops

    fake = _FakeLib(P, N.lib())
    monkeypatch.setattr(N, "lib", lambda: fake)
    monkeypatch.setattr(autotune, "_key", lambda comm, coll, dtype: f"NVIDIA B200|{P}|{coll}|" + {torch.float32: "fp32", torch.bfloat16: "bf16"}[dtype])
    monkeypatch.setattr(ops, "_stream_ptr", lambda s: None)
    autotune.reload()
    errors = []
    comm = SimpleNamespace(P=P, nlocal=1, _h=None, _choices={}, launches=0, ll_max_bytes=4 << 20, ll2_max_bytes=(4 << 20) // 16 * 8 * P,
                           has_multicast=multicast, device=0, is_symmetric=lambda t: True, _err=lambda rc: errors.append(rc))
    for dtype in (torch.float32, torch.bfloat16):
        esz = 4 if dtype == torch.float32 else 2
        sz = 8
        while sz <= (1 << 30):
            ne = max(1, sz // esz)
            x = torch.empty(0, dtype=dtype).new_empty(0)      # no storage of that size on this box: fake tensors below
            t = SimpleNamespace(numel=lambda ne=ne: ne, element_size=lambda esz=esz: esz, dtype=dtype, data_ptr=lambda: 4096,
                                device="cpu")
            before = len(fake.calls)
            ops._run(comm, "allreduce", [t], [t], ne, "sum", "auto", 2, 1, 0, 1.0, 0, None, ne * esz, ops.LL_AR)
            blk = max(1, ne // P)
            ops._run(comm, "reduce_scatter", [t], [t], blk, "sum", "auto", 2, 1, 0, 1.0, 0, None, blk * esz, ops.LL_RS)
            ops._run(comm, "allgather", [t], [t], blk, "sum", "auto", 2, 1, 0, 1.0, 0, None, blk * esz, ops.LL_AG)
            assert len(fake.calls) >= before + 3
            sz *= 4
    autotune.reload()
    assert not errors, (errors, [c for c in fake.calls][-6:])
    # the tuned hierarchical cell is still used where the length allows it (8 ranks: the 32-byte vector of the sweep)
    if P == 8 and multicast:
        assert any(name.startswith("radix_batch:ll") and coll == 0 and b == P for coll, name, k, b, count in fake.calls)
