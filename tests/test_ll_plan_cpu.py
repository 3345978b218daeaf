"""Host half of the flagged-line (push) execution of step programs: which messages are forwarded line by line
from the previous round's steps, and where a rank-local barrier is still needed (csrc/kernels/llprog.cu)."""
import pytest

from configurable_hierarchical_allreduce_algorithms_b200 import Program


def _prog(coll, algo, P, count, k=2, b=1, in_place=False):
    return Program(coll, algo, P, count, k, b, in_symmetric=True, out_symmetric=True, in_place=in_place)


def test_flat_two_round_allreduce_needs_no_barrier_and_forwards_the_whole_broadcast():
    P, n = 8, 1024
    info = _prog("allreduce", "radix_batch", P, n * P, 2, 1).ll_info(4)
    # reduce round: every rank pushes P-1 chunks; broadcast round: all P * (P-1) messages are forwarded by the reducers
    assert info["levels"] == 3                         # entry round (empty in this mode), reduce, broadcast
    assert info["pushed"] == P * (P - 1) and info["forwarded"] == P * (P - 1)
    assert info["barriers"] == 0
    assert info["inbox_lines"] == 2 * (P - 1) * n * 4 // 8


def test_one_round_collectives_are_one_push_phase():
    P, n = 4, 100
    for coll in ("allgather", "reduce_scatter"):
        info = _prog(coll, "radix_batch", P, n, 2, 1).ll_info(2)
        assert info["pushed"] == P * (P - 1) and info["forwarded"] == 0 and info["barriers"] == 0


@pytest.mark.parametrize("k,b", [(2, 2), (2, 4), (4, 4), (8, 8)])
def test_hierarchical_shapes_forward_and_keep_only_the_barriers_that_order_something(k, b):
    P, n = 8, 64
    prog = _prog("allreduce", "radix_batch", P, n * P, k, b)
    info = prog.ll_info(4)
    total = info["pushed"] + info["forwarded"]
    assert total == prog.remote_msgs                     # every remote source is a message, pushed or forwarded
    assert info["forwarded"] > 0
    assert info["barriers"] < P * (info["levels"] - 1)   # fewer than one per rank and round boundary


def test_in_place_form_reads_the_staged_copy_and_therefore_keeps_a_barrier():
    P, n = 4, 256
    a = _prog("allreduce", "radix_batch", P, n * P, 2, 1).ll_info(4)
    b = _prog("allreduce", "radix_batch", P, n * P, 2, 1, in_place=True).ll_info(4)
    assert a["barriers"] == 0 and b["barriers"] > 0


def test_element_size_scales_the_lines():
    P, n = 4, 1000
    prog = _prog("allreduce", "recursive_doubling", P, n, 2, 1)
    assert prog.ll_info(8)["inbox_lines"] == 2 * prog.ll_info(4)["inbox_lines"]
    assert prog.ll_info(2)["inbox_lines"] * 4 == prog.ll_info(8)["inbox_lines"]
