"""Invariants of the schedule arithmetic, checked through the programs it produces."""
import numpy as np
import pytest

from configurable_hierarchical_allreduce_algorithms_b200.parallel.program import Program


@pytest.mark.parametrize("P", range(1, 33))
def test_flat_radix_reduce_scatter_all_radices(P):
    ins = [np.arange(P * 2, dtype=np.int64) * (r + 1) for r in range(P)]
    tot = sum(ins)
    for k in range(2, 10):
        p = Program("reduce_scatter", "radix", P, 2, k, 1)
        p.verify()
        outs = p.simulate(ins)
        for r in range(P):
            np.testing.assert_array_equal(outs[r], tot[2 * r:2 * r + 2])


def test_rounds_shrink_with_radix():
    # more neighbours per round, fewer rounds: the point of the configurable radix
    r2 = Program("allreduce", "radix_batch", 16, 16 * 8, 2, 16, 0, True, True).nrounds
    r4 = Program("allreduce", "radix_batch", 16, 16 * 8, 4, 16, 0, True, True).nrounds
    r16 = Program("allreduce", "radix_batch", 16, 16 * 8, 16, 16, 0, True, True).nrounds
    assert r2 > r4 > r16


def test_batch_controls_round_count_of_store_and_forward():
    few = Program("reduce_scatter", "radix_block", 9, 4, 9, 8).nrounds   # all digits of a position at once
    many = Program("reduce_scatter", "radix_block", 9, 4, 9, 1).nrounds  # one exchange per synchronisation
    assert many > few
