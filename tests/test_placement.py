"""CPU: sessions are spread over GPUs so that the summed context length (what a
decode step streams) is even, under the per-step batch cap."""
import numpy as np
import pytest

from wayruntime_b200 import placement


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("seed", [0, 1, 20261125])
def test_assignment_is_a_balanced_partition(world, seed):
    rng = np.random.Generator(np.random.Philox(seed))
    lens = [int(x) for x in rng.integers(1024, 4097, size=16 * world)]
    bins = placement.assign_sessions(lens, world)
    assert sorted(i for b in bins for i in b) == list(range(len(lens)))
    assert all(len(b) <= placement.BATCH_MAX for b in bins)
    assert placement.imbalance(lens, bins) <= 1.01
    assert bins == placement.assign_sessions(lens, world)          # deterministic


def test_assignment_edge_cases():
    assert placement.assign_sessions([], 3) == [[], [], []]
    assert placement.assign_sessions([5], 2) == [[0], []]
    bins = placement.assign_sessions([10, 10, 10, 1], 2, per_gpu=2)
    assert sorted(len(b) for b in bins) == [2, 2]
    with pytest.raises(ValueError):
        placement.assign_sessions([1] * 5, 2, per_gpu=2)
    with pytest.raises(ValueError):
        placement.assign_sessions([1], 0)
