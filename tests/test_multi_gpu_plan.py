"""Shard planners of the C ABI (plain host functions, no device needed): N-slab ranges and the greedy assignment of expert
groups to ranks, checked against the Python planner the two-rank gloo test uses and against their defining properties."""
import numpy as np
import pytest

import ascb200 as ab
from sharding import dirichlet_counts, lpt_partition, n_slab


@pytest.mark.parametrize("n,world,align", [(11008, 1, 16), (11008, 2, 16), (11008, 4, 16), (11008, 8, 16), (8192, 8, 128), (1000, 3, 16), (40, 8, 16), (0, 4, 16)])
def test_nslab_ranges_tile_the_columns(n, world, align):
    ranges = [ab.shard_nslab(n, r, world, align) for r in range(world)]
    assert ranges == [n_slab(n, r, world, align) for r in range(world)]
    assert ranges[0][0] == 0 and ranges[-1][1] == n
    for (lo0, hi0), (lo1, hi1) in zip(ranges, ranges[1:]):
        assert hi0 == lo1 and lo0 <= hi0
    for lo, hi in ranges[:-1]:
        assert (hi - lo) % align == 0 or hi == n


@pytest.mark.parametrize("groups,world,seed", [(64, 1, 1), (64, 2, 2), (64, 4, 3), (64, 8, 0xA5C00003), (5, 8, 4), (1024, 8, 5)])
def test_groups_lpt_matches_the_python_planner_and_balances_rows(groups, world, seed):
    counts = dirichlet_counts(groups, 32768, seed)
    owner = ab.shard_groups_lpt(counts, world)
    mine = lpt_partition(counts, world)
    for r in range(world):
        assert sorted(np.flatnonzero(owner == r).tolist()) == mine[r]
    load = np.array([counts[owner == r].sum() for r in range(world)])
    assert load.sum() == counts.sum()
    assert load.max() - load.min() <= counts.max()   # greedy by size: no rank is ahead by more than one group


def test_planner_argument_errors():
    import ctypes as C
    lo, hi = C.c_int64(), C.c_int64()
    assert ab.lib().ascb200_shard_nslab(100, 4, 4, 16, C.byref(lo), C.byref(hi)) == ab.EINVAL
    assert ab.lib().ascb200_shard_nslab(100, 0, 0, 16, C.byref(lo), C.byref(hi)) == ab.EINVAL
    assert ab.lib().ascb200_shard_groups_lpt(None, 4, 2, None) == ab.EINVAL
    neg = np.array([5, -3, 0, 7], np.int64)   # non-positive counts are empty groups
    owner = ab.shard_groups_lpt(neg, 2)
    assert owner[3] != owner[0]
