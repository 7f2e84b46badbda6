"""Host logic of the feature-cache policies (CACHE_POLICY degree | sample | random, CACHE_TYPE gpu_memory):
slot maps against the oracle's ranking, and the sizing arithmetic of
toolkits/GCN_GPU_NEIGHBOR.hpp:1427-1441."""
import numpy as np

import oracle
from neutronbench_b200 import (cache_nodes_for_memory, cache_slots_by_degree, cache_slots_by_sample_count,
                               cache_slots_random)


def test_sample_count_policy_ranks_like_the_oracle():
    rng = np.random.RandomState(5)
    V = 3000
    counts = rng.poisson(2.0, size=V).astype(np.uint32)      # many ties, many zeros
    for num in (0, 1, 700, V, V + 10):
        hm_ref, ids = oracle.cache_by_degree(counts, min(num, V))   # same rule: descending key, ties by id
        hm = cache_slots_by_sample_count(counts, num)
        np.testing.assert_array_equal(hm, hm_ref)
        assert (hm != 0xFFFFFFFF).sum() == min(num, V)
    # a node that is never sampled is cached last
    order = np.argsort(cache_slots_by_sample_count(counts, V))
    assert counts[order[0]] == counts.max() and counts[order[-1]] == counts.min()
    np.testing.assert_array_equal(cache_slots_by_degree(counts, 100), cache_slots_by_sample_count(counts, 100))


def test_random_policy_is_a_seeded_uniform_subset():
    V, num = 5000, 1200
    a, b, c = cache_slots_random(V, num, 7), cache_slots_random(V, num, 7), cache_slots_random(V, num, 8)
    np.testing.assert_array_equal(a, b)
    assert not np.array_equal(a, c)
    slots = a[a != 0xFFFFFFFF]
    assert len(slots) == num and np.array_equal(np.sort(slots), np.arange(num, dtype=np.uint32))
    # uniform: the cached ids are spread over the id range (mean id near V/2)
    ids = np.nonzero(a != 0xFFFFFFFF)[0]
    assert abs(ids.mean() - V / 2) < 4 * V / np.sqrt(12 * num)
    assert (cache_slots_random(V, V + 5, 1) != 0xFFFFFFFF).all()


def test_gpu_memory_sizing_arithmetic():
    mb = 1024 * 1024
    assert cache_nodes_for_memory(1124 * mb, 256, 10 ** 9) == 1024 * mb // (4 * 256)     # (free - 100 MB) / row bytes
    assert cache_nodes_for_memory(50 * mb, 602, 1000) == 0                                # nothing left after the reserve
    assert cache_nodes_for_memory(100 * 1024 * mb, 602, 232965) == 232965                 # clamped to the graph
