"""Sampler: the CUDA Philox/Floyd sampler must equal the oracle's draw for draw, and must have the
reference's structural properties (core/ntsSampler.hpp:936-1042): k = min(deg, fanout) distinct
neighbour positions per destination, all neighbours when deg <= fanout, uniform over neighbours."""
import numpy as np
import pytest
import torch

import oracle
from helpers import assert_block_equal, dev_i32, dev_i64, host_u32, small_graph
from neutronbench_b200 import FullyRepGraph, Sampler

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fanouts", [(25, 10), (15, 10, 5), (3,), (40, 2)])
def test_sampler_matches_oracle_stream(cuda_device, ws, fanouts):
    V = 5000
    edges, co, ri = small_graph(V, 120000, seed=5)
    seeds = np.random.RandomState(1).choice(V, 300, replace=False).astype(np.uint32)
    g = FullyRepGraph(dev_i64(co, cuda_device), dev_i32(ri, cuda_device), V)
    smp = Sampler(g, seeds, fanouts, batch_size=128, ws=ws, seed=1234)
    draw = 0
    while smp.sample_not_finished():
        lo = smp.work_offset
        ssg = smp.sample_one()
        ref, _ = oracle.sample_batch(co, ri, V, seeds[lo: lo + 128], list(fanouts), seed=1234, draw=draw)
        for dev_blk, ref_blk in zip(ssg.sampled_sgs, ref):
            assert_block_equal(dev_blk, ref_blk)
        draw += 1
    assert draw == 3   # 128 + 128 + 44: the last batch is short (core/ntsSampler.hpp:846)


def test_structure_and_uniformity(cuda_device, ws):
    V, fan = 400, 5
    rng = np.random.RandomState(3)
    # vertex 0 has 40 distinct in-neighbours, vertex 1 has 3, vertex 2 has none
    edges = np.concatenate([
        np.stack([np.arange(100, 140), np.zeros(40, dtype=np.int64)], axis=1),
        np.stack([np.arange(200, 203), np.ones(3, dtype=np.int64)], axis=1)]).astype(np.int32)
    co, ri = oracle.build_csc(edges, V)
    g = FullyRepGraph(dev_i64(co, cuda_device), dev_i32(ri, cuda_device), V)
    seeds = np.array([0, 1, 2], dtype=np.uint32)
    smp = Sampler(g, np.tile(seeds, 4000), [fan], batch_size=3, ws=ws, seed=77)
    counts = np.zeros(V, dtype=np.int64)
    for _ in range(4000):
        blk = smp.sample_one().sampled_sgs[0]
        co_h = host_u32(blk.column_offset, 4)
        np.testing.assert_array_equal(co_h, [0, 5, 8, 8])
        src = host_u32(blk.source, blk.src_size)
        loc = host_u32(blk.row_indices, blk.e_size)
        col0 = src[loc[0:5]]
        assert len(set(col0.tolist())) == 5 and ((col0 >= 100) & (col0 < 140)).all()
        assert sorted(src[loc[5:8]].tolist()) == [200, 201, 202]
        counts[col0] += 1
    picked = counts[100:140]
    expected = 4000 * fan / 40.0
    chi2 = ((picked - expected) ** 2 / expected).sum()
    assert chi2 < 80.0, chi2          # 39 degrees of freedom: 99.99 % quantile is about 79
    assert picked.min() > 0


@pytest.mark.parametrize("rate,lower", [(0.5, 3), (0.1, 6), (1.0, 1)])
def test_sample_rate_mode_matches_oracle(cuda_device, ws, rate, lower):
    """SAMPLE_RATE / LOWER_FANOUT (core/ntsSampler.hpp:901-912): counts, Floyd draws for small subsets and
    selection sampling for subsets above 128 positions (a hub with ~900 in-neighbours) equal the oracle's."""
    V = 2500
    rng = np.random.RandomState(8)
    hub = np.stack([rng.randint(0, V, 900), np.zeros(900, np.int64)], axis=1)
    edges = np.concatenate([hub, small_graph(V, 30000, seed=2)[0].astype(np.int64)]).astype(np.uint32)
    co, ri = oracle.build_csc(edges, V)
    seeds = np.concatenate([[0], rng.choice(np.arange(1, V), 149, replace=False)]).astype(np.uint32)
    g = FullyRepGraph(dev_i64(co, cuda_device), dev_i32(ri, cuda_device), V)
    smp = Sampler(g, seeds, (4, 4), batch_size=100, ws=ws, seed=77, sample_rate=rate, lower_fanout=lower)
    draw = 0
    while smp.sample_not_finished():
        lo = smp.work_offset
        ssg = smp.sample_one(phase=True)
        ref, _ = oracle.sample_batch(co, ri, V, seeds[lo: lo + 100], [4, 4], seed=77, draw=draw, sample_rate=rate,
                                     lower_fanout=lower)
        for dev_blk, ref_blk in zip(ssg.sampled_sgs, ref):
            assert_block_equal(dev_blk, ref_blk)
        draw += 1
    # outside the training phase the fan-out rule applies again
    smp.restart()
    ssg = smp.sample_one(phase=False)
    ref, _ = oracle.sample_batch(co, ri, V, seeds[:100], [4, 4], seed=77, draw=draw)
    for dev_blk, ref_blk in zip(ssg.sampled_sgs, ref):
        assert_block_equal(dev_blk, ref_blk)


def test_random_batches_are_fresh_uniform_subsets(cuda_device, ws):
    V = 3000
    edges, co, ri = small_graph(V, 30000, seed=5)
    ids = np.arange(100, 1100, dtype=np.uint32)
    g = FullyRepGraph(dev_i64(co, cuda_device), dev_i32(ri, cuda_device), V)
    smp = Sampler(g, ids, (3,), batch_size=256, ws=ws, seed=5)
    smp.random_batches = True
    seen = []
    while smp.sample_not_finished():
        d, n = smp.next_seeds()
        got = host_u32(d)[:n]
        assert len(np.unique(got)) == n and np.isin(got, ids).all()     # distinct members of the seed list
        seen.append(got)
    assert [len(s) for s in seen] == [256, 256, 256, 232]                # batch sizes as in the plain loop
    assert len(np.intersect1d(seen[0], seen[1])) > 0                     # batches are drawn independently
