"""CACHE_POLICY:sample / random and CACHE_TYPE:gpu_memory on the device: the sampling-frequency counts
equal those of the oracle's sampler on the same draws, the cache holds the right rows, and training
results do not depend on what is cached."""
import numpy as np
import pytest
import torch

import oracle
from helpers import dev_i32, small_graph
from neutronbench_b200 import (FullyRepGraph, GCN_GPU_NEIGHBOR_impl, GCNConfig, GNNDatum, Sampler, Workspace, _lib,
                               cache_slots_by_sample_count)
from neutronbench_b200.cuda_stream import ptr

pytestmark = pytest.mark.gpu


def test_count_ids_equals_bincount(cuda_device):
    rng = np.random.RandomState(1)
    V = 1000
    ids = rng.randint(0, V + 50, size=20000).astype(np.uint32)      # some ids lie outside the graph
    counts = torch.zeros(V, dtype=torch.int32, device=cuda_device)
    st = torch.cuda.current_stream().cuda_stream
    d_ids = dev_i32(ids, cuda_device)
    _lib.call("nb_count_ids", ptr(d_ids), len(ids), V, ptr(counts), st)
    _lib.call("nb_count_ids", ptr(d_ids), 0, V, ptr(counts), st)     # empty list: no-op
    _lib.call("nb_count_ids", ptr(d_ids), 5000, V, ptr(counts), st)  # accumulates
    ref = np.bincount(ids[ids < V], minlength=V) + np.bincount(ids[:5000][ids[:5000] < V], minlength=V)
    np.testing.assert_array_equal(counts.cpu().numpy(), ref)


def _make(cuda_device, cache_type, policy, rate=0.3, pipelines=1, V=3000, F=50):
    edges, co, ri = small_graph(V, 40000, seed=9)
    rng = np.random.RandomState(0)
    feat = rng.randn(V, F).astype(np.float32)
    label = rng.randint(0, 5, size=V).astype(np.int64)
    cfg = GCNConfig(layers=[F, 16, 5], fanout=(6, 4), batch_size=200, drop_rate=0.3, cache_type=cache_type,
                    cache_rate=rate, cache_policy=policy, seed=77, pipelines=pipelines)
    g = FullyRepGraph.from_edges(torch.from_numpy(edges).to(cuda_device), V, Workspace(64 << 20))
    datum = GNNDatum(torch.from_numpy(feat).pin_memory(), torch.from_numpy(label).to(cuda_device), np.zeros(V, np.int32))
    tk = GCN_GPU_NEIGHBOR_impl(g, datum, cfg)
    train_ids = np.arange(0, 900, dtype=np.uint32)
    smp = Sampler(g, train_ids, cfg.fanout, cfg.batch_size, tk.ws, seed=cfg.seed, with_edge_weights=False)
    return co, ri, feat, cfg, g, tk, smp, train_ids


def test_sample_policy_counts_and_cache_rows(cuda_device):
    V = 3000
    co, ri, feat, cfg, g, tk, smp, train_ids = _make(cuda_device, "rate", "sample", V=V)
    tk.init_cache(smp)
    # the oracle's sampler on the same seeds and draw numbers gives the same source lists
    ref = np.zeros(V, np.int64)
    for draw, lo in enumerate(range(0, len(train_ids), cfg.batch_size)):
        blocks, _ = oracle.sample_batch(co, ri, V, train_ids[lo: lo + cfg.batch_size], list(cfg.fanout), cfg.seed, draw)
        for b in blocks:
            ref += np.bincount(b.source, minlength=V)
    hm_ref = cache_slots_by_sample_count(ref.astype(np.uint32), int(V * cfg.cache_rate))
    hm = tk.dev_cache_node_hashmap.cpu().numpy().view(np.uint32)
    np.testing.assert_array_equal(hm, hm_ref)
    assert tk.cache_node_num == int(V * cfg.cache_rate)
    cached = np.nonzero(hm != 0xFFFFFFFF)[0]
    rows = tk.dev_cache_feature.cpu().numpy()[:, :feat.shape[1]]
    np.testing.assert_array_equal(rows[hm[cached]], feat[cached])
    assert ref[cached].min() >= np.delete(ref, cached).max()      # the most frequently sampled nodes are cached
    assert smp.work_offset == smp.work_range[0]                    # the dry run leaves the sampler restarted


@pytest.mark.parametrize("cache_type,policy", [("rate", "random"), ("rate", "sample"), ("gpu_memory", "degree"),
                                               ("random", "degree")])
def test_training_does_not_depend_on_the_cache(cuda_device, cache_type, policy):
    outs = []
    for ct, pol in (("none", "degree"), (cache_type, policy)):
        co, ri, feat, cfg, g, tk, smp, train_ids = _make(cuda_device, ct, pol, pipelines=2)
        tk.init_cache(smp)
        if ct == "gpu_memory":
            assert tk.cache_node_num == g.global_vertices          # a small graph fits whole
        rng = np.random.RandomState(3)
        curve = [tk.Forward(smp, rng=rng, train=True) for _ in range(2)]
        outs.append((tk.P.W.cpu().numpy().copy(), curve))
    np.testing.assert_array_equal(outs[0][0].view(np.uint32), outs[1][0].view(np.uint32))
    assert outs[0][1] == outs[1][1]
