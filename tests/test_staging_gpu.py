"""Staging of uncached rows, the node-id-sharded feature table, per-handle tuning switches and the device error
word, all through the C ABI.  None of them may change a result: every variant trains to bit-identical weights."""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import dev_f32, dev_i32, dev_i64, small_graph
from neutronbench_b200 import (FullyRepGraph, GCN_GPU_NEIGHBOR_impl, GCNConfig, GNNDatum, Sampler, Workspace, _lib)
from neutronbench_b200.cuda_stream import ptr
from neutronbench_b200.peer import ShardedFeatureTable, shard_rows_for

pytestmark = pytest.mark.gpu


def _train(cuda_device, F, hidden, classes, fanout, cache_rate, where, stage, options=(), shards=0, pipelines=1,
           steps=4, V=5000, batch=300, E=70000):
    edges, co, ri = small_graph(V, E, seed=8)
    rng = np.random.RandomState(1)
    feat = rng.randn(V, F).astype(np.float32)
    label = rng.randint(0, classes, size=V).astype(np.int64)
    cfg = GCNConfig(layers=[F] + [hidden] * (len(fanout) - 1) + [classes], fanout=fanout, batch_size=batch,
                    drop_rate=0.3, cache_type="rate" if cache_rate > 0 else "none", cache_rate=cache_rate, seed=2000,
                    pipelines=pipelines, stage_misses=stage)
    g = FullyRepGraph.from_edges(torch.from_numpy(edges).to(cuda_device), V, Workspace(64 << 20))
    lab = torch.from_numpy(label).to(cuda_device)
    if shards:
        rows = shard_rows_for(V, shards)
        parts = [torch.from_numpy(feat[k * rows: (k + 1) * rows]).to(cuda_device) for k in range(shards)]
        table = ShardedFeatureTable.from_local_parts(parts, rows)
        datum = GNNDatum(None, lab, np.zeros(V, np.int32), shards=table)
        cache_source = torch.from_numpy(feat).to(cuda_device)
    else:
        f = torch.from_numpy(feat)
        datum = GNNDatum(f.to(cuda_device) if where == "device" else f.pin_memory(), lab, np.zeros(V, np.int32))
        cache_source = None
    tk = GCN_GPU_NEIGHBOR_impl(g, datum, cfg)
    if shards and cache_rate > 0:      # the cache is filled from a whole table; the shards serve the misses
        tk.datum = GNNDatum(cache_source, lab, np.zeros(V, np.int32))
        tk.init_cache()
        tk.datum = datum
    else:
        tk.init_cache()
    for name, value in options:
        _lib.call("nb_gcn_set_option", tk._ensure_engine(), name.encode(), int(value))
    smp = Sampler(g, np.arange(steps * batch, dtype=np.uint32), fanout, batch, tk.ws, seed=cfg.seed, with_edge_weights=False)
    losses = []
    if pipelines > 1:
        tk.run_pipelined(smp, train=True, on_batch=None)
    else:
        for _ in range(steps):
            tk.train_step(smp)
            losses.append(tk.read_stats())
    torch.cuda.synchronize()
    tk.check_device_errors()
    return tk.P.W.cpu().numpy().copy(), losses


@pytest.mark.parametrize("F,fanout,cache_rate", [(100, (5, 4, 3), 0.2), (602, (10, 5), 0.3), (100, (6, 4), 0.0),
                                                 (300, (6, 4), 0.0), (602, (8, 4), 1.0)])
@pytest.mark.parametrize("where", ["device", "pinned_host"])
def test_staged_misses_change_no_result(cuda_device, F, fanout, cache_rate, where):
    """Rows without a cache slot read once per distinct source into the staging table (nb_gcn_config.stage_misses)
    against once per edge from the table itself: identical weights and losses."""
    w0, l0 = _train(cuda_device, F, 64, 7, fanout, cache_rate, where, stage=False)
    w1, l1 = _train(cuda_device, F, 64, 7, fanout, cache_rate, where, stage=True)
    np.testing.assert_array_equal(w0.view(np.uint32), w1.view(np.uint32))
    assert l0 == l1


@pytest.mark.parametrize("F,cache_rate,shards", [(128, 0.0, 4), (100, 0.25, 3), (602, 0.3, 2)])
def test_sharded_feature_table_equals_whole_table(cuda_device, F, cache_rate, shards):
    """owner = id // shard_rows over a pointer table (here all shards in one GPU's memory; the 2-GPU test maps real
    peers): same weights as the unsharded run, plain loop and pipelined loop."""
    w0, l0 = _train(cuda_device, F, 64, 7, (6, 4), cache_rate, "device", stage=False)
    w1, l1 = _train(cuda_device, F, 64, 7, (6, 4), cache_rate, "device", stage=True, shards=shards)
    w2, _ = _train(cuda_device, F, 64, 7, (6, 4), cache_rate, "device", stage=True, shards=shards, pipelines=3)
    np.testing.assert_array_equal(w0.view(np.uint32), w1.view(np.uint32))
    np.testing.assert_array_equal(w0.view(np.uint32), w2.view(np.uint32))
    assert l0 == l1


def test_sharded_table_needs_staging(cuda_device):
    with pytest.raises(_lib.NbError):
        _train(cuda_device, 64, 32, 5, (4, 3), 0.0, "device", stage=False, shards=2, steps=1)


@pytest.mark.parametrize("options", [(("l2_hint", 0),), (("l2_hint", 2),), (("y_stream_stores", 0),),
                                     (("reserve_sms", 8),), (("ring_group_shift", 0),), (("gemm_mode", 1), ("pdl", 0)),
                                     (("l2_hint", 3), ("l2_keep_min_uses", 3)), (("wide_direct", 1),), (("ring_prefetch", 4),),
                                     (("ring_prefetch", 14), ("l2_hint", 0)), (("ring_balance", 0),),
                                     (("ring_balance", 1),), (("ring_balance", 1), ("reserve_sms", 5)),
                                     (("fuse_relu", 1),), (("hub_min_edges", 0),), (("ring_warps", 22),),
                                     (("fuse_last_aggregation", 0),),
                                     (("ring_warps", 24),), (("ring_warps", 24), ("reserve_sms", 4), ("ring_balance", 1)),
                                     (("wide_direct", 1), ("wide_rows_in_flight", 1)),
                                     (("wide_direct", 1), ("wide_rows_in_flight", 4), ("y_stream_stores", 0))])
def test_handle_options_change_no_result(cuda_device, options):
    """nb_gcn_set_option acts on one handle only and never on results (wide rows: the ring kernel runs)."""
    w0, l0 = _train(cuda_device, 602, 128, 41, (10, 5), 1.0, "device", stage=None)
    w1, l1 = _train(cuda_device, 602, 128, 41, (10, 5), 1.0, "device", stage=None, options=options)
    np.testing.assert_array_equal(w0.view(np.uint32), w1.view(np.uint32))
    assert l0 == l1


@pytest.mark.parametrize("F,hidden,classes,fanout", [(100, 128, 47, (5, 4, 3)), (64, 256, 7, (6, 4)), (32, 100, 64, (4, 4)),
                                                     (48, 36, 3, (30, 3))])
def test_output_layer_that_aggregates_its_own_rows_changes_no_result(cuda_device, F, hidden, classes, fanout):
    """The last block's aggregation inside the fused output-layer kernel (hidden widths up to 256, rows longer than
    one 32-edge pass) against the separate aggregation launch: bit-identical weights and losses."""
    w0, l0 = _train(cuda_device, F, hidden, classes, fanout, 0.3, "device", stage=None,
                    options=(("fuse_last_aggregation", 0),))
    w1, l1 = _train(cuda_device, F, hidden, classes, fanout, 0.3, "device", stage=None)
    np.testing.assert_array_equal(w0.view(np.uint32), w1.view(np.uint32))
    assert l0 == l1


@pytest.mark.parametrize("F,hidden,fanout", [(100, 128, (4, 4)), (64, 64, (3, 3, 3)), (100, 100, (4, 4))])
def test_relu_and_dropout_in_the_gemm_epilogue_change_no_result(cuda_device, F, hidden, fanout):
    """Blocks of more than 148 x 160 rows take the tensor-core kernel with 128-row tiles, smaller ones the row-balanced
    one; both can apply ReLU + dropout as the product leaves TMEM (`fuse_relu`), drawing the same Philox words as the
    separate kernel: weights after three steps are bit-identical."""
    kw = dict(steps=3, V=120000, batch=12000, E=900000)
    w0, l0 = _train(cuda_device, F, hidden, 10, fanout, 0.0, "device", stage=None, **kw)
    w1, l1 = _train(cuda_device, F, hidden, 10, fanout, 0.0, "device", stage=None, options=(("fuse_relu", 1),), **kw)
    np.testing.assert_array_equal(w0.view(np.uint32), w1.view(np.uint32))
    assert l0 == l1


def test_unknown_option_is_refused(cuda_device):
    with pytest.raises(_lib.NbError):
        _train(cuda_device, 64, 32, 5, (4, 3), 0.0, "device", stage=None, options=(("no_such_switch", 1),), steps=1)


def _flags():
    f = C.c_uint32(0)
    _lib.call("nb_device_error_flags", C.byref(f))
    return f.value


def test_id_beyond_the_last_shard_is_reported_not_read(cuda_device):
    """A vertex id that no shard holds sets bit 2 of the device error word; the row is left untouched."""
    _lib.call("nb_device_error_reset")
    F, rows = 16, 100
    parts = [torch.full((rows, F), float(k + 1), device=cuda_device) for k in range(2)]
    table = ShardedFeatureTable.from_local_parts(parts, rows)
    src = dev_i32(np.array([5, 150, 199, 200, 4000000], dtype=np.uint32), cuda_device)
    x0 = torch.full((5, F), -1.0, device=cuda_device)
    _lib.call("nb_feature_gather", ptr(x0), None, F, ptr(table.table), 2, rows, None, 0, None, ptr(src), 5, F,
              torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert _flags() == 4
    got = x0.cpu().numpy()
    assert (got[0] == 1).all() and (got[1] == 2).all() and (got[2] == 2).all()
    assert (got[3] == -1).all() and (got[4] == -1).all()
    _lib.call("nb_device_error_reset")
    assert _flags() == 0


def test_uncached_row_without_a_table_is_reported(cuda_device):
    """Cache-only configuration (feat == NULL) and a source that has no slot: reported, never dereferenced."""
    _lib.call("nb_device_error_reset")
    F = 8
    cache = torch.ones((4, F), device=cuda_device)
    hm = dev_i32(np.array([0, 0xFFFFFFFF, 1, 2], dtype=np.uint32), cuda_device)
    src = dev_i32(np.array([0, 1, 3], dtype=np.uint32), cuda_device)
    x0 = torch.full((3, F), -1.0, device=cuda_device)
    _lib.call("nb_feature_gather", ptr(x0), None, F, None, 0, 0, ptr(cache), F, ptr(hm), ptr(src), 3, F,
              torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert _flags() == 4
    assert (x0.cpu().numpy()[1] == -1).all() and (x0.cpu().numpy()[0] == 1).all()
    _lib.call("nb_device_error_reset")


def test_label_outside_the_class_range_is_reported(cuda_device, ws):
    """Unlabelled vertices are commonly marked -1: such a row counts with loss 0, no hit and a zero gradient."""
    _lib.call("nb_device_error_reset")
    B, Cn = 6, 5
    rng = np.random.RandomState(0)
    z = rng.randn(B, Cn).astype(np.float32)
    lab = np.array([0, 4, -1, 2, 5, 1], dtype=np.int64)
    dz = torch.empty((B, Cn), device=cuda_device)
    stats = torch.zeros(2, device=cuda_device)
    _lib.call("nb_softmax_nll", ws.handle, ptr(dev_f32(z, cuda_device)), ptr(dev_i64(lab, cuda_device)), B, Cn, ptr(dz),
              ptr(stats), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert _flags() == 8
    g = dz.cpu().numpy()
    assert (g[2] == 0).all() and (g[4] == 0).all() and np.abs(g[0]).sum() > 0
    ok = [0, 1, 3, 5]
    zs = z[ok] - z[ok].max(axis=1, keepdims=True)
    ref = -(zs[np.arange(4), lab[ok]] - np.log(np.exp(zs).sum(axis=1))).sum() / B
    assert abs(float(stats[0]) - ref) < 1e-5
    _lib.call("nb_device_error_reset")
    assert _flags() == 0


def test_phase_times_of_the_epoch_line(cuda_device):
    """nb_gcn_read_phase_times: sample (host wall time of the sampling halves), trans (staging), graph (aggregation
    launches) and nn (rest of the training half) are all measured, and reading them resets them."""
    edges, co, ri = small_graph(5000, 70000, seed=8)
    rng = np.random.RandomState(1)
    V, F = 5000, 100
    cfg = GCNConfig(layers=[F, 64, 7], fanout=(6, 4), batch_size=300, drop_rate=0.3, cache_type="rate", cache_rate=0.3,
                    seed=2000, pipelines=3, stage_misses=True)
    g = FullyRepGraph.from_edges(torch.from_numpy(edges).to(cuda_device), V, Workspace(64 << 20))
    datum = GNNDatum(torch.from_numpy(rng.randn(V, F).astype(np.float32)).pin_memory(),
                     torch.from_numpy(rng.randint(0, 7, size=V).astype(np.int64)).to(cuda_device), np.zeros(V, np.int32))
    tk = GCN_GPU_NEIGHBOR_impl(g, datum, cfg)
    tk.init_cache()
    _lib.call("nb_gcn_set_timing", tk._ensure_engine(), 1)
    smp = Sampler(g, np.arange(1500, dtype=np.uint32), cfg.fanout, 300, tk.ws, seed=cfg.seed, with_edge_weights=False)
    tk.Forward(smp, train=True)
    torch.cuda.synchronize()
    ms = (C.c_double * 4)()
    _lib.call("nb_gcn_read_phase_times", tk._ensure_engine(), ms)
    sample, trans, graph, nn = list(ms)
    assert sample > 0 and trans > 0 and graph > 0 and nn > 0, list(ms)
    _lib.call("nb_gcn_read_phase_times", tk._ensure_engine(), ms)
    assert list(ms) == [0.0, 0.0, 0.0, 0.0]


@pytest.mark.parametrize("cache_rate,stage,where", [(0.3, True, "pinned_host"), (0.3, False, "device"), (0.0, True, "device"),
                                                    (1.0, None, "device")])
@pytest.mark.parametrize("in_flight", [1, 2, 4])
def test_plain_load_wide_row_kernel_equals_the_ring(cuda_device, cache_rate, stage, where, in_flight):
    """The one-warp-per-row plain-load aggregation for wide rows (option wide_direct) against the shared-memory ring:
    cache hits, rows of the staging table and rows of a device table, 1 / 2 / 4 source rows in flight per warp."""
    w0, l0 = _train(cuda_device, 602, 128, 41, (10, 5), cache_rate, where, stage=stage)
    w1, l1 = _train(cuda_device, 602, 128, 41, (10, 5), cache_rate, where, stage=stage,
                    options=(("wide_direct", 1), ("wide_rows_in_flight", in_flight)))
    np.testing.assert_array_equal(w0.view(np.uint32), w1.view(np.uint32))
    assert l0 == l1
