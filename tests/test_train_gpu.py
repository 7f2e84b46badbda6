"""End-to-end parity of the training path: the CUDA trainer and the CPU oracle run the same batches
(identical sampled edge lists — both use the same Philox sampler) from the same initial weights.
Bar (north star): loss curves within 1e-3 over 5 epochs; aggregation outputs 1e-5 relative."""
import numpy as np
import pytest
import torch

import oracle
from helpers import dev_i32, dev_i64, small_graph
from neutronbench_b200 import (FullyRepGraph, GCN_GPU_NEIGHBOR_impl, GCNConfig, GNNDatum, Sampler,
                               SingleGPUSampleGraphOp, Workspace)

pytestmark = pytest.mark.gpu


def _setup(cuda_device, V=4000, E=60000, F=100, hidden=32, classes=7, fanout=(10, 5), batch=256, drop=0.5,
           cache_rate=0.0, fuse=True, layers=None, use_engine=True, pipelines=1):
    edges, co, ri = small_graph(V, E, seed=6)
    rng = np.random.RandomState(0)
    feat = rng.randn(V, F).astype(np.float32)
    label = rng.randint(0, classes, size=V).astype(np.int64)
    sizes = layers or [F] + [hidden] * (len(fanout) - 1) + [classes]
    cfg = GCNConfig(layers=sizes, fanout=fanout, batch_size=batch, drop_rate=drop, learn_rate=0.01,
                    weight_decay=0.0001, cache_type="rate" if cache_rate > 0 else "none", cache_rate=cache_rate,
                    fuse_gather=fuse, seed=2000, pipelines=pipelines)
    g = FullyRepGraph.from_edges(torch.from_numpy(edges).to(cuda_device), V, Workspace(64 << 20))
    datum = GNNDatum(torch.from_numpy(feat).to(cuda_device), torch.from_numpy(label).to(cuda_device),
                     np.zeros(V, np.int32))
    tk = GCN_GPU_NEIGHBOR_impl(g, datum, cfg, use_engine=use_engine)
    tk.init_cache()
    ref = oracle.GCN(sizes, tk.P.W.cpu().numpy(), cfg.learn_rate, cfg.weight_decay, drop, cfg.seed)
    return edges, co, ri, feat, label, cfg, g, tk, ref


@pytest.mark.parametrize("fanout,drop,cache_rate,fuse", [((10, 5), 0.5, 0.0, True), ((10, 5), 0.0, 0.3, True),
                                                         ((5, 4, 3), 0.5, 1.0, False), ((5, 4, 3), 0.2, 0.0, True)])
@pytest.mark.parametrize("use_engine", [True, False], ids=["native_step", "python_step"])
def test_loss_curve_matches_oracle_over_5_epochs(cuda_device, fanout, drop, cache_rate, fuse, use_engine):
    V = 4000
    edges, co, ri, feat, label, cfg, g, tk, ref = _setup(cuda_device, V=V, fanout=fanout, drop=drop,
                                                         cache_rate=cache_rate, fuse=fuse, use_engine=use_engine)
    train_ids = np.arange(0, 1200, dtype=np.uint32)
    smp = Sampler(g, train_ids, fanout, cfg.batch_size, tk.ws, seed=cfg.seed, with_edge_weights=False)
    rng_gpu, rng_cpu = np.random.RandomState(2000), np.random.RandomState(2000)
    ids_cpu = train_ids.copy()
    draw = 0
    for epoch in range(5):
        acc, loss, batches = tk.Forward(smp, rng=rng_gpu, train=True)
        rng_cpu.shuffle(ids_cpu)
        ref_loss = ref_correct = 0
        for lo in range(0, len(ids_cpu), cfg.batch_size):
            blocks, _ = oracle.sample_batch(co, ri, V, ids_cpu[lo: lo + cfg.batch_size], list(fanout), cfg.seed, draw)
            l, c, _, _ = ref.train_step(blocks, feat, label)
            ref_loss += l
            ref_correct += c
            draw += 1
        ref_loss /= batches
        assert batches == 5
        assert abs(loss - ref_loss) < 1e-3, (epoch, loss, ref_loss)
        assert abs(acc - ref_correct / len(ids_cpu)) < 0.01
    w_gpu = tk.P.W.cpu().numpy()
    assert np.abs(w_gpu - ref.W).max() < 1e-3


def test_operator_surface_forward_backward(cuda_device):
    """SingleGPUSampleGraphOp (explicit edge weights, the reference's call shape) against
    MiniBatchFuseOp's restatement, layer by layer; fused-weight variant gives identical bits."""
    V, F = 4000, 64
    edges, co, ri, feat, label, cfg, g, tk, ref = _setup(cuda_device, V=V)
    seeds = np.arange(100, 356, dtype=np.uint32)
    smp = Sampler(g, seeds, (10, 5), 256, tk.ws, seed=5)
    ssg = smp.sample_one()
    blocks, _ = oracle.sample_batch(co, ri, V, seeds, [10, 5], 5, 0)
    rng = np.random.RandomState(1)
    for layer in range(2):
        b = blocks[layer]
        x = rng.randn(b.src_size + 3, F).astype(np.float32)     # more rows than src_size, like X[0]
        gy = rng.randn(b.v_size, F).astype(np.float32)
        y_ref = oracle.spmm_fwd(x, b.edge_weight_forward, b.row_indices, b.column_offset)
        gx_ref = oracle.spmm_bwd(gy, b.edge_weight_backward, b.row_offset, b.column_indices)
        for fused in (False, True):
            op = SingleGPUSampleGraphOp(ssg, None, layer, None, fused_weights=fused)
            y = op.forward(torch.from_numpy(x).to(cuda_device))
            gx = op.backward(torch.from_numpy(gy).to(cuda_device))
            assert y.requires_grad and y.is_leaf and tuple(y.shape) == (b.v_size, F)
            assert not gx.requires_grad and tuple(gx.shape) == (b.src_size, F)
            np.testing.assert_array_equal(y.detach().cpu().numpy().view(np.uint32), y_ref.view(np.uint32))
            np.testing.assert_array_equal(gx.cpu().numpy().view(np.uint32), gx_ref.view(np.uint32))


def test_eval_forward_has_no_side_effects(cuda_device):
    edges, co, ri, feat, label, cfg, g, tk, ref = _setup(cuda_device)
    w0 = tk.P.W.clone()
    smp = Sampler(g, np.arange(500, dtype=np.uint32), cfg.fanout, 500, tk.ws, seed=1)
    acc, loss, batches = tk.Forward(smp, train=False)
    assert batches == 1 and np.isfinite(loss) and 0.0 <= acc <= 1.0
    assert torch.equal(w0, tk.P.W)


def test_native_step_and_python_step_are_the_same_computation(cuda_device):
    """nb_gcn_step issues the kernels the Python mirror issues, in the same order: after three
    optimizer steps the weights are identical bit for bit."""
    outs = []
    for use_engine in (True, False):
        edges, co, ri, feat, label, cfg, g, tk, ref = _setup(cuda_device, fanout=(5, 4, 3), drop=0.3, cache_rate=0.4,
                                                             use_engine=use_engine)
        smp = Sampler(g, np.arange(700, dtype=np.uint32), cfg.fanout, cfg.batch_size, tk.ws, seed=cfg.seed,
                      with_edge_weights=False)
        for _ in range(3):
            tk.train_step(smp)
        loss, hits = tk.read_stats()
        outs.append((tk.P.W.cpu().numpy().copy(), loss, hits))
    np.testing.assert_array_equal(outs[0][0].view(np.uint32), outs[1][0].view(np.uint32))
    assert outs[0][1] == outs[1][1] and outs[0][2] == outs[1][2]


@pytest.mark.parametrize("staged", [False, True], ids=["host_seeds", "device_seeds"])
def test_pipelined_loop_equals_plain_loop(cuda_device, staged):
    """Sampling batch i+1 on a second stream while batch i trains (nb_gcn_sample / nb_gcn_compute)
    changes no result: per-epoch loss and accuracy and the final weights are bit-identical."""
    outs = []
    for pipelines in (1, 2, 4):
        edges, co, ri, feat, label, cfg, g, tk, ref = _setup(cuda_device, fanout=(10, 5), drop=0.5, cache_rate=0.3,
                                                             pipelines=pipelines)
        smp = Sampler(g, np.arange(1100, dtype=np.uint32), cfg.fanout, cfg.batch_size, tk.ws, seed=cfg.seed,
                      with_edge_weights=False)
        rng = np.random.RandomState(11)
        curve = []
        for _ in range(3):
            if staged:
                smp.shuffle(rng)
                smp.stage_seeds_on_device()
                curve.append(tk.Forward(smp, train=True))
            else:
                curve.append(tk.Forward(smp, rng=rng, train=True))
        outs.append((tk.P.W.cpu().numpy().copy(), curve))
    for other in outs[1:]:
        np.testing.assert_array_equal(outs[0][0].view(np.uint32), other[0].view(np.uint32))
        assert outs[0][1] == other[1]
    assert outs[0][1][0][2] == 5


def test_sample_rate_training_matches_oracle(cuda_device):
    """The native step with SAMPLE_RATE set draws degree-proportional neighbourhoods for training batches
    (and only for those): loss curve equal to the oracle's on the same draws, pipelined."""
    V, fanout = 4000, (10, 5)
    edges, co, ri = small_graph(V, 60000, seed=6)
    rng = np.random.RandomState(0)
    feat = rng.randn(V, 40).astype(np.float32)
    label = rng.randint(0, 6, size=V).astype(np.int64)
    sizes = [40, 24, 6]
    cfg = GCNConfig(layers=sizes, fanout=fanout, batch_size=200, drop_rate=0.2, seed=2000, pipelines=2,
                    sample_rate=0.3, lower_fanout=2)
    g = FullyRepGraph.from_edges(torch.from_numpy(edges).to(cuda_device), V, Workspace(64 << 20))
    datum = GNNDatum(torch.from_numpy(feat).to(cuda_device), torch.from_numpy(label).to(cuda_device), np.zeros(V, np.int32))
    tk = GCN_GPU_NEIGHBOR_impl(g, datum, cfg)
    ref = oracle.GCN(sizes, tk.P.W.cpu().numpy(), cfg.learn_rate, cfg.weight_decay, cfg.drop_rate, cfg.seed)
    ids = np.arange(0, 1000, dtype=np.uint32)
    smp = Sampler(g, ids, fanout, cfg.batch_size, tk.ws, seed=cfg.seed, with_edge_weights=False,
                  sample_rate=cfg.sample_rate, lower_fanout=cfg.lower_fanout)
    draw = 0
    for epoch in range(2):
        acc, loss, batches = tk.Forward(smp, train=True)
        ref_loss = 0.0
        for lo in range(0, len(ids), cfg.batch_size):
            blocks, _ = oracle.sample_batch(co, ri, V, ids[lo: lo + cfg.batch_size], list(fanout), cfg.seed, draw,
                                            sample_rate=cfg.sample_rate, lower_fanout=cfg.lower_fanout)
            l, c, _, _ = ref.train_step(blocks, feat, label)
            ref_loss += l
            draw += 1
        assert batches == 5 and abs(loss - ref_loss / batches) < 1e-3
    assert np.abs(tk.P.W.cpu().numpy() - ref.W).max() < 1e-3


@pytest.mark.parametrize("pipelines", [1, 2], ids=["plain", "pipelined"])
def test_multi_label_training_matches_oracle(cuda_device, pipelines):
    """CLASSES > 1: BCE loss and per-batch F1 (utils/torch_func.hpp:31-75) through the native step."""
    V, fanout, classes = 3000, (8, 4), 9
    edges, co, ri = small_graph(V, 40000, seed=3)
    rng = np.random.RandomState(0)
    feat = rng.randn(V, 30).astype(np.float32)
    label = (rng.rand(V, classes) < 0.3).astype(np.int64)
    sizes = [30, 16, classes]
    cfg = GCNConfig(layers=sizes, fanout=fanout, batch_size=150, drop_rate=0.1, seed=2000, pipelines=pipelines,
                    classes=classes)
    g = FullyRepGraph.from_edges(torch.from_numpy(edges).to(cuda_device), V, Workspace(64 << 20))
    datum = GNNDatum(torch.from_numpy(feat).to(cuda_device), torch.from_numpy(label).to(cuda_device), np.zeros(V, np.int32))
    tk = GCN_GPU_NEIGHBOR_impl(g, datum, cfg)
    ref = oracle.GCN(sizes, tk.P.W.cpu().numpy(), cfg.learn_rate, cfg.weight_decay, cfg.drop_rate, cfg.seed,
                     multi_label=True)
    ids = np.arange(0, 700, dtype=np.uint32)
    smp = Sampler(g, ids, fanout, cfg.batch_size, tk.ws, seed=cfg.seed, with_edge_weights=False)
    draw = 0
    for epoch in range(3):
        f1, loss, batches = tk.Forward(smp, train=True)
        ref_loss = ref_f1 = 0.0
        for lo in range(0, len(ids), cfg.batch_size):
            blocks, _ = oracle.sample_batch(co, ri, V, ids[lo: lo + cfg.batch_size], list(fanout), cfg.seed, draw)
            l, f, _, _ = ref.train_step(blocks, feat, label)
            ref_loss += l
            ref_f1 += f
            draw += 1
        assert batches == 5
        assert abs(loss - ref_loss / batches) < 1e-3
        assert abs(f1 - ref_f1 / batches) < 0.02
    assert np.abs(tk.P.W.cpu().numpy() - ref.W).max() < 1e-3
    # the Python mirror of the step gives the same numbers as the native one
    tk2 = GCN_GPU_NEIGHBOR_impl(g, datum, cfg, use_engine=False)
    tk3 = GCN_GPU_NEIGHBOR_impl(g, datum, GCNConfig(**{**cfg.__dict__, "pipelines": 1}))
    for t in (tk2, tk3):
        s2 = Sampler(g, ids, fanout, cfg.batch_size, t.ws, seed=cfg.seed, with_edge_weights=False)
        t.Forward(s2, train=True)
    np.testing.assert_array_equal(tk2.P.W.cpu().numpy().view(np.uint32), tk3.P.W.cpu().numpy().view(np.uint32))


@pytest.mark.parametrize("pipelines", [1, 3], ids=["plain", "pipelined"])
def test_update_on_its_own_stream_changes_nothing(cuda_device, pipelines):
    """overlap_update runs the gradient sum and Adam on a second stream, ordered by events against the step that
    produced the gradients and the step that next reads the weights: weights and loss curve stay bit-identical."""
    outs = []
    for overlap in (False, True):
        edges, co, ri, feat, label, cfg, g, tk, ref = _setup(cuda_device, fanout=(10, 5), drop=0.5, cache_rate=0.3,
                                                             pipelines=pipelines)
        tk.overlap_update = overlap
        smp = Sampler(g, np.arange(1100, dtype=np.uint32), cfg.fanout, cfg.batch_size, tk.ws, seed=cfg.seed,
                      with_edge_weights=False)
        rng = np.random.RandomState(5)
        curve = [tk.Forward(smp, rng=rng, train=True) for _ in range(3)]
        val = tk.Forward(Sampler(g, np.arange(2000, 2200, dtype=np.uint32), cfg.fanout, 200, tk.ws, seed=1), train=False)
        outs.append((tk.P.W.cpu().numpy().copy(), curve, val))
    np.testing.assert_array_equal(outs[0][0].view(np.uint32), outs[1][0].view(np.uint32))
    assert outs[0][1] == outs[1][1] and outs[0][2] == outs[1][2]


def test_programmatic_dependent_launch_changes_nothing(cuda_device):
    """nb_set_pdl(1) lets each kernel of the training half be scheduled while its predecessor drains; every kernel
    waits for the predecessor before touching memory, so weights and losses stay bit-identical."""
    from neutronbench_b200 import _lib
    outs = []
    try:
        for pdl in (0, 1):
            _lib.load().nb_set_pdl(pdl)
            edges, co, ri, feat, label, cfg, g, tk, ref = _setup(cuda_device, V=6000, E=90000, F=300, hidden=128, classes=41,
                                                                 fanout=(10, 5), batch=512, drop=0.5, cache_rate=1.0, pipelines=2)
            smp = Sampler(g, np.arange(2000, dtype=np.uint32), cfg.fanout, cfg.batch_size, tk.ws, seed=cfg.seed,
                          with_edge_weights=False)
            curve = [tk.Forward(smp, train=True) for _ in range(2)]
            outs.append((tk.P.W.cpu().numpy().copy(), curve))
    finally:
        _lib.load().nb_set_pdl(1)   # the default
    np.testing.assert_array_equal(outs[0][0].view(np.uint32), outs[1][0].view(np.uint32))
    assert outs[0][1] == outs[1][1]



def test_native_step_on_seeds_without_neighbours(cuda_device):
    """Seeds with no in-edges give blocks without edges (and an input-side block without vertices): the step
    still runs, the loss is log(C) under zero aggregates, and nothing is read out of bounds."""
    V, F, C = 500, 12, 4
    rng = np.random.RandomState(0)
    src = rng.randint(0, 250, 3000)
    dst = rng.randint(0, 250, 3000)                       # vertices 250.. have no edges at all
    edges = np.stack([src, dst], axis=1).astype(np.int32)
    feat = rng.randn(V, F).astype(np.float32)
    label = rng.randint(0, C, size=V).astype(np.int64)
    cfg = GCNConfig(layers=[F, 8, C], fanout=(4, 3), batch_size=64, drop_rate=0.0, seed=3)
    g = FullyRepGraph.from_edges(torch.from_numpy(edges).to(cuda_device), V, Workspace(32 << 20))
    datum = GNNDatum(torch.from_numpy(feat).to(cuda_device), torch.from_numpy(label).to(cuda_device), np.zeros(V, np.int32))
    for use_engine in (True, False):
        tk = GCN_GPU_NEIGHBOR_impl(g, datum, cfg, use_engine=use_engine)
        w0 = tk.P.W.clone()
        smp = Sampler(g, np.arange(300, 428, dtype=np.uint32), cfg.fanout, cfg.batch_size, tk.ws, seed=cfg.seed,
                      with_edge_weights=False)
        acc, loss, batches = tk.Forward(smp, train=True)
        assert batches == 2 and abs(loss - np.log(C)) < 1e-5 and 0.0 <= acc <= 1.0
        assert torch.isfinite(tk.P.W).all()
        # mixed batch: some seeds with neighbours, some without
        smp2 = Sampler(g, np.arange(200, 328, dtype=np.uint32), cfg.fanout, cfg.batch_size, tk.ws, seed=cfg.seed,
                       with_edge_weights=False)
        acc2, loss2, _ = tk.Forward(smp2, train=True)
        assert np.isfinite(loss2) and torch.isfinite(tk.P.W).all() and not torch.equal(w0, tk.P.W)
