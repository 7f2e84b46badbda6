"""The full-graph operator and trainer (ForwardSingleGPUfuseOp, GCN_GPU_impl) on a Cora-shaped graph — 2,708
vertices, 5,278 undirected random edges made symmetric plus self loops (13,264 edges), binary bag-of-words features
of width 1,433 with about 1.3 % ones, 7 classes, hidden 16 — against the CPU oracle's restatement of the same step
(whole-graph degree weights core/ntsBaseOp.hpp:183-186, aggregation core/NtsScheduler.hpp:146-178, 239-271, dense
layers, masked NLL, Adam).  Bars: operator outputs bit-exact against the oracle's aggregation (same arithmetic, same
order), loss within 1e-3 per epoch, final weights within 1e-3."""
import numpy as np
import pytest
import torch

import oracle
from neutronbench_b200 import (ForwardSingleGPUfuseOp, FullyRepGraph, GCN_GPU_impl, GCNConfig, GNNDatum, PartitionedGraph,
                               Workspace, synth)

pytestmark = pytest.mark.gpu


def cora_shaped(seed=3):
    V, F, C = 2708, 1433, 7
    edges = synth.uniform_undirected_numpy(V, 5278, seed)
    rng = np.random.RandomState(seed + 1)
    feat = (rng.random_sample((V, F)) < 0.013).astype(np.float32)
    label = rng.randint(0, C, size=V).astype(np.int64)
    mask = synth.split_mask(V, seed)
    return V, F, C, edges, feat, label, mask


def whole_graph_reference(edges, V):
    """CSC, CSR and the two weight arrays as the reference's full-graph operator holds them."""
    co64, ri = oracle.build_csc(edges, V)
    co = co64.astype(np.uint32)
    ro, ci = oracle.csr_from_csc(co, ri, V)
    out_d, in_d = oracle.degrees(edges, V, clamp=True)
    s_out = np.sqrt(out_d.astype(np.float64)).astype(np.float32)
    s_in = np.sqrt(in_d.astype(np.float64)).astype(np.float32)
    dst = np.repeat(np.arange(V), np.diff(co.astype(np.int64)))
    src = np.repeat(np.arange(V), np.diff(ro.astype(np.int64)))
    wf = np.float32(1.0) / (s_out[ri] * s_in[dst])
    wb = np.float32(1.0) / (s_out[src] * s_in[ci])
    return co, ri, ro, ci, wf, wb


def test_full_graph_operator_forward_backward(cuda_device):
    V, F, C, edges, feat, label, mask = cora_shaped()
    assert len(edges) == 2 * 5278 + V == 13264
    co, ri, ro, ci, wf, wb = whole_graph_reference(edges, V)
    g = FullyRepGraph.from_edges(torch.from_numpy(edges).to(cuda_device), V, Workspace(64 << 20))
    pg = PartitionedGraph(g, Workspace(64 << 20))
    np.testing.assert_array_equal(pg.column_offset.cpu().numpy().view(np.uint32), co)
    np.testing.assert_array_equal(pg.row_offset.cpu().numpy().view(np.uint32), ro)
    np.testing.assert_array_equal(pg.column_indices.cpu().numpy().view(np.uint32)[: len(ci)], ci)
    np.testing.assert_array_equal(pg.edge_weight_forward.cpu().numpy().view(np.uint32), wf.view(np.uint32))
    np.testing.assert_array_equal(pg.edge_weight_backward.cpu().numpy().view(np.uint32), wb.view(np.uint32))
    op = ForwardSingleGPUfuseOp(pg, None)
    rng = np.random.RandomState(5)
    for width in (1433, 16, 7):
        x = rng.randn(V, width).astype(np.float32)
        gy = rng.randn(V, width).astype(np.float32)
        y = op.forward(torch.from_numpy(x).to(cuda_device))
        gx = op.backward(torch.from_numpy(gy).to(cuda_device))
        assert y.requires_grad and y.is_leaf and tuple(y.shape) == (V, width) and not gx.requires_grad
        np.testing.assert_array_equal(y.detach().cpu().numpy().view(np.uint32), oracle.spmm_fwd(x, wf, ri, co).view(np.uint32))
        np.testing.assert_array_equal(gx.cpu().numpy().view(np.uint32), oracle.spmm_bwd(gy, wb, ro, ci).view(np.uint32))


@pytest.mark.parametrize("drop", [0.0, 0.5])
def test_full_graph_training_matches_the_oracle(cuda_device, drop):
    V, F, C, edges, feat, label, mask = cora_shaped()
    co, ri, ro, ci, wf, wb = whole_graph_reference(edges, V)
    sizes = [F, 16, C]
    cfg = GCNConfig(layers=sizes, fanout=(-1, -1), batch_size=V, drop_rate=drop, learn_rate=0.01, weight_decay=0.0005,
                    seed=2000)
    g = FullyRepGraph.from_edges(torch.from_numpy(edges).to(cuda_device), V, Workspace(64 << 20))
    pg = PartitionedGraph(g, Workspace(64 << 20))
    datum = GNNDatum(torch.from_numpy(feat).to(cuda_device), torch.from_numpy(label).to(cuda_device), mask)
    tk = GCN_GPU_impl(pg, datum, cfg)
    # the same step on the CPU
    W = tk.P.W.cpu().numpy().copy()
    M, Vv, grad = np.zeros_like(W), np.zeros_like(W), np.zeros_like(W)
    offs = tk.P.offsets
    b1t, b2t = np.float32(0.9), np.float32(0.999)
    train = np.nonzero(mask == 0)[0]
    scale = 1.0 / (1.0 - drop) if drop > 0 else 1.0
    for epoch in range(6):
        tk.epoch(train=True)
        loss_gpu, hits_gpu = tk.read_stats()
        w = [W[offs[l]: offs[l + 1]].reshape(sizes[l], sizes[l + 1]) for l in range(2)]
        y0 = oracle.spmm_fwd(feat, wf, ri, co)
        x1 = oracle.relu_dropout(oracle.gemm_nn(y0, w[0]), drop, 2000, 0, epoch)
        y1 = oracle.spmm_fwd(x1, wf, ri, co)
        z = oracle.gemm_nn(y1, w[1])
        loss, dz_train, hits = oracle.softmax_nll(z[train], label[train])
        dz = np.zeros_like(z)
        dz[train] = dz_train
        grad[offs[1]: offs[2]] = oracle.gemm_tn(y1, dz).reshape(-1)
        dx1 = oracle.spmm_bwd(oracle.gemm_nt(dz, w[1]), wb, ro, ci, act=x1, scale=scale)
        grad[offs[0]: offs[1]] = oracle.gemm_tn(y0, dx1).reshape(-1)
        oracle.adam(W, grad, M, Vv, 0.01, 0.9, 0.999, 1e-9, 0.0005, float(b1t), float(b2t))
        b1t, b2t = np.float32(b1t * np.float32(0.9)), np.float32(b2t * np.float32(0.999))
        assert abs(loss_gpu - loss) < 1e-3, (epoch, loss_gpu, loss)
        assert abs(hits_gpu - hits) <= 2
    assert np.abs(tk.P.W.cpu().numpy() - W).max() < 1e-3
    logits = tk.epoch(train=False)
    acc = tk.Test(1, logits)
    assert 0.0 <= acc <= 1.0
