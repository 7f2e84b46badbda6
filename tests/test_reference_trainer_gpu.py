"""The CUDA path (through the C ABI) against a run of the REFERENCE's own trainer and against its aggregation
operator at benchmark widths (tests/golden/train_*.npz, agg_*.npz: Sampler::sample_one, MiniBatchFuseOp,
NtsContext, libtorch mm / log_softmax / nll_loss / autograd, Parameter::learnC2C_with_decay_Adam, compiled from
the reference tree by oracle/Makefile and run by tests/golden/make_golden.py).

Every batch of the reference run is replayed from the reference's initial weights on the reference's sampled
edge lists, once through the native step (nb_gcn_sample_from_edges + nb_gcn_compute + nb_gcn_update) and once
kernel by kernel from the Python mirror.  Bars: loss within 1e-3 for every batch and every epoch mean over 5
epochs, final weights within 1e-3, correct counts equal (a tie in an argmax may flip one prediction: at most one
per batch is tolerated); aggregation within 1e-5 relative (fp32)."""
import os

import numpy as np
import pytest
import torch

from helpers import dev_f32, dev_i32, host_u32
from neutronbench_b200 import (FullyRepGraph, GCN_GPU_NEIGHBOR_impl, GCNConfig, GNNDatum, Sampler,
                               SingleGPUSampleGraphOp, Workspace)
from test_reference_trainer_cpu import AGG, TRAIN, batch_raw, batch_seeds, load_train, make_golden

pytestmark = pytest.mark.gpu


def _trainer(g, cuda_device, use_engine):
    lr, wd = [float(x) for x in g["lr_wd"]]
    cfg = GCNConfig(layers=g["layers"], fanout=g["fanout"], batch_size=g["batch"], drop_rate=0.0, learn_rate=lr,
                    weight_decay=wd, seed=2000)
    edges = torch.from_numpy(g["edges"].reshape(-1, 2).astype(np.int32)).to(cuda_device)
    graph = FullyRepGraph.from_edges(edges, g["V"], Workspace(64 << 20))
    datum = GNNDatum(torch.from_numpy(g["feat"]).to(cuda_device), torch.from_numpy(g["label"]).to(cuda_device),
                     np.zeros(g["V"], np.int32))
    tk = GCN_GPU_NEIGHBOR_impl(graph, datum, cfg, use_engine=use_engine)
    tk.P.W.copy_(torch.from_numpy(g["W0"]))       # the reference's xavier draw, not ours
    return graph, tk, cfg


@pytest.mark.parametrize("use_engine", [True, False], ids=["native_step", "python_step"])
@pytest.mark.parametrize("path", TRAIN, ids=[os.path.basename(p)[:-4] for p in TRAIN])
def test_replay_of_the_reference_trainer(cuda_device, path, use_engine):
    g = load_train(path)
    graph, tk, cfg = _trainer(g, cuda_device, use_engine)
    n = len(g["loss"])
    loss = np.zeros(n)
    smp = Sampler(graph, g["seeds"], g["fanout"], g["batch"], tk.ws, seed=cfg.seed, with_edge_weights=False)
    for k in range(n):
        raw = [dev_i32(r, cuda_device) for r in batch_raw(g, k)]
        if use_engine:
            seeds = dev_i32(batch_seeds(g, k), cuda_device)
            tk.sample_from_edges(seeds, raw, slot=0)
            tk.compute_batch(0, train=True)
        else:
            if not smp.sample_not_finished():
                smp.restart()                      # next epoch: the reference walks the same list again
            ssg = smp.sample_one(raw_edges=raw)
            np.testing.assert_array_equal(host_u32(ssg.sampled_sgs[-1].destination, len(batch_seeds(g, k))),
                                          batch_seeds(g, k))
            tk.forward_backward(ssg, train=True)
        tk.Update()
        tk.step_count += 1
        loss[k], hits = tk.read_stats()
        assert abs(loss[k] - g["loss"][k]) < 1e-3, (k, loss[k], g["loss"][k])
        assert abs(hits - int(g["correct"][k])) <= 1, (k, hits, int(g["correct"][k]))
    ref_epoch = g["loss"].astype(np.float64).reshape(g["epochs"], -1).mean(axis=1)
    assert np.abs(loss.reshape(g["epochs"], -1).mean(axis=1) - ref_epoch).max() < 1e-3
    tk._join_update_stream()
    torch.cuda.synchronize()
    assert np.abs(tk.P.W.cpu().numpy() - g["W_final"]).max() < 1e-3


@pytest.mark.parametrize("path", AGG, ids=[os.path.basename(p)[:-4] for p in AGG])
def test_wide_hub_aggregation_against_reference_operator(cuda_device, ws, path):
    """F = 602 / 128 on a block with a column and a row of more than 4,096 edges, every aggregation variant."""
    z = np.load(path)
    V, F = int(z["V"][0]), int(z["F"][0])
    edges = torch.from_numpy(z["edges"].reshape(-1, 2).astype(np.int32)).to(cuda_device)
    graph = FullyRepGraph.from_edges(edges, V, ws)
    smp = Sampler(graph, z["seeds"], [-1], batch_size=len(z["seeds"]), ws=ws)
    ssg = smp.sample_one(raw_edges=[dev_i32(z["raw_edges"], cuda_device)])
    blk = ssg.sampled_sgs[0]
    assert [blk.v_size, blk.e_size, blk.src_size] == z["sizes"].tolist()
    x, gy = make_golden.agg_operands(blk.src_size, blk.v_size, F, int(z["operand_seed"][0]))
    for fused in (False, True):
        op = SingleGPUSampleGraphOp(ssg, None, 0, None, fused_weights=fused)
        y = op.forward(dev_f32(x, cuda_device)).detach().cpu().numpy()[z["y_rows"]]
        gx = op.backward(dev_f32(gy, cuda_device)).cpu().numpy()[z["gx_rows"]]
        np.testing.assert_array_equal(y.view(np.uint32), z["y"].view(np.uint32))      # bar: 1e-5 relative; met bit for bit
        np.testing.assert_array_equal(gx.view(np.uint32), z["gx"].view(np.uint32))
