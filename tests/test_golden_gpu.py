"""The CUDA path (through the C ABI) against outputs of the REFERENCE's own code (tests/golden/*.npz).
Bars of the north star: block construction bit-exact on identical sampled edge lists; aggregation
forward/backward within 1e-5 relative (fp32)."""
import os

import numpy as np
import pytest
import torch

from helpers import dev_f32, dev_i32, host_f32, host_u32
from neutronbench_b200 import FullyRepGraph, Sampler, SingleGPUSampleGraphOp
from test_golden_cpu import GOLDEN, load, raw_lists

pytestmark = pytest.mark.gpu
IDS = [os.path.basename(p)[:-4] for p in GOLDEN]


@pytest.mark.parametrize("path", GOLDEN, ids=IDS)
def test_graph_blocks_and_aggregation_against_reference(cuda_device, ws, path):
    g = load(path)
    V, F, L = int(g["V"][0]), int(g["F"][0]), g["L"]
    edges = torch.from_numpy(g["edges"].reshape(-1, 2).astype(np.int32)).to(cuda_device)
    graph = FullyRepGraph.from_edges(edges, V, ws)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(graph.column_offset.cpu().numpy().astype(np.uint32), g["graph_column_offset"])
    np.testing.assert_array_equal(host_u32(graph.row_indices), g["graph_row_indices"])

    fanout = [int(f) for f in g["fanout"]]
    smp = Sampler(graph, g["seeds"], fanout, batch_size=len(g["seeds"]), ws=ws)
    ssg = smp.sample_one(raw_edges=[dev_i32(r, cuda_device) for r in raw_lists(g)])
    torch.cuda.synchronize()
    for l, blk in enumerate(ssg.sampled_sgs):
        p = f"block{l}_"
        v, e, s = [int(x) for x in g[p + "sizes"]]
        assert (blk.v_size, blk.e_size, blk.src_size) == (v, e, s)
        np.testing.assert_array_equal(host_u32(blk.destination, v), g[p + "destination"])
        np.testing.assert_array_equal(host_u32(blk.source, s), g[p + "source"])
        np.testing.assert_array_equal(host_u32(blk.column_offset, v + 1), g[p + "column_offset"])
        np.testing.assert_array_equal(host_u32(blk.row_indices, e), g[p + "row_indices"])
        np.testing.assert_array_equal(host_u32(blk.row_offset, s + 1), g[p + "row_offset"])
        np.testing.assert_array_equal(host_u32(blk.column_indices, e), g[p + "column_indices"])
        np.testing.assert_array_equal(host_f32(blk.edge_weight_forward, e).view(np.uint32),
                                      g[p + "edge_weight_forward"].view(np.uint32))
        np.testing.assert_array_equal(host_f32(blk.edge_weight_backward, e).view(np.uint32),
                                      g[p + "edge_weight_backward"].view(np.uint32))
        x, gy = g[p + "x"].reshape(-1, F), g[p + "gy"].reshape(-1, F)
        ry, rgx = g[p + "y"].reshape(-1, F), g[p + "gx"].reshape(-1, F)
        for fused in (False, True):
            op = SingleGPUSampleGraphOp(ssg, None, l, None, fused_weights=fused)
            y = op.forward(dev_f32(x, cuda_device)).detach().cpu().numpy()
            gx = op.backward(dev_f32(gy, cuda_device)).cpu().numpy()
            # bar of the north star: 1e-5 relative; met with zero difference (same fused multiply-add per edge)
            np.testing.assert_array_equal(y.view(np.uint32), ry.view(np.uint32))
            np.testing.assert_array_equal(gx.view(np.uint32), rgx.view(np.uint32))
