"""Block construction parity: dedup, reindex, CSC offsets, CSR transpose, degrees and weights must be
BIT-EXACT against the oracle on identical sampled edge lists."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from helpers import assert_block_equal, dev_i32, dev_i64, host_u32, small_graph
from neutronbench_b200 import FullyRepGraph, Sampler, _lib, build_block
from neutronbench_b200.cuda_stream import ptr

pytestmark = pytest.mark.gpu


def _device_graph(co, ri, V, device):
    return FullyRepGraph(dev_i64(co, device), dev_i32(ri, device), V)


@pytest.mark.parametrize("V,E,kind", [(3000, 40000, "rmat"), (2708, 10556, "uniform"), (50, 400, "rmat"),
                                      (100000, 600000, "rmat")])
@pytest.mark.parametrize("fanouts", [(10, 5), (25, 10), (5, 4, 3)])
def test_blocks_from_identical_edge_lists(cuda_device, ws, V, E, kind, fanouts):
    edges, co, ri = small_graph(V, E, seed=V % 97, kind=kind)
    rng = np.random.RandomState(4)
    seeds = rng.choice(V, size=min(V // 2, 512), replace=False).astype(np.uint32)
    ref_blocks, raws = oracle.sample_batch(co, ri, V, seeds, list(fanouts), seed=99)
    g = _device_graph(co, ri, V, cuda_device)
    smp = Sampler(g, seeds, fanouts, batch_size=len(seeds), ws=ws)
    ssg = smp.sample_one(raw_edges=[dev_i32(r, cuda_device) for r in raws])
    torch.cuda.synchronize()
    assert len(ssg.sampled_sgs) == len(ref_blocks)
    for dev_blk, ref_blk in zip(ssg.sampled_sgs, ref_blocks):
        assert_block_equal(dev_blk, ref_blk)
    # chain property: destinations of block l are the sources of block l+1 (core/ntsSampler.hpp:884)
    for l in range(len(fanouts) - 1):
        np.testing.assert_array_equal(host_u32(ssg.sampled_sgs[l].destination, ssg.sampled_sgs[l].v_size),
                                      host_u32(ssg.sampled_sgs[l + 1].source, ssg.sampled_sgs[l + 1].src_size))


def test_full_neighbour_hop_with_hub_rows(cuda_device, ws):
    """fanout < 0 keeps every neighbour: long CSR rows exercise the CTA sort (shared-memory bitonic) and
    the windowed counting sort (rows longer than 4096)."""
    V = 20000
    rng = np.random.RandomState(8)
    hub = np.stack([np.zeros(9000, dtype=np.int64), rng.randint(0, V, 9000)], axis=1)        # vertex 0 -> many
    mid = np.stack([np.full(3000, 7, dtype=np.int64), rng.randint(0, V, 3000)], axis=1)      # vertex 7 -> some
    rest = np.stack([rng.randint(0, V, 60000), rng.randint(0, V, 60000)], axis=1)
    edges = np.concatenate([hub, mid, rest]).astype(np.int32)
    co, ri = oracle.build_csc(edges, V)
    seeds = np.arange(V, dtype=np.uint32)
    ref_blocks, raws = oracle.sample_batch(co, ri, V, seeds, [-1], seed=1)
    assert (np.diff(ref_blocks[0].row_offset) > 4096).any()
    g = _device_graph(co, ri, V, cuda_device)
    smp = Sampler(g, seeds, [-1], batch_size=V, ws=ws)
    ssg = smp.sample_one(raw_edges=[dev_i32(r, cuda_device) for r in raws])
    torch.cuda.synchronize()
    assert_block_equal(ssg.sampled_sgs[0], ref_blocks[0])


def test_duplicate_edges_and_self_loops(cuda_device, ws):
    V = 64
    edges = np.array([[1, 0], [1, 0], [1, 0], [0, 0], [2, 1], [2, 1], [63, 1], [5, 5]], dtype=np.int32)
    co, ri = oracle.build_csc(edges, V)
    seeds = np.array([0, 1, 5, 9], dtype=np.uint32)   # vertex 9 has no in-edges: empty column
    ref_blocks, raws = oracle.sample_batch(co, ri, V, seeds, [-1], seed=1)
    g = _device_graph(co, ri, V, cuda_device)
    smp = Sampler(g, seeds, [-1], batch_size=4, ws=ws)
    ssg = smp.sample_one(raw_edges=[dev_i32(r, cuda_device) for r in raws])
    assert_block_equal(ssg.sampled_sgs[0], ref_blocks[0])
    assert ssg.sampled_sgs[0].src_size == 5


def test_block_without_edges(cuda_device, ws):
    V = 32
    co = np.zeros(V + 1, dtype=np.uint64)
    ri = np.zeros(0, dtype=np.uint32)
    seeds = np.array([3, 4], dtype=np.uint32)
    g = _device_graph(co, np.zeros(1, dtype=np.uint32), V, cuda_device)
    smp = Sampler(g, seeds, [5], batch_size=2, ws=ws)
    ssg = smp.sample_one()
    blk = ssg.sampled_sgs[0]
    assert (blk.v_size, blk.e_size, blk.src_size) == (2, 0, 0)
    np.testing.assert_array_equal(host_u32(blk.column_offset, 3), [0, 0, 0])


def test_out_of_range_source_id_is_reported(cuda_device, ws):
    co = dev_i32(np.array([0, 2], dtype=np.uint32), cuda_device)
    ri = dev_i32(np.array([1, 4000], dtype=np.uint32), cuda_device)
    dst = dev_i32(np.array([0], dtype=np.uint32), cuda_device)
    with pytest.raises(_lib.NbError, match="num_vertices"):
        build_block(ws, 100, dst, co, ri, 1, 2)


def test_graph_csc_build_is_stable_in_file_order(cuda_device, ws):
    for V, E, seed in [(3000, 40000, 2), (257, 90000, 3)]:   # the second one has columns longer than 32
        edges, co, ri = small_graph(V, E, seed)
        out_d, in_d = oracle.degrees(edges, V, clamp=False)
        g = FullyRepGraph.from_edges(torch.from_numpy(edges).to(cuda_device), V, ws)
        torch.cuda.synchronize()
        np.testing.assert_array_equal(g.column_offset.cpu().numpy().astype(np.uint64), co)
        np.testing.assert_array_equal(host_u32(g.row_indices), ri)
        np.testing.assert_array_equal(host_u32(g.out_degree), out_d)
        np.testing.assert_array_equal(host_u32(g.in_degree), in_d)
