"""Shared builders for the parity tests: small seeded graphs, host<->device moves, comparisons."""
from __future__ import annotations

import numpy as np
import torch

import oracle
from neutronbench_b200 import synth


def small_graph(V=3000, E=40000, seed=1, kind="rmat"):
    if kind == "rmat":
        edges = synth.rmat_numpy(V, E, (0.57, 0.19, 0.19), seed)
    else:
        edges = synth.uniform_undirected_numpy(V, E // 2, seed)
    co, ri = oracle.build_csc(edges, V)
    return edges, co, ri


# Device tensors made by the dev_* helpers stay referenced until the test ends: the C ABI takes raw
# addresses, so a temporary whose last Python reference is gone could be recycled by torch's caching
# allocator while a kernel still reads it.  tests/conftest.py clears the list after every test.
KEEP_ALIVE = []


def _keep(t):
    KEEP_ALIVE.append(t)
    return t


def dev_i32(a, device):
    return _keep(torch.from_numpy(np.ascontiguousarray(a).astype(np.uint32).view(np.int32)).to(device))


def dev_i64(a, device):
    return _keep(torch.from_numpy(np.ascontiguousarray(a).astype(np.int64)).to(device))


def dev_f32(a, device):
    return _keep(torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(device))


def host_u32(t, n=None):
    a = t.detach().cpu().numpy().view(np.uint32)
    return a if n is None else a[:n]


def host_f32(t, n=None):
    a = t.detach().cpu().numpy()
    return a if n is None else a[:n]


def assert_block_equal(dev_blk, ref_blk, weights=True):
    """Bit-exact comparison of a device sampCSC with the oracle's block."""
    assert dev_blk.v_size == ref_blk.v_size
    assert dev_blk.e_size == ref_blk.e_size
    assert dev_blk.src_size == ref_blk.src_size
    v, e, s = ref_blk.v_size, ref_blk.e_size, ref_blk.src_size
    np.testing.assert_array_equal(host_u32(dev_blk.destination, v), ref_blk.destination)
    np.testing.assert_array_equal(host_u32(dev_blk.source, s), ref_blk.source)
    np.testing.assert_array_equal(host_u32(dev_blk.column_offset, v + 1), ref_blk.column_offset)
    np.testing.assert_array_equal(host_u32(dev_blk.row_indices, e), ref_blk.row_indices[:e])
    np.testing.assert_array_equal(host_u32(dev_blk.row_offset, s + 1), ref_blk.row_offset)
    np.testing.assert_array_equal(host_u32(dev_blk.column_indices, e), ref_blk.column_indices[:e])
    # float arrays compared as bit patterns: the weights are required to be bit-identical
    np.testing.assert_array_equal(host_f32(dev_blk.src_norm, s).view(np.uint32), ref_blk.src_norm.view(np.uint32))
    np.testing.assert_array_equal(host_f32(dev_blk.dst_norm, v).view(np.uint32), ref_blk.dst_norm.view(np.uint32))
    if weights:
        np.testing.assert_array_equal(host_f32(dev_blk.edge_weight_forward, e).view(np.uint32),
                                      ref_blk.edge_weight_forward.view(np.uint32))
        np.testing.assert_array_equal(host_f32(dev_blk.edge_weight_backward, e).view(np.uint32),
                                      ref_blk.edge_weight_backward.view(np.uint32))
