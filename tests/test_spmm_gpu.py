"""Aggregation parity: CUDA SpMM (through the C ABI) against the CPU oracle on identical blocks.

Bar: the north star asks for 1e-5 relative (fp32).  The kernels keep the arithmetic of the reference's CPU
operator (one fused multiply-add per edge and element, edge by edge), so the comparison below is bit-exact; the
tolerance is only stated for the full-size property test at the end.
"""
import numpy as np
import pytest
import torch

import oracle
from helpers import dev_f32, dev_i32, host_f32, small_graph
from neutronbench_b200 import Cuda_Stream, _lib
from neutronbench_b200.cuda_stream import ptr

pytestmark = pytest.mark.gpu


def _block(V=3000, E=40000, seeds=256, fanouts=(10, 5), seed=3, kind="rmat"):
    edges, co, ri = small_graph(V, E, seed, kind)
    rng = np.random.RandomState(seed)
    s = rng.choice(V, size=seeds, replace=False).astype(np.uint32)
    blocks, _ = oracle.sample_batch(co, ri, V, s, list(fanouts), seed=seed)
    return blocks


@pytest.mark.parametrize("F", [1, 2, 3, 16, 41, 100, 128, 602, 1433])
def test_forward_explicit_weights_bit_exact(cuda_device, F):
    blk = _block()[0]
    rng = np.random.RandomState(F)
    x = rng.randn(blk.src_size, F).astype(np.float32)
    ref = oracle.spmm_fwd(x, blk.edge_weight_forward, blk.row_indices, blk.column_offset)
    dx = dev_f32(x, cuda_device)
    dy = torch.full((blk.v_size, F), float("nan"), device=cuda_device)
    cs = Cuda_Stream()
    cs.Gather_By_Dst_From_Src(ptr(dx), ptr(dy), ptr(dev_f32(blk.edge_weight_forward, cuda_device)),
                              ptr(dev_i32(blk.row_indices, cuda_device)), ptr(dev_i32(blk.column_offset, cuda_device)),
                              0, 0, 0, 0, blk.e_size, blk.v_size, F, True, False)
    cs.CUDA_DEVICE_SYNCHRONIZE()
    np.testing.assert_array_equal(host_f32(dy).view(np.uint32), ref.view(np.uint32))


@pytest.mark.parametrize("F", [1, 16, 100, 128, 602])
def test_backward_explicit_weights_bit_exact(cuda_device, F):
    blk = _block()[1]
    rng = np.random.RandomState(100 + F)
    gy = rng.randn(blk.v_size, F).astype(np.float32)
    ref = oracle.spmm_bwd(gy, blk.edge_weight_backward, blk.row_offset, blk.column_indices)
    dgy = dev_f32(gy, cuda_device)
    dgx = torch.full((blk.src_size, F), float("nan"), device=cuda_device)
    cs = Cuda_Stream()
    cs.Gather_By_Src_From_Dst(ptr(dgy), ptr(dgx), ptr(dev_f32(blk.edge_weight_backward, cuda_device)),
                              ptr(dev_i32(blk.row_offset, cuda_device)), ptr(dev_i32(blk.column_indices, cuda_device)),
                              0, 0, 0, 0, blk.e_size, blk.src_size, F, True, False)
    cs.CUDA_DEVICE_SYNCHRONIZE()
    np.testing.assert_array_equal(host_f32(dgx).view(np.uint32), ref.view(np.uint32))


@pytest.mark.parametrize("F", [16, 128, 602])
def test_fused_weight_variants_equal_explicit(cuda_device, F):
    blk = _block(fanouts=(25, 10))[0]
    rng = np.random.RandomState(7 + F)
    x = rng.randn(blk.src_size, F).astype(np.float32)
    gy = rng.randn(blk.v_size, F).astype(np.float32)
    act = np.maximum(rng.randn(blk.src_size, F), 0).astype(np.float32)
    ref_f = oracle.spmm_fwd(x, blk.edge_weight_forward, blk.row_indices, blk.column_offset)
    ref_b = oracle.spmm_bwd(gy, blk.edge_weight_backward, blk.row_offset, blk.column_indices, act=act, scale=2.0)
    st = torch.cuda.current_stream().cuda_stream
    d = cuda_device
    ri, co = dev_i32(blk.row_indices, d), dev_i32(blk.column_offset, d)
    ro, ci = dev_i32(blk.row_offset, d), dev_i32(blk.column_indices, d)
    sn, dn = dev_f32(blk.src_norm, d), dev_f32(blk.dst_norm, d)
    dy = torch.empty((blk.v_size, F), device=d)
    _lib.call("nb_spmm_csc_fwd_fused", ptr(dev_f32(x, d)), ptr(dy), ptr(ri), ptr(co), ptr(sn), ptr(dn), blk.v_size, F,
              st)
    dgx = torch.empty((blk.src_size, F), device=d)
    _lib.call("nb_spmm_csr_bwd_fused", ptr(dev_f32(gy, d)), ptr(dgx), ptr(ro), ptr(ci), ptr(sn), ptr(dn),
              ptr(dev_f32(act, d)), 2.0, blk.src_size, F, st)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(host_f32(dy).view(np.uint32), ref_f.view(np.uint32))
    np.testing.assert_array_equal(host_f32(dgx).view(np.uint32), ref_b.view(np.uint32))


@pytest.mark.parametrize("panel_bytes", [None, 1 << 20, 200_000])
@pytest.mark.parametrize("F,use_cache", [(602, True), (602, False), (100, True), (128, True)])
def test_gather_fused_forward_equals_gather_then_spmm(cuda_device, ws, F, use_cache, panel_bytes):
    """panel_bytes forces the staged kernel to cut rows into 2..many column panels (the cut is a
    schedule, not arithmetic: the bits must not change)."""
    V = 3000
    blk = _block(V=V)[0]
    rng = np.random.RandomState(11)
    feat = rng.randn(V, F).astype(np.float32)
    out_deg = rng.randint(1, 50, size=V).astype(np.uint32)
    hm, ids = oracle.cache_by_degree(out_deg, V // 3)
    ld = (F + 3) // 4 * 4
    cache = np.zeros((len(ids), ld), dtype=np.float32)
    cache[:, :F] = feat[ids]
    x0 = oracle.feature_gather(feat, blk.source)
    ref = oracle.spmm_fwd(x0, blk.edge_weight_forward, blk.row_indices, blk.column_offset)
    d = cuda_device
    dy = torch.empty((blk.v_size, F), device=d)
    dfeat = dev_f32(feat, d)
    dcache = dev_f32(cache, d) if use_cache else None
    dhm = dev_i32(hm, d) if use_cache else None
    old_panel = _lib.load().nb_set_l2_panel_bytes(panel_bytes) if panel_bytes is not None else None
    _lib.call("nb_spmm_csc_fwd_gather_fused", ws.handle, ptr(dfeat), F, ptr(dcache), ld if use_cache else 0, ptr(dhm),
              ptr(dev_i32(blk.source, d)), ptr(dy), ptr(dev_i32(blk.row_indices, d)),
              ptr(dev_i32(blk.column_offset, d)), ptr(dev_f32(blk.src_norm, d)), ptr(dev_f32(blk.dst_norm, d)),
              blk.v_size, blk.src_size, blk.e_size, F, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    if old_panel is not None:
        _lib.load().nb_set_l2_panel_bytes(old_panel)
    np.testing.assert_array_equal(host_f32(dy).view(np.uint32), ref.view(np.uint32))


def test_empty_columns_and_empty_block(cuda_device):
    # two destinations without in-edges around one with three
    co = np.array([0, 0, 3, 3], dtype=np.uint32)
    ri = np.array([1, 0, 1], dtype=np.uint32)
    w = np.array([0.5, 0.25, 2.0], dtype=np.float32)
    x = np.arange(8, dtype=np.float32).reshape(2, 4)
    ref = oracle.spmm_fwd(x, w, ri, co)
    d = cuda_device
    dy = torch.full((3, 4), float("nan"), device=d)
    st = torch.cuda.current_stream().cuda_stream
    _lib.call("nb_spmm_csc_fwd", ptr(dev_f32(x, d)), ptr(dy), ptr(dev_f32(w, d)), ptr(dev_i32(ri, d)),
              ptr(dev_i32(co, d)), 3, 4, st)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(host_f32(dy), ref)
    assert (host_f32(dy)[0] == 0).all() and (host_f32(dy)[2] == 0).all()
    _lib.call("nb_spmm_csc_fwd", 0, 0, 0, 0, 0, 0, 4, st)  # v == 0: nothing to do


@pytest.mark.parametrize("misalign", [1, 0])
def test_long_rows_and_unaligned_views(cuda_device, misalign):
    """A hub row of 5000 edges (many segments / 32-edge passes); with misalign=1 the x tensor starts
    4 bytes off a 16-byte boundary, so the staged path is not applicable and the vector width of the
    direct-load path must fall back to scalar."""
    rng = np.random.RandomState(5)
    s, F = 700, 128
    lens = np.array([5000, 0, 33, 32, 31, 1], dtype=np.uint32)
    co = np.concatenate([[0], np.cumsum(lens)]).astype(np.uint32)
    ri = rng.randint(0, s, size=int(co[-1])).astype(np.uint32)
    w = rng.rand(int(co[-1])).astype(np.float32)
    x = rng.randn(s, F).astype(np.float32)
    ref = oracle.spmm_fwd(x, w, ri, co)
    d = cuda_device
    buf = torch.empty(s * F + 1, device=d)
    xv = buf[misalign: misalign + s * F].view(s, F)
    xv.copy_(dev_f32(x, d))
    assert xv.data_ptr() % 16 == 4 * misalign
    dy = torch.empty((len(lens), F), device=d)
    _lib.call("nb_spmm_csc_fwd", ptr(xv), ptr(dy), ptr(dev_f32(w, d)), ptr(dev_i32(ri, d)), ptr(dev_i32(co, d)),
              len(lens), F, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(host_f32(dy).view(np.uint32), ref.view(np.uint32))


@pytest.mark.parametrize("F", [128, 100, 41, 256, 7])
@pytest.mark.parametrize("hub_min", [None, 64, 0])
def test_rows_of_thousands_of_edges_take_the_team_path_with_identical_bits(cuda_device, ws, F, hub_min):
    """A block whose transposed form has a few sources with 300 .. 3,000 edges among 2,000 short rows (what a popular
    vertex of a Products-shaped batch looks like in the backward pass).  Rows of at least `hub_min_edges` edges are
    walked by a team of warps with one column per lane; every element is still one fused multiply-add per edge in edge
    order, so explicit and fused weights, with and without the activation mask, give the oracle's bits whatever the
    threshold (None: the default, 0: every row on the one-warp path)."""
    rng = np.random.RandomState(11 + F)
    n, s = 2000, 900
    lens = rng.randint(0, 12, size=n).astype(np.uint32)
    for r, l in ((3, 3000), (4, 257), (700, 256), (701, 255), (1500, 1031), (1999, 640), (256, 300), (255, 999)):
        lens[r] = l
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.uint32)
    e = int(offs[-1])
    idx = rng.randint(0, s, size=e).astype(np.uint32)
    w = rng.rand(e).astype(np.float32)
    x = rng.randn(s, F).astype(np.float32)
    act = np.maximum(rng.randn(n, F), 0).astype(np.float32)
    row_norm = np.sqrt(rng.randint(1, 50, size=n)).astype(np.float32)
    idx_norm = np.sqrt(rng.randint(1, 50, size=s)).astype(np.float32)
    rows = np.repeat(np.arange(n), lens)
    w_fused = (np.float32(1.0) / (idx_norm[idx] * row_norm[rows])).astype(np.float32)
    d = cuda_device
    st = torch.cuda.current_stream().cuda_stream
    if hub_min is not None:
        _lib.call("nb_set_option", b"hub_min_edges", hub_min)
    try:
        dy = torch.full((n, F), float("nan"), device=d)
        _lib.call("nb_spmm_csc_fwd", ptr(dev_f32(x, d)), ptr(dy), ptr(dev_f32(w, d)), ptr(dev_i32(idx, d)),
                  ptr(dev_i32(offs, d)), n, F, st)
        torch.cuda.synchronize()
        np.testing.assert_array_equal(host_f32(dy).view(np.uint32), oracle.spmm_fwd(x, w, idx, offs).view(np.uint32))
        # transposed form with fused weights and the relu/dropout mask: rows are sources, x rows are destinations
        dgx = torch.full((n, F), float("nan"), device=d)
        _lib.call("nb_spmm_csr_bwd_fused", ptr(dev_f32(x, d)), ptr(dgx), ptr(dev_i32(offs, d)), ptr(dev_i32(idx, d)),
                  ptr(dev_f32(row_norm, d)), ptr(dev_f32(idx_norm, d)), ptr(dev_f32(act, d)), 2.0, n, F, st)
        torch.cuda.synchronize()
        ref = oracle.spmm_bwd(x, w_fused, offs, idx, act=act, scale=2.0)
        np.testing.assert_array_equal(host_f32(dgx).view(np.uint32), ref.view(np.uint32))
    finally:
        if hub_min is not None:
            _lib.call("nb_set_option", b"hub_min_edges", 256)


def test_linearity_at_full_size(cuda_device):
    """Reddit-shaped input block sizes (v=25k, fanout 10, F=602): A(x1 + 2 x2) == A x1 + 2 A x2 within
    1e-5 relative — a size-independent property checked without the CPU oracle."""
    rng = np.random.RandomState(9)
    v, s, F, fan = 25000, 140000, 602, 10
    co = (np.arange(v + 1) * fan).astype(np.uint32)
    ri = rng.randint(0, s, size=v * fan).astype(np.uint32)
    w = rng.rand(v * fan).astype(np.float32)
    d = cuda_device
    g = torch.Generator(device=d).manual_seed(1)
    x1 = torch.randn((s, F), device=d, generator=g)
    x2 = torch.randn((s, F), device=d, generator=g)
    dri, dco, dw = dev_i32(ri, d), dev_i32(co, d), dev_f32(w, d)
    st = torch.cuda.current_stream().cuda_stream

    def agg(x):
        y = torch.empty((v, F), device=d)
        _lib.call("nb_spmm_csc_fwd", ptr(x), ptr(y), ptr(dw), ptr(dri), ptr(dco), v, F, st)
        return y

    lhs = agg(x1 + 2 * x2)
    rhs = agg(x1) + 2 * agg(x2)
    err = (lhs - rhs).abs().max().item() / rhs.abs().max().item()
    assert err < 1e-5, err


@pytest.mark.parametrize("F", [16, 100, 128, 256, 1024])
def test_staged_and_direct_paths_give_identical_bits(cuda_device, F):
    """The TMA-staged kernel and the direct-load kernel are two schedules of the same arithmetic."""
    blk = _block(fanouts=(25, 10))[1]
    rng = np.random.RandomState(F)
    x = rng.randn(blk.src_size, F).astype(np.float32)
    d = cuda_device
    dx, dw = dev_f32(x, d), dev_f32(blk.edge_weight_forward, d)
    ri, co = dev_i32(blk.row_indices, d), dev_i32(blk.column_offset, d)
    st = torch.cuda.current_stream().cuda_stream
    outs = []
    lib = _lib.load()
    for staged in (2, 4, 0):    # ring kernel, two-stage segment kernel, direct loads
        old = lib.nb_set_staged_spmm(staged)
        y = torch.empty((blk.v_size, F), device=d)
        _lib.call("nb_spmm_csc_fwd", ptr(dx), ptr(y), ptr(dw), ptr(ri), ptr(co), blk.v_size, F, st)
        torch.cuda.synchronize()
        lib.nb_set_staged_spmm(1 if old else 0)
        outs.append(host_f32(y))
    np.testing.assert_array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))
    np.testing.assert_array_equal(outs[0].view(np.uint32), outs[2].view(np.uint32))
    ref = oracle.spmm_fwd(x, blk.edge_weight_forward, blk.row_indices, blk.column_offset)
    np.testing.assert_array_equal(outs[0].view(np.uint32), ref.view(np.uint32))
    import ctypes
    flags = ctypes.c_uint32(7)
    _lib.call("nb_device_error_flags", ctypes.byref(flags))
    assert flags.value == 0


@pytest.mark.parametrize("mode", [1, 5])
@pytest.mark.parametrize("F", [256, 602, 1024])
def test_ring_groupings_give_identical_bits(cuda_device, ws, F, mode):
    """The ring kernel waits once per pair of rows (mode 1, the default, where four row slots fit: F = 1024 has three
    and keeps a barrier per row) or once per row (mode 5).  Same arithmetic, same order: plain, masked backward and
    gather-fused forms (cache hits and misses) keep their bits."""
    V = 3000
    blk = _block(V=V, fanouts=(25, 10))[0]
    rng = np.random.RandomState(F + mode)
    d = cuda_device
    st = torch.cuda.current_stream().cuda_stream
    lib = _lib.load()
    feat = rng.randn(V, F).astype(np.float32)
    hm, ids = oracle.cache_by_degree(rng.randint(1, 50, size=V).astype(np.uint32), V // 3)
    ld = (F + 31) // 32 * 32
    cache = np.zeros((len(ids), ld), dtype=np.float32)
    cache[:, :F] = feat[ids]
    x0 = oracle.feature_gather(feat, blk.source)
    ref_g = oracle.spmm_fwd(x0, blk.edge_weight_forward, blk.row_indices, blk.column_offset)
    gy = rng.randn(blk.v_size, F).astype(np.float32)
    act = np.maximum(rng.randn(blk.src_size, F), 0).astype(np.float32)
    ref_b = oracle.spmm_bwd(gy, blk.edge_weight_backward, blk.row_offset, blk.column_indices, act=act, scale=2.0)
    ri, co = dev_i32(blk.row_indices, d), dev_i32(blk.column_offset, d)
    ro, ci = dev_i32(blk.row_offset, d), dev_i32(blk.column_indices, d)
    sn, dn = dev_f32(blk.src_norm, d), dev_f32(blk.dst_norm, d)
    dfeat, dcache, dhm, dsrc = dev_f32(feat, d), dev_f32(cache, d), dev_i32(hm, d), dev_i32(blk.source, d)
    old = lib.nb_set_staged_spmm(mode)
    try:
        dy = torch.full((blk.v_size, F), float("nan"), device=d)
        _lib.call("nb_spmm_csc_fwd_gather_fused", ws.handle, ptr(dfeat), F, ptr(dcache), ld, ptr(dhm), ptr(dsrc), ptr(dy),
                  ptr(ri), ptr(co), ptr(sn), ptr(dn), blk.v_size, blk.src_size, blk.e_size, F, st)
        dy2 = torch.full((blk.v_size, F), float("nan"), device=d)
        _lib.call("nb_spmm_csc_fwd_fused", ptr(dev_f32(x0, d)), ptr(dy2), ptr(ri), ptr(co), ptr(sn), ptr(dn),
                  blk.v_size, F, st)
        dgx = torch.full((blk.src_size, F), float("nan"), device=d)
        _lib.call("nb_spmm_csr_bwd_fused", ptr(dev_f32(gy, d)), ptr(dgx), ptr(ro), ptr(ci), ptr(sn), ptr(dn),
                  ptr(dev_f32(act, d)), 2.0, blk.src_size, F, st)
        torch.cuda.synchronize()
    finally:
        lib.nb_set_staged_spmm(1 if old else 0)
    np.testing.assert_array_equal(host_f32(dy).view(np.uint32), ref_g.view(np.uint32))
    np.testing.assert_array_equal(host_f32(dy2).view(np.uint32), ref_g.view(np.uint32))
    np.testing.assert_array_equal(host_f32(dgx).view(np.uint32), ref_b.view(np.uint32))
    import ctypes
    flags = ctypes.c_uint32(7)
    _lib.call("nb_device_error_flags", ctypes.byref(flags))
    assert flags.value == 0
