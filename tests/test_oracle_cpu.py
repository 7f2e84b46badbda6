"""The CPU oracle checked against independent statements of the same mathematics (numpy, dense
algebra, finite differences) and against published known-answer vectors.  No GPU needed."""
import numpy as np
import pytest

import oracle
from neutronbench_b200 import cache_slots_by_degree, synth


def _graph(V=800, E=9000, seed=2):
    edges = synth.rmat_numpy(V, E, (0.57, 0.19, 0.19), seed)
    co, ri = oracle.build_csc(edges, V)
    return edges, co, ri


def test_philox_known_answers():
    # Known-answer vectors of Philox4x32-10 published with the Random123 library (Salmon et al., SC'11).
    kat = [((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
           ((0xffffffff,) * 4, (0xffffffff,) * 2, (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
           ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0),
            (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1))]
    for c, k, want in kat:
        assert tuple(int(x) for x in oracle.philox(c, k)) == want


def test_csc_is_stable_counting_sort():
    edges, co, ri = _graph()
    order = np.argsort(edges[:, 1], kind="stable")
    np.testing.assert_array_equal(ri, edges[order, 0].astype(np.uint32))
    np.testing.assert_array_equal(np.diff(co.astype(np.int64)), np.bincount(edges[:, 1], minlength=800))


def test_block_arrays_against_numpy():
    V = 800
    edges, co, ri = _graph(V)
    seeds = np.random.RandomState(0).choice(V, 100, replace=False).astype(np.uint32)
    blocks, raws = oracle.sample_batch(co, ri, V, seeds, [6, 4], seed=5)
    assert len(blocks) == 2
    np.testing.assert_array_equal(blocks[1].destination, seeds)               # seed block last
    np.testing.assert_array_equal(blocks[0].destination, blocks[1].source)   # chained
    for b, raw in zip(blocks, reversed(raws)):
        uniq = np.unique(raw)                                                # ascending distinct ids
        np.testing.assert_array_equal(b.source, uniq)
        np.testing.assert_array_equal(b.source[b.row_indices], raw)
        # CSR = stable sort of the CSC edges by local source
        dst_of_edge = np.repeat(np.arange(b.v_size), np.diff(b.column_offset.astype(np.int64)))
        order = np.argsort(b.row_indices, kind="stable")
        np.testing.assert_array_equal(b.column_indices, dst_of_edge[order].astype(np.uint32))
        np.testing.assert_array_equal(np.diff(b.row_offset.astype(np.int64)), np.bincount(b.row_indices, minlength=b.src_size))
        # weights: 1/((float)sqrt(out) * (float)sqrt(in)) with block degrees
        out_d = np.diff(b.row_offset.astype(np.int64))
        in_d = np.diff(b.column_offset.astype(np.int64))
        wf = np.float32(1) / (np.sqrt(out_d[b.row_indices].astype(np.float64)).astype(np.float32)
                              * np.sqrt(in_d[dst_of_edge].astype(np.float64)).astype(np.float32))
        np.testing.assert_array_equal(b.edge_weight_forward.view(np.uint32), wf.astype(np.float32).view(np.uint32))
        src_of_csr = np.repeat(np.arange(b.src_size), out_d)
        wb = np.float32(1) / (np.sqrt(out_d[src_of_csr].astype(np.float64)).astype(np.float32)
                              * np.sqrt(in_d[b.column_indices].astype(np.float64)).astype(np.float32))
        np.testing.assert_array_equal(b.edge_weight_backward.view(np.uint32), wb.astype(np.float32).view(np.uint32))


def test_sampling_structure():
    V = 800
    edges, co, ri = _graph(V)
    seeds = np.arange(200, dtype=np.uint32)
    fan = 5
    c, e = oracle.init_co(co, seeds, fan)
    raw = oracle.sample_hop(co, ri, seeds, fan, c, seed=9, hop=0)
    deg = np.diff(co.astype(np.int64))[seeds]
    np.testing.assert_array_equal(np.diff(c.astype(np.int64)), np.minimum(deg, fan))
    for i, d in enumerate(seeds):
        col = raw[c[i]: c[i + 1]]
        nbrs = ri[co[d]: co[d + 1]]
        if deg[i] <= fan:
            np.testing.assert_array_equal(col, nbrs)          # all neighbours, CSC order
        else:
            # k distinct POSITIONS: as a multiset the column is contained in the neighbour multiset
            from collections import Counter
            assert not (Counter(col.tolist()) - Counter(nbrs.tolist()))
    c_all, e_all = oracle.init_co(co, seeds, -1)
    assert e_all == deg.sum()


def test_aggregation_equals_dense_algebra_and_transposes():
    V = 800
    edges, co, ri = _graph(V)
    blocks, _ = oracle.sample_batch(co, ri, V, np.arange(64, dtype=np.uint32), [5, 3], seed=1)
    for b in blocks:
        A = np.zeros((b.v_size, b.src_size))
        dst_of_edge = np.repeat(np.arange(b.v_size), np.diff(b.column_offset.astype(np.int64)))
        np.add.at(A, (dst_of_edge, b.row_indices), b.edge_weight_forward.astype(np.float64))
        rng = np.random.RandomState(3)
        x, gy = rng.randn(b.src_size, 9).astype(np.float32), rng.randn(b.v_size, 9).astype(np.float32)
        np.testing.assert_allclose(oracle.spmm_fwd(x, b.edge_weight_forward, b.row_indices, b.column_offset), A @ x,
                                   rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(oracle.spmm_bwd(gy, b.edge_weight_backward, b.row_offset, b.column_indices),
                                   A.T @ gy, rtol=1e-5, atol=1e-6)
        act = rng.randn(b.src_size, 9).astype(np.float32)
        masked = oracle.spmm_bwd(gy, b.edge_weight_backward, b.row_offset, b.column_indices, act=act, scale=2.0)
        np.testing.assert_allclose(masked, np.where(act > 0, 2.0 * (A.T @ gy), 0.0), rtol=1e-5, atol=1e-6)


def test_cache_slots_host_logic_equals_oracle():
    rng = np.random.RandomState(1)
    deg = rng.randint(1, 9, size=5000).astype(np.uint32)        # many ties
    for num in (0, 1, 1000, 5000, 9999):
        hm, ids = oracle.cache_by_degree(deg, min(num, 5000))
        np.testing.assert_array_equal(cache_slots_by_degree(deg, num), hm)
    assert (np.diff(deg[ids].astype(np.int64)) <= 0).all()       # descending degree


def test_training_step_gradient_by_finite_differences():
    """dW from the oracle's hand-written backward equals the numerical derivative of its own loss
    (dropout off), including the 'input-side block is not back-propagated' shortcut."""
    V, F, H, C = 300, 6, 5, 4
    edges = synth.rmat_numpy(V, 2500, (0.57, 0.19, 0.19), 4)
    co, ri = oracle.build_csc(edges, V)
    rng = np.random.RandomState(0)
    feat = rng.randn(V, F).astype(np.float32)
    label = rng.randint(0, C, V).astype(np.int64)
    sizes = [F, H, H, C]
    W0 = (rng.randn(F * H + H * H + H * C) * 0.3).astype(np.float32)
    blocks, _ = oracle.sample_batch(co, ri, V, np.arange(40, dtype=np.uint32), [4, 3, 2], seed=3)
    net = oracle.GCN(sizes, W0, lr=0.0, wd=0.0, drop=0.0, seed=1)
    net.train_step(blocks, feat, label)
    grad = net.grad.copy()

    def loss_at(W):
        n = oracle.GCN(sizes, W, lr=0.0, wd=0.0, drop=0.0, seed=1)
        return n.train_step(blocks, feat, label, train=False)[0]

    eps = 1e-2
    for idx in rng.choice(len(W0), 25, replace=False):
        Wp, Wm = W0.copy(), W0.copy()
        Wp[idx] += eps
        Wm[idx] -= eps
        num = (loss_at(Wp) - loss_at(Wm)) / (2 * eps)
        assert abs(num - grad[idx]) < 2e-3 + 0.05 * abs(num), (idx, num, grad[idx])


def test_adam_against_numpy_formula():
    rng = np.random.RandomState(2)
    n = 1000
    W, g = rng.randn(n).astype(np.float32), rng.randn(n).astype(np.float32)
    M, V = np.zeros(n, np.float32), np.zeros(n, np.float32)
    W0 = W.copy()
    oracle.adam(W, g, M, V, 0.01, 0.9, 0.999, 1e-9, 0.0001, 0.9, 0.999)
    gg = g.astype(np.float64) + 0.0001 * W0
    m = 0.1 * gg
    v = 0.001 * gg * gg
    want = W0 - 0.01 * (m / 0.1) / (np.sqrt(v / 0.001) + 1e-9)
    np.testing.assert_allclose(W, want, rtol=2e-5, atol=1e-6)


def test_label_and_feature_gather():
    rng = np.random.RandomState(3)
    feat = rng.randn(50, 7).astype(np.float32)
    src = np.array([3, 3, 49, 0], dtype=np.uint32)
    np.testing.assert_array_equal(oracle.feature_gather(feat, src), feat[src])
    lab = rng.randint(0, 5, 50).astype(np.int64)
    np.testing.assert_array_equal(oracle.label_gather(lab, src), lab[src])


def test_sample_rate_counts_and_large_subsets():
    """SAMPLE_RATE mode (core/ntsSampler.hpp:901-912): per destination max(int(deg * rate), min(lower, deg));
    subsets above 128 positions are drawn by selection sampling and are still exact-size, distinct and
    inside the neighbourhood."""
    rng = np.random.RandomState(4)
    V = 600
    hub = np.stack([rng.randint(0, V, 900), np.zeros(900, np.int64)], axis=1)          # vertex 0: in-degree ~900
    rest = np.stack([rng.randint(0, V, 6000), rng.randint(0, V, 6000)], axis=1)
    edges = np.concatenate([hub, rest]).astype(np.uint32)
    co, ri = oracle.build_csc(edges, V)
    deg = np.diff(co.astype(np.int64))
    dst = np.array([0, 5, 17, 300, 599, 5], dtype=np.uint32)
    for rate, lower in ((0.5, 3), (0.05, 8), (1.0, 1)):
        offs, e = oracle.init_co_rate(co, dst, rate, lower)
        want = np.maximum((deg[dst].astype(np.float32) * np.float32(rate)).astype(np.int64), np.minimum(lower, deg[dst]))
        np.testing.assert_array_equal(np.diff(offs.astype(np.int64)), want)
        assert e == want.sum()
        picked = oracle.sample_hop(co, ri, dst, -1, offs, 99, 3)
        for i, d in enumerate(dst):
            mine = picked[offs[i]: offs[i + 1]]
            nbrs = ri[co[d]: co[d + 1]]
            # a sample is a sub-multiset of the column: no neighbour position is used twice
            cnt_m = np.bincount(mine, minlength=V)
            cnt_n = np.bincount(nbrs, minlength=V)
            assert (cnt_m <= cnt_n).all() and len(mine) == want[i]
    offs, _ = oracle.init_co_rate(co, dst, 0.5, 3)
    assert offs[1] - offs[0] > 128                       # the hub takes the selection-sampling path
    a = oracle.sample_hop(co, ri, dst, -1, offs, 99, 3)
    b = oracle.sample_hop(co, ri, dst, -1, offs, 100, 3)
    assert not np.array_equal(a, b)                      # the seed matters


def test_drop_train_ids_by_degree_follows_the_reference_code():
    from neutronbench_b200 import drop_train_ids_by_degree
    in_deg = np.array([5, 1, 9, 3, 7, 2, 8, 4], dtype=np.int64)
    ids = np.arange(8, dtype=np.uint32)
    np.testing.assert_array_equal(drop_train_ids_by_degree(ids, in_deg, "shuffle", 0.5), ids)
    # delhigh: descending order, last quarter dropped -> the two lowest-degree ids go
    np.testing.assert_array_equal(drop_train_ids_by_degree(ids, in_deg, "delhigh", 0.25), [2, 6, 4, 0, 7, 3])
    # dellow: ascending order, last quarter dropped -> the two highest-degree ids go
    np.testing.assert_array_equal(drop_train_ids_by_degree(ids, in_deg, "dellow", 0.25), [1, 5, 3, 7, 0, 4])
    assert len(drop_train_ids_by_degree(ids, in_deg, "dellow", 1.0)) == 0


def test_sigmoid_bce_oracle_equals_libtorch():
    """The multi-label loss of the reference is libtorch's binary_cross_entropy(sigmoid(z), y)
    (utils/torch_func.hpp:67-75); the oracle restates it and is checked here against torch itself,
    including logits large enough to reach the log clamp at -100."""
    import torch
    rng = np.random.RandomState(2)
    B, Cn = 37, 11
    z = (rng.randn(B, Cn) * 4).astype(np.float32)
    z[0, 0], z[0, 1], z[1, 0] = 120.0, -120.0, 30.0
    y = (rng.rand(B, Cn) < 0.3).astype(np.int64)
    y[0, 0], y[0, 1] = 0, 1                                   # confidently wrong: clamped logs
    loss, d, counters = oracle.sigmoid_bce(z, y)
    zt = torch.tensor(z, requires_grad=True)
    lt = torch.nn.functional.binary_cross_entropy(torch.sigmoid(zt), torch.tensor(y, dtype=torch.float32))
    lt.backward()
    assert abs(loss - float(lt.detach())) < 1e-5 * max(1.0, abs(float(lt.detach())))
    np.testing.assert_allclose(d, zt.grad.numpy(), rtol=1e-4, atol=1e-8)
    pred = (torch.sigmoid(torch.tensor(z)) > 0.5).numpy()
    assert counters == (int((pred & (y != 0)).sum()), int(pred.sum()), int((y != 0).sum()))
    # f1_score of the reference (utils/torch_func.hpp:31-60) on the same batch
    tp, pre, tru = counters
    f1 = 2 * (tp / pre) * (tp / tru) / (tp / pre + tp / tru)
    assert abs(oracle.f1_of(counters) - f1) < 1e-6
    assert oracle.f1_of((0, 5, 9)) == 0.0 and oracle.f1_of((0, 0, 9)) == 0.0
