"""Dense pieces against the oracle: GEMM (NN/TN/NT), ReLU+dropout (bit-exact mask), softmax/NLL loss,
Adam (bit-exact)."""
import numpy as np
import pytest
import torch

import oracle
from helpers import dev_f32, dev_i64, host_f32
from neutronbench_b200 import _lib
from neutronbench_b200.cuda_stream import ptr

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[17, 0, 18, 1], ids=["tcgen05_3xtf32", "cuda_cores", "tcgen05_tf32", "default"])
def gemm_mode(request):
    """Every GEMM test runs on the tensor-core path (default), the CUDA-core path and plain TF32."""
    lib = _lib.load()
    old = lib.nb_set_gemm_mode(request.param)
    yield request.param
    lib.nb_set_gemm_mode(old)
    import ctypes
    flags = ctypes.c_uint32(0)
    _lib.call("nb_device_error_flags", ctypes.byref(flags))
    assert flags.value == 0


RTOL = 1e-5   # fp32 tolerance of the north star; the GEMMs differ from the oracle only in summation order


def _close(a, b, k, mode=1):
    scale = np.abs(b).max() + 1e-30
    tol = 2e-3 if mode == 18 else RTOL * max(1.0, np.sqrt(k) / 8)   # plain TF32 keeps 10 mantissa bits
    assert np.abs(a - b).max() / scale < tol, (np.abs(a - b).max(), scale)


@pytest.mark.parametrize("M,K,N", [(1, 1, 1), (63, 17, 65), (1024, 128, 41), (3000, 602, 128), (200, 1433, 16),
                                   (3000, 604, 128), (777, 100, 128), (19000, 128, 64), (130, 32, 32), (19777, 604, 128),
                                   (8200, 36, 96), (23600, 100, 128)])
def test_gemm_nn(cuda_device, ws, gemm_mode, M, K, N):
    rng = np.random.RandomState(M + K + N)
    a, b = rng.randn(M, K).astype(np.float32), rng.randn(K, N).astype(np.float32)
    c = torch.empty((M, N), device=cuda_device)
    _lib.call("nb_gemm", ws.handle, ptr(dev_f32(a, cuda_device)), ptr(dev_f32(b, cuda_device)), ptr(c), M, N, K, 0, 0,
              torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    _close(host_f32(c), oracle.gemm_nn(a, b), K, gemm_mode)


@pytest.mark.parametrize("M,K,N", [(5000, 602, 128), (1024, 128, 41), (70, 3, 5), (25000, 100, 128), (5000, 604, 128),
                                   (4001, 36, 64)])
def test_gemm_tn_weight_gradient(cuda_device, ws, gemm_mode, M, K, N):
    """dW[K x N] = Y^T[K x M] dZ[M x N]; the long reduction over M runs split-K."""
    rng = np.random.RandomState(M + N)
    y, dz = rng.randn(M, K).astype(np.float32), rng.randn(M, N).astype(np.float32)
    c = torch.empty((K, N), device=cuda_device)
    _lib.call("nb_gemm", ws.handle, ptr(dev_f32(y, cuda_device)), ptr(dev_f32(dz, cuda_device)), ptr(c), K, N, M, 1, 0,
              torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    _close(host_f32(c), oracle.gemm_tn(y, dz), M, gemm_mode)


@pytest.mark.parametrize("M,N,K", [(1024, 41, 128), (3000, 128, 128), (7, 5, 3), (1000, 64, 96), (20000, 128, 128)])
def test_gemm_nt_input_gradient(cuda_device, ws, gemm_mode, M, N, K):
    """dY[M x K] = dZ[M x N] W^T with W[K x N]."""
    rng = np.random.RandomState(M + N + K)
    dz, w = rng.randn(M, N).astype(np.float32), rng.randn(K, N).astype(np.float32)
    c = torch.empty((M, K), device=cuda_device)
    _lib.call("nb_gemm", ws.handle, ptr(dev_f32(dz, cuda_device)), ptr(dev_f32(w, cuda_device)), ptr(c), M, K, N, 0, 1,
              torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    _close(host_f32(c), oracle.gemm_nt(dz, w), N, gemm_mode)


@pytest.mark.parametrize("n,p", [(1, 0.5), (1023, 0.5), (4096, 0.0), (100003, 0.3)])
def test_relu_dropout_bit_exact(cuda_device, n, p):
    z = np.random.RandomState(n).randn(n).astype(np.float32)
    ref = oracle.relu_dropout(z, p, seed=2000, layer=1, step=17)
    dz = dev_f32(z, cuda_device)
    _lib.call("nb_relu_dropout", ptr(dz), n, p, 2000, 1, 17, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(host_f32(dz).view(np.uint32), ref.view(np.uint32))
    if p > 0 and n > 50000:
        kept = (ref[z > 0] != 0).mean()
        assert abs(kept - (1 - p)) < 0.01


@pytest.mark.parametrize("B,C", [(1, 2), (1024, 41), (4096, 47), (777, 172)])
def test_softmax_nll(cuda_device, ws, B, C):
    rng = np.random.RandomState(B)
    logits = (rng.randn(B, C) * 3).astype(np.float32)
    label = rng.randint(0, C, size=B).astype(np.int64)
    loss, dref, correct = oracle.softmax_nll(logits, label)
    d = torch.empty((B, C), device=cuda_device)
    stats = torch.zeros(2, device=cuda_device)
    _lib.call("nb_softmax_nll", ws.handle, ptr(dev_f32(logits, cuda_device)), ptr(dev_i64(label, cuda_device)), B, C,
              ptr(d), ptr(stats), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    got = stats.cpu().numpy()
    assert abs(got[0] - loss) <= 1e-5 * max(1.0, abs(loss))
    assert int(got[1]) == correct
    np.testing.assert_allclose(host_f32(d), dref, rtol=1e-4, atol=1e-7 / B)


def test_adam_bit_exact_over_steps(cuda_device):
    rng = np.random.RandomState(0)
    n = 82304 + 3
    W = rng.randn(n).astype(np.float32) * 0.1
    M, V = np.zeros(n, np.float32), np.zeros(n, np.float32)
    dW, dM, dV = dev_f32(W, cuda_device), dev_f32(M, cuda_device), dev_f32(V, cuda_device)
    b1, b2 = np.float32(0.9), np.float32(0.999)
    b1_t, b2_t = b1, b2
    for step in range(4):
        g = rng.randn(n).astype(np.float32) * 0.01
        oracle.adam(W, g, M, V, 0.01, 0.9, 0.999, 1e-9, 0.0001, float(b1_t), float(b2_t))
        _lib.call("nb_adam", ptr(dW), ptr(dev_f32(g, cuda_device)), ptr(dM), ptr(dV), n, 0.01, 0.9, 0.999, 1e-9, 0.0001,
                  float(b1_t), float(b2_t), torch.cuda.current_stream().cuda_stream)
        b1_t, b2_t = np.float32(b1_t * b1), np.float32(b2_t * b2)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(host_f32(dW).view(np.uint32), W.view(np.uint32))
    np.testing.assert_array_equal(host_f32(dM).view(np.uint32), M.view(np.uint32))
    np.testing.assert_array_equal(host_f32(dV).view(np.uint32), V.view(np.uint32))


@pytest.mark.parametrize("B,C", [(1, 1), (37, 11), (1024, 121), (300, 33)])
def test_sigmoid_bce_matches_oracle(cuda_device, ws, B, C):
    """Multi-label loss, gradient and F1 counters (CLASSES > 1) against the oracle; the counters are exact."""
    rng = np.random.RandomState(B + C)
    z = (rng.randn(B, C) * 3).astype(np.float32)
    z.flat[0] = 110.0
    y = (rng.rand(B, C) < 0.25).astype(np.int64)
    y.flat[0] = 0
    loss, d_ref, counters = oracle.sigmoid_bce(z, y)
    dz = torch.full((B, C), float("nan"), device=cuda_device)
    stats = torch.zeros(4, device=cuda_device)
    st = torch.cuda.current_stream().cuda_stream
    _lib.call("nb_sigmoid_bce", ws.handle, ptr(dev_f32(z, cuda_device)), ptr(dev_i64(y, cuda_device)), B, C, ptr(dz),
              ptr(stats), st)
    s = stats.cpu().numpy()
    assert abs(s[0] - loss) <= 2e-5 * max(1.0, abs(loss))
    assert (int(s[1]), int(s[2]), int(s[3])) == counters
    np.testing.assert_allclose(dz.cpu().numpy(), d_ref, rtol=2e-4, atol=1e-9)
    # forward only: no gradient buffer
    _lib.call("nb_sigmoid_bce", ws.handle, ptr(dev_f32(z, cuda_device)), ptr(dev_i64(y, cuda_device)), B, C, None,
              ptr(stats), st)
    assert abs(float(stats[0]) - loss) <= 2e-5 * max(1.0, abs(loss))


@pytest.mark.parametrize("kind,M,N,K", [("NN", 3000, 128, 604), ("TN", 604, 128, 9000), ("NT", 5000, 128, 128),
                                        ("NN", 19777, 128, 604), ("NN", 9000, 64, 100)])
def test_tma_and_cp_async_kernels_give_identical_bits(cuda_device, ws, kind, M, N, K):
    """The TMA-fed kernel and the cp.async kernel issue the same MMAs in the same order and cut K at the same
    places, so a caller whose operands do not qualify for tensor maps gets the same bits as one whose do."""
    import os
    lib = _lib.load()
    old = lib.nb_set_gemm_mode(17)
    rng = np.random.RandomState(M + N + K)
    if kind == "NN":
        a, b, ta, tb = rng.randn(M, K), rng.randn(K, N), 0, 0
    elif kind == "TN":
        a, b, ta, tb = rng.randn(K, M), rng.randn(K, N), 1, 0
    else:
        a, b, ta, tb = rng.randn(M, K), rng.randn(N, K), 0, 1
    da, db = dev_f32(a.astype(np.float32), cuda_device), dev_f32(b.astype(np.float32), cuda_device)
    outs = []
    try:
        for no_tma in ("", "1"):
            if no_tma:
                os.environ["NB_TC_NO_TMA"] = "1"
            c = torch.full((M, N), float("nan"), device=cuda_device)
            _lib.call("nb_gemm", ws.handle, ptr(da), ptr(db), ptr(c), M, N, K, ta, tb, torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            outs.append(host_f32(c).copy())
    finally:
        os.environ.pop("NB_TC_NO_TMA", None)
        lib.nb_set_gemm_mode(old)
    np.testing.assert_array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))


@pytest.mark.parametrize("B,H,C", [(1024, 128, 41), (37, 16, 7), (300, 32, 64), (9, 5, 1), (1000, 100, 47)])
def test_fused_output_layer_matches_oracle(cuda_device, ws, B, H, C):
    """nb_output_layer = Y W, softmax/NLL on gathered labels, dW = Y^T dZ, dY = dZ W^T in two launches."""
    assert _lib.load().nb_output_layer_supported(H, C) == 1
    rng = np.random.RandomState(B + H + C)
    V = B * 3
    y, w = rng.randn(B, H).astype(np.float32), (rng.randn(H, C) * 0.3).astype(np.float32)
    table = rng.randint(0, C, size=V).astype(np.int64)
    dst = rng.choice(V, B, replace=False).astype(np.uint32)
    z = oracle.gemm_nn(y, w)
    loss, dz, correct = oracle.softmax_nll(z, table[dst])
    dw_ref, dy_ref = oracle.gemm_tn(y, dz), oracle.gemm_nt(dz, w)
    st = torch.cuda.current_stream().cuda_stream
    dy = torch.full((B, H), float("nan"), device=cuda_device)
    dw = torch.full((H, C), float("nan"), device=cuda_device)
    stats = torch.zeros(4, device=cuda_device)
    from helpers import dev_i32
    args = (ws.handle, ptr(dev_f32(y, cuda_device)), ptr(dev_f32(w, cuda_device)), ptr(dev_i64(table, cuda_device)),
            ptr(dev_i32(dst, cuda_device)), B, H, C)
    _lib.call("nb_output_layer", *args, 1, ptr(dw), ptr(dy), ptr(stats), st)
    s = stats.cpu().numpy()
    assert abs(s[0] - loss) < 1e-5 * max(1.0, abs(loss)) and int(s[1]) == correct
    _close(host_f32(dw), dw_ref, B)
    _close(host_f32(dy), dy_ref, C)
    # evaluation: loss and hits only, gradients untouched
    dw.fill_(7.0)
    _lib.call("nb_output_layer", *args, 0, ptr(dw), 0, ptr(stats), st)
    s2 = stats.cpu().numpy()
    assert s2[0] == s[0] and s2[1] == s[1] and float(dw.min()) == 7.0
    # wider layers are refused, not mis-computed
    assert _lib.load().nb_output_layer_supported(128, 65) == 0 and _lib.load().nb_output_layer_supported(4096, 64) == 0


def test_native_step_with_and_without_the_fused_output_layer(cuda_device):
    """Switching nb_output_layer off changes the last layer's summation order only: same loss curve to 1e-5."""
    from neutronbench_b200 import FullyRepGraph, GCN_GPU_NEIGHBOR_impl, GCNConfig, GNNDatum, Sampler, Workspace
    from helpers import small_graph
    V = 3000
    edges, co, ri = small_graph(V, 40000, seed=4)
    rng = np.random.RandomState(0)
    feat, label = rng.randn(V, 24).astype(np.float32), rng.randint(0, 5, size=V).astype(np.int64)
    curves = []
    for fused in (True, False):
        cfg = GCNConfig(layers=[24, 16, 5], fanout=(6, 4), batch_size=128, drop_rate=0.2, seed=11)
        g = FullyRepGraph.from_edges(torch.from_numpy(edges).to(cuda_device), V, Workspace(64 << 20))
        datum = GNNDatum(torch.from_numpy(feat).to(cuda_device), torch.from_numpy(label).to(cuda_device), np.zeros(V, np.int32))
        tk = GCN_GPU_NEIGHBOR_impl(g, datum, cfg)
        tk.fuse_output_layer = fused
        smp = Sampler(g, np.arange(600, dtype=np.uint32), cfg.fanout, cfg.batch_size, tk.ws, seed=cfg.seed,
                      with_edge_weights=False)
        curves.append([tk.Forward(smp, train=True)[1] for _ in range(3)])
    _lib.load().nb_set_fused_output_layer(1)
    np.testing.assert_allclose(curves[0], curves[1], rtol=2e-5)
