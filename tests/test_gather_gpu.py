"""Feature / label gather parity (bit-exact copies) including cache hits, zero-copy host misses and
a node-id-sharded table."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from helpers import dev_f32, dev_i32, dev_i64, host_f32
from neutronbench_b200 import Cuda_Stream, _lib
from neutronbench_b200.cuda_stream import ptr

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("F", [1, 7, 100, 128, 602])
def test_plain_gather_from_device_table(cuda_device, F):
    rng = np.random.RandomState(F)
    V, n = 5000, 1777
    feat = rng.randn(V, F).astype(np.float32)
    src = np.sort(rng.choice(V, n, replace=False)).astype(np.uint32)
    ref = oracle.feature_gather(feat, src)
    x0 = torch.full((n, F), float("nan"), device=cuda_device)
    cs = Cuda_Stream()
    cs.zero_copy_feature_move_gpu(ptr(x0), ptr(dev_f32(feat, cuda_device)), ptr(dev_i32(src, cuda_device)), F, n)
    cs.CUDA_DEVICE_SYNCHRONIZE()
    np.testing.assert_array_equal(host_f32(x0), ref)


def test_zero_copy_from_pinned_host(cuda_device):
    rng = np.random.RandomState(2)
    V, n, F = 3000, 900, 100
    feat = torch.from_numpy(rng.randn(V, F).astype(np.float32)).pin_memory()
    src = rng.choice(V, n, replace=False).astype(np.uint32)
    ref = oracle.feature_gather(feat.numpy(), src)
    x0 = torch.empty((n, F), device=cuda_device)
    cs = Cuda_Stream()
    cs.zero_copy_feature_move_gpu(ptr(x0), ptr(feat), ptr(dev_i32(src, cuda_device)), F, n)
    cs.CUDA_DEVICE_SYNCHRONIZE()
    np.testing.assert_array_equal(host_f32(x0), ref)


@pytest.mark.parametrize("F,rate", [(602, 0.2), (100, 0.2), (128, 1.0), (602, 0.0)])
def test_cached_gather_hits_and_misses(cuda_device, F, rate):
    from neutronbench_b200 import cache_slots_by_degree
    rng = np.random.RandomState(3)
    V, n = 4000, 2500
    feat = rng.randn(V, F).astype(np.float32)
    deg = rng.randint(1, 30, size=V).astype(np.uint32)
    num = int(V * rate)
    hm_ref, ids = oracle.cache_by_degree(deg, num)
    hm = cache_slots_by_degree(deg, num)
    np.testing.assert_array_equal(hm, hm_ref)           # host-side slot map equals the oracle's
    src = np.sort(rng.choice(V, n, replace=False)).astype(np.uint32)
    ref = oracle.feature_gather(feat, src)
    ld = (F + 3) // 4 * 4
    d = cuda_device
    dfeat = torch.from_numpy(feat).pin_memory()          # misses come from mapped host memory
    dhm = dev_i32(hm, d)
    cache = torch.zeros((max(num, 1), ld), device=d)
    if num:
        _lib.call("nb_cache_fill", ptr(cache), ld, ptr(dfeat), F, ptr(dhm), V, F,
                  torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        np.testing.assert_array_equal(host_f32(cache)[:, :F], feat[ids])
    x0 = torch.empty((n, F), device=d)
    cs = Cuda_Stream()
    cs.gather_feature_cached(ptr(x0), ptr(dfeat), ptr(cache), ptr(dev_i32(src, d)), F, n, ptr(dhm), ld)
    cs.CUDA_DEVICE_SYNCHRONIZE()
    np.testing.assert_array_equal(host_f32(x0), ref)


def test_sharded_table(cuda_device):
    rng = np.random.RandomState(4)
    V, n, F, shards = 4001, 1500, 128, 4
    rows = (V + shards - 1) // shards
    feat = rng.randn(V, F).astype(np.float32)
    parts = [dev_f32(feat[i * rows: (i + 1) * rows], cuda_device) for i in range(shards)]
    table = torch.tensor([p.data_ptr() for p in parts], dtype=torch.int64, device=cuda_device)
    src = rng.choice(V, n, replace=False).astype(np.uint32)
    ref = oracle.feature_gather(feat, src)
    x0 = torch.empty((n, F), device=cuda_device)
    _lib.call("nb_feature_gather", ptr(x0), None, F, ptr(table), shards, rows, None, 0, None,
              ptr(dev_i32(src, cuda_device)), n, F, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(host_f32(x0), ref)


@pytest.mark.parametrize("label_size", [1, 5])
def test_label_gather(cuda_device, label_size):
    rng = np.random.RandomState(5)
    V, n = 1000, 333
    label = rng.randint(0, 40, size=(V, label_size)).astype(np.int64)
    dst = rng.choice(V, n, replace=False).astype(np.uint32)
    ref = oracle.label_gather(label.reshape(-1), dst, label_size)
    out = torch.empty((n, label_size), dtype=torch.int64, device=cuda_device)
    cs = Cuda_Stream()
    if label_size == 1:
        cs.global_copy_label_move_gpu(ptr(out), ptr(dev_i64(label, cuda_device)), ptr(dev_i32(dst, cuda_device)), n)
    else:
        cs.global_copy_mulilabel_move_gpu(ptr(out), ptr(dev_i64(label, cuda_device)), ptr(dev_i32(dst, cuda_device)),
                                          n, label_size)
    cs.CUDA_DEVICE_SYNCHRONIZE()
    np.testing.assert_array_equal(out.cpu().numpy().reshape(ref.shape), ref)
