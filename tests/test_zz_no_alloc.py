"""The workspace-free loss entry point (nb_softmax_nll_static) against the regular one.

It exists for callers that may not allocate or pass scratch at call time (all device memory already
committed to the host application's pool, or an allocation ban after start-up): its scratch is a fixed
array inside the library.  The file name keeps this test last in collection order, so a run that stops
at the first failure has already exercised everything else.  Two calls in a row with different batch
sizes check that nothing left in the shared array by one call leaks into the next."""
import ctypes as C

import numpy as np
import pytest
import torch

from neutronbench_b200 import Workspace, _lib
from neutronbench_b200.cuda_stream import ptr

pytestmark = pytest.mark.gpu


def _both(device, ws, B, Cn, seed):
    g = torch.Generator(device=device).manual_seed(seed)
    logits = torch.randn((B, Cn), device=device, generator=g) * 3
    label = torch.randint(0, Cn, (B,), device=device, generator=g, dtype=torch.int64)
    st = torch.cuda.current_stream().cuda_stream
    d_ref, s_ref = torch.empty((B, Cn), device=device), torch.zeros(2, device=device)
    _lib.call("nb_softmax_nll", ws.handle, ptr(logits), ptr(label), B, Cn, ptr(d_ref), ptr(s_ref), st)
    d_new, s_new = torch.full((B, Cn), float("nan"), device=device), torch.full((2,), float("nan"), device=device)
    used_before = _lib.load().nb_ws_used(ws.handle)
    _lib.call("nb_softmax_nll_static", ptr(logits), ptr(label), B, Cn, ptr(d_new), ptr(s_new), st)
    assert _lib.load().nb_ws_used(ws.handle) == used_before
    torch.cuda.synchronize()
    # same kernels, same launch shapes: the outputs must be identical, not merely close
    np.testing.assert_array_equal(d_new.cpu().numpy().view(np.uint32), d_ref.cpu().numpy().view(np.uint32))
    np.testing.assert_array_equal(s_new.cpu().numpy().view(np.uint32), s_ref.cpu().numpy().view(np.uint32))
    return s_new.cpu().numpy()


def test_static_scratch_loss_matches_workspace_loss_twice():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    ws = Workspace(8 << 20)
    first = _both(device, ws, 4096, 47, seed=1)      # larger batch first ...
    second = _both(device, ws, 1000, 41, seed=2)     # ... then a smaller one over the same array
    assert np.isfinite(first).all() and np.isfinite(second).all()
    ws.close()


def test_static_scratch_loss_rejects_oversized_batch():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    lib = _lib.load()
    st = lib.nb_softmax_nll_static(1, 1, 65537, 4, None, 1, None)   # pointers are not touched before the size check
    assert st == -1
    assert b"65536" in lib.nb_last_error()
