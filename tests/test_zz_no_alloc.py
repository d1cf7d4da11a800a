"""The entry point that allocates nothing (tmt_moe_router_dw_noalloc): its scratch is a fixed
array in the library image, shared by every call on a GPU. Checked through the C ABI against
the router weight gradient the handle-based tmt_moe_backward returns, on two calls in a row
with different sizes, so that whatever the first call left in the shared array would show up
in the second. Collected last on purpose (file name), so a run that stops at the first failure
has already run every other test."""
import ctypes

import numpy as np
import pytest
import torch

from tmt_moe_b200 import synth

pytestmark = pytest.mark.gpu


def _case(T, D, H, E, K, seed):
    import gpu_util as G
    data = synth.make(T, D, H, E, K, seed=seed, w_std=0.05, router_std=0.1, dy_std=0.1)
    layer = G.Layer(data, T, D, E, K, H)
    layer.forward()
    g = layer.backward(data["dY"], 0.1, 0.001)
    return layer, g["dWr"], layer.moe.read("dlogits")


def test_no_alloc_router_gradient_twice_in_a_row():
    import tmt_moe_b200 as M
    lib = M.load()
    assert torch.cuda.is_available()
    # second case is smaller: stale partial sums of the first would land in rows it reads
    for (T, D, H, E, K, seed) in ((1500, 256, 128, 8, 2, 21), (333, 128, 64, 5, 2, 22)):
        layer, ref, dlogits = _case(T, D, H, E, K, seed)
        dl = torch.from_numpy(dlogits).cuda()
        out = torch.full((E, D), float("nan"), device="cuda")
        rc = lib.tmt_moe_router_dw_noalloc(ctypes.c_void_p(dl.data_ptr()), ctypes.c_void_p(layer.X.data_ptr()),
                                           T, D, E, ctypes.c_void_p(out.data_ptr()), None)
        assert rc == 0, lib.tmt_moe_last_error().decode()
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        assert np.isfinite(got).all()
        assert synth.rel_l2(got, ref) <= 3e-2          # the gradient tolerance of the other GPU tests
        assert synth.rel_l2(got, ref) <= 1e-5          # same products, only the summation order differs


def test_no_alloc_rejects_sizes_beyond_the_scratch():
    import tmt_moe_b200 as M
    lib = M.load()
    x = torch.zeros(16, device="cuda")
    rc = lib.tmt_moe_router_dw_noalloc(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(x.data_ptr()), 4, 4096, 64,
                                       ctypes.c_void_p(x.data_ptr()), None)
    assert rc == -1
    assert b"exceeds the built-in scratch" in lib.tmt_moe_last_error()
