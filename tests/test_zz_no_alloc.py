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


@pytest.mark.parametrize("T,D,E", [(70, 2048, 64), (90, 512, 80), (45, 256, 16), (130, 384, 32)],
                         ids=["64_experts_x_2048_exactly_the_limit", "80_experts_two_passes", "16_experts", "32_experts"])
def test_no_alloc_all_expert_widths_on_a_side_stream(T, D, E):
    """Every accumulator width of the first kernel (8 is covered above; here 16, 32, 64), the loop over more than 64
    experts and the largest size the built-in scratch holds, on a stream of its own, against the product written out in
    numpy: sum over tokens of bf16(dlogits[t, e]) * X[t, d] in float64."""
    import tmt_moe_b200 as M
    from oracle import oracle as O
    lib = M.load()
    rng = np.random.default_rng(1000 + E)
    dl = (rng.standard_normal((T, E)) * 0.05).astype(np.float32)
    X = O.f32_to_bf16(rng.standard_normal((T, D), dtype=np.float32))
    want = O.bf16_to_f32(O.f32_to_bf16(dl)).astype(np.float64).T @ O.bf16_to_f32(X).astype(np.float64)
    d_dl = torch.from_numpy(dl).cuda()
    d_X = torch.from_numpy(X.view(np.int16).copy()).cuda()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    for _ in range(2):                                   # the second call finds the first one's partial sums in the array
        out = torch.full((E, D), float("nan"), device="cuda")
        side.wait_stream(torch.cuda.current_stream())
        rc = lib.tmt_moe_router_dw_noalloc(ctypes.c_void_p(d_dl.data_ptr()), ctypes.c_void_p(d_X.data_ptr()), T, D, E,
                                           ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(side.cuda_stream))
        assert rc == 0, lib.tmt_moe_last_error().decode()
        side.synchronize()
        got = out.cpu().numpy()
        assert np.isfinite(got).all()
        assert synth.rel_l2(got, want) <= 1e-5


def test_no_alloc_rejects_sizes_beyond_the_scratch():
    import tmt_moe_b200 as M
    lib = M.load()
    x = torch.zeros(16, device="cuda")
    rc = lib.tmt_moe_router_dw_noalloc(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(x.data_ptr()), 4, 4096, 64,
                                       ctypes.c_void_p(x.data_ptr()), None)
    assert rc == -1
    assert b"exceeds the built-in scratch" in lib.tmt_moe_last_error()
