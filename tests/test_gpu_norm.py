"""LayerNorm on the GPU (include/tmt_norm.h) against the CPU oracle: outputs, statistics, input gradient and the
gamma / beta gradients are bit-identical (the summation orders are part of the interface)."""
import numpy as np
import pytest
import torch

import tmt_moe_b200 as M
from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,D", [(1, 64), (37, 256), (300, 512), (260, 2048), (129, 4096), (5, 8192), (131, 320)])
def test_forward_and_backward_are_bit_identical_to_the_oracle(rows, D):
    rng = np.random.default_rng(rows * 1000 + D)
    xb = O.f32_to_bf16(rng.normal(0.3, 1.2, (rows, D)).astype(np.float32))
    dyb = O.f32_to_bf16(rng.normal(0, 1e-1, (rows, D)).astype(np.float32))
    g = rng.normal(1, 0.2, D).astype(np.float32)
    b = rng.normal(0, 0.2, D).astype(np.float32)
    dev = lambda a: torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).cuda()
    X, dY, G, B = dev(xb), dev(dyb), dev(g), dev(b)
    Y = torch.zeros_like(X)
    mean, rstd = torch.zeros(rows, device="cuda"), torch.zeros(rows, device="cuda")
    M.ln_forward(X, G, B, Y, mean, rstd)
    wY, wm, wr = O.ln_forward(xb, g, b)
    np.testing.assert_array_equal(mean.cpu().numpy().view(np.uint32), wm.view(np.uint32))
    np.testing.assert_array_equal(rstd.cpu().numpy().view(np.uint32), wr.view(np.uint32))
    np.testing.assert_array_equal(Y.cpu().numpy().view(np.uint16), wY)
    dX = torch.zeros_like(X)
    dG, dB = torch.full((D,), float("nan"), device="cuda"), torch.full((D,), float("nan"), device="cuda")
    scratch = torch.zeros(M.ln_backward_scratch_bytes(rows, D) // 4, device="cuda")
    M.ln_backward(X, dY, G, mean, rstd, dX, dG, dB, scratch)
    wdX, wdG, wdB = O.ln_backward(xb, dyb, g, wm, wr)
    np.testing.assert_array_equal(dX.cpu().numpy().view(np.uint16), wdX)
    np.testing.assert_array_equal(dG.cpu().numpy().view(np.uint32), wdG.view(np.uint32))
    np.testing.assert_array_equal(dB.cpu().numpy().view(np.uint32), wdB.view(np.uint32))


def test_bad_shapes_are_refused():
    x = torch.zeros((4, 100), dtype=torch.int16, device="cuda")
    f = torch.zeros(100, device="cuda")
    with pytest.raises(M.MoeError):
        M.ln_forward(x, f, f, x, f, f)            # dim not a multiple of 8
