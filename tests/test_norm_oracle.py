"""CPU checks of the LayerNorm oracle (oracle_ln_forward / oracle_ln_backward, the restatement of
tmt-cuda/src/norm.cu:8-94) against a float64 evaluation of the reference's formulas, and a finite-difference
check of the backward pass. The reference holds no stored vectors for its LayerNorm (its own test is the
end-to-end learning test): parity of this component is unpinned by the reference."""
import numpy as np

from oracle import oracle as O


def _f64(xb, g, b):
    x = O.bf16_to_f32(xb).astype(np.float64)
    mu = x.mean(1)
    var = (x * x).mean(1) - mu * mu                   # norm.cu:39: E[x^2] - mean^2
    rs = 1.0 / np.sqrt(var + 1e-5)
    return x, mu, rs, (x - mu[:, None]) * rs[:, None] * g + b


def test_forward_and_backward_match_float64():
    rng = np.random.default_rng(1)
    for rows, D in ((7, 64), (300, 512), (130, 2048)):
        xb = O.f32_to_bf16(rng.normal(0.5, 1.5, (rows, D)).astype(np.float32))
        g = rng.normal(1, 0.2, D).astype(np.float32)
        b = rng.normal(0, 0.2, D).astype(np.float32)
        Y, mean, rstd = O.ln_forward(xb, g, b)
        x, mu, rs, ref = _f64(xb, g, b)
        np.testing.assert_allclose(mean, mu, rtol=0, atol=2e-6)
        np.testing.assert_allclose(rstd, rs, rtol=3e-6)
        np.testing.assert_allclose(O.bf16_to_f32(Y), ref, rtol=8e-3, atol=1e-6)      # bf16 output
        dyb = O.f32_to_bf16(rng.normal(0, 1, (rows, D)).astype(np.float32))
        dX, dG, dB = O.ln_backward(xb, dyb, g, mean, rstd)
        dy = O.bf16_to_f32(dyb).astype(np.float64)
        xh = (x - mu[:, None]) * rs[:, None]
        gg = dy * g
        want = rs[:, None] * (gg - gg.mean(1)[:, None] - xh * (gg * xh).mean(1)[:, None])
        np.testing.assert_allclose(O.bf16_to_f32(dX), want, rtol=8e-3, atol=2e-3)
        np.testing.assert_allclose(dG, (dy * xh).sum(0), rtol=2e-4, atol=2e-4)
        np.testing.assert_allclose(dB, dy.sum(0), rtol=2e-5, atol=2e-5)


def test_backward_is_the_gradient_of_forward():
    rng = np.random.default_rng(2)
    rows, D = 3, 64
    x = rng.normal(0, 1, (rows, D))
    g = rng.normal(1, 0.2, D).astype(np.float32)
    b = np.zeros(D, np.float32)
    dy = rng.normal(0, 1, (rows, D))

    def loss(xx):
        mu = xx.mean(1, keepdims=True)
        rs = 1.0 / np.sqrt((xx * xx).mean(1, keepdims=True) - mu * mu + 1e-5)
        return float((((xx - mu) * rs * g + b) * dy).sum())
    xb = O.f32_to_bf16(x.astype(np.float32))
    xq = O.bf16_to_f32(xb).astype(np.float64)
    dyb = O.f32_to_bf16(dy.astype(np.float32))
    dy = O.bf16_to_f32(dyb).astype(np.float64)
    _, mean, rstd = O.ln_forward(xb, g, b)
    dX, _, _ = O.ln_backward(xb, dyb, g, mean, rstd)
    num = np.zeros_like(xq)
    for i in range(rows):
        for j in range(0, D, 7):
            e = np.zeros_like(xq); e[i, j] = 1e-4
            num[i, j] = (loss(xq + e) - loss(xq - e)) / 2e-4
    sel = np.zeros_like(xq, bool); sel[:, ::7] = True
    np.testing.assert_allclose(O.bf16_to_f32(dX)[sel], num[sel], rtol=2e-2, atol=2e-2)
