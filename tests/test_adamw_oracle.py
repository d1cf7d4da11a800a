"""CPU checks of the AdamW oracle (oracle_adamw / oracle_sumsq, the restatement of tmt-cuda/src/adam.cu:57-99):
against a float64 evaluation of the same formulas, and the properties the reference's optimizer relies on.
The reference holds no golden vectors for its optimizer: parity of this component is unpinned by the reference."""
import numpy as np

from oracle import oracle as O


def _ref64(w, m, v, g, scale, lr, b1, b2, eps, wd, step):
    w, m, v, g = (a.astype(np.float64) for a in (w, m, v, g))
    g = g * scale
    m = b1 * m + (1 - b1) * g
    v = b2 * v + (1 - b2) * g * g
    bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
    w = w - lr * ((m / bc1) / (np.sqrt(v / bc2) + eps) + wd * w)
    return w, m, v


def test_adamw_matches_float64_formulas():
    rng = np.random.default_rng(3)
    n = 10007
    w = rng.normal(0, 0.02, n).astype(np.float32)
    m = rng.normal(0, 1e-3, n).astype(np.float32)
    v = (rng.normal(0, 1e-3, n).astype(np.float32)) ** 2
    g = rng.normal(0, 1e-2, n).astype(np.float32)
    for step in (1, 2, 1000):
        w2, m2, v2, work = O.adamw(w, m, v, g, 0.37, 3e-4, 0.9, 0.999, 1e-8, 0.01, step)
        rw, rm, rv = _ref64(w, m, v, g, np.float32(0.37), np.float32(3e-4), np.float32(0.9), np.float32(0.999), np.float32(1e-8),
                            np.float32(0.01), step)
        np.testing.assert_allclose(m2, rm, rtol=3e-7, atol=3e-10)     # m is a difference of terms near 1e-3
        np.testing.assert_allclose(v2, rv, rtol=3e-7, atol=1e-16)
        np.testing.assert_allclose(w2, rw, rtol=1e-6, atol=1e-9)
        np.testing.assert_array_equal(work, O.f32_to_bf16(w2))


def test_zero_gradient_only_decays_and_scale_one_without_clip():
    w = np.full(64, 2.0, np.float32)
    z = np.zeros(64, np.float32)
    w2, m2, v2, _ = O.adamw(w, z, z, z, 1.0, 0.1, 0.9, 0.999, 1e-8, 0.01, 1)
    np.testing.assert_array_equal(m2, z)
    np.testing.assert_array_equal(v2, z)
    np.testing.assert_allclose(w2, 2.0 - 0.1 * 0.01 * 2.0, rtol=1e-7)
    assert O.clip_scale(123.0, 0.0) == 1.0
    assert O.clip_scale(4.0, 1.0) == 0.5
    assert O.clip_scale(0.25, 1.0) == 1.0


def test_sumsq_is_double_precision():
    g = np.full(1 << 20, 1e-4, np.float32)
    s = O.sumsq([g, g])
    want = 2 * (1 << 20) * float(np.float32(1e-4)) ** 2
    assert abs(s - want) < 1e-9 * want           # a float32 accumulator would be off by ~1e-3 relative
