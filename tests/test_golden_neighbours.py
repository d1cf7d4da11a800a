"""The two neighbours of the MoE block against the REFERENCE's own outputs: tests/golden/ref_ln_*.npz and
ref_adam_*.npz were made by tests/golden/make_ref_vectors.py from tmt-cuda/src/norm.cu and adam.cu recompiled for
sm_100a and run on a B200. The CPU oracle is checked here without a GPU, the CUDA kernels in the tests marked gpu.

Tolerances (the reference is built with fast-math, sums in another order and adds block results with atomics):
LayerNorm: mean / rstd relative 1e-5; Y and dX relative L2 <= 4e-3 and at most one bf16 step (2^-7 relative) per
element; dGamma / dBeta relative L2 <= 1e-4. AdamW: squared norm relative 1e-12 (both in double); master weights
relative 2e-6 of the update's size, moments relative 1e-6; bf16 working copies within one bf16 step. The update
formula here is fma(-lr, fma(wd, w, u), w), the reference's is w - lr * (u + wd * w): the same real-number function,
rounded in a different sequence, which is what the master-weight tolerance bounds."""
import os
import sys

import numpy as np
import pytest

from tmt_moe_b200 import synth
from oracle import oracle as O

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
from make_ref_vectors import ADAM_CASES, ADAM_HYP, LN_CASES, adam_inputs, ln_inputs  # noqa: E402

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _load(name):
    return np.load(os.path.join(GOLD, "ref_%s.npz" % name))


def _bf16_close(got, want, steps=1):
    """bf16 bit patterns: every element within `steps` bf16 steps of the reference's value."""
    g, w = O.bf16_to_f32(got).astype(np.float64), O.bf16_to_f32(want).astype(np.float64)
    tol = steps * np.maximum(np.abs(w), 1e-30) * 2.0 ** -7
    assert (np.abs(g - w) <= tol).all(), float(np.max(np.abs(g - w) / np.maximum(np.abs(w), 1e-30)))


def _check_ln(got, ref):
    np.testing.assert_allclose(got["mean"], ref["mean"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(got["rstd"], ref["rstd"], rtol=1e-5)
    assert synth.rel_l2(O.bf16_to_f32(got["Y"]), O.bf16_to_f32(ref["Y"])) <= 4e-3
    assert synth.rel_l2(O.bf16_to_f32(got["dX"]), O.bf16_to_f32(ref["dX"])) <= 4e-3
    # one bf16 step, measured against the row's largest magnitude (cancellation makes tiny outputs relatively noisy)
    for k in ("Y", "dX"):
        g, w = O.bf16_to_f32(got[k]).astype(np.float64), O.bf16_to_f32(ref[k]).astype(np.float64)
        assert (np.abs(g - w) <= np.abs(w).max(axis=1, keepdims=True) * 2.0 ** -7).all(), k
    assert synth.rel_l2(got["dGamma"], ref["dGamma"]) <= 1e-4
    assert synth.rel_l2(got["dBeta"], ref["dBeta"]) <= 1e-4


def _check_adam(c, got, ref, before):
    assert abs(got["sumsq"] - float(ref["sumsq"])) <= 1e-12 * float(ref["sumsq"])
    np.testing.assert_allclose(got["m"], ref["m"], rtol=1e-6, atol=1e-12)
    np.testing.assert_allclose(got["v"], ref["v"], rtol=1e-6, atol=1e-20)
    upd = np.abs(ref["master"] - before).max()
    assert upd > 0
    assert np.abs(got["master"] - ref["master"]).max() <= 2e-6 * upd + 2.0 ** -24 * np.abs(ref["master"]).max()
    off = 0
    for n, fl in zip(c["sizes"], c["flags"]):
        sl = slice(off, off + n)
        if fl & 2:
            _bf16_close(got["work"][sl], ref["work"][sl])
        else:       # frozen: untouched by both
            np.testing.assert_array_equal(got["master"][sl], before[sl])
            np.testing.assert_array_equal(ref["master"][sl], before[sl])
        off += n


def _oracle_adam(c):
    master, m, v, grad = adam_inputs(c)
    ss = O.sumsq([grad[sum(c["sizes"][:i]):sum(c["sizes"][:i + 1])] for i, f in enumerate(c["flags"]) if f & 1])
    scale = O.clip_scale(ss, c["clip"])
    out = dict(master=master.copy(), m=m.copy(), v=v.copy(), work=np.zeros(master.size, np.uint16), sumsq=ss)
    off = 0
    for n, fl in zip(c["sizes"], c["flags"]):
        sl = slice(off, off + n)
        if fl & 2:
            out["master"][sl], out["m"][sl], out["v"][sl], out["work"][sl] = O.adamw(
                master[sl], m[sl], v[sl], grad[sl], scale, ADAM_HYP["lr"], ADAM_HYP["b1"], ADAM_HYP["b2"], ADAM_HYP["eps"],
                ADAM_HYP["wd"], c["step"])
        off += n
    return out, master


@pytest.mark.parametrize("name", sorted(LN_CASES))
def test_layernorm_oracle_matches_reference_outputs(oracle, name):
    X, dY, gamma, beta = ln_inputs(LN_CASES[name])
    Y, mean, rstd = oracle.ln_forward(X, gamma, beta)
    dX, dG, dB = oracle.ln_backward(X, dY, gamma, mean, rstd)
    _check_ln(dict(Y=Y, mean=mean, rstd=rstd, dX=dX, dGamma=dG, dBeta=dB), _load(name))


@pytest.mark.parametrize("name", sorted(ADAM_CASES))
def test_adamw_oracle_matches_reference_outputs(oracle, name):
    c = ADAM_CASES[name]
    got, before = _oracle_adam(c)
    _check_adam(c, got, _load(name), before)


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(LN_CASES))
def test_layernorm_cuda_matches_reference_outputs(name):
    import torch
    import tmt_moe_b200 as M
    X, dY, gamma, beta = ln_inputs(LN_CASES[name])
    rows, D = X.shape
    dev = lambda a: torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).cuda()
    dXd, dYd, G, B = dev(X), dev(dY), dev(gamma), dev(beta)
    Y, dX = torch.zeros_like(dXd), torch.zeros_like(dXd)
    mean, rstd = torch.zeros(rows, device="cuda"), torch.zeros(rows, device="cuda")
    dG, dB = torch.zeros(D, device="cuda"), torch.zeros(D, device="cuda")
    scratch = torch.zeros(M.ln_backward_scratch_bytes(rows, D) // 4, device="cuda")
    M.ln_forward(dXd, G, B, Y, mean, rstd)
    M.ln_backward(dXd, dYd, G, mean, rstd, dX, dG, dB, scratch)
    torch.cuda.synchronize()
    u16 = lambda t: t.cpu().numpy().view(np.uint16)
    _check_ln(dict(Y=u16(Y), mean=mean.cpu().numpy(), rstd=rstd.cpu().numpy(), dX=u16(dX), dGamma=dG.cpu().numpy(),
                   dBeta=dB.cpu().numpy()), _load(name))


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(ADAM_CASES))
def test_adamw_cuda_matches_reference_outputs(name):
    import torch
    import tmt_moe_b200 as M
    c = ADAM_CASES[name]
    master, m, v, grad = adam_inputs(c)
    flat = {k: torch.from_numpy(a.copy()).cuda() for k, a in dict(master=master, m=m, v=v, grad=grad).items()}
    work = torch.zeros(master.size, dtype=torch.int16, device="cuda")
    views = {k: [] for k in ("master", "m", "v", "grad", "work")}
    off = 0
    for n in c["sizes"]:
        for k in ("master", "m", "v", "grad"):
            views[k].append(flat[k][off:off + n])
        views["work"].append(work[off:off + n])
        off += n
    opt = M.AdamW(c["sizes"])
    ss = opt.step(views["master"], views["m"], views["v"], views["grad"], views["work"], c["flags"], clip=c["clip"],
                  step=c["step"], zero_grads=True, want_norm=True, **ADAM_HYP)
    torch.cuda.synchronize()
    got = dict(master=flat["master"].cpu().numpy(), m=flat["m"].cpu().numpy(), v=flat["v"].cpu().numpy(),
               work=work.cpu().numpy().view(np.uint16), sumsq=ss)
    ref = _load(name)
    _check_adam(c, got, ref, master)
    assert float(flat["grad"].abs().max()) == 0.0 and float(np.abs(ref["grad"]).max()) == 0.0     # both clear every gradient
    opt.close()
