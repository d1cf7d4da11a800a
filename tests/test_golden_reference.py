"""The reference's own outputs (tests/golden/ref_moe_*.npz, made by tests/golden/make_ref_vectors.py
from tmt-cuda/src/moe.cu recompiled for sm_100a and run on a B200) against the CPU oracle (here,
no GPU needed) and against the CUDA path (marked gpu). Reference mode: one DxD matrix per expert.

Tolerances: indices and counts exact; logits 2e-3 absolute (the reference accumulates in another
order); outputs relative L2 <= 1e-2; gradients relative L2 <= 3e-2 per tensor, the reference's own
bar (architecture_test.cu:254); aux and z relative 1e-3 (its router uses fast-math exp)."""
import os
import sys

import numpy as np
import pytest

from tmt_moe_b200 import synth
from oracle import oracle as O

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
from make_ref_vectors import CASES, inputs  # noqa: E402

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _load(name):
    return np.load(os.path.join(GOLD, "ref_moe_%s.npz" % name))


def _check(case, got_fwd, got_bwd, ref):
    E, K = case["E"], case["K"]
    if E > 1:
        np.testing.assert_array_equal(got_fwd["idx"], ref["idx"])
        np.testing.assert_array_equal(got_fwd["counts"], ref["counts"])
        np.testing.assert_allclose(got_fwd["logits"], ref["logits"], atol=2e-3)
        np.testing.assert_allclose(got_fwd["probs"], ref["probs"], atol=1e-3)
        assert abs(got_fwd["aux"] - float(ref["aux"])) <= 1e-3 * abs(float(ref["aux"]))
        assert abs(got_fwd["z"] - float(ref["zloss"])) <= 1e-3 * abs(float(ref["zloss"]))
    assert synth.rel_l2(O.bf16_to_f32(got_fwd["Y"]), O.bf16_to_f32(ref["Y"])) <= 1e-2
    assert synth.rel_l2(O.bf16_to_f32(got_bwd["dX"]), O.bf16_to_f32(ref["dX"])) <= 3e-2
    assert synth.rel_l2(got_bwd["dWup"], ref["dWexp"]) <= 3e-2
    if E > 1:
        assert synth.rel_l2(got_bwd["dWr"], ref["dWr"]) <= 3e-2
    else:
        assert (ref["dWr"] == 0).all() and (got_bwd["dWr"] == 0).all()


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_matches_reference_outputs(oracle, name):
    c = CASES[name]
    d = inputs(c)
    ref = _load(name)
    f = oracle.forward(d["X"], d["Wr"], d["Wup"], None, c["K"], Y=d["Y0"] if c["beta"] else None, beta=c["beta"])
    b = oracle.backward(f, d["dY"], c["aux"], c["zcoef"])
    fwd = dict(idx=f["idx"], counts=f["counts"], logits=f["logits"], probs=f["probs"], aux=f["aux"],
               z=float(f["stat"][c["E"]]), Y=f["Y"])
    _check(c, fwd, b, ref)


def _identity_down(c):
    """hidden = dim and Wdown[e] = I: the two-matrix layer computes gate * silu(x Wup^T), the reference's
    single-matrix layer up to one more bf16 rounding (of the SiLU output and of the gated row)."""
    eye = O.f32_to_bf16(np.eye(c["D"], dtype=np.float32))
    return np.ascontiguousarray(np.broadcast_to(eye, (c["E"], c["D"], c["D"])))


MULTI = sorted(n for n in CASES if CASES[n]["E"] > 1)


@pytest.mark.parametrize("name", MULTI)
def test_two_matrix_oracle_pinned_by_reference_outputs(oracle, name):
    """The oracle's two-matrix mode (up-projection + SiLU, down-projection + gate, and their backward chain) against
    the reference's own outputs: with an identity down-projection both compute the same function. Same tolerances as
    the single-matrix comparison."""
    c = CASES[name]
    d = inputs(c)
    ref = _load(name)
    f = oracle.forward(d["X"], d["Wr"], d["Wup"], _identity_down(c), c["K"], Y=d["Y0"] if c["beta"] else None, beta=c["beta"])
    b = oracle.backward(f, d["dY"], c["aux"], c["zcoef"])
    fwd = dict(idx=f["idx"], counts=f["counts"], logits=f["logits"], probs=f["probs"], aux=f["aux"],
               z=float(f["stat"][c["E"]]), Y=f["Y"])
    _check(c, fwd, b, ref)


@pytest.mark.gpu
@pytest.mark.parametrize("impl", [pytest.param(2, id="tcgen05_2cta"), pytest.param(3, id="tcgen05")])
@pytest.mark.parametrize("name", MULTI)
def test_cuda_two_matrix_mode_pinned_by_reference_outputs(name, impl):
    """The CUDA up / down / dH epilogue chain against the reference's outputs, identity down-projection."""
    import gpu_util as G
    c = CASES[name]
    d = dict(inputs(c))
    d["Wdown"] = _identity_down(c)
    ref = _load(name)
    layer = G.Layer(d, c["T"], c["D"], c["E"], c["K"], c["D"], gemm_impl=impl)
    Y = layer.forward(d["Y0"] if c["beta"] else None, c["beta"])
    stat, counts, aux = layer.moe.stats()
    g = layer.backward(d["dY"], c["aux"], c["zcoef"])
    assert layer.moe.device_status() == 0
    fwd = dict(idx=layer.moe.read("idx"), counts=counts.astype(np.int32), logits=layer.moe.read("logits"),
               probs=layer.moe.read("probs"), aux=aux, z=float(stat[c["E"]]), Y=Y)
    _check(c, fwd, g, ref)


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(CASES))
def test_cuda_matches_reference_outputs(name):
    import gpu_util as G
    c = CASES[name]
    d = inputs(c)
    ref = _load(name)
    layer = G.Layer(d, c["T"], c["D"], c["E"], c["K"], 0)
    Y = layer.forward(d["Y0"] if c["beta"] else None, c["beta"])
    stat, counts, aux = layer.moe.stats()
    g = layer.backward(d["dY"], c["aux"], c["zcoef"])
    assert layer.moe.device_status() == 0
    fwd = dict(idx=layer.moe.read("idx"), counts=counts.astype(np.int32), logits=layer.moe.read("logits"),
               probs=layer.moe.read("probs"), aux=aux, z=float(stat[c["E"]]), Y=Y)
    _check(c, fwd, g, ref)
