"""Multi-tensor AdamW on the GPU (include/tmt_adamw.h) against the CPU oracle: master weights, moments and the bf16
working copies are bit-identical, the squared gradient norm agrees to double rounding, clipping, frozen tensors,
odd sizes and a non-finite gradient behave as tmt-cuda/src/adam.cu:57-105 and model.cu:716-729 do."""
import numpy as np
import pytest
import torch

import tmt_moe_b200 as M
from oracle import oracle as O

pytestmark = pytest.mark.gpu

HYP = dict(lr=3e-4, b1=0.9, b2=0.999, eps=1e-8, wd=0.01)


def _tensors(sizes, seed):
    rng = np.random.default_rng(seed)
    host = []
    for n in sizes:
        host.append(dict(w=rng.normal(0, 0.02, n).astype(np.float32), m=rng.normal(0, 1e-3, n).astype(np.float32),
                         v=rng.normal(0, 1e-3, n).astype(np.float32) ** 2, g=rng.normal(0, 1e-2, n).astype(np.float32)))
    return host


def _dev(host, key, offset=0):
    out = []
    for t in host:
        buf = torch.zeros(t[key].size + offset, dtype=torch.float32, device="cuda")
        buf[offset:] = torch.from_numpy(t[key]).cuda()
        out.append(buf[offset:])
    return out


@pytest.mark.parametrize("clip", [0.0, 0.05])
@pytest.mark.parametrize("offset", [0, 1])      # 1: unaligned views, the scalar path
def test_step_is_bit_identical_to_the_oracle(clip, offset):
    sizes = [8192 * 3, 100003, 1, 4096, 8192 + 4]
    host = _tensors(sizes, 11)
    w, m, v, g = (_dev(host, k, offset) for k in "wmvg")
    work = [torch.zeros(n + 2 * offset, dtype=torch.int16, device="cuda")[2 * offset:] for n in sizes]
    work[2] = None
    flags = [3, 3, 3, 1, 3]                      # tensor 3: in the norm, frozen
    opt = M.AdamW(sizes)
    for step in (1, 2):
        ss = opt.step(w, m, v, g, work, flags, clip=clip, step=step, zero_grads=False, want_norm=True, **HYP)
        want_ss = O.sumsq([t["g"] for t in host])
        assert abs(ss - want_ss) <= 1e-10 * want_ss     # different (fixed) summation orders, both in double
        scale = O.clip_scale(ss, clip)
        if clip > 0:
            assert scale < 1.0
        for i, t in enumerate(host):
            if flags[i] & 2:
                t["w"], t["m"], t["v"], wk = O.adamw(t["w"], t["m"], t["v"], t["g"], scale, HYP["lr"], HYP["b1"], HYP["b2"],
                                                     HYP["eps"], HYP["wd"], step)
                if work[i] is not None:
                    np.testing.assert_array_equal(work[i].cpu().numpy().view(np.uint16), wk)
            np.testing.assert_array_equal(w[i].cpu().numpy().view(np.uint32), t["w"].view(np.uint32))
            np.testing.assert_array_equal(m[i].cpu().numpy().view(np.uint32), t["m"].view(np.uint32))
            np.testing.assert_array_equal(v[i].cpu().numpy().view(np.uint32), t["v"].view(np.uint32))
    opt.close()


def test_gradients_are_cleared_and_nonfinite_norm_refuses_the_step():
    sizes = [5000, 8192]
    host = _tensors(sizes, 5)
    w, m, v, g = (_dev(host, k) for k in "wmvg")
    work = [torch.zeros(n, dtype=torch.int16, device="cuda") for n in sizes]
    opt = M.AdamW(sizes)
    opt.step(w, m, v, g, work, None, step=1, zero_grads=True, **HYP)
    torch.cuda.synchronize()
    assert all(float(x.abs().max()) == 0.0 for x in g)
    before = [x.clone() for x in w]
    g[1][17] = float("inf")
    with pytest.raises(M.MoeError, match="non-finite"):
        opt.step(w, m, v, g, work, None, step=2, zero_grads=True, want_norm=True, **HYP)
    for a, b in zip(w, before):
        assert torch.equal(a, b)                 # nothing was updated (adam.cu:81-82)
    assert float(g[1][17]) == float("inf")       # and nothing was cleared
    opt.close()
