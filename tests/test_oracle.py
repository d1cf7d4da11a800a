"""CPU tests: the oracle against the reference's own known-answer tests and against an
independent float64 autograd statement of the same math."""
import numpy as np
import pytest
import torch


def _rand_bf16(o, rng, shape, std):
    return o.f32_to_bf16(rng.standard_normal(shape).astype(np.float32) * std)


def test_router_closed_form(oracle):
    """The reference's test_router (tmt-cuda/src/architecture_test.cu:62-87): N=5, E=4, K=2,
    logits 2*sin(0.43 i); router backward with s_j = 0 and (aux, z) = (0.7, 0), (0, 0.3) must
    equal the central finite difference of z*lse^2/N + aux*E/N*sum p_e*cnt_e/(N*K)."""
    N, E, K = 5, 4, 2
    logits = (np.sin(np.arange(N * E, dtype=np.float32) * np.float32(0.43)) * 2).astype(np.float32).reshape(N, E)
    probs, idx, w, lse = oracle.topk_from_logits(logits, K)
    counts, _, _, _ = oracle.layout(idx, E)
    assert counts.sum() == N * K
    np.testing.assert_allclose(w.sum(1), 1.0, rtol=1e-6)
    # top-2 by value, lowest index first on ties
    for r in range(N):
        order = sorted(range(E), key=lambda e: (-logits[r, e], e))[:K]
        assert list(idx[r]) == order
    sj = np.zeros((N, K), np.float32)
    for aux, z in ((0.7, 0.0), (0.0, 0.3)):
        got = oracle.router_bwd(probs, idx, sj, logits, counts, aux, z)

        def objective(zz):
            loss = 0.0
            for r in range(N):
                s = np.exp(zz[r]).sum()
                l = np.log(s)
                loss += z * l * l / N
                loss += (aux * E / N * np.exp(zz[r]) / s * counts / (N * K)).sum()
            return loss
        zz = logits.astype(np.float64)
        for r in range(N):
            for e in range(E):
                old = zz[r, e]
                zz[r, e] = old + 1e-4
                hi = objective(zz)
                zz[r, e] = old - 1e-4
                lo = objective(zz)
                zz[r, e] = old
                ref = (hi - lo) / 2e-4
                assert abs(got[r, e] - ref) <= 2e-6 + 2e-4 * abs(ref)


def test_router_dot_order_is_the_stated_one(oracle):
    """Independent numpy restatement of the router's fp32 order: 8 interleaved FMA chains
    (element d in chain (d/8)%8), tree ((c0+c1)+(c2+c3))+((c4+c5)+(c6+c7))."""
    rng = np.random.default_rng(3)
    T, D, E = 7, 192, 5
    X = _rand_bf16(oracle, rng, (T, D), 1.0)
    for wr in (_rand_bf16(oracle, rng, (E, D), 0.02), (rng.standard_normal((E, D)) * 0.02).astype(np.float32)):
        r = oracle.router(X, wr, 2)
        xf = oracle.bf16_to_f32(X)
        wf = oracle.bf16_to_f32(wr) if wr.dtype == np.uint16 else wr
        for t in range(T):
            for e in range(E):
                c = [np.float32(0)] * 8
                for d in range(D):
                    s = (d >> 3) & 7
                    # fp32 FMA = round(double product + double addend): exact for fp32 inputs
                    c[s] = np.float32(np.float64(xf[t, d]) * np.float64(wf[e, d]) + np.float64(c[s]))
                v = np.float32(np.float32(np.float32(c[0] + c[1]) + np.float32(c[2] + c[3])) +
                               np.float32(np.float32(c[4] + c[5]) + np.float32(c[6] + c[7])))
                assert v == r["logits"][t, e]


def test_tie_break_lowest_index(oracle):
    logits = np.array([[1.0, 3.0, 3.0, 3.0], [2.0, 2.0, 2.0, 2.0], [0.0, -1.0, 0.0, 5.0]], np.float32)
    _, idx, w, _ = oracle.topk_from_logits(logits, 2)
    assert idx.tolist() == [[1, 2], [0, 1], [3, 0]]
    np.testing.assert_allclose(w[1], [0.5, 0.5])


def test_layout_stable_and_padded(oracle):
    rng = np.random.default_rng(0)
    T, E, K = 1000, 6, 2
    idx = np.stack([rng.permutation(E)[:K] for _ in range(T)]).astype(np.int32)
    idx[:, 0] = np.where(idx[:, 0] == 5, 0, idx[:, 0])
    idx[:, 1] = np.where(idx[:, 1] == 5, (idx[:, 0] + 1) % 5, idx[:, 1])  # expert 5 stays empty
    counts, off, poff, slot_of = oracle.layout(idx, E)
    assert counts[5] == 0 and counts.sum() == T * K
    assert (poff % 128 == 0).all() and poff[E] == sum((c + 127) // 128 * 128 for c in counts)
    assert off[E] == T * K
    for e in range(E):
        s = slot_of[idx == e]
        assert (np.diff(s) == 1).all() if len(s) > 1 else True     # token order kept, dense
        if len(s):
            assert s[0] == poff[e] and s[-1] == poff[e] + counts[e] - 1


@pytest.mark.parametrize("hidden", [0, 96])
@pytest.mark.parametrize("router_f32", [False, True])
def test_backward_matches_float64_autograd(oracle, hidden, router_f32):
    from torch_ref import moe_loss
    rng = np.random.default_rng(11 + hidden)
    T, D, E, K = 96, 64, 4, 2
    X = _rand_bf16(oracle, rng, (T, D), 1.0)
    Wr = (rng.standard_normal((E, D)) * 0.3).astype(np.float32)
    Wr = Wr if router_f32 else oracle.f32_to_bf16(Wr)
    if hidden:
        Wup = _rand_bf16(oracle, rng, (E, hidden, D), 0.15)
        Wdown = _rand_bf16(oracle, rng, (E, D, hidden), 0.15)
    else:
        Wup = _rand_bf16(oracle, rng, (E, D, D), 0.15)
        Wdown = None
    dY = _rand_bf16(oracle, rng, (T, D), 0.1)
    aux, z = 0.1, 0.05
    f = oracle.forward(X, Wr, Wup, Wdown, K)
    b = oracle.backward(f, dY, aux, z)
    td = torch.float64
    tX = torch.tensor(oracle.bf16_to_f32(X), dtype=td, requires_grad=True)
    tWr = torch.tensor(Wr if router_f32 else oracle.bf16_to_f32(Wr), dtype=td, requires_grad=True)
    tWu = torch.tensor(oracle.bf16_to_f32(Wup), dtype=td, requires_grad=True)
    tWd = None if Wdown is None else torch.tensor(oracle.bf16_to_f32(Wdown), dtype=td, requires_grad=True)
    loss, Y = moe_loss(tX, tWr, tWu, tWd, torch.tensor(f["idx"], dtype=torch.long),
                       torch.tensor(oracle.bf16_to_f32(dY), dtype=td), hidden, aux, z,
                       torch.tensor(f["counts"]))
    loss.backward()

    def rel(a, ref):
        ref = ref.detach().numpy()
        return np.linalg.norm(a.astype(np.float64) - ref) / max(np.linalg.norm(ref), 1e-30)
    assert rel(oracle.bf16_to_f32(f["Y"]), Y) < 1e-2
    assert rel(oracle.bf16_to_f32(b["dX"]), tX.grad) < 2e-2
    assert rel(b["dWr"], tWr.grad) < 2e-2
    assert rel(b["dWup"], tWu.grad) < 2e-2
    if hidden:
        assert rel(b["dWdown"], tWd.grad) < 2e-2
    # aux scalar: E * sum_e mean_p * frac
    p = torch.softmax(tX.detach() @ tWr.detach().t(), 1)
    aux_ref = E * ((p.mean(0)) * (torch.tensor(f["counts"], dtype=td) / (T * K))).sum().item()
    assert abs(f["aux"] - aux_ref) < 1e-4 * abs(aux_ref)
    z_ref = (torch.logsumexp(tX.detach() @ tWr.detach().t(), 1) ** 2).mean().item()
    assert abs(f["stat"][E] - z_ref) < 1e-4 * abs(z_ref) + 1e-7


def test_identical_experts_equal_dense(oracle):
    """The reference's test_moe_backward property (architecture_test.cu:234-264): two experts
    with identical weights, top-2 (weights sum to 1) compute exactly the dense (experts=1)
    layer; the summed expert gradients and the input gradient match within 3 % (L2)."""
    rng = np.random.default_rng(5)
    T, D = 70, 32
    X = _rand_bf16(oracle, rng, (T, D), 1.0)
    W = _rand_bf16(oracle, rng, (1, D, D), 0.2)
    dY = _rand_bf16(oracle, rng, (T, D), 0.1)
    Wr1 = _rand_bf16(oracle, rng, (1, D), 0.1)
    Wr2 = _rand_bf16(oracle, rng, (2, D), 0.1)
    dense = oracle.forward(X, Wr1, W, None, 1)
    moe = oracle.forward(X, Wr2, np.concatenate([W, W]), None, 2)
    yd, ym = oracle.bf16_to_f32(dense["Y"]), oracle.bf16_to_f32(moe["Y"])
    assert np.linalg.norm(yd - ym) <= 1e-2 * np.linalg.norm(yd)
    assert dense["aux"] == 0 and dense["stat"][1] == 0
    bd = oracle.backward(dense, dY)
    bm = oracle.backward(moe, dY)   # aux = z = 0 as in the reference test
    g = bm["dWup"][0] + bm["dWup"][1]
    assert np.linalg.norm(g - bd["dWup"][0]) <= 1e-6 + 0.03 * np.linalg.norm(bd["dWup"][0])
    xd, xm = oracle.bf16_to_f32(bd["dX"]), oracle.bf16_to_f32(bm["dX"])
    assert np.linalg.norm(xd - xm) <= 1e-6 + 0.03 * np.linalg.norm(xd)
    assert (bd["dWr"] == 0).all()


def test_empty_expert_and_beta(oracle):
    rng = np.random.default_rng(9)
    T, D, H, E, K = 40, 32, 48, 5, 2
    X = _rand_bf16(oracle, rng, (T, D), 1.0)
    Wr = _rand_bf16(oracle, rng, (E, D), 0.05)
    bias = np.array([0, 0, -1e4, 0, 0], np.float32)       # expert 2 never selected
    Wup = _rand_bf16(oracle, rng, (E, H, D), 0.1)
    Wdown = _rand_bf16(oracle, rng, (E, D, H), 0.1)
    Y0 = _rand_bf16(oracle, rng, (T, D), 1.0)
    f0 = oracle.forward(X, Wr, Wup, Wdown, K, bias=bias)
    f1 = oracle.forward(X, Wr, Wup, Wdown, K, Y=Y0, beta=1.0, bias=bias)
    assert f0["counts"][2] == 0
    d = oracle.bf16_to_f32(f1["Y"]) - (oracle.bf16_to_f32(Y0) + oracle.bf16_to_f32(f0["Y"]))
    assert np.abs(d).max() <= 2 ** -7 * np.abs(oracle.bf16_to_f32(f1["Y"])).max()
    b = oracle.backward(f0, _rand_bf16(oracle, rng, (T, D), 0.1), 0.1, 0.001)
    assert (b["dWup"][2] == 0).all() and (b["dWdown"][2] == 0).all()


def test_nvfp4_roundtrip(oracle):
    rng = np.random.default_rng(2)
    W = _rand_bf16(oracle, rng, (24, 64), 0.02)
    packed, scales, ts = oracle.nvfp4_quantize(W)
    Wq = oracle.bf16_to_f32(oracle.nvfp4_dequantize(packed, scales, 1.0)) * ts
    Wf = oracle.bf16_to_f32(W)
    amax = np.abs(Wf).max()
    assert np.isclose(ts, amax / (6 * 448), rtol=1e-6)
    # per block: error at most half an e2m1 step (1.0 at the top of the range) times the block scale
    blk = np.abs(Wf).reshape(24, 4, 16).max(2, keepdims=True)
    err = np.abs(Wq - Wf).reshape(24, 4, 16)
    assert (err <= blk / 6 * 1.0 * 1.07 + 1e-12).all()
    # quantising the dequantised tensor is a fixed point
    W2 = oracle.f32_to_bf16(oracle.bf16_to_f32(oracle.nvfp4_dequantize(packed, scales, ts)))
    p2, s2, ts2 = oracle.nvfp4_quantize(W2)
    Wq2 = oracle.bf16_to_f32(oracle.nvfp4_dequantize(p2, s2, 1.0)) * ts2
    assert np.abs(Wq2 - oracle.bf16_to_f32(W2)).max() <= np.abs(Wq - Wf).max() + 1e-9
    # zero tensor
    p0, s0, t0 = oracle.nvfp4_quantize(np.zeros((2, 32), np.uint16))
    assert t0 == 1.0 and (p0 == 0).all() and (s0 == 0).all()
    # e2m1 grid values survive exactly when the block scale is a power of two
    grid = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0.5, -1, -1.5, -2, -3, -4, -6, 0], np.float32)
    pg, sg, tg = oracle.nvfp4_quantize(oracle.f32_to_bf16(np.tile(grid, (1, 1))))
    back = oracle.bf16_to_f32(oracle.nvfp4_dequantize(pg, sg, 1.0)) * tg
    np.testing.assert_allclose(back[0], grid, rtol=2 ** -7)
