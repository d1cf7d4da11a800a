"""NVFP4 expert weights: the CUDA quantiser must reproduce the CPU statement byte for byte, and the
NVFP4 forward (config 3's shape: 64 streams, 16 experts, top-2) must match the oracle run on the
dequantised weights (output gate: relative L2 <= 1e-2, as for bf16). The error against the
unquantised weights is printed for information."""
import numpy as np
import pytest
import torch

from tmt_moe_b200 import synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _quantize_gpu(M, G, W):
    rows, cols = W.shape
    Wd = G.dev(W)
    packed = torch.empty((rows, cols // 2), dtype=torch.uint8, device="cuda")
    scales = torch.empty((rows, cols // 16), dtype=torch.uint8, device="cuda")
    ts = M.quantize_nvfp4(Wd, rows, cols, packed, scales)
    torch.cuda.synchronize()
    return packed, scales, ts


def test_quantiser_byte_exact():
    import gpu_util as G
    import tmt_moe_b200 as M
    rng = np.random.default_rng(4)
    for shape, std in (((256, 512), 0.02), ((64, 64), 1.0), ((128, 1024), 3e-4)):
        W = O.f32_to_bf16(rng.standard_normal(shape, dtype=np.float32) * std)
        W[3, :16] = 0                                   # an all-zero block
        W[5, 7] = O.f32_to_bf16(np.array([std * 40], np.float32))[0]   # an outlier sets the tensor scale
        p_ref, s_ref, ts_ref = O.nvfp4_quantize(W)
        p, s, ts = _quantize_gpu(M, G, W)
        assert ts == ts_ref
        np.testing.assert_array_equal(s.cpu().numpy(), s_ref)
        np.testing.assert_array_equal(p.cpu().numpy(), p_ref)


def _setup(M, G, T, D, H, E, K, seed, tiny_blocks=False):
    data = synth.make(T, D, H, E, K, seed=seed, need_dy=False)
    up_q, down_q, up_dq, down_dq, us, ds, keep = [], [], [], [], [], [], []
    for e in range(E):
        for W, qs, dqs, sc in ((data["Wup"][e], up_q, up_dq, us), (data["Wdown"][e], down_q, down_dq, ds)):
            if tiny_blocks:                              # blocks far below the tensor's amax: subnormal e4m3 scales, zero scales
                W = W.copy()
                f = O.bf16_to_f32(W)
                f[1::4, 16:64] *= 2.0 ** -15
                f[2::4, 64:96] *= 2.0 ** -20
                W[...] = O.f32_to_bf16(f)
            p, s, ts = _quantize_gpu(M, G, W)
            keep += [p, s]
            qs.append((p, s, ts, W.shape[0], W.shape[1]))
            dqs.append(O.nvfp4_dequantize(p.cpu().numpy(), s.cpu().numpy(), 1.0))
            sc.append(ts)
    return data, up_q, down_q, np.stack(up_dq), np.stack(down_dq), np.array(us, np.float32), np.array(ds, np.float32), keep


# Two routes: steps of a few tokens read the packed weights directly (register-operand MMA); larger steps expand the
# weights once and run the grouped tcgen05 kernels. TMT_MOE_DECODE_MAX_TOKENS = 0 forces the second route.
@pytest.mark.parametrize("route", ["small_batch", "expanded"])
@pytest.mark.parametrize("impl", [pytest.param(3, id="tcgen05"), pytest.param(2, id="tcgen05_2cta")])
def test_forward_nvfp4_decode_shape(impl, route, monkeypatch):
    import gpu_util as G
    import tmt_moe_b200 as M
    if route == "expanded":
        monkeypatch.setenv("TMT_MOE_DECODE_MAX_TOKENS", "0")
    T, D, H, E, K = 64, 1024, 2048, 16, 2
    data, up_q, down_q, up_dq, down_dq, us, ds, keep = _setup(M, G, T, D, H, E, K, 31)
    pad = 256 if impl == 2 else 128
    ref = O.forward(data["X"], data["Wr"], up_dq, down_dq, K, up_scale=us, down_scale=ds, pad=pad)
    moe = M.MoE(T, D, E, K, hidden=H, training=False, gemm_impl=impl)
    X, Wr = G.dev(data["X"]), G.dev(data["Wr"])
    Y = torch.zeros((T, D), dtype=torch.int16, device="cuda")
    for _ in range(2):                                   # second call reuses the weight tables
        moe.forward_nvfp4(X, Wr, up_q, down_q, Y)
        torch.cuda.synchronize()
    assert moe.device_status() == 0
    np.testing.assert_array_equal(moe.read("idx"), ref["idx"])
    got = O.bf16_to_f32(G.host_u16(Y))
    assert synth.rel_l2(got, O.bf16_to_f32(ref["Y"])) <= 1e-2
    full = O.forward(data["X"], data["Wr"], data["Wup"], data["Wdown"], K, pad=pad)
    print("NVFP4 vs unquantised weights: relative L2 = %.3f" % synth.rel_l2(got, O.bf16_to_f32(full["Y"])))


@pytest.mark.parametrize("case", [
    pytest.param(dict(T=37, D=256, H=512, E=4, K=2, beta=0.5, tiny=False), id="ragged_37_tokens_beta_two_passes_per_expert"),
    pytest.param(dict(T=64, D=512, H=256, E=8, K=3, beta=0.0, tiny=True), id="top3_subnormal_and_zero_block_scales"),
    pytest.param(dict(T=1, D=256, H=256, E=16, K=2, beta=0.0, tiny=False), id="one_token_most_experts_idle"),
])
@pytest.mark.parametrize("row_groups", ["1", "2"])
def test_small_batch_route_matches_expanded_route(case, row_groups, monkeypatch):
    """Both routes multiply the same bf16 values (q * block scale) with fp32 accumulation; only the order of the sums and
    one bf16 rounding of the SiLU input can differ. Against the oracle: relative L2 <= 1e-2; between routes: <= 3e-3."""
    import gpu_util as G
    import tmt_moe_b200 as M
    monkeypatch.setenv("TMT_MOE_FP4_ROW_GROUPS", row_groups)     # 64 or 128 weight rows per block
    T, D, H, E, K = case["T"], case["D"], case["H"], case["E"], case["K"]
    data, up_q, down_q, up_dq, down_dq, us, ds, keep = _setup(M, G, T, D, H, E, K, 77, tiny_blocks=case["tiny"])
    ref = O.forward(data["X"], data["Wr"], up_dq, down_dq, K, up_scale=us, down_scale=ds, pad=128)
    rng = np.random.default_rng(5)
    Y0 = O.f32_to_bf16(rng.standard_normal((T, D), dtype=np.float32) * 0.1)
    X, Wr = G.dev(data["X"]), G.dev(data["Wr"])
    outs = {}
    for route in ("small_batch", "expanded"):
        monkeypatch.setenv("TMT_MOE_DECODE_MAX_TOKENS", "256" if route == "small_batch" else "0")
        moe = M.MoE(64, D, E, K, hidden=H, training=False, gemm_impl=3)
        Y = G.dev(Y0.copy())
        moe.forward_nvfp4(X, Wr, up_q, down_q, Y, beta=case["beta"], tokens=T)
        torch.cuda.synchronize()
        assert moe.device_status() == 0
        np.testing.assert_array_equal(moe.read("idx", tokens=T), ref["idx"])
        outs[route] = O.bf16_to_f32(G.host_u16(Y))
        moe.close()
    want = O.bf16_to_f32(ref["Y"]) + case["beta"] * O.bf16_to_f32(Y0)
    assert synth.rel_l2(outs["small_batch"], want) <= 1e-2
    assert synth.rel_l2(outs["small_batch"], outs["expanded"]) <= 3e-3


def test_small_batch_route_is_deterministic_and_independent_of_batch_composition():
    """Same inputs, same bits: across calls, across handles, and for a token whichever other tokens share its step (a
    column of the expert products depends on its own token only; the token list is built in ascending order)."""
    import gpu_util as G
    import tmt_moe_b200 as M
    T, D, H, E, K = 64, 1024, 2048, 16, 2
    data, up_q, down_q, up_dq, down_dq, us, ds, keep = _setup(M, G, T, D, H, E, K, 5)
    X, Wr = G.dev(data["X"]), G.dev(data["Wr"])
    outs = []
    for handle in range(2):
        moe = M.MoE(T, D, E, K, hidden=H, training=False, gemm_impl=2)
        for _ in range(2):
            Y = torch.zeros((T, D), dtype=torch.int16, device="cuda")
            moe.forward_nvfp4(X, Wr, up_q, down_q, Y)
            torch.cuda.synchronize()
            assert moe.device_status() == 0
            outs.append(G.host_u16(Y))
        moe.close()
    for o in outs[1:]:
        np.testing.assert_array_equal(o, outs[0])
    # the first 20 tokens alone
    moe = M.MoE(T, D, E, K, hidden=H, training=False, gemm_impl=2)
    Y = torch.zeros((T, D), dtype=torch.int16, device="cuda")
    moe.forward_nvfp4(X, Wr, up_q, down_q, Y, tokens=20)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(G.host_u16(Y)[:20], outs[0][:20])


def test_requantising_in_place_is_followed_by_both_routes(monkeypatch):
    """Weights re-quantised INTO THE SAME BUFFERS with an unchanged tensor scale (rows reversed: same amax): the
    descriptors do not change, so the handle is told with tmt_moe_nvfp4_weights_changed; after that the expanded route
    (which caches a bf16 expansion) and the small-batch route (which reads the packed bytes) both compute with the new
    weights."""
    import gpu_util as G
    import tmt_moe_b200 as M
    T, D, H, E, K = 48, 256, 256, 4, 2
    data, up_q, down_q, up_dq, down_dq, us, ds, keep = _setup(M, G, T, D, H, E, K, 91)
    X, Wr = G.dev(data["X"]), G.dev(data["Wr"])
    handles = {}
    for route, limit in (("small_batch", "256"), ("expanded", "0")):
        monkeypatch.setenv("TMT_MOE_DECODE_MAX_TOKENS", limit)
        moe = M.MoE(64, D, E, K, hidden=H, training=False, gemm_impl=3)
        Y = torch.zeros((T, D), dtype=torch.int16, device="cuda")
        moe.forward_nvfp4(X, Wr, up_q, down_q, Y, tokens=T)           # builds the expansion / the table from the old weights
        torch.cuda.synchronize()
        handles[route] = moe
    # new weights into the same packed / scale buffers
    new_up, new_down = data["Wup"][:, ::-1].copy(), data["Wdown"][:, ::-1].copy()
    up_dq2, down_dq2 = [], []
    for e in range(E):
        for W, q, dq in ((new_up[e], up_q[e], up_dq2), (new_down[e], down_q[e], down_dq2)):
            ts = M.quantize_nvfp4(G.dev(W), W.shape[0], W.shape[1], q[0], q[1])
            assert ts == q[2]                                         # same tensor scale: nothing in the descriptor changed
            dq.append(O.nvfp4_dequantize(q[0].cpu().numpy(), q[1].cpu().numpy(), 1.0))
    torch.cuda.synchronize()
    ref = O.forward(data["X"], data["Wr"], np.stack(up_dq2), np.stack(down_dq2), K, up_scale=us, down_scale=ds, pad=128)
    old = O.forward(data["X"], data["Wr"], up_dq, down_dq, K, up_scale=us, down_scale=ds, pad=128)
    want, stale = O.bf16_to_f32(ref["Y"]), O.bf16_to_f32(old["Y"])
    assert synth.rel_l2(stale, want) > 0.5                            # the two weight sets give clearly different outputs
    for route, limit in (("small_batch", "256"), ("expanded", "0")):
        monkeypatch.setenv("TMT_MOE_DECODE_MAX_TOKENS", limit)
        moe = handles[route]
        moe.nvfp4_weights_changed()
        Y = torch.zeros((T, D), dtype=torch.int16, device="cuda")
        moe.forward_nvfp4(X, Wr, up_q, down_q, Y, tokens=T)
        torch.cuda.synchronize()
        assert moe.device_status() == 0
        assert synth.rel_l2(O.bf16_to_f32(G.host_u16(Y)), want) <= 1e-2, route
        moe.close()


@pytest.mark.parametrize("case", [
    pytest.param(dict(T=64, D=1024, H=2048, E=16, K=2, rf=False, limit="256"), id="sampler_step_fused_into_the_router"),
    pytest.param(dict(T=33, D=512, H=256, E=8, K=2, rf=True, limit="256"), id="ragged_fp32_router_fused"),
    pytest.param(dict(T=300, D=256, H=256, E=4, K=2, rf=False, limit="0"), id="larger_batch_stand_alone_kernel"),
])
def test_layernorm_taken_into_the_forward_gives_the_same_bits(case, monkeypatch):
    """tmt_moe_forward_nvfp4_ln on the rows before the LayerNorm = tmt_ln_forward followed by tmt_moe_forward_nvfp4, bit for
    bit: routing products and output. (The stand-alone kernel is itself bit-identical to its oracle and pinned by the
    reference's golden outputs; the fused router does the same arithmetic in the same order.)"""
    import gpu_util as G
    import tmt_moe_b200 as M
    monkeypatch.setenv("TMT_MOE_DECODE_MAX_TOKENS", case["limit"])
    T, D, H, E, K = case["T"], case["D"], case["H"], case["E"], case["K"]
    data, up_q, down_q, up_dq, down_dq, us, ds, keep = _setup(M, G, T, D, H, E, K, 55)
    rng = np.random.default_rng(56)
    raw = O.f32_to_bf16(rng.standard_normal((T, D), dtype=np.float32) * 1.7 + 0.4)
    gamma = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    beta_ln = (0.1 * rng.standard_normal(D)).astype(np.float32)
    Wr = G.dev(data["Wr"] if not case["rf"] else O.bf16_to_f32(data["Wr"]))
    dt = M.F32 if case["rf"] else M.BF16
    Xraw, Gm, Bt = G.dev(raw), G.dev(gamma), G.dev(beta_ln)
    # two steps: LayerNorm kernel, then the block
    Xn = torch.zeros_like(Xraw)
    mean, rstd = torch.zeros(T, device="cuda"), torch.zeros(T, device="cuda")
    M.ln_forward(Xraw, Gm, Bt, Xn, mean, rstd)
    a = M.MoE(T, D, E, K, hidden=H, router_dtype=dt, training=False)
    Ya = torch.zeros((T, D), dtype=torch.int16, device="cuda")
    a.forward_nvfp4(Xn, Wr, up_q, down_q, Ya)
    torch.cuda.synchronize()
    # one call
    b = M.MoE(T, D, E, K, hidden=H, router_dtype=dt, training=False)
    Yb = torch.zeros((T, D), dtype=torch.int16, device="cuda")
    l0 = b.launch_count
    for _ in range(2):
        b.forward_nvfp4_ln(Xraw, Gm, Bt, Wr, up_q, down_q, Yb)
        torch.cuda.synchronize()
    assert a.device_status() == 0 and b.device_status() == 0
    for n in ("logits", "idx", "w", "counts"):
        np.testing.assert_array_equal(a.read(n), b.read(n), err_msg=n)
    np.testing.assert_array_equal(G.host_u16(Ya), G.host_u16(Yb))
    # and against the oracle: LayerNorm oracle, then the block's oracle on the normalised rows
    xn_ref, _, _ = O.ln_forward(raw, gamma, beta_ln)
    np.testing.assert_array_equal(G.host_u16(Xn), xn_ref)
    wr_ref = data["Wr"] if not case["rf"] else O.bf16_to_f32(data["Wr"])
    ref = O.forward(xn_ref, wr_ref, up_dq, down_dq, K, up_scale=us, down_scale=ds, pad=256)
    np.testing.assert_array_equal(b.read("idx"), ref["idx"])
    assert synth.rel_l2(O.bf16_to_f32(G.host_u16(Yb)), O.bf16_to_f32(ref["Y"])) <= 1e-2
