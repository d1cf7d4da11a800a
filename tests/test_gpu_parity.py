"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle.

Tolerances (bf16 path, fp32 accumulation): routing (logits, indices, counts, offsets, slots)
bit-exact; outputs relative L2 <= 1e-2 and max-abs <= 2e-2 * max|ref|; gradients relative L2
<= 3e-2 per tensor (the reference's own bar, architecture_test.cu:254); aux / z relative 1e-4."""
import ctypes

import numpy as np
import pytest
import torch

from tmt_moe_b200 import synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu

M = None
G = None


@pytest.fixture(scope="module", autouse=True)
def _mods():
    global M, G
    import tmt_moe_b200
    import gpu_util
    M, G = tmt_moe_b200, gpu_util
    assert torch.cuda.is_available()
    O.build()


# gemm_impl values of include/tmt_moe.h: 0 = AUTO (the CTA-pair kernel), 1 = SIMT cross-check, 2 = CTA pairs, 3 = one CTA per tile
IMPLS = [pytest.param(3, id="tcgen05"), pytest.param(1, id="simt"), pytest.param(2, id="tcgen05_2cta")]
PAD = {0: 256, 1: 128, 2: 256, 3: 128}
OUT_L2, OUT_MAX, GRAD_L2 = 1e-2, 2e-2, 3e-2


def _fwd_bwd(cfg, impl, seed=0, bias=None, beta=0.0, aux=0.1, zcoef=0.001, backward=True, w_std=0.02,
             router_std=0.02):
    T, D, H, E, K = cfg["T"], cfg["D"], cfg["H"], cfg["E"], cfg["K"]
    rf = cfg.get("router_f32", False)
    data = synth.make(T, D, H, E, K, rf, seed=seed, need_res=beta != 0.0, w_std=w_std, router_std=router_std)
    ref = O.forward(data["X"], data["Wr"], data["Wup"], data["Wdown"], K, Y=data.get("Y0"), beta=beta, bias=bias,
                    pad=PAD[impl])
    layer = G.Layer(data, T, D, E, K, H, rf, training=backward, gemm_impl=impl, bias=bias)
    Y = layer.forward(data.get("Y0"), beta)
    assert layer.moe.device_status() == 0
    G.check_routing(layer, ref)
    yr, yg = O.bf16_to_f32(ref["Y"]), O.bf16_to_f32(Y)
    assert np.isfinite(yg).all()
    assert synth.rel_l2(yg, yr) <= OUT_L2 and synth.max_rel(yg, yr) <= OUT_MAX
    stat, counts, aux_v = layer.moe.stats()
    np.testing.assert_array_equal(counts, ref["counts"])
    if E > 1:
        np.testing.assert_allclose(stat, ref["stat"], rtol=1e-4, atol=1e-6)
        assert abs(aux_v - ref["aux"]) <= 1e-4 * abs(ref["aux"])
    else:
        assert aux_v == 0 and (stat == 0).all()
    if not backward:
        return layer, ref, None
    rb = O.backward(ref, data["dY"], aux, zcoef)
    g = layer.backward(data["dY"], aux, zcoef)
    assert layer.moe.device_status() == 0
    assert synth.rel_l2(O.bf16_to_f32(g["dX"]), O.bf16_to_f32(rb["dX"])) <= GRAD_L2
    assert synth.rel_l2(g["dWup"], rb["dWup"]) <= GRAD_L2
    if H > 0:
        assert synth.rel_l2(g["dWdown"], rb["dWdown"]) <= GRAD_L2
    if E > 1:
        assert synth.rel_l2(g["dWr"], rb["dWr"]) <= GRAD_L2
        np.testing.assert_allclose(layer.moe.read("s_j"), rb["s_j"], rtol=3e-2, atol=3e-2 * np.abs(rb["s_j"]).max())
    else:
        assert (g["dWr"] == 0).all()
    for e in range(E):      # an expert without tokens gets an exactly zero gradient
        if ref["counts"][e] == 0:
            assert (g["dWup"][e] == 0).all()
    return layer, ref, g


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("hidden", [0, 256])
def test_small_ragged(impl, hidden):
    """Token count that is no multiple of the 64-token router block or of 8; 5 experts."""
    _fwd_bwd(dict(T=301, D=128, H=hidden, E=5, K=2), impl, seed=1, w_std=0.1, router_std=0.2)


@pytest.mark.parametrize("impl", IMPLS)
def test_fp32_router_and_residual(impl):
    _fwd_bwd(dict(T=512, D=256, H=320, E=8, K=2, router_f32=True), impl, seed=2, beta=1.0, w_std=0.08, router_std=0.1)


@pytest.mark.parametrize("impl", IMPLS)
def test_empty_expert_and_heavy_skew(impl):
    """Expert 2 never selected (empty group -> zero gradient); expert 0 takes a slot of every token."""
    bias = np.array([30, 0, -1e4, 0, 0, 0], np.float32)
    layer, ref, _ = _fwd_bwd(dict(T=700, D=128, H=128, E=6, K=2), impl, seed=3, bias=bias, w_std=0.1)
    assert ref["counts"][2] == 0 and ref["counts"][0] == 700


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("hidden", [0, 128])
def test_dense_shortcut(impl, hidden):
    """experts = 1 (the reference's default config): no router gradient, no statistics."""
    _fwd_bwd(dict(T=200, D=128, H=hidden, E=1, K=1), impl, seed=4, w_std=0.1)


def test_tie_break_lowest_index():
    """Identical router rows give exactly equal logits: the lowest indices must win."""
    T, D, E, K = 130, 64, 6, 3
    data = synth.make(T, D, 64, E, K, seed=5)
    data["Wr"][:] = data["Wr"][0]
    layer = G.Layer(data, T, D, E, K, 64)
    layer.forward()
    idx = layer.moe.read("idx")
    assert (idx == np.array([0, 1, 2])).all()
    ref = O.forward(data["X"], data["Wr"], data["Wup"], data["Wdown"], K)
    G.check_routing(layer, ref)


@pytest.mark.parametrize("impl", [pytest.param(3, id="tcgen05"), pytest.param(2, id="tcgen05_2cta")])
def test_topk4_64_experts(impl):
    """Config-5 routing shape at reduced size: 64 experts, top-4, fp32 router."""
    _fwd_bwd(dict(T=1024, D=256, H=256, E=64, K=4, router_f32=True), impl, seed=6, w_std=0.08, router_std=0.1)


@pytest.mark.parametrize("impl", [pytest.param(2, id="tcgen05_2cta"), pytest.param(3, id="tcgen05")])
def test_config5_true_widths(impl):
    """The benchmarked configuration at its own widths (dim 2048, hidden 2048, 64 experts, top-4, fp32 router) on a
    token sample the oracle finishes in seconds: routing bit-exact, forward and every gradient in tolerance."""
    _fwd_bwd(dict(synth.CONFIGS["c5"], T=2048), impl, seed=17)


def test_single_token_and_partial_batch():
    cfg = dict(T=257, D=128, H=192, E=4, K=2)
    data = synth.make(257, 128, 192, 4, 2, seed=7, w_std=0.1)
    layer = G.Layer(data, 257, 128, 4, 2, 192, training=False)
    for tokens in (1, 63, 257):
        sub = dict(data, X=data["X"][:tokens])
        ref = O.forward(sub["X"], data["Wr"], data["Wup"], data["Wdown"], 2)
        Y = layer.forward(tokens=tokens)
        G.check_routing(layer, ref, tokens)
        assert synth.rel_l2(O.bf16_to_f32(Y), O.bf16_to_f32(ref["Y"])) <= OUT_L2


def test_tcgen05_matches_simt_buffers():
    """Every grouped GEMM of the two tensor-core kernels against the independent SIMT kernel on the
    same inputs: pre-activation, SiLU output, gated output, dP, dXg and the weight gradients. Group
    padding differs between the kernels, so grouped buffers are compared on their real rows."""
    cfg = dict(T=900, D=192, H=448, E=4, K=2)
    data = synth.make(cfg["T"], cfg["D"], cfg["H"], cfg["E"], cfg["K"], seed=8, w_std=0.08)
    got = {}
    for impl in (3, 1, 2):
        layer = G.Layer(data, cfg["T"], cfg["D"], cfg["E"], cfg["K"], cfg["H"], gemm_impl=impl)
        layer.forward()
        g = layer.backward(data["dY"], 0.1, 0.001)
        poff, counts = layer.moe.read("poff"), layer.moe.read("counts")
        real = np.concatenate([np.arange(poff[e], poff[e] + counts[e]) for e in range(cfg["E"])])
        bufs = {n: O.bf16_to_f32(layer.moe.read(n)[real]) for n in ("Xg", "P", "Hact", "Yg", "dYg", "dP", "dXg")}
        bufs.update(dWup=g["dWup"], dWdown=g["dWdown"], dWr=g["dWr"], dX=O.bf16_to_f32(g["dX"]),
                    sw=layer.moe.read("sw_part")[real].sum(1))
        got[impl] = bufs
        assert layer.moe.device_status() == 0
    for impl in (3, 2):
        for n in got[impl]:
            assert np.isfinite(got[impl][n]).all(), (impl, n)
            assert synth.rel_l2(got[impl][n], got[1][n]) <= 4e-3, (impl, n)


def test_config1_full():
    """Config 1 at full size, forward only, fp32 router: identical top-2 indices, outputs within
    1e-2 relative error."""
    _fwd_bwd(synth.CONFIGS["c1"], 0, seed=11, backward=False)


@pytest.mark.parametrize("impl", [pytest.param(3, id="tcgen05"), pytest.param(2, id="tcgen05_2cta")])
@pytest.mark.parametrize("name,tokens", [("c2", 1024), ("c4", 2048)])
def test_training_configs_reduced_tokens(name, tokens, impl):
    """Configs 2 and 4 with their true widths and expert counts on a token subsample the CPU
    oracle finishes in seconds; config 4 with its Zipf(1.2) logit bias."""
    cfg = dict(synth.CONFIGS[name], T=tokens)
    bias = synth.zipf_bias(cfg["E"], 2.0) if name == "c4" else None
    _fwd_bwd(cfg, impl, seed=12, bias=bias)


def test_full_size_routing_and_invariants():
    """Config 2 at full size: routing bit-exact against the oracle's router; the layer is
    position-wise, so permuting the tokens permutes the outputs (exactly) and the weight
    gradients agree up to summation order."""
    cfg = synth.CONFIGS["c2"]
    T, D, H, E, K = cfg["T"], cfg["D"], cfg["H"], cfg["E"], cfg["K"]
    data = synth.make(T, D, H, E, K, seed=13)
    r = O.router(data["X"], data["Wr"], K)
    counts, off, poff, slot_of = O.layout(r["idx"], E)
    layer = G.Layer(data, T, D, E, K, H)
    Y = layer.forward()
    ref = dict(r, counts=counts, poff=poff, slot_of=slot_of)
    G.check_routing(layer, ref)
    g = layer.backward(data["dY"], 0.1, 0.001)
    perm = np.random.default_rng(0).permutation(T)
    data2 = dict(data, X=data["X"][perm], dY=data["dY"][perm])
    layer2 = G.Layer(data2, T, D, E, K, H)
    Y2 = layer2.forward()
    np.testing.assert_array_equal(Y2, Y[perm])
    g2 = layer2.backward(data2["dY"], 0.1, 0.001)
    assert synth.rel_l2(O.bf16_to_f32(g2["dX"]), O.bf16_to_f32(g["dX"][perm])) <= 2e-3
    assert synth.rel_l2(g2["dWup"], g["dWup"]) <= 1e-3
    assert synth.rel_l2(g2["dWdown"], g["dWdown"]) <= 1e-3
    assert synth.rel_l2(g2["dWr"], g["dWr"]) <= 1e-3
    assert layer.moe.device_status() == 0 and layer2.moe.device_status() == 0


def test_deterministic_reruns():
    cfg = dict(T=2048, D=256, H=512, E=8, K=2)
    data = synth.make(cfg["T"], cfg["D"], cfg["H"], cfg["E"], cfg["K"], seed=14)
    layer = G.Layer(data, cfg["T"], cfg["D"], cfg["E"], cfg["K"], cfg["H"])
    a = layer.forward().copy()
    ga = layer.backward(data["dY"], 0.1, 0.001)
    b = layer.forward().copy()
    gb = layer.backward(data["dY"], 0.1, 0.001)
    np.testing.assert_array_equal(a, b)
    for k in ("dX", "dWr", "dWup", "dWdown"):
        np.testing.assert_array_equal(ga[k], gb[k])


def test_host_step_equals_device_path():
    """The host-buffer entry point (pinned host X / dY in, Y / dX / statistics out, copies overlapped with
    compute on a second stream) returns exactly what the device-pointer calls return."""
    cfg = dict(T=3000, D=256, H=384, E=8, K=2)
    data = synth.make(cfg["T"], cfg["D"], cfg["H"], cfg["E"], cfg["K"], seed=15, need_res=True)
    layer = G.Layer(data, cfg["T"], cfg["D"], cfg["E"], cfg["K"], cfg["H"])
    Y = layer.forward(data["Y0"], 1.0).copy()
    g = layer.backward(data["dY"], 0.1, 0.001)
    stat, _, _ = layer.moe.stats()
    host = M.MoE(cfg["T"], cfg["D"], cfg["E"], cfg["K"], hidden=cfg["H"], host_io=True, gemm_impl=M.GEMM_TCGEN05)
    pin = lambda a: torch.from_numpy(a.view(np.int16).copy()).pin_memory()
    hX, hdY, hY = pin(data["X"]), pin(data["dY"]), pin(data["Y0"])
    hdX = torch.zeros_like(hX).pin_memory()
    hstat = torch.zeros(cfg["E"] + 1).pin_memory()
    E = cfg["E"]
    dWr = torch.zeros_like(layer.dWr)
    dWup_all, dWdown_all = torch.zeros_like(layer.dWup_all), torch.zeros_like(layer.dWdown_all)
    for _ in range(2):
        hY.copy_(pin(data["Y0"]))
        host.step_host(hX, hdY, layer.Wr, layer.Wup, layer.Wdown, dWr, [dWup_all[e] for e in range(E)],
                       [dWdown_all[e] for e in range(E)], hY, hdX, hstat, 1.0, 0.1, 0.001)
    assert host.device_status() == 0
    np.testing.assert_array_equal(hY.numpy().view(np.uint16), Y)
    np.testing.assert_array_equal(hdX.numpy().view(np.uint16), g["dX"])
    np.testing.assert_array_equal(dWr.cpu().numpy(), g["dWr"])
    np.testing.assert_array_equal(dWup_all.cpu().numpy(), g["dWup"])
    np.testing.assert_array_equal(hstat.numpy(), stat)


def test_host_steps_queued_back_to_back():
    """Host steps queued without waiting (uploads of step n+1 under the GEMMs of step n, downloads under the
    following compute): two different batches give exactly the results of the device-pointer calls."""
    cfg = dict(T=3000, D=256, H=384, E=8, K=2)
    E = cfg["E"]
    batches = [synth.make(cfg["T"], cfg["D"], cfg["H"], E, cfg["K"], seed=15), synth.make(cfg["T"], cfg["D"], cfg["H"], E, cfg["K"], seed=16)]
    layer = G.Layer(batches[0], cfg["T"], cfg["D"], E, cfg["K"], cfg["H"])
    want = []
    for b in batches:
        layer.X = G.dev(b["X"])
        Y = layer.forward(None, 0.0).copy()
        g = layer.backward(b["dY"], 0.1, 0.001)
        want.append((Y, g["dX"].copy()))
    host = M.MoE(cfg["T"], cfg["D"], E, cfg["K"], hidden=cfg["H"], host_io=True, gemm_impl=M.GEMM_TCGEN05)
    pin = lambda a: torch.from_numpy(a.view(np.int16).copy()).pin_memory()
    bufs = [(pin(b["X"]), pin(b["dY"]), torch.zeros(cfg["T"], cfg["D"], dtype=torch.int16).pin_memory(),
             torch.zeros(cfg["T"], cfg["D"], dtype=torch.int16).pin_memory(), torch.zeros(E + 1).pin_memory()) for b in batches]
    dWr = torch.zeros_like(layer.dWr)
    dWup_all, dWdown_all = torch.zeros_like(layer.dWup_all), torch.zeros_like(layer.dWdown_all)
    for rep in range(3):                      # six steps in flight order A B A B A B, one wait at the end
        for hX, hdY, hY, hdX, hstat in bufs:
            host.step_host(hX, hdY, layer.Wr, layer.Wup, layer.Wdown, dWr, [dWup_all[e] for e in range(E)],
                           [dWdown_all[e] for e in range(E)], hY, hdX, hstat, 0.0, 0.1, 0.001, wait=False)
    host.host_wait()
    assert host.device_status() == 0
    for (hX, hdY, hY, hdX, hstat), (Y, dX) in zip(bufs, want):
        np.testing.assert_array_equal(hY.numpy().view(np.uint16), Y)
        np.testing.assert_array_equal(hdX.numpy().view(np.uint16), dX)


def test_bounded_wait_runs_out_and_context_survives():
    """Failure detection without a fault: a wait on a barrier nothing signals runs out after its limit,
    the kernel records the time-out status and returns, and the same handle keeps working."""
    cfg = dict(T=256, D=128, H=128, E=4, K=2)
    data = synth.make(cfg["T"], cfg["D"], cfg["H"], cfg["E"], cfg["K"], seed=16)
    layer = G.Layer(data, cfg["T"], cfg["D"], cfg["E"], cfg["K"], cfg["H"], training=False)
    a = layer.forward().copy()
    rc = layer.moe.lib.tmt_moe_selftest_bounded_wait(layer.moe.h, ctypes.c_longlong(2_000_000))   # about 1 ms
    assert rc == 2, (rc, layer.moe.lib.tmt_moe_last_error())
    assert layer.moe.device_status() == 0          # the handle's own status word is untouched
    np.testing.assert_array_equal(layer.forward(), a)


def test_argument_errors():
    with pytest.raises(M.MoeError):
        M.MoE(64, 100, 4, 2)           # dim not a multiple of 64
    with pytest.raises(M.MoeError):
        M.MoE(64, 128, 4, 5)           # topk > experts (the reference rejects it too, config.h:51-52)
    m = M.MoE(64, 128, 4, 2, hidden=128, training=False)
    x = torch.zeros(64, 128, dtype=torch.int16, device="cuda")
    with pytest.raises(M.MoeError):
        m.forward(x, x, [x] * 4, [x] * 4, x, tokens=65)
    with pytest.raises(M.MoeError):
        m.backward(x, x, [x] * 4, [x] * 4, x, [x] * 4, [x] * 4, x)


def test_router_usage_telemetry_accumulates_on_the_device():
    """tmt_moe_usage: counts of every forward pass since the last reset, and the reference's summary of them
    (train_main.cu:232-248: share 1.0 = uniform, dead below 0.01)."""
    T, D, H, E, K = 700, 128, 128, 8, 2
    bias = np.array([0, 0, 0, 0, 0, 0, 0, -60.0], np.float32)          # expert 7 never wins
    total = np.zeros(E, np.int64)
    layer = None
    for seed in (31, 32, 33):
        data = synth.make(T, D, H, E, K, seed=seed)
        if layer is None:
            layer = G.Layer(data, T, D, E, K, H, bias=bias)
            assert layer.moe.usage(reset=True)["passes"] == 0
        layer.X = G.dev(data["X"])
        layer.forward()
        total += layer.moe.read("counts").astype(np.int64)
    u = layer.moe.usage()
    np.testing.assert_array_equal(u["totals"], total)
    assert u["passes"] == 3 and total[7] == 0 and u["dead"] == 1
    share = total / total.sum() * E
    assert abs(u["min_share"] - share.min()) < 1e-12 and abs(u["max_share"] - share.max()) < 1e-12
    assert layer.moe.usage(reset=True)["passes"] == 3
    assert layer.moe.usage()["passes"] == 0 and layer.moe.usage()["totals"].sum() == 0


@pytest.mark.parametrize("cfg,bias_on", [
    (dict(T=37, D=256, H=256, E=4, K=2), False),
    (dict(T=200, D=512, H=128, E=16, K=2, router_f32=True), True),
    (dict(T=130, D=256, H=128, E=40, K=4), False),
], ids=["37_tokens_4_experts", "200_tokens_fp32_router_bias", "130_tokens_40_experts_top4"])
def test_per_token_router_and_tiled_router_agree_bitwise(cfg, bias_on, monkeypatch):
    """Short batches compute the logits with one block per token, long ones with 64-token tiles; the chains, their
    order and the butterfly are the same, so every routing product is identical bit for bit (and equals the oracle's)."""
    T, D, H, E, K = cfg["T"], cfg["D"], cfg["H"], cfg["E"], cfg["K"]
    rf = cfg.get("router_f32", False)
    data = synth.make(T, D, H, E, K, rf, seed=11)
    bias = (np.random.default_rng(3).standard_normal(E) * 0.5).astype(np.float32) if bias_on else None
    ref = O.forward(data["X"], data["Wr"], data["Wup"], data["Wdown"], K, bias=bias, pad=128)
    got = {}
    for flag in ("0", "1"):
        monkeypatch.setenv("TMT_MOE_ROUTER_SMALL", flag)
        layer = G.Layer(data, T, D, E, K, H, rf, training=False, gemm_impl=3, bias=bias)
        layer.forward(None, 0.0)
        assert layer.moe.device_status() == 0
        G.check_routing(layer, ref)
        got[flag] = {n: layer.moe.read(n) for n in ("logits", "probs", "lse", "idx", "w", "slot_of", "counts", "poff")}
        got[flag]["stat"] = layer.moe.stats()[0]
    for n, v in got["0"].items():
        np.testing.assert_array_equal(v, got["1"][n], err_msg=n)
