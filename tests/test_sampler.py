"""Batched multi-stream sampler (include/tmt_sampler.h). Without a GPU: the oracle's restatement of Generator::sample
(tmt-cuda/src/generate.h:47-58) on known answers. On a GPU: the session's replayed decode steps equal direct
tmt_moe_forward_nvfp4 calls bit for bit on every ring slot, and the batched sampling kernel picks the oracle's bytes
(a draw closer than 1e-9 of the probability mass to the boundary between two bytes may fall either way: the device's
and the host's double exp can differ in the last bit)."""
import numpy as np
import pytest

from tmt_moe_b200 import synth
from oracle import oracle as O


def test_oracle_sample_known_answers(oracle):
    lg = np.full((3, 256), -30.0, np.float32)
    lg[0, 17] = 5.0; lg[0, 200] = 5.0            # two equal maxima: argmax keeps the first (std::max_element)
    lg[1, 255] = 9.0
    lg[2, 3] = 1.0
    bits = O.f32_to_bf16(lg)
    nxt, _ = oracle.sample(bits, 0.0, 7, 0)
    np.testing.assert_array_equal(nxt, [17, 255, 3])
    # temp > 0 with all other bytes at exp(-35 / 0.5) ~ 1e-31 of the mass: stream 0 draws 17 or 200, the others their peak
    for pos in range(50):
        nxt, _ = oracle.sample(bits, 0.5, 7, pos)
        assert nxt[0] in (17, 200) and nxt[1] == 255 and nxt[2] == 3
    # the draw depends on (seed, stream, position) only
    a, _ = oracle.sample(bits, 0.5, 7, 11)
    b, _ = oracle.sample(bits[:1], 0.5, 7, 11)
    assert a[0] == b[0]
    # uniform draws: in [0, 1), mean 1/2, both halves of stream 0's two-way choice occur
    us = np.array([oracle.sampler_uniform(9, s, p) for s in range(64) for p in range(64)])
    assert us.min() >= 0.0 and us.max() < 1.0 and abs(us.mean() - 0.5) < 0.02
    picks = {int(oracle.sample(bits[:1], 0.5, 7, p)[0][0]) for p in range(64)}
    assert picks == {17, 200}


def test_oracle_sample_follows_the_distribution(oracle):
    """Empirical frequencies over many positions against softmax(logits / temp)."""
    rng = np.random.default_rng(3)
    lg = np.full((1, 256), -40.0, np.float32)
    lg[0, :8] = rng.standard_normal(8).astype(np.float32)
    bits = O.f32_to_bf16(lg)
    temp = 0.8
    l = O.bf16_to_f32(bits)[0].astype(np.float64)
    p = np.exp((l - l.max()) / temp); p /= p.sum()
    counts = np.zeros(256)
    n = 4000
    for pos in range(n):
        counts[oracle.sample(bits, temp, 123, pos)[0][0]] += 1
    assert counts[8:].sum() == 0
    assert np.abs(counts[:8] / n - p[:8]).max() < 0.03


@pytest.mark.gpu
def test_session_steps_equal_direct_calls_on_every_slot():
    import torch
    import gpu_util as G
    import tmt_moe_b200 as M
    from test_gpu_nvfp4 import _setup
    S, D, H, E, K, ring = 64, 512, 512, 8, 2, 3
    data, up_q, down_q, up_dq, down_dq, us, ds, keep = _setup(M, G, S, D, H, E, K, 41)
    Wr = G.dev(data["Wr"])
    rng = np.random.default_rng(8)
    batches = [O.f32_to_bf16(rng.standard_normal((S, D), dtype=np.float32)) for _ in range(2 * ring)]
    # direct calls
    moe = M.MoE(S, D, E, K, hidden=H, training=False)
    want = []
    for xb in batches:
        Y = torch.zeros((S, D), dtype=torch.int16, device="cuda")
        moe.forward_nvfp4(G.dev(xb), Wr, up_q, down_q, Y)
        torch.cuda.synchronize()
        want.append(G.host_u16(Y).copy())
    # the session: two rounds over the ring, host rows in and out, one wait per round
    ses = M.Sampler(S, D, H, E, K, ring=ring, seed=5)
    ses.set_weights(Wr, up_q, down_q)
    pin = lambda a: torch.from_numpy(a.view(np.int16).copy()).pin_memory()
    hx = [pin(b) for b in batches]
    hy = [torch.zeros((S, D), dtype=torch.int16).pin_memory() for _ in batches]
    for rnd in range(2):
        for slot in range(ring):
            i = rnd * ring + slot
            ses.upload(slot, hx[i])
            ses.step(slot, 0.0)
            ses.download(slot, hy[i])
        ses.sync()
    assert ses.steps == 2 * ring and ses.graphs == ring          # the second round replayed the recorded steps
    for i, w in enumerate(want):
        np.testing.assert_array_equal(hy[i].numpy().view(np.uint16), w, err_msg="batch %d" % i)
    # beta: Y = beta * Y + moe(X) re-records the slot once
    ses.step(0, 1.0)
    ses.download(0, hy[0])
    ses.sync()
    assert ses.graphs == ring + 1
    acc = O.bf16_to_f32(hy[0].numpy().view(np.uint16))
    # slot 0 holds batch `ring`'s input and output from the second round: beta = 1 doubles it (up to one bf16 rounding)
    ref = 2.0 * O.bf16_to_f32(want[ring])
    assert synth.rel_l2(acc, ref) <= 4e-3
    # with the LayerNorm in front of the block taken into the step: the slot's X rows are the rows before it
    gamma = torch.from_numpy((1 + 0.1 * rng.standard_normal(D)).astype(np.float32)).cuda()
    beta_ln = torch.from_numpy((0.1 * rng.standard_normal(D)).astype(np.float32)).cuda()
    ses.set_layernorm(gamma, beta_ln)
    Xn = torch.zeros((S, D), dtype=torch.int16, device="cuda")
    mean, rstd = torch.zeros(S, device="cuda"), torch.zeros(S, device="cuda")
    M.ln_forward(G.dev(batches[1]), gamma, beta_ln, Xn, mean, rstd)
    Yd = torch.zeros((S, D), dtype=torch.int16, device="cuda")
    moe.forward_nvfp4(Xn, Wr, up_q, down_q, Yd)
    torch.cuda.synchronize()
    for _ in range(2):
        ses.upload(1, hx[1])
        ses.step(1, 0.0)
        ses.download(1, hy[1])
    ses.sync()
    np.testing.assert_array_equal(hy[1].numpy().view(np.uint16), G.host_u16(Yd))
    ses.close()
    with pytest.raises(M.MoeError):
        M.Sampler(S, D, 0, E, K)                                  # reference-mode experts have no NVFP4 path


@pytest.mark.gpu
@pytest.mark.parametrize("temp", [0.0, 0.7, 1.3])
def test_sampling_kernel_picks_the_oracles_bytes(temp):
    import torch
    import gpu_util as G
    import tmt_moe_b200 as M
    S = 64
    ses = M.Sampler(S, 256, 256, 4, 2, ring=1, seed=77)
    rng = np.random.default_rng(21)
    nxt = torch.full((S,), -1, dtype=torch.int32, device="cuda")
    close = 0
    for pos in (0, 1, 5, 1000, 2 ** 40):
        lg = O.f32_to_bf16(rng.standard_normal((S, 256), dtype=np.float32) * 4)
        if pos == 1:
            lg[:, 40] = lg[:, 9]                                  # ties
        ses.sample(G.dev(lg), temp, pos, nxt)
        ses.sync()
        got = nxt.cpu().numpy()
        want, margin = O.sample(lg, temp, 77, pos)
        bad = got != want
        assert (margin[bad] < 1e-9).all(), (pos, np.nonzero(bad)[0], margin[bad])
        close += int(bad.sum())
        assert got.min() >= 0 and got.max() <= 255
    assert close <= 1
    ses.close()
