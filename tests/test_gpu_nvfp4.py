"""NVFP4 expert weights: the CUDA quantiser must reproduce the CPU statement byte for byte, and the
NVFP4 forward (config 3's shape: 64 streams, 16 experts, top-2) must match the oracle run on the
dequantised weights (output gate: relative L2 <= 1e-2, as for bf16). The error against the
unquantised weights is printed for information."""
import numpy as np
import pytest
import torch

import synth
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


@pytest.mark.parametrize("impl", [pytest.param(0, id="tcgen05"), pytest.param(2, id="tcgen05_2cta")])
def test_forward_nvfp4_decode_shape(impl):
    import gpu_util as G
    import tmt_moe_b200 as M
    T, D, H, E, K = 64, 1024, 2048, 16, 2
    data = synth.make(T, D, H, E, K, seed=31, need_dy=False)
    up_q, down_q, up_dq, down_dq, us, ds, keep = [], [], [], [], [], [], []
    for e in range(E):
        for W, qs, dqs, sc in ((data["Wup"][e], up_q, up_dq, us), (data["Wdown"][e], down_q, down_dq, ds)):
            p, s, ts = _quantize_gpu(M, G, W)
            keep += [p, s]
            qs.append((p, s, ts, W.shape[0], W.shape[1]))
            dqs.append(O.nvfp4_dequantize(p.cpu().numpy(), s.cpu().numpy(), 1.0))
            sc.append(ts)
    pad = 256 if impl == 2 else 128
    ref = O.forward(data["X"], data["Wr"], np.stack(up_dq), np.stack(down_dq), K, up_scale=np.array(us, np.float32),
                    down_scale=np.array(ds, np.float32), pad=pad)
    moe = M.MoE(T, D, E, K, hidden=H, training=False, gemm_impl=impl)
    X, Wr = G.dev(data["X"]), G.dev(data["Wr"])
    Y = torch.zeros((T, D), dtype=torch.int16, device="cuda")
    for _ in range(2):                                   # second call reuses the expanded weights
        moe.forward_nvfp4(X, Wr, up_q, down_q, Y)
        torch.cuda.synchronize()
    assert moe.device_status() == 0
    np.testing.assert_array_equal(moe.read("idx"), ref["idx"])
    got = O.bf16_to_f32(G.host_u16(Y))
    assert synth.rel_l2(got, O.bf16_to_f32(ref["Y"])) <= 1e-2
    full = O.forward(data["X"], data["Wr"], data["Wup"], data["Wdown"], K, pad=pad)
    print("NVFP4 vs unquantised weights: relative L2 = %.3f" % synth.rel_l2(got, O.bf16_to_f32(full["Y"])))
