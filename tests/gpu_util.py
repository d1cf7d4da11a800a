"""Glue between torch device memory and the C ABI wrapper for the GPU parity tests."""
import numpy as np
import torch

import tmt_moe_b200 as M
from oracle import oracle as O


def dev(a):
    """numpy -> cuda tensor, uint16 bit patterns travel as int16."""
    if a is None:
        return None
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16).copy()).cuda()
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host_u16(t):
    return t.cpu().numpy().view(np.uint16)


class Layer:
    """One MoE layer on the GPU with its weights, driven through the C ABI."""

    def __init__(self, data, T, D, E, K, H, router_f32=False, training=True, gemm_impl=M.GEMM_TCGEN05, bias=None):
        self.moe = M.MoE(T, D, E, K, hidden=H, router_dtype=M.F32 if router_f32 else M.BF16,
                         training=training, gemm_impl=gemm_impl)
        self.T, self.D, self.E, self.K, self.H = T, D, E, K, H
        self.X = dev(data["X"])
        self.Wr = dev(data["Wr"])
        self.Wup_all = dev(data["Wup"])
        self.Wdown_all = dev(data["Wdown"])
        self.Wup = [self.Wup_all[e] for e in range(E)]
        self.Wdown = None if H == 0 else [self.Wdown_all[e] for e in range(E)]
        if bias is not None:
            self.moe.set_router_bias(bias)

    def forward(self, Y0=None, beta=0.0, tokens=None):
        T = self.T if tokens is None else tokens
        self.Y = torch.zeros((T, self.D), dtype=torch.int16, device="cuda") if Y0 is None else dev(Y0)
        self.moe.forward(self.X, self.Wr, self.Wup, self.Wdown, self.Y, beta, tokens)
        torch.cuda.synchronize()
        return host_u16(self.Y)

    def backward(self, dY, aux=0.0, zcoef=0.0):
        E, D, H = self.E, self.D, self.H
        self.dY = dev(dY)
        self.dX = torch.full((dY.shape[0], D), 0x7fc0, dtype=torch.int16, device="cuda")   # NaN canary
        self.dWr = torch.full((E, D), float("nan"), device="cuda")
        self.dWup_all = torch.full(tuple(self.Wup_all.shape), float("nan"), device="cuda")
        self.dWdown_all = None if H == 0 else torch.full(tuple(self.Wdown_all.shape), float("nan"), device="cuda")
        dWup = [self.dWup_all[e] for e in range(E)]
        dWdown = None if H == 0 else [self.dWdown_all[e] for e in range(E)]
        self.moe.backward(self.dY, self.Wr, self.Wup, self.Wdown, self.dWr, dWup, dWdown, self.dX, aux, zcoef)
        torch.cuda.synchronize()
        return dict(dX=host_u16(self.dX), dWr=self.dWr.cpu().numpy(), dWup=self.dWup_all.cpu().numpy(),
                    dWdown=None if H == 0 else self.dWdown_all.cpu().numpy())


def check_routing(layer, ref, tokens=None):
    """Bit-exact: logits, indices, counts, padded offsets, slots."""
    m = layer.moe
    np.testing.assert_array_equal(m.read("logits", tokens).view(np.uint32), ref["logits"].view(np.uint32))
    np.testing.assert_array_equal(m.read("idx", tokens), ref["idx"])
    np.testing.assert_array_equal(m.read("counts"), ref["counts"])
    np.testing.assert_array_equal(m.read("poff"), ref["poff"])
    np.testing.assert_array_equal(m.read("slot_of", tokens), ref["slot_of"])
    np.testing.assert_allclose(m.read("probs", tokens), ref["probs"], rtol=2e-5, atol=1e-7)
    np.testing.assert_allclose(m.read("w", tokens), ref["w"], rtol=2e-5, atol=1e-7)
    np.testing.assert_allclose(m.read("lse", tokens), ref["lse"], rtol=2e-6, atol=2e-6)
