"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configs
(LayerNorm-like N(0,1) activations, N(0,0.02^2) weights, N(0,1e-2^2) upstream gradient), and
the comparison helpers the parity tests share. bf16 tensors are uint16 bit patterns."""
import numpy as np


class O:
    """bf16 bit patterns <-> fp32 (round to nearest even), in numpy."""

    @staticmethod
    def f32_to_bf16(x):
        u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
        return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)

    @staticmethod
    def bf16_to_f32(b):
        return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)

CONFIGS = {
    # name: tokens, dim, hidden, experts, topk, router fp32
    "c1": dict(T=2048, D=512, H=1024, E=4, K=2, router_f32=True),
    "c2": dict(T=16384, D=1024, H=4096, E=8, K=2, router_f32=False),
    "c3": dict(T=64, D=1024, H=2048, E=16, K=2, router_f32=False),
    "c4": dict(T=65536, D=1024, H=4096, E=16, K=2, router_f32=False),
    "c5": dict(T=131072, D=2048, H=2048, E=64, K=4, router_f32=True),
}


def zipf_bias(E, scale, s=1.2):
    """Per-expert logit bias of Zipf(s) magnitude: scale * rank^-s (config 4's skew)."""
    return (scale * np.arange(1, E + 1, dtype=np.float64) ** (-s)).astype(np.float32)


def make(T, D, H, E, K, router_f32=False, seed=0, w_std=0.02, router_std=0.02, x_std=1.0, dy_std=1e-2,
         need_dy=True, need_res=False):
    rng = np.random.default_rng(seed)
    X = O.f32_to_bf16(rng.standard_normal((T, D), dtype=np.float32) * x_std)
    Wr = (rng.standard_normal((E, D), dtype=np.float32) * router_std).astype(np.float32)
    if not router_f32:
        Wr = O.f32_to_bf16(Wr)
    if H > 0:
        Wup = O.f32_to_bf16(rng.standard_normal((E, H, D), dtype=np.float32) * w_std)
        Wdown = O.f32_to_bf16(rng.standard_normal((E, D, H), dtype=np.float32) * w_std)
    else:
        Wup = O.f32_to_bf16(rng.standard_normal((E, D, D), dtype=np.float32) * w_std)
        Wdown = None
    out = dict(X=X, Wr=Wr, Wup=Wup, Wdown=Wdown, K=K, H=H)
    if need_dy:
        out["dY"] = O.f32_to_bf16(rng.standard_normal((T, D), dtype=np.float32) * dy_std)
    if need_res:
        out["Y0"] = O.f32_to_bf16(rng.standard_normal((T, D), dtype=np.float32))
    return out


def rel_l2(a, ref):
    a = np.asarray(a, np.float64).ravel()
    ref = np.asarray(ref, np.float64).ravel()
    return float(np.linalg.norm(a - ref) / max(np.linalg.norm(ref), 1e-30))


def max_rel(a, ref):
    a = np.asarray(a, np.float64).ravel()
    ref = np.asarray(ref, np.float64).ravel()
    return float(np.abs(a - ref).max() / max(np.abs(ref).max(), 1e-30))
