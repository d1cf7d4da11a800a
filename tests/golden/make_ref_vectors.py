"""Generates tests/golden/ref_moe_*.npz, ref_ln_*.npz and ref_adam_*.npz: outputs of the REFERENCE's own moe_forward /
moe_backward, layernorm_fwd / layernorm_bwd and multi-tensor optimizer kernels (recompiled for sm_100a,
oracle/_ref/libtmt_ref.so) on seeded inputs.

Run on a machine with a GPU:  python tests/golden/make_ref_vectors.py [out_dir]
Inputs are regenerated from the seed by the tests (tmt_moe_b200/synth.py), so only outputs are stored.
Cases stay inside what the reference computes correctly (experts <= 4, see oracle/ref_driver.cu)."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path[:0] = [ROOT, os.path.join(ROOT, "test-model-thing-cuda_b200")]

from tmt_moe_b200 import synth  # noqa: E402
from oracle import ref  # noqa: E402

# name: tokens, dim, experts, topk, seed, beta, aux, zcoef, weight std, router std
CASES = {
    "e4k2": dict(T=300, D=128, E=4, K=2, seed=101, beta=0.0, aux=0.1, zcoef=0.001, w_std=0.1, router_std=0.2),
    "e4k2_residual": dict(T=257, D=192, E=4, K=2, seed=102, beta=1.0, aux=0.01, zcoef=0.001, w_std=0.08, router_std=0.1),
    "e3k2": dict(T=130, D=64, E=3, K=2, seed=103, beta=0.0, aux=0.0, zcoef=0.0, w_std=0.15, router_std=0.3),
    "e2k1": dict(T=200, D=128, E=2, K=1, seed=104, beta=0.0, aux=0.1, zcoef=0.01, w_std=0.1, router_std=0.2),
    "dense": dict(T=96, D=128, E=1, K=1, seed=105, beta=1.0, aux=0.0, zcoef=0.0, w_std=0.1, router_std=0.1),
}


def inputs(c):
    return synth.make(c["T"], c["D"], 0, c["E"], c["K"], False, seed=c["seed"], w_std=c["w_std"],
                      router_std=c["router_std"], dy_std=0.1, need_res=True)


# LayerNorm (tmt-cuda/src/norm.cu): rows, dim, seed
LN_CASES = {"ln_300x256": dict(N=300, D=256, seed=201), "ln_65x2048": dict(N=65, D=2048, seed=202),
            "ln_129x64": dict(N=129, D=64, seed=203)}
# multi-tensor AdamW (tmt-cuda/src/adam.cu): tensor sizes, flags (bit 0 in the norm, bit 1 updated), clip, step
ADAM_CASES = {"adam_clip": dict(sizes=[4096 * 3 + 17, 1000, 8192], flags=[3, 3, 3], clip=0.5, step=3, seed=301),
              "adam_noclip_frozen": dict(sizes=[5000, 4097, 64], flags=[3, 1, 3], clip=0.0, step=1, seed=302)}
ADAM_HYP = dict(lr=3e-3, b1=0.9, b2=0.999, eps=1e-8, wd=0.01)


def ln_inputs(c):
    rng = np.random.default_rng(c["seed"])
    O = synth.O
    X = O.f32_to_bf16(rng.standard_normal((c["N"], c["D"]), dtype=np.float32) * 1.5 + 0.3)
    dY = O.f32_to_bf16(rng.standard_normal((c["N"], c["D"]), dtype=np.float32) * 0.1)
    gamma = (1 + 0.1 * rng.standard_normal(c["D"])).astype(np.float32)
    beta = (0.1 * rng.standard_normal(c["D"])).astype(np.float32)
    return X, dY, gamma, beta


def adam_inputs(c):
    rng = np.random.default_rng(c["seed"])
    n = sum(c["sizes"])
    master = (rng.standard_normal(n) * 0.02).astype(np.float32)
    m = (rng.standard_normal(n) * 1e-3).astype(np.float32)
    v = ((rng.standard_normal(n) * 1e-3) ** 2).astype(np.float32)
    grad = (rng.standard_normal(n) * 1e-2).astype(np.float32)
    return master, m, v, grad


def main(out_dir):
    os.makedirs(out_dir, exist_ok=True)
    for name, c in LN_CASES.items():
        r = ref.ln_run(*ln_inputs(c))
        np.savez_compressed(os.path.join(out_dir, "ref_%s.npz" % name), **r)
        print(name, "mean[0]", r["mean"][0], "rstd[0]", r["rstd"][0], flush=True)
    for name, c in ADAM_CASES.items():
        master, m, v, grad = adam_inputs(c)
        r = ref.adam_run(c["sizes"], c["flags"], master, m, v, grad, c["clip"], step=c["step"], **ADAM_HYP)
        np.savez_compressed(os.path.join(out_dir, "ref_%s.npz" % name), **{k: np.asarray(x) for k, x in r.items()})
        print(name, "sumsq", r["sumsq"], flush=True)
    for name, c in CASES.items():
        d = inputs(c)
        r = ref.run(d["X"], d["Wr"], d["Wup"], c["K"], Y0=d["Y0"] if c["beta"] else None, beta=c["beta"],
                    dY=d["dY"], aux=c["aux"], zcoef=c["zcoef"])
        np.savez_compressed(os.path.join(out_dir, "ref_moe_%s.npz" % name),
                            Y=r["Y"], logits=r["logits"], probs=r["probs"], idx=r["idx"], counts=r["counts"],
                            dX=r["dX"], dWr=r["dWr"], dWexp=r["dWexp"].astype(np.float32),
                            aux=np.float32(r["aux"]), zloss=np.float32(r["zloss"]))
        print(name, "counts", r["counts"], "aux", r["aux"], "z", r["zloss"], flush=True)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__)))
