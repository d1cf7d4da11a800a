"""Generates tests/golden/ref_moe_*.npz: outputs of the REFERENCE's own moe_forward /
moe_backward (recompiled for sm_100a, oracle/_ref/libtmt_ref.so) on seeded inputs.

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


def main(out_dir):
    os.makedirs(out_dir, exist_ok=True)
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
