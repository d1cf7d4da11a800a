"""ctypes front end of oracle/_ref/libtmt_ref.so: the reference's own moe_forward /
moe_backward (tmt-cuda/src/moe.cu) recompiled for sm_100a by oracle/Makefile. Test
infrastructure only; needs a GPU. Reference mode only (one DxD matrix per expert), E <= 4."""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libtmt_ref.so")


def available():
    return os.path.exists(LIB_PATH)


def run(X, Wr, Wexp, K, Y0=None, beta=0.0, dY=None, aux=0.0, zcoef=0.0):
    """X (N,D) u16, Wr (E,D) u16, Wexp (E,D,D) u16. Returns a dict of host arrays."""
    lib = ctypes.CDLL(LIB_PATH)
    N, D = X.shape
    E = Wr.shape[0]
    p = lambda a: None if a is None else a.ctypes.data_as(ctypes.c_void_p)
    Y = np.zeros((N, D), np.uint16) if Y0 is None else np.array(Y0, np.uint16, copy=True)
    out = dict(Y=Y, logits=np.zeros((N, E), np.float32), probs=np.zeros((N, E), np.float32),
               idx=np.zeros((N, K), np.int32), counts=np.zeros(E, np.int32), dX=np.zeros((N, D), np.uint16),
               dWr=np.zeros((E, D), np.float32), dWexp=np.zeros((E, D, D), np.float32))
    a, z = ctypes.c_float(0), ctypes.c_float(0)
    X, Wr, Wexp = (np.ascontiguousarray(v, np.uint16) for v in (X, Wr, Wexp))
    dYc = None if dY is None else np.ascontiguousarray(dY, np.uint16)
    rc = lib.ref_moe_run(N, E, K, D, p(X), p(Wr), p(Wexp), p(Y), ctypes.c_float(beta), p(dYc), ctypes.c_float(aux),
                         ctypes.c_float(zcoef), p(out["logits"]), p(out["probs"]), p(out["idx"]), p(out["counts"]),
                         p(out["dX"]), p(out["dWr"]), p(out["dWexp"]), ctypes.byref(a), ctypes.byref(z))
    if rc != 0:
        raise RuntimeError("ref_moe_run refused the shape (rc=%d)" % rc)
    out["aux"], out["zloss"] = a.value, z.value
    return out
