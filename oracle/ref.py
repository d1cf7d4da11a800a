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


def time_moe(X, Wr, Wexp, K, dY, aux=0.01, zcoef=0.001, warmup=15, iters=60):
    """Steady-state milliseconds of the reference's moe_forward and moe_forward + moe_backward (CUDA events, the
    method of tmt-cuda/src/profile.cu:34-63) on the given inputs. Returns (ms_fwd, ms_fwd_bwd)."""
    lib = ctypes.CDLL(LIB_PATH)
    N, D = X.shape
    E = Wr.shape[0]
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    X, Wr, Wexp, dY = (np.ascontiguousarray(v, np.uint16) for v in (X, Wr, Wexp, dY))
    f, fb = ctypes.c_float(0), ctypes.c_float(0)
    rc = lib.ref_moe_time(N, E, K, D, p(X), p(Wr), p(Wexp), p(dY), ctypes.c_float(aux), ctypes.c_float(zcoef),
                          int(warmup), int(iters), ctypes.byref(f), ctypes.byref(fb))
    if rc != 0:
        raise RuntimeError("ref_moe_time refused the shape (rc=%d)" % rc)
    return f.value, fb.value


def ln_run(X, dY, gamma, beta):
    """The reference's layernorm_fwd + layernorm_bwd (tmt-cuda/src/norm.cu:92-110). X, dY (N,D) u16."""
    lib = ctypes.CDLL(LIB_PATH)
    N, D = X.shape
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    X, dY = np.ascontiguousarray(X, np.uint16), np.ascontiguousarray(dY, np.uint16)
    gamma, beta = np.ascontiguousarray(gamma, np.float32), np.ascontiguousarray(beta, np.float32)
    out = dict(Y=np.zeros((N, D), np.uint16), mean=np.zeros(N, np.float32), rstd=np.zeros(N, np.float32),
               dX=np.zeros((N, D), np.uint16), dGamma=np.zeros(D, np.float32), dBeta=np.zeros(D, np.float32))
    rc = lib.ref_ln_run(N, D, p(X), p(dY), p(gamma), p(beta), p(out["Y"]), p(out["mean"]), p(out["rstd"]), p(out["dX"]),
                        p(out["dGamma"]), p(out["dBeta"]))
    if rc != 0:
        raise RuntimeError("ref_ln_run failed (rc=%d)" % rc)
    return out


def adam_run(sizes, flags, master, m, v, grad, clip, lr, b1, b2, eps, wd, step):
    """One step of the reference's multi-tensor optimizer (tmt-cuda/src/adam.cu:44-96) over tensors laid back to back
    in the flat fp32 arrays. Returns dict(master, m, v, grad, work (bf16 bits), sumsq)."""
    lib = ctypes.CDLL(LIB_PATH)
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    master, m, v, grad = (np.array(a, dtype=np.float32, copy=True).ravel() for a in (master, m, v, grad))
    work = np.zeros(master.size, np.uint16)
    sz = (ctypes.c_longlong * len(sizes))(*[int(s) for s in sizes])
    fl = (ctypes.c_ubyte * len(sizes))(*[int(f) for f in flags])
    ss = ctypes.c_double(0)
    rc = lib.ref_adam_run(len(sizes), sz, fl, p(master), p(m), p(v), p(grad), p(work), ctypes.c_float(clip), ctypes.c_float(lr),
                          ctypes.c_float(b1), ctypes.c_float(b2), ctypes.c_float(eps), ctypes.c_float(wd), int(step),
                          ctypes.byref(ss))
    if rc != 0:
        raise RuntimeError("ref_adam_run failed (rc=%d)" % rc)
    return dict(master=master, m=m, v=v, grad=grad, work=work, sumsq=ss.value)
