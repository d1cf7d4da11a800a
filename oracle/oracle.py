"""ctypes front end of the CPU oracle (oracle/moe_oracle.cpp). Test infrastructure only.

Nothing in the product package imports this module: it is the checker used by the
test-suite, by the smoke check and by the benchmark's CPU baseline. bf16 tensors
travel as numpy uint16 arrays holding the raw bit patterns.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libmoe_oracle.so")
_lib = None


def build(force=False):
    """Compile the oracle with the recipe in oracle/Makefile."""
    if force or not os.path.exists(_LIB_PATH) or \
            os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "moe_oracle.cpp")):
        subprocess.check_call(["make", "-C", _HERE, "-B", "all"], stdout=subprocess.DEVNULL)


class _Cfg(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in
                ("tokens", "dim", "hidden", "experts", "topk", "router_f32", "threads", "pad")]


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.oracle_stats.restype = ctypes.c_float
        _lib.oracle_layout.restype = ctypes.c_int
        _lib.oracle_abi_version.restype = ctypes.c_int
        _lib.oracle_sumsq.restype = ctypes.c_double
        _lib.oracle_clip_scale.restype = ctypes.c_float
        _lib.oracle_sampler_uniform.restype = ctypes.c_double
        assert _lib.oracle_abi_version() == 7, "stale oracle library: run make -C oracle -B"
    return _lib


def host_threads():
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def f32_to_bf16(x):
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    return ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)


def bf16_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _cfg(T, D, H, E, K, router_f32, threads, pad=128):
    return _Cfg(T, D, H, E, K, int(router_f32), threads or host_threads(), pad)


def topk_from_logits(logits, K):
    """moe.cu:72-94 on given fp32 logits. Returns probs, idx, w, lse."""
    T, E = logits.shape
    logits = np.ascontiguousarray(logits, np.float32)
    probs = np.empty((T, E), np.float32)
    idx = np.empty((T, K), np.int32)
    w = np.empty((T, K), np.float32)
    lse = np.empty(T, np.float32)
    lib().oracle_topk_from_logits(T, E, K, _p(logits), _p(probs), _p(idx), _p(w), _p(lse))
    return probs, idx, w, lse


def router(X, Wr, K, bias=None, threads=None):
    T, D = X.shape
    E = Wr.shape[0]
    f32 = Wr.dtype == np.float32
    cfg = _cfg(T, D, 0, E, K, f32, threads)
    logits = np.empty((T, E), np.float32)
    probs = np.empty((T, E), np.float32)
    idx = np.empty((T, K), np.int32)
    w = np.empty((T, K), np.float32)
    lse = np.empty(T, np.float32)
    X = np.ascontiguousarray(X)
    Wr = np.ascontiguousarray(Wr)
    bias = None if bias is None else np.ascontiguousarray(bias, np.float32)
    lib().oracle_router(ctypes.byref(cfg), _p(X), _p(Wr), _p(bias), _p(logits), _p(probs), _p(idx),
                        _p(w), _p(lse))
    return dict(logits=logits, probs=probs, idx=idx, w=w, lse=lse)


def layout(idx, E, pad=128):
    T, K = idx.shape
    idx = np.ascontiguousarray(idx, np.int32)
    counts = np.empty(E, np.int32)
    off = np.empty(E + 1, np.int32)
    poff = np.empty(E + 1, np.int32)
    slot_of = np.empty((T, K), np.int32)
    lib().oracle_layout(T, E, K, pad, _p(idx), _p(counts), _p(off), _p(poff), _p(slot_of))
    return counts, off, poff, slot_of


def router_bwd(probs, idx, s_j, logits, counts, aux, zcoef):
    T, E = probs.shape
    K = idx.shape[1]
    out = np.empty((T, E), np.float32)
    lib().oracle_router_bwd(T, E, K, _p(np.ascontiguousarray(probs, np.float32)),
                            _p(np.ascontiguousarray(idx, np.int32)),
                            _p(np.ascontiguousarray(s_j, np.float32)),
                            _p(np.ascontiguousarray(logits, np.float32)),
                            _p(np.ascontiguousarray(counts, np.int32)),
                            ctypes.c_float(aux), ctypes.c_float(zcoef), _p(out))
    return out


def forward(X, Wr, Wup, Wdown, K, Y=None, beta=0.0, bias=None, up_scale=None, down_scale=None,
            threads=None, pad=128):
    """Full forward. X (T,D) u16; Wr (E,D) u16 or f32; Wup (E,H,D) u16 [hidden>0] or (E,D,D)
    [hidden==0, Wdown=None]; Wdown (E,D,H). Returns a dict with Y and every saved tensor."""
    T, D = X.shape
    E = Wr.shape[0]
    H = 0 if Wdown is None else Wup.shape[1]
    cfg = _cfg(T, D, H, E, K, Wr.dtype == np.float32, threads, pad)
    cap = (T * K + pad - 1) // pad * pad + pad * E
    X = np.ascontiguousarray(X)
    Wr = np.ascontiguousarray(Wr)
    Wup = np.ascontiguousarray(Wup)
    Wdown = None if Wdown is None else np.ascontiguousarray(Wdown)
    Yio = np.zeros((T, D), np.uint16) if Y is None else np.array(Y, dtype=np.uint16, copy=True)
    r = dict(
        logits=np.empty((T, E), np.float32), probs=np.empty((T, E), np.float32),
        idx=np.empty((T, K), np.int32), w=np.empty((T, K), np.float32), lse=np.empty(T, np.float32),
        counts=np.empty(E, np.int32), off=np.empty(E + 1, np.int32), poff=np.empty(E + 1, np.int32),
        slot_of=np.empty((T, K), np.int32), Xg=np.zeros((cap, D), np.uint16),
        P=np.zeros((cap, max(H, 1)), np.uint16), Hact=np.zeros((cap, max(H, 1)), np.uint16),
        Yg=np.zeros((cap, D), np.uint16), stat=np.zeros(E + 1, np.float32))
    aux = ctypes.c_float(0)
    bias = None if bias is None else np.ascontiguousarray(bias, np.float32)
    us = None if up_scale is None else np.ascontiguousarray(up_scale, np.float32)
    ds = None if down_scale is None else np.ascontiguousarray(down_scale, np.float32)
    lib().oracle_forward(ctypes.byref(cfg), _p(X), _p(Wr), _p(bias), _p(Wup), _p(Wdown), _p(us), _p(ds),
                         _p(Yio), ctypes.c_float(beta), _p(r["logits"]), _p(r["probs"]), _p(r["idx"]),
                         _p(r["w"]), _p(r["lse"]), _p(r["counts"]), _p(r["off"]), _p(r["poff"]),
                         _p(r["slot_of"]), _p(r["Xg"]), _p(r["P"]), _p(r["Hact"]), _p(r["Yg"]),
                         _p(r["stat"]), ctypes.byref(aux))
    r["Y"] = Yio
    r["aux"] = aux.value
    r["rows"] = int(r["poff"][E])
    r["_in"] = dict(X=X, Wr=Wr, Wup=Wup, Wdown=Wdown, K=K, H=H)
    return r


def backward(fwd, dY, aux=0.0, zcoef=0.0, threads=None):
    """Backward from a forward() result. Returns dX (u16), dWr, dWup, dWdown (f32), s_j, dlogits."""
    i = fwd["_in"]
    X, Wr, Wup, Wdown, K, H = i["X"], i["Wr"], i["Wup"], i["Wdown"], i["K"], i["H"]
    T, D = X.shape
    E = Wr.shape[0]
    cfg = _cfg(T, D, H, E, K, Wr.dtype == np.float32, threads)
    dY = np.ascontiguousarray(dY, np.uint16)
    out = dict(dX=np.zeros((T, D), np.uint16), dWr=np.zeros((E, D), np.float32),
               dWup=np.zeros(Wup.shape, np.float32),
               dWdown=None if Wdown is None else np.zeros(Wdown.shape, np.float32),
               s_j=np.zeros((T, K), np.float32), dlogits=np.zeros((T, E), np.float32))
    lib().oracle_backward(ctypes.byref(cfg), _p(X), _p(dY), _p(Wr), _p(Wup), _p(Wdown),
                          _p(fwd["logits"]), _p(fwd["probs"]), _p(fwd["idx"]), _p(fwd["w"]),
                          _p(fwd["counts"]), _p(fwd["poff"]), _p(fwd["slot_of"]), _p(fwd["Xg"]),
                          _p(fwd["P"]), _p(fwd["Hact"]), _p(fwd["Yg"]), ctypes.c_float(aux),
                          ctypes.c_float(zcoef), _p(out["dX"]), _p(out["dWr"]), _p(out["dWup"]),
                          _p(out["dWdown"]), _p(out["s_j"]), _p(out["dlogits"]))
    return out


def nvfp4_quantize(W):
    """W (rows, cols) u16 bf16 -> packed (rows, cols/2) u8, scales (rows, cols/16) u8, tensor scale."""
    rows, cols = W.shape
    assert cols % 16 == 0
    W = np.ascontiguousarray(W, np.uint16)
    packed = np.empty((rows, cols // 2), np.uint8)
    scales = np.empty((rows, cols // 16), np.uint8)
    ts = ctypes.c_float(0)
    lib().oracle_nvfp4_quantize(_p(W), ctypes.c_long(rows), ctypes.c_long(cols), _p(packed), _p(scales),
                                ctypes.byref(ts))
    return packed, scales, ts.value


def nvfp4_dequantize(packed, scales, tensor_scale=1.0):
    rows, half = packed.shape
    cols = half * 2
    W = np.empty((rows, cols), np.uint16)
    lib().oracle_nvfp4_dequantize(_p(np.ascontiguousarray(packed)), _p(np.ascontiguousarray(scales)),
                                  ctypes.c_float(tensor_scale), ctypes.c_long(rows), ctypes.c_long(cols),
                                  _p(W))
    return W


def adamw(master, m, v, grad, scale, lr, b1, b2, eps, wd, step, want_work=True):
    """One AdamW step on one tensor, in place on copies. Returns (master, m, v, work bf16 bits)."""
    master, m, v = (np.array(a, dtype=np.float32, copy=True).ravel() for a in (master, m, v))
    grad = np.ascontiguousarray(grad, np.float32).ravel()
    work = np.zeros(master.size, np.uint16) if want_work else None
    lib().oracle_adamw(_p(master), _p(m), _p(v), _p(grad), _p(work), ctypes.c_long(master.size), ctypes.c_float(scale),
                       ctypes.c_float(lr), ctypes.c_float(b1), ctypes.c_float(b2), ctypes.c_float(eps), ctypes.c_float(wd),
                       ctypes.c_int(step))
    return master, m, v, work


def sumsq(grads):
    """Squared norm of a list of gradient arrays, accumulated in double in list and index order."""
    return float(sum(lib().oracle_sumsq(_p(np.ascontiguousarray(g, np.float32).ravel()), ctypes.c_long(g.size)) for g in grads))


def clip_scale(ss, clip):
    return float(lib().oracle_clip_scale(ctypes.c_double(ss), ctypes.c_float(clip)))


def ln_forward(X, gamma, beta):
    """LayerNorm forward (norm.cu:8-50). X (rows, D) bf16 bits. Returns Y (bf16 bits), mean, rstd."""
    rows, D = X.shape
    X = np.ascontiguousarray(X, np.uint16)
    Y = np.empty((rows, D), np.uint16)
    mean, rstd = np.empty(rows, np.float32), np.empty(rows, np.float32)
    lib().oracle_ln_forward(_p(X), _p(np.ascontiguousarray(gamma, np.float32)), _p(np.ascontiguousarray(beta, np.float32)), _p(Y),
                            _p(mean), _p(rstd), ctypes.c_long(rows), ctypes.c_int(D))
    return Y, mean, rstd


def ln_backward(X, dY, gamma, mean, rstd):
    """LayerNorm backward (norm.cu:54-94). Returns dX (bf16 bits), dGamma, dBeta."""
    rows, D = X.shape
    dX = np.empty((rows, D), np.uint16)
    dG, dB = np.empty(D, np.float32), np.empty(D, np.float32)
    lib().oracle_ln_backward(_p(np.ascontiguousarray(X, np.uint16)), _p(np.ascontiguousarray(dY, np.uint16)),
                             _p(np.ascontiguousarray(gamma, np.float32)), _p(np.ascontiguousarray(mean, np.float32)),
                             _p(np.ascontiguousarray(rstd, np.float32)), _p(dX), _p(dG), _p(dB), ctypes.c_long(rows), ctypes.c_int(D))
    return dX, dG, dB


def sample(logits, temp, seed, pos):
    """Generator::sample (generate.h:47-58) for a batch: logits (streams, 256) bf16 bits. Returns (next byte per stream,
    margin per stream = relative distance of the draw from the nearest boundary between two bytes)."""
    S = logits.shape[0]
    assert logits.shape[1] == 256
    nxt = np.zeros(S, np.int32)
    margin = np.zeros(S, np.float64)
    lib().oracle_sample(_p(np.ascontiguousarray(logits, np.uint16)), ctypes.c_int(S), ctypes.c_float(temp), ctypes.c_uint64(seed),
                        ctypes.c_longlong(pos), _p(nxt), _p(margin))
    return nxt, margin


def sampler_uniform(seed, stream, pos):
    return float(lib().oracle_sampler_uniform(ctypes.c_uint64(seed), ctypes.c_int(stream), ctypes.c_longlong(pos)))
