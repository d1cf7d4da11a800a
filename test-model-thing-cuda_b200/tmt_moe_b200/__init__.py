"""Python front end of the B200 MoE block: a thin ctypes layer over the C ABI in
include/tmt_moe.h (libtmt_moe_b200.so, built in-tree by build.py).

The class mirrors the reference's operator interface for this path
(tmt-cuda/src/moe.cu:330-545): create once (moe_keep_alloc + moe_ws_alloc), then
forward / stats / backward with the same argument meaning. Tensors are anything with a
`data_ptr()` (torch CUDA tensors) or raw integer device addresses. There is no CPU or
library fallback: if the shared library is missing or a call fails, an exception is raised.
"""
import ctypes
import os

from . import build as _build

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtmt_moe_b200.so")

BF16, F32 = 0, 1
GEMM_AUTO, GEMM_SIMT, GEMM_TCGEN05_2CTA, GEMM_TCGEN05 = 0, 1, 2, 3
EP_PEER, EP_NCCL, EP_DMA = 0, 1, 2

EXPORTS = (
    "tmt_moe_create", "tmt_moe_destroy", "tmt_moe_last_error", "tmt_moe_set_router_bias",
    "tmt_moe_forward", "tmt_moe_stats", "tmt_moe_backward", "tmt_moe_step_host", "tmt_moe_read",
    "tmt_moe_launch_count", "tmt_moe_device_status", "tmt_moe_quantize_nvfp4",
    "tmt_moe_forward_nvfp4", "tmt_moe_ep_unique_id", "tmt_moe_ep_init", "tmt_moe_set_profile",
    "tmt_moe_profile", "tmt_moe_num_phases", "tmt_moe_phase_name", "tmt_moe_ep_plan",
    "tmt_moe_copy_stats", "tmt_moe_selftest_bounded_wait", "tmt_moe_router_dw_noalloc",
    "tmt_moe_debug_gemm_cycles", "tmt_moe_step_host_async", "tmt_moe_host_wait",
    "tmt_adamw_create", "tmt_adamw_destroy", "tmt_adamw_step",
    "tmt_ln_forward", "tmt_ln_backward", "tmt_ln_backward_scratch_bytes", "tmt_moe_usage",
    "tmt_moe_ep_check_capacity", "tmt_moe_nvfp4_weights_changed",
    "tmt_moe_forward_nvfp4_ln", "tmt_moe_ep_plan_device",
    "tmt_ckpt_hash", "tmt_ckpt_record_bytes", "tmt_ckpt_save_param", "tmt_ckpt_load_param",
    "tmt_sampler_create", "tmt_sampler_destroy", "tmt_sampler_set_weights", "tmt_sampler_x", "tmt_sampler_y",
    "tmt_sampler_stream", "tmt_sampler_step", "tmt_sampler_upload", "tmt_sampler_download", "tmt_sampler_sync",
    "tmt_sampler_sample", "tmt_sampler_steps", "tmt_sampler_graphs", "tmt_sampler_set_layernorm",
)


class MoeError(RuntimeError):
    pass


class Desc(ctypes.Structure):
    _fields_ = [("tokens", ctypes.c_int), ("dim", ctypes.c_int), ("hidden", ctypes.c_int),
                ("experts", ctypes.c_int), ("topk", ctypes.c_int), ("router_dtype", ctypes.c_int),
                ("training", ctypes.c_int), ("gemm_impl", ctypes.c_int), ("device", ctypes.c_int),
                ("host_io", ctypes.c_int), ("stream", ctypes.c_void_p), ("ep_world", ctypes.c_int),
                ("ep_rank", ctypes.c_int), ("ep_capacity_factor", ctypes.c_float), ("ep_transport", ctypes.c_int)]


class Nvfp4Weight(ctypes.Structure):
    _fields_ = [("packed", ctypes.c_void_p), ("scales", ctypes.c_void_p),
                ("tensor_scale", ctypes.c_float), ("rows", ctypes.c_int), ("cols", ctypes.c_int)]


_lib = None


def load():
    """Loads the shared library (never builds it implicitly on a machine without nvcc)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise MoeError("libtmt_moe_b200.so is missing: run `python -m tmt_moe_b200.build` "
                       "(or __graft_entry__.build()) first; there is no fallback path")
    lib = ctypes.CDLL(LIB_PATH)
    lib.tmt_moe_last_error.restype = ctypes.c_char_p
    lib.tmt_moe_read.restype = ctypes.c_longlong
    lib.tmt_moe_launch_count.restype = ctypes.c_longlong
    lib.tmt_moe_ep_plan.restype = ctypes.c_longlong
    lib.tmt_moe_destroy.restype = None
    lib.tmt_moe_phase_name.restype = ctypes.c_char_p
    for name in EXPORTS:
        getattr(lib, name)
    _lib = lib
    return lib


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, int):
        return ctypes.c_void_p(x)
    if hasattr(x, "data_ptr"):
        return ctypes.c_void_p(x.data_ptr())
    if hasattr(x, "ctypes"):
        return x.ctypes.data_as(ctypes.c_void_p)
    raise TypeError("expected a tensor, a numpy array or an address, got %r" % type(x))


def _ptr_array(xs):
    if xs is None:
        return None
    arr = (ctypes.c_void_p * len(xs))()
    for i, x in enumerate(xs):
        p = _ptr(x)
        arr[i] = None if p is None else p.value
    return arr


def _check(rc, lib):
    if rc != 0:
        raise MoeError(lib.tmt_moe_last_error().decode())


class MoE:
    """One MoE layer's state (the reference's MoeKeep + MoeWs)."""

    def __init__(self, tokens, dim, experts, topk, hidden=0, router_dtype=BF16, training=True,
                 gemm_impl=GEMM_AUTO, device=0, host_io=False, stream=None, ep_world=1, ep_rank=0,
                 ep_capacity_factor=0.0, ep_transport=0):
        self.lib = load()
        self.desc = Desc(tokens, dim, hidden, experts, topk, router_dtype, int(training), gemm_impl, device,
                         int(host_io), stream, ep_world, ep_rank, ep_capacity_factor, ep_transport)
        self.h = ctypes.c_void_p()
        _check(self.lib.tmt_moe_create(ctypes.byref(self.desc), ctypes.byref(self.h)), self.lib)
        self.tokens, self.dim, self.hidden, self.experts, self.topk = tokens, dim, hidden, experts, topk
        self.pad = 256 if gemm_impl in (GEMM_AUTO, GEMM_TCGEN05_2CTA) else 128      # rows every expert group is padded to
        self._keep = None

    def close(self):
        if getattr(self, "h", None) is not None and self.h.value:
            self.lib.tmt_moe_destroy(self.h)
            self.h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_router_bias(self, bias):
        import numpy as np
        arr = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        _check(self.lib.tmt_moe_set_router_bias(self.h, _ptr(arr)), self.lib)

    def forward(self, X, Wrouter, Wup, Wdown, Y, beta=0.0, tokens=None):
        t = self.tokens if tokens is None else tokens
        up, down = _ptr_array(Wup), _ptr_array(Wdown)
        self._keep = (up, down)
        _check(self.lib.tmt_moe_forward(self.h, _ptr(X), _ptr(Wrouter), up, down, _ptr(Y), ctypes.c_float(beta), t),
               self.lib)

    def backward(self, dY, Wrouter, Wup, Wdown, dWrouter, dWup, dWdown, dX, aux=0.0, zcoef=0.0):
        _check(self.lib.tmt_moe_backward(self.h, _ptr(dY), _ptr(Wrouter), _ptr_array(Wup), _ptr_array(Wdown),
                                         _ptr(dWrouter), _ptr_array(dWup), _ptr_array(dWdown), _ptr(dX),
                                         ctypes.c_float(aux), ctypes.c_float(zcoef)), self.lib)

    def step_host(self, X_host, dY_host, Wrouter, Wup, Wdown, dWrouter, dWup, dWdown, Y_host, dX_host, stat_host,
                  beta=0.0, aux=0.0, zcoef=0.0, tokens=None, wait=True):
        """wait=False queues the step and returns (tmt_moe_step_host_async); call host_wait() before reading results."""
        t = self.tokens if tokens is None else tokens
        fn = self.lib.tmt_moe_step_host if wait else self.lib.tmt_moe_step_host_async
        _check(fn(self.h, _ptr(X_host), _ptr(dY_host), _ptr(Wrouter), _ptr_array(Wup),
                                          _ptr_array(Wdown), _ptr(dWrouter), _ptr_array(dWup), _ptr_array(dWdown),
                                          _ptr(Y_host), _ptr(dX_host), _ptr(stat_host), ctypes.c_float(beta),
                                          ctypes.c_float(aux), ctypes.c_float(zcoef), t), self.lib)

    def usage(self, reset=False):
        """Router-balance telemetry since the last reset: dict(min_share, max_share, dead, passes, totals[E])."""
        import numpy as np
        mn, mx = ctypes.c_double(), ctypes.c_double()
        dead, passes = ctypes.c_longlong(), ctypes.c_longlong()
        totals = np.zeros(self.experts, np.int64)
        _check(self.lib.tmt_moe_usage(self.h, ctypes.byref(mn), ctypes.byref(mx), ctypes.byref(dead), ctypes.byref(passes),
                                      totals.ctypes.data_as(ctypes.c_void_p), int(reset)), self.lib)
        return dict(min_share=mn.value, max_share=mx.value, dead=dead.value, passes=passes.value, totals=totals)

    def host_wait(self):
        _check(self.lib.tmt_moe_host_wait(self.h), self.lib)

    def stats(self):
        """Returns (stat[E+1], counts[E], aux) as numpy arrays / float (moe_aux_from, moe.cu:470-475)."""
        import numpy as np
        stat = np.zeros(self.experts + 1, np.float32)
        counts = np.zeros(self.experts, np.int64)
        aux = ctypes.c_float(0)
        _check(self.lib.tmt_moe_stats(self.h, _ptr(stat), _ptr(counts), ctypes.byref(aux)), self.lib)
        return stat, counts, aux.value

    def read(self, name, tokens=None):
        import numpy as np
        t = self.tokens if tokens is None else tokens
        E, K = self.experts, self.topk
        shapes = {"logits": ((t, E), np.float32), "probs": ((t, E), np.float32), "idx": ((t, K), np.int32),
                  "slot_of": ((t, K), np.int32), "w": ((t, K), np.float32), "lse": ((t,), np.float32),
                  "counts": ((E,), np.int32), "poff": ((E + 1,), np.int32), "dlogits": ((t, E), np.float32),
                  "s_j": ((t, K), np.float32)}
        if name not in shapes:
            cap = np.zeros(1, np.int32)
            self.lib.tmt_moe_read(self.h, b"cap", _ptr(cap), ctypes.c_size_t(4))
            cap = int(cap[0])
            gcap = np.zeros(1, np.int32)              # rows of the grouped GEMM buffers (differs from cap under expert parallelism)
            self.lib.tmt_moe_read(self.h, b"gcap", _ptr(gcap), ctypes.c_size_t(4))
            gcap = int(gcap[0])
            D, H = self.dim, self.hidden
            shapes.update({"slotw": ((cap,), np.float32), "tok_of_slot": ((cap,), np.int32),
                           "tile_expert": ((cap // 128,), np.int32), "num_m_tiles": ((1,), np.int32),
                           "Xg": ((gcap, D), np.uint16), "Yg": ((gcap, D), np.uint16), "dYg": ((gcap, D), np.uint16),
                           "dXg": ((gcap, D), np.uint16), "P": ((gcap, H), np.uint16), "Hact": ((gcap, H), np.uint16),
                           "dP": ((gcap, H), np.uint16), "sw_part": ((gcap, (H + 127) // 128), np.float32)})
        shape, dt = shapes[name]
        out = np.empty(shape, dt)
        n = self.lib.tmt_moe_read(self.h, name.encode(), _ptr(out), ctypes.c_size_t(out.nbytes))
        if n < 0:
            raise MoeError(self.lib.tmt_moe_last_error().decode())
        assert n == out.nbytes, (n, out.nbytes)
        return out

    def forward_nvfp4(self, X, Wrouter, Wup, Wdown, Y, beta=0.0, tokens=None):
        """Wup / Wdown: lists of (packed, scales, tensor_scale, rows, cols)."""
        t = self.tokens if tokens is None else tokens

        def arr(ws):
            a = (Nvfp4Weight * len(ws))()
            for i, (p, s, ts, r, c) in enumerate(ws):
                a[i] = Nvfp4Weight(_ptr(p), _ptr(s), ts, r, c)
            return a
        # a sampler calls this once per byte with the same weights: the descriptor arrays are built once per set of
        # pointers, scales and shapes (a list mutated in place gets new arrays; the tensors are kept alive by the entry)
        def sig(ws):
            return tuple((_ptr(p).value, _ptr(s).value, float(ts), r, c) for p, s, ts, r, c in ws)
        key = (sig(Wup), sig(Wdown))
        hit = getattr(self, "_nvfp4_desc", None)
        if hit is None or hit[0] != key:
            hit = (key, list(Wup), list(Wdown), arr(Wup), arr(Wdown))
            self._nvfp4_desc = hit
        _check(self.lib.tmt_moe_forward_nvfp4(self.h, _ptr(X), _ptr(Wrouter), hit[3], hit[4], _ptr(Y),
                                              ctypes.c_float(beta), t), self.lib)

    def forward_nvfp4_ln(self, X, gamma, beta_ln, Wrouter, Wup, Wdown, Y, beta=0.0, tokens=None):
        """forward_nvfp4 with the LayerNorm in front of the block taken in (X: rows before the normalisation)."""
        t = self.tokens if tokens is None else tokens

        def arr(ws):
            a = (Nvfp4Weight * len(ws))()
            for i, (p, s, ts, r, c) in enumerate(ws):
                a[i] = Nvfp4Weight(_ptr(p), _ptr(s), ts, r, c)
            return a
        keep = (arr(Wup), arr(Wdown))
        _check(self.lib.tmt_moe_forward_nvfp4_ln(self.h, _ptr(X), _ptr(gamma), _ptr(beta_ln), _ptr(Wrouter), keep[0], keep[1],
                                                 _ptr(Y), ctypes.c_float(beta), t), self.lib)

    def nvfp4_weights_changed(self):
        """Call after re-quantising into the same buffers: derived copies are rebuilt at the next forward_nvfp4."""
        _check(self.lib.tmt_moe_nvfp4_weights_changed(self.h), self.lib)

    def ep_init_torch(self, dist):
        """Creates the handle's NCCL communicator: rank 0 makes the id, torch.distributed ships it."""
        import torch
        buf = torch.zeros(128, dtype=torch.uint8)
        if dist.get_rank() == 0:
            raw = (ctypes.c_ubyte * 128)()
            _check(self.lib.tmt_moe_ep_unique_id(raw), self.lib)
            buf = torch.tensor(list(raw), dtype=torch.uint8)
        dev = buf.cuda() if dist.get_backend() == "nccl" else buf
        dist.broadcast(dev, src=0)
        raw = (ctypes.c_ubyte * 128)(*dev.cpu().tolist())
        _check(self.lib.tmt_moe_ep_init(self.h, raw), self.lib)

    @property
    def ep_waves(self):
        """Expert waves an expert-parallel step runs in (1: one exchange per pass); known after ep_init."""
        w = ctypes.c_int(0)
        if self.lib.tmt_moe_read(self.h, b"ep_waves", ctypes.byref(w), ctypes.c_size_t(4)) != 4:
            _check(-1, self.lib)
        return int(w.value)

    def set_profile(self, on):
        _check(self.lib.tmt_moe_set_profile(self.h, int(on)), self.lib)

    def profile(self, reset=True):
        """{phase name: (milliseconds, launches)} accumulated since the last reset."""
        n = self.lib.tmt_moe_num_phases()
        ms = (ctypes.c_float * n)()
        cnt = (ctypes.c_longlong * n)()
        _check(self.lib.tmt_moe_profile(self.h, ms, cnt, int(reset)), self.lib)
        return {self.lib.tmt_moe_phase_name(i).decode(): (ms[i], cnt[i]) for i in range(n) if cnt[i]}

    def gemm_cycles(self):
        """Measurement only (TMT_MOE_GEMM_CYCLES=1 at creation): (launches so far, array
        [ring slot][cta][counter]) of the per-role cycle counters of the last GEMM launches."""
        import numpy as np
        a, b, c = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        self.lib.tmt_moe_debug_gemm_cycles(self.h, None, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c))
        out = np.zeros((a.value, b.value, c.value), np.int64)
        n = self.lib.tmt_moe_debug_gemm_cycles(self.h, out.ctypes.data_as(ctypes.c_void_p), None, None, None)
        if n < 0:
            raise MoeError(self.lib.tmt_moe_last_error().decode())
        return n, out

    @property
    def launch_count(self):
        return self.lib.tmt_moe_launch_count(self.h)

    def device_status(self):
        return self.lib.tmt_moe_device_status(self.h)


def ln_forward(X, gamma, beta, Y, mean, rstd, stream=None):
    """LayerNorm forward (include/tmt_norm.h; layernorm_fwd, tmt-cuda/src/norm.cu:96-100). Torch CUDA tensors."""
    lib = load()
    rows, dim = X.shape
    _check(lib.tmt_ln_forward(_ptr(X), _ptr(gamma), _ptr(beta), _ptr(Y), _ptr(mean), _ptr(rstd), int(rows), int(dim), _ptr(stream)), lib)


def ln_backward_scratch_bytes(rows, dim):
    lib = load()
    lib.tmt_ln_backward_scratch_bytes.restype = ctypes.c_size_t
    return int(lib.tmt_ln_backward_scratch_bytes(int(rows), int(dim)))


def ln_backward(X, dY, gamma, mean, rstd, dX, dGamma, dBeta, scratch, stream=None):
    """LayerNorm backward (layernorm_bwd, norm.cu:102-110); scratch: ln_backward_scratch_bytes(rows, dim) bytes."""
    lib = load()
    rows, dim = X.shape
    _check(lib.tmt_ln_backward(_ptr(X), _ptr(dY), _ptr(gamma), _ptr(mean), _ptr(rstd), _ptr(dX), _ptr(dGamma), _ptr(dBeta),
                               int(rows), int(dim), _ptr(scratch), _ptr(stream)), lib)


class AdamW:
    """Multi-tensor AdamW over a fixed list of tensors (include/tmt_adamw.h; the reference's optimizer_step,
    tmt-cuda/src/model.cu:716-729). Tensors are torch CUDA tensors (fp32 master / m / v / grad, bf16 work or None)."""

    def __init__(self, sizes, device=0, stream=None):
        self.lib = load()
        self.n = len(sizes)
        self.h = ctypes.c_void_p()
        arr = (ctypes.c_longlong * self.n)(*[int(s) for s in sizes])
        _check(self.lib.tmt_adamw_create(self.n, arr, int(device), _ptr(stream), ctypes.byref(self.h)), self.lib)

    def step(self, master, m, v, grad, work, flags=None, clip=0.0, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, wd=0.01, step=1,
             zero_grads=True, want_norm=False):
        fl = (ctypes.c_ubyte * self.n)(*([3] * self.n if flags is None else [int(f) for f in flags]))
        ss = ctypes.c_double(0.0)
        _check(self.lib.tmt_adamw_step(self.h, _ptr_array(master), _ptr_array(m), _ptr_array(v), _ptr_array(grad),
                                       _ptr_array(work), fl, ctypes.c_float(clip), ctypes.c_float(lr), ctypes.c_float(b1),
                                       ctypes.c_float(b2), ctypes.c_float(eps), ctypes.c_float(wd), int(step),
                                       int(bool(zero_grads)), ctypes.byref(ss) if want_norm else None), self.lib)
        return ss.value if want_norm else None

    def close(self):
        if self.h:
            self.lib.tmt_adamw_destroy(self.h)
            self.h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:   # noqa: BLE001
            pass


class SamplerDesc(ctypes.Structure):
    _fields_ = [("streams", ctypes.c_int), ("dim", ctypes.c_int), ("hidden", ctypes.c_int), ("experts", ctypes.c_int),
                ("topk", ctypes.c_int), ("router_dtype", ctypes.c_int), ("ring", ctypes.c_int), ("device", ctypes.c_int),
                ("stream", ctypes.c_void_p), ("seed", ctypes.c_uint64)]


class Sampler:
    """Batched multi-stream sampler session (include/tmt_sampler.h; the reference's Generator, generate.h:9-60, for many
    streams): NVFP4 decode steps replayed as CUDA graphs over device-resident ring slots, and Generator::sample on the
    device for all streams at once."""

    def __init__(self, streams, dim, hidden, experts, topk, router_dtype=BF16, ring=4, device=0, stream=None, seed=1):
        self.lib = load()
        for name in ("tmt_sampler_x", "tmt_sampler_y", "tmt_sampler_stream"):
            getattr(self.lib, name).restype = ctypes.c_void_p
        self.lib.tmt_sampler_steps.restype = ctypes.c_longlong
        self.lib.tmt_sampler_destroy.restype = None
        self.desc = SamplerDesc(streams, dim, hidden, experts, topk, router_dtype, ring, device, stream, seed)
        self.h = ctypes.c_void_p()
        _check(self.lib.tmt_sampler_create(ctypes.byref(self.desc), ctypes.byref(self.h)), self.lib)
        self.streams, self.dim, self.ring = streams, dim, ring
        self._keep = None

    def set_weights(self, Wrouter, Wup, Wdown):
        """Wup / Wdown: lists of (packed, scales, tensor_scale, rows, cols), one entry per expert."""
        def arr(ws):
            a = (Nvfp4Weight * len(ws))()
            for i, (p, sc, ts, r, c) in enumerate(ws):
                a[i] = Nvfp4Weight(_ptr(p), _ptr(sc), ts, r, c)
            return a
        self._keep = (Wrouter, list(Wup), list(Wdown))
        _check(self.lib.tmt_sampler_set_weights(self.h, _ptr(Wrouter), arr(Wup), arr(Wdown)), self.lib)

    def set_layernorm(self, gamma, beta):
        """The slots' X rows become the rows before the LayerNorm in front of the block (None, None: off)."""
        self._ln = (gamma, beta)
        _check(self.lib.tmt_sampler_set_layernorm(self.h, _ptr(gamma), _ptr(beta)), self.lib)

    def x_ptr(self, slot):
        return self.lib.tmt_sampler_x(self.h, slot)

    def y_ptr(self, slot):
        return self.lib.tmt_sampler_y(self.h, slot)

    @property
    def cuda_stream(self):
        return self.lib.tmt_sampler_stream(self.h)

    def step(self, slot, beta=0.0):
        _check(self.lib.tmt_sampler_step(self.h, slot, ctypes.c_float(beta)), self.lib)

    def upload(self, slot, X_host):
        _check(self.lib.tmt_sampler_upload(self.h, slot, _ptr(X_host)), self.lib)

    def download(self, slot, Y_host):
        _check(self.lib.tmt_sampler_download(self.h, slot, _ptr(Y_host)), self.lib)

    def sync(self):
        _check(self.lib.tmt_sampler_sync(self.h), self.lib)

    def sample(self, logits, temp, position, next_device):
        _check(self.lib.tmt_sampler_sample(self.h, _ptr(logits), ctypes.c_float(temp), ctypes.c_longlong(position),
                                           _ptr(next_device)), self.lib)

    @property
    def steps(self):
        return self.lib.tmt_sampler_steps(self.h)

    @property
    def graphs(self):
        return self.lib.tmt_sampler_graphs(self.h)

    def close(self):
        if getattr(self, "h", None) is not None and self.h.value:
            self.lib.tmt_sampler_destroy(self.h)
            self.h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:   # noqa: BLE001
            pass


CKPT_HASH_INIT = 14695981039346656037


def ckpt_hash(h, data):
    """The reference's streaming checkpoint checksum (FNV-1a 64, checkpoint.h:11-17) over a bytes-like object."""
    lib = load()
    lib.tmt_ckpt_hash.restype = ctypes.c_uint64
    buf = (ctypes.c_char * len(data)).from_buffer_copy(bytes(data)) if len(data) else None
    return int(lib.tmt_ckpt_hash(ctypes.c_uint64(h), buf, ctypes.c_size_t(len(data))))


def ckpt_record_bytes(n):
    lib = load()
    lib.tmt_ckpt_record_bytes.restype = ctypes.c_size_t
    return int(lib.tmt_ckpt_record_bytes(ctypes.c_longlong(n)))


def ckpt_save_param(master, m, v, stream=None):
    """One V3 parameter record (u64 n | master | m | v, checkpoint.h:142-148) of fp32 CUDA tensors, as bytes."""
    lib = load()
    n = master.numel()
    rec = bytearray(ckpt_record_bytes(n))
    buf = (ctypes.c_char * len(rec)).from_buffer(rec)
    _check(lib.tmt_ckpt_save_param(_ptr(master), _ptr(m), _ptr(v), ctypes.c_longlong(n), buf, ctypes.c_size_t(len(rec)),
                                   _ptr(stream)), lib)
    return bytes(rec)


def ckpt_load_param(record, master, m=None, v=None, work=None, stream=None):
    """Reads one record into fp32 CUDA tensors and re-materialises the bf16 working copy (checkpoint.h:149)."""
    lib = load()
    buf = (ctypes.c_char * len(record)).from_buffer_copy(bytes(record))
    _check(lib.tmt_ckpt_load_param(buf, ctypes.c_size_t(len(record)), ctypes.c_longlong(master.numel()), _ptr(master), _ptr(m),
                                   _ptr(v), _ptr(work), _ptr(stream)), lib)


def quantize_nvfp4(W, rows, cols, packed, scales, stream=None):
    """Quantises a bf16 device matrix; returns the per-tensor scale."""
    lib = load()
    ts = ctypes.c_float(0)
    _check(lib.tmt_moe_quantize_nvfp4(_ptr(W), rows, cols, _ptr(packed), _ptr(scales), ctypes.byref(ts),
                                      ctypes.c_void_p(stream)), lib)
    return ts.value
