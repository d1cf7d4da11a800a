"""Dry run of the ctypes front end against a stand-in library, on CPU.

Every method of tmt_moe_b200 that talks to the shared library is called once with host arrays of plausible shapes while
a fake library records the calls and answers success. Nothing is computed: the point is that the Python side of the
GPU-only paths (argument marshalling, shape tables, the properties the bench reads at N > 1) runs without a NameError,
AttributeError or TypeError before it ever reaches a GPU box. The real library's behaviour is the GPU tests' business.
"""
import ctypes
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path[:0] = [os.path.join(ROOT, "test-model-thing-cuda_b200")]


class FakeFn:
    def __init__(self, lib, name):
        self.lib, self.name, self.restype = lib, name, ctypes.c_int

    def __call__(self, *args):
        self.lib.calls.append(self.name)
        n = self.name
        if n == "tmt_moe_last_error":
            return b"stand-in library"
        if n.endswith("_create"):
            args[-1]._obj.value = 0x1000                      # byref(c_void_p): a non-null handle
            return 0
        if n == "tmt_moe_read":
            what, dst, size = args[1], args[2], args[3].value
            if what in (b"cap", b"gcap", b"ep_waves"):
                val = ctypes.c_int(4 if what == b"ep_waves" else 1024)
                ctypes.memmove(dst, ctypes.byref(val), 4)
                return 4
            return size
        if n == "tmt_moe_debug_gemm_cycles":
            if args[1] is None:
                for a, v in zip(args[2:5], (2, 3, 4)):
                    a._obj.value = v
            return 0
        if n == "tmt_moe_num_phases":
            return 2
        if n == "tmt_moe_phase_name":
            return b"phase%d" % args[0]
        if n == "tmt_moe_profile":
            args[2][0] = 3                                     # one phase has launches
            return 0
        if n in ("tmt_ckpt_record_bytes", "tmt_ln_backward_scratch_bytes"):
            return 8 + 12 * 16
        if n == "tmt_moe_ep_unique_id":
            return 0
        return 0


class FakeLib:
    def __init__(self):
        self.calls, self._fns = [], {}

    def __getattr__(self, name):
        if not name.startswith("tmt_"):
            raise AttributeError(name)
        return self._fns.setdefault(name, FakeFn(self, name))


@pytest.fixture
def front_end(monkeypatch):
    import tmt_moe_b200 as M
    fake = FakeLib()
    monkeypatch.setattr(M, "_lib", fake)
    return M, fake


class HostTensor(np.ndarray):
    """numpy array with the two torch methods the helpers use."""
    def numel(self):
        return self.size


def _t(shape, dtype):
    return np.zeros(shape, dtype).view(HostTensor)


def test_moe_handle_methods(front_end):
    M, fake = front_end
    T, D, H, E, K = 64, 128, 64, 8, 2
    moe = M.MoE(T, D, E, K, hidden=H, router_dtype=M.F32, training=True, gemm_impl=M.GEMM_AUTO, ep_world=2, ep_rank=1,
                ep_transport=M.EP_PEER)
    assert moe.pad == 256
    X, Y, dY, dX = (_t((T, D), np.uint16) for _ in range(4))
    Wr, dWr = _t((E, D), np.float32), _t((E, D), np.float32)
    Wup, Wdown = [_t((H, D), np.uint16) for _ in range(E)], [_t((D, H), np.uint16) for _ in range(E)]
    dWup, dWdown = [_t((H, D), np.float32) for _ in range(E)], [_t((D, H), np.float32) for _ in range(E)]
    stat = _t((E + 1,), np.float32)
    moe.set_router_bias(np.zeros(E))
    moe.set_router_bias(None)
    moe.forward(X, Wr, Wup, Wdown, Y, beta=0.5)
    moe.backward(dY, Wr, Wup, Wdown, dWr, dWup, dWdown, dX, aux=0.01, zcoef=0.001)
    moe.step_host(X, dY, Wr, Wup, Wdown, dWr, dWup, dWdown, Y, dX, stat, wait=True)
    moe.step_host(X, dY, Wr, Wup, Wdown, dWr, dWup, dWdown, Y, dX, stat, wait=False)
    moe.host_wait()
    assert set(moe.usage(reset=True)) == {"min_share", "max_share", "dead", "passes", "totals"}
    st, counts, aux = moe.stats()
    assert st.shape == (E + 1,) and counts.shape == (E,) and aux == 0.0
    for name in ("logits", "probs", "idx", "slot_of", "w", "lse", "counts", "poff", "dlogits", "s_j", "slotw", "tok_of_slot",
                 "tile_expert", "num_m_tiles", "Xg", "Yg", "dYg", "dXg", "P", "Hact", "dP", "sw_part"):
        assert moe.read(name).size > 0
    assert moe.ep_waves == 4
    moe.set_profile(True)
    assert list(moe.profile()) == ["phase0"]
    n, cyc = moe.gemm_cycles()
    assert cyc.shape == (2, 3, 4)
    assert moe.launch_count == 0 and moe.device_status() == 0
    q = [(_t((H, D // 2), np.uint8), _t((H, D // 16), np.uint8), 1.0, H, D) for _ in range(E)]
    qd = [(_t((D, H // 2), np.uint8), _t((D, H // 16), np.uint8), 1.0, D, H) for _ in range(E)]
    moe.forward_nvfp4(X, Wr, q, qd, Y)
    moe.forward_nvfp4(X, Wr, q, qd, Y)                       # second call: the cached descriptor arrays
    moe.forward_nvfp4_ln(X, _t((D,), np.float32), _t((D,), np.float32), Wr, q, qd, Y)
    moe.nvfp4_weights_changed()
    assert M.quantize_nvfp4(Wup[0], H, D, q[0][0], q[0][1]) == 0.0
    moe.close()
    moe.close()                                              # idempotent
    for f in ("tmt_moe_create", "tmt_moe_forward", "tmt_moe_backward", "tmt_moe_step_host", "tmt_moe_step_host_async",
              "tmt_moe_forward_nvfp4", "tmt_moe_forward_nvfp4_ln", "tmt_moe_nvfp4_weights_changed", "tmt_moe_destroy"):
        assert f in fake.calls, f
    assert fake.calls.count("tmt_moe_destroy") == 1


def test_ep_init_through_a_process_group(front_end):
    M, fake = front_end
    torch = pytest.importorskip("torch")

    class OneRank:                                           # the three calls ep_init_torch makes, for a single CPU rank
        @staticmethod
        def get_rank():
            return 0

        @staticmethod
        def get_backend():
            return "gloo"

        @staticmethod
        def broadcast(t, src):
            assert t.dtype == torch.uint8 and t.numel() == 128 and src == 0
    moe = M.MoE(64, 128, 8, 2, hidden=64, ep_world=2, ep_rank=0)
    moe.ep_init_torch(OneRank)
    assert fake.calls[-2:] == ["tmt_moe_ep_unique_id", "tmt_moe_ep_init"]


def test_neighbours_sampler_and_checkpoint_helpers(front_end):
    M, fake = front_end
    rows, dim = 8, 64
    X, Yo, dY, dX = (_t((rows, dim), np.uint16) for _ in range(4))
    g, b, dg, db = (_t((dim,), np.float32) for _ in range(4))
    mean, rstd = _t((rows,), np.float32), _t((rows,), np.float32)
    M.ln_forward(X, g, b, Yo, mean, rstd)
    scratch = _t((M.ln_backward_scratch_bytes(rows, dim),), np.uint8)
    M.ln_backward(X, dY, g, mean, rstd, dX, dg, db, scratch)
    opt = M.AdamW([16, 32])
    ts = lambda n, dt=np.float32: [_t((16,), dt), _t((32,), dt)]
    assert opt.step(ts(2), ts(2), ts(2), ts(2), ts(2, np.uint16), want_norm=True) == 0.0
    assert opt.step(ts(2), ts(2), ts(2), ts(2), [None, None], flags=[1, 1]) is None
    opt.close()
    s = M.Sampler(64, 128, 64, 8, 2, router_dtype=M.F32, ring=2, seed=7)
    q = [(_t((64, 64), np.uint8), _t((64, 8), np.uint8), 1.0, 64, 128) for _ in range(8)]
    s.set_weights(_t((8, 128), np.float32), q, q)
    s.set_layernorm(_t((128,), np.float32), _t((128,), np.float32))
    s.set_layernorm(None, None)
    assert s.x_ptr(0) == 0 and s.y_ptr(1) == 0 and s.cuda_stream == 0
    s.upload(0, _t((64, 128), np.uint16)); s.step(0, 0.0); s.download(0, _t((64, 128), np.uint16)); s.sync()
    s.sample(_t((64, 256), np.uint16), 0.8, 3, _t((64,), np.int32))
    assert s.steps == 0 and s.graphs == 0
    s.close()
    assert M.ckpt_record_bytes(16) == 8 + 12 * 16
    rec = M.ckpt_save_param(_t((16,), np.float32), _t((16,), np.float32), _t((16,), np.float32))
    assert len(rec) == 8 + 12 * 16
    M.ckpt_load_param(rec, _t((16,), np.float32), _t((16,), np.float32), _t((16,), np.float32), _t((16,), np.uint16))
    assert M.ckpt_hash(M.CKPT_HASH_INIT, b"abc") == 0 and M.ckpt_hash(M.CKPT_HASH_INIT, b"") == 0
    for f in ("tmt_ln_forward", "tmt_ln_backward", "tmt_adamw_step", "tmt_sampler_set_weights", "tmt_sampler_sample",
              "tmt_ckpt_save_param", "tmt_ckpt_load_param", "tmt_ckpt_hash"):
        assert f in fake.calls, f
