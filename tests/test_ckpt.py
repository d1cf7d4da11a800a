"""Checkpoint pass-through of the block's parameters (include/tmt_ckpt.h). Here, without a GPU: the checksum against
published FNV-1a 64 known answers and a plain restatement of checkpoint.h:11-16, the record size, and the checks a load
makes before it touches the device. On a GPU (marked gpu): records written from device memory have the reference's byte
layout (checkpoint.h:142-148), and save -> load -> re-materialised bf16 / NVFP4 copies give a bit-identical forward."""
import ctypes
import struct

import numpy as np
import pytest

import tmt_moe_b200 as M
from tmt_moe_b200 import synth
from oracle import oracle as O


def _fnv1a(h, data):
    for b in data:
        h = ((h ^ b) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


def test_checksum_known_answers():
    init = M.CKPT_HASH_INIT
    assert M.ckpt_hash(init, b"") == init == 0xcbf29ce484222325
    assert M.ckpt_hash(init, b"a") == 0xaf63dc4c8601ec8c            # FNV-1a 64 test vectors
    assert M.ckpt_hash(init, b"foobar") == 0x85944171f73967e8
    data = np.random.default_rng(1).integers(0, 256, 5000, dtype=np.uint8).tobytes()
    assert M.ckpt_hash(init, data) == _fnv1a(init, data)
    # streaming: the hash of a file is the hash of its pieces in order (Checkpoint::bytes, checkpoint.h:31-35)
    assert M.ckpt_hash(M.ckpt_hash(init, data[:1234]), data[1234:]) == _fnv1a(init, data)


def test_record_size_and_load_checks_before_any_device_work():
    assert M.ckpt_record_bytes(1) == 20 and M.ckpt_record_bytes(2048 * 2048) == 8 + 12 * 2048 * 2048
    lib = M.load()
    rec = struct.pack("<Q", 7) + bytes(12 * 7)
    buf = (ctypes.c_char * len(rec)).from_buffer_copy(rec)
    dummy = ctypes.c_void_p(16)                 # never dereferenced: both calls fail before any copy
    assert lib.tmt_ckpt_load_param(buf, ctypes.c_size_t(len(rec)), ctypes.c_longlong(8), dummy, None, None, None, None) == -1
    assert b"shape mismatch" in lib.tmt_moe_last_error()
    assert lib.tmt_ckpt_load_param(buf, ctypes.c_size_t(len(rec) - 4), ctypes.c_longlong(7), dummy, None, None, None, None) == -1
    assert b"truncated" in lib.tmt_moe_last_error()


@pytest.mark.gpu
def test_round_trip_gives_a_bit_identical_forward():
    import torch
    import gpu_util as G
    T, D, H, E, K = 300, 256, 256, 4, 2
    data = synth.make(T, D, H, E, K, seed=61, need_dy=False)
    rng = np.random.default_rng(62)
    # fp32 masters (what the optimizer owns), moments, and the bf16 working copies derived from them
    shapes = [("Wr", (E, D))] + [("Wup%d" % e, (H, D)) for e in range(E)] + [("Wdown%d" % e, (D, H)) for e in range(E)]
    masters = {n: torch.from_numpy((rng.standard_normal(s) * (0.1 if n == "Wr" else 0.02)).astype(np.float32)).cuda() for n, s in shapes}
    moments = {n: (torch.from_numpy(rng.standard_normal(s).astype(np.float32) * 1e-3).cuda(),
                   torch.from_numpy((rng.standard_normal(s).astype(np.float32) * 1e-3) ** 2).cuda()) for n, s in shapes}

    def work_of(ms):
        return {n: t.to(torch.bfloat16) for n, t in ms.items()}          # torch rounds to nearest even as well

    def forward(work, nvfp4):
        moe = M.MoE(T, D, E, K, hidden=H, training=False)
        X = G.dev(data["X"])
        Y = torch.zeros((T, D), dtype=torch.int16, device="cuda")
        up, down = [work["Wup%d" % e] for e in range(E)], [work["Wdown%d" % e] for e in range(E)]
        if not nvfp4:
            moe.forward(X, work["Wr"], up, down, Y)
        else:
            q = {"up": [], "down": []}
            for name, ws in (("up", up), ("down", down)):
                for W in ws:
                    r, c = W.shape
                    p = torch.empty((r, c // 2), dtype=torch.uint8, device="cuda")
                    s = torch.empty((r, c // 16), dtype=torch.uint8, device="cuda")
                    q[name].append((p, s, M.quantize_nvfp4(W, r, c, p, s), r, c))
            moe.forward_nvfp4(X, work["Wr"], q["up"], q["down"], Y)
        torch.cuda.synchronize()
        assert moe.device_status() == 0
        return G.host_u16(Y).copy()

    want_bf16, want_fp4 = forward(work_of(masters), False), forward(work_of(masters), True)
    # save: the payload section of the block's parameters, in parameter order, with the running checksum
    payload, h = b"", M.CKPT_HASH_INIT
    for n, _ in shapes:
        rec = M.ckpt_save_param(masters[n], moments[n][0], moments[n][1])
        cnt = masters[n].numel()
        host = b"".join(t.cpu().numpy().tobytes() for t in (masters[n], moments[n][0], moments[n][1]))
        assert rec == struct.pack("<Q", cnt) + host                       # u64 n | master | m | v (checkpoint.h:144-148)
        payload += rec
        h = M.ckpt_hash(h, rec)
    assert h == _fnv1a(M.CKPT_HASH_INIT, payload)
    # load into fresh buffers; the bf16 copies come from the library (copy_bf16_kernel's job, checkpoint.h:149)
    off, loaded, work = 0, {}, {}
    for n, s in shapes:
        cnt = int(np.prod(s))
        size = M.ckpt_record_bytes(cnt)
        master = torch.full(s, float("nan"), device="cuda")
        m1, v1 = torch.full(s, float("nan"), device="cuda"), torch.full(s, float("nan"), device="cuda")
        wk = torch.zeros(s, dtype=torch.bfloat16, device="cuda")
        M.ckpt_load_param(payload[off:off + size], master, m1, v1, wk)
        off += size
        assert torch.equal(master, masters[n]) and torch.equal(m1, moments[n][0]) and torch.equal(v1, moments[n][1])
        loaded[n], work[n] = master, wk
    assert off == len(payload)
    for n in work:
        assert torch.equal(work[n], masters[n].to(torch.bfloat16)), n
    np.testing.assert_array_equal(forward(work, False), want_bf16)
    np.testing.assert_array_equal(forward(work, True), want_fp4)
    # weights only (the sampler's load, generate.h:25) on an unaligned view: the scalar path of the re-materialisation
    base = torch.zeros(masters["Wr"].numel() + 1, device="cuda")
    wk = torch.zeros(masters["Wr"].numel() + 1, dtype=torch.bfloat16, device="cuda")
    M.ckpt_load_param(payload[:M.ckpt_record_bytes(E * D)], base[1:], None, None, wk[1:])
    assert torch.equal(wk[1:], masters["Wr"].reshape(-1).to(torch.bfloat16))
