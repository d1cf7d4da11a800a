"""CPU checks of the C ABI: the shared library loads without a GPU and exports every function
include/tmt_moe.h declares; compute entry points fail with a message (no GPU here), never crash."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    import tmt_moe_b200 as M
    from tmt_moe_b200 import build
    build.build()
    return M.load()


def test_every_declared_symbol_is_exported(lib):
    names = set()
    for header in sorted(os.listdir(os.path.join(ROOT, "include"))):
        text = open(os.path.join(ROOT, "include", header)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(tmt_(?:moe|adamw|ln|ckpt|sampler)_[a-z0-9_]+)\s*\(", text))
    assert len(names) >= 26 and "tmt_adamw_step" in names and "tmt_ln_backward" in names
    for n in sorted(names):
        assert hasattr(lib, n), n
    import tmt_moe_b200 as M
    assert set(M.EXPORTS) <= names


def test_adamw_fails_cleanly_on_bad_arguments(lib):
    assert lib.tmt_adamw_create(0, None, 0, None, None) == -1
    h = ctypes.c_void_p()
    assert lib.tmt_adamw_create(0, None, 0, None, ctypes.byref(h)) == -1
    assert b"tensor" in lib.tmt_moe_last_error()
    assert lib.tmt_adamw_step(None, None, None, None, None, None, None, ctypes.c_float(0), ctypes.c_float(0), ctypes.c_float(0),
                              ctypes.c_float(0), ctypes.c_float(0), ctypes.c_float(0), 1, 0, None) == -1


def test_create_fails_cleanly_without_gpu_or_with_bad_arguments(lib):
    import torch
    import tmt_moe_b200 as M
    with pytest.raises(M.MoeError):
        M.MoE(64, 100, 4, 2)          # dim not a multiple of 64 (checked before any CUDA call)
    with pytest.raises(M.MoeError):
        M.MoE(64, 128, 17, 18)        # topk > experts: the reference rejects this too (config.h:51-52)
    if not torch.cuda.is_available():
        with pytest.raises(M.MoeError):
            M.MoE(64, 128, 4, 2)
    assert lib.tmt_moe_create(None, None) == -1
    assert b"null" in lib.tmt_moe_last_error()


def test_phase_names(lib):
    n = lib.tmt_moe_num_phases()
    names = [lib.tmt_moe_phase_name(i).decode() for i in range(n)]
    assert names[0] == "router" and "gemm_up" in names and "exchange" in names and len(set(names)) == n


def test_reference_shim_compiles(tmp_path):
    """The source-level drop-in (shim/moe.h) accepts the calls the reference's own harness makes
    (tmt-cuda/src/profile.cu:32-55) with the reference's argument lists."""
    import shutil
    import subprocess
    cuda_inc = "/usr/local/cuda/include"
    if shutil.which("g++") is None or not os.path.exists(os.path.join(cuda_inc, "cuda_bf16.h")):
        pytest.skip("needs g++ and the CUDA headers")
    src = tmp_path / "use_shim.cpp"
    src.write_text("""
#include "%s/test-model-thing-cuda_b200/shim/moe.h"
int run() {
    int N = 2048, E = 8, K = 2, D = 1280;
    bf16 *X = nullptr, *Y = nullptr, *dY = nullptr, *dX = nullptr, *Wr = nullptr, *Wx[16] = {nullptr};
    float *dWr = nullptr, *dWx[16] = {nullptr};
    MoeKeep keep; MoeWs ws;
    moe_keep_alloc(keep, N, E, K, D);
    moe_ws_alloc(ws, N, E, K, D);
    float aux = moe_forward(X, Wr, Wx, Y, keep, ws, N, E, K, D);
    moe_backward(dY, Wx, Wr, dWr, dWx, dX, keep, ws, 0.01f, 0.001f);
    float hsum[17] = {0};
    aux += moe_aux_from(keep, hsum) + keep.zloss + keep.hcnt[0];
    moe_keep_free(keep); moe_ws_free(ws);
    return (int)aux;
}
""" % ROOT)
    r = subprocess.run(["g++", "-std=c++17", "-I", cuda_inc, "-c", str(src), "-o", str(tmp_path / "use_shim.o")],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert r.returncode == 0, r.stdout
