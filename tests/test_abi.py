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
    text = open(os.path.join(ROOT, "include", "tmt_moe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(tmt_moe_[a-z0-9_]+)\s*\(", text))
    assert len(names) >= 20
    for n in sorted(names):
        assert hasattr(lib, n), n
    import tmt_moe_b200 as M
    assert set(M.EXPORTS) <= names


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
