"""The source-level drop-in (shim/moe.h) linked into the reference's own caller and RUN: oracle/_ref/profile_via_shim is
tmt-cuda/src/profile.cu compiled unchanged (oracle/Makefile, target `shim`) with shim/moe.h standing in for moe.cu. The
harness allocates MoeKeep / MoeWs, runs 15 warm-up and 2 x 60 timed moe_forward / moe_backward calls (8 experts, top-2,
dim 1280, 2048 tokens) and prints two timing lines; a failure inside the library would throw and abort it."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "oracle", "_ref", "profile_via_shim")


@pytest.mark.skipif(not os.path.exists(BIN), reason="oracle/_ref/profile_via_shim is built where the reference tree is present")
def test_reference_harness_runs_on_the_shim():
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = os.path.join(ROOT, "test-model-thing-cuda_b200", "tmt_moe_b200") + ":" + env.get("LD_LIBRARY_PATH", "")
    r = subprocess.run([BIN], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    print(r.stdout)
    assert r.returncode == 0, r.stdout
    lines = [l for l in r.stdout.splitlines() if l.startswith("MoE fwd")]
    assert len(lines) == 2 and "N=2048 E=8 K=2 D=1280" in lines[0] and lines[1].startswith("MoE fwd+bwd"), r.stdout
