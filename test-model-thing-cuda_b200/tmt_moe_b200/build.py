"""Builds libtmt_moe_b200.so in-tree from csrc/*.cu for sm_100a (nvcc cross-compiles without a GPU)."""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(HERE), "csrc")
LIB = os.path.join(HERE, "libtmt_moe_b200.so")
OBJ = os.path.join(HERE, "build")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "-Xptxas", "-v"]
if os.environ.get("TMT_MOE_MEASURE"):       # measurement build: compiles the kernels' phase switches in (results can be wrong)
    FLAGS.append("-DTMT_MOE_MEASURE")


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _newest_source():
    return max(os.path.getmtime(os.path.join(CSRC, f)) for f in os.listdir(CSRC)) if os.path.isdir(CSRC) else 0
    

def stale():
    inc = os.path.join(os.path.dirname(os.path.dirname(HERE)), "include", "tmt_moe.h")
    newest = max(_newest_source(), os.path.getmtime(inc) if os.path.exists(inc) else 0)
    return not os.path.exists(LIB) or os.path.getmtime(LIB) < newest


def build(force=False, verbose=False):
    if not force and not stale():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")

    def compile_one(src):
        obj = os.path.join(OBJ, src[:-3] + ".o")
        r = subprocess.run([nvcc, *FLAGS, "-c", os.path.join(CSRC, src), "-o", obj],
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        with open(os.path.join(OBJ, src[:-3] + ".ptxas.txt"), "w") as f:
            f.write(r.stdout)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed on %s:\n%s" % (src, r.stdout))
        if verbose:
            print(r.stdout)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, sources()))
    r = subprocess.run([nvcc, "-shared", "-o", LIB, *objs, "-ldl"], stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stdout)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
