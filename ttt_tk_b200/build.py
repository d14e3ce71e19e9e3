"""Build libttt_mlp_b200.so (CUDA kernels + C ABI) in-tree with nvcc for sm_100a.

    python -m ttt_tk_b200.build            # rebuild if sources are newer than the library
    python -m ttt_tk_b200.build --force

nvcc cross-compiles without a GPU.  The library links only against cudart; the driver
entry point it needs (cuTensorMapEncodeTiled) is looked up at run time.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libttt_mlp_b200.so")
SOURCES = ["ttt_capi.cu", "ttt_fwd_sm100.cu", "ttt_bwd_sm100.cu", "umma_selftest.cu"]
HEADERS = ["sm100_ptx.cuh", "ttt_internal.h", os.path.join("..", "..", "include", "ttt_mlp_b200.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC)")


def needs_build():
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    if not force and not needs_build():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [_nvcc()] + NVCC_FLAGS + ["-o", LIB_PATH] + SOURCES + ["-lcudart"]
    res = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libttt_mlp_b200.so")
    with open(os.path.join(LIB_DIR, "ptxas.log"), "w") as f:
        f.write(res.stdout + res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
