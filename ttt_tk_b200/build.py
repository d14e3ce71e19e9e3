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
SOURCES = ["ttt_capi.cu", "ttt_fwd_sm100.cu", "ttt_bwd_sm100.cu", "ttt_fwd_cluster_sm100.cu", "ttt_bwd_cluster_sm100.cu", "ttt_linear_fwd_sm100.cu", "ttt_linear_bwd_sm100.cu",
           "ttt_layout.cu", "ttt_glue.cu", "umma_selftest.cu"]
HEADERS = ["sm100_ptx.cuh", "ttt_device.cuh", "ttt_cluster.cuh", "ttt_internal.h", os.path.join("..", "..", "include", "ttt_mlp_b200.h")]
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


# ---------------------------------------------------------------------------------------------
# The PyTorch extension module `test_time_training` (the reference's module name): a C++ shim
# over the C ABI, built in-tree next to the library it links against.
EXT_NAME = "test_time_training"
EXT_SOURCE = os.path.join(CSRC, "test_time_training.cpp")


def extension_path():
    import sysconfig
    return os.path.join(LIB_DIR, EXT_NAME + sysconfig.get_config_var("EXT_SUFFIX"))


def build_extension(force=False, verbose=False):
    """Compile ttt_tk_b200/lib/test_time_training*.so with g++ against the installed torch."""
    build(force=False, verbose=verbose)
    out = extension_path()
    deps = [EXT_SOURCE, os.path.join(CSRC, "..", "..", "include", "ttt_mlp_b200.h")]
    if not force and os.path.exists(out) and all(os.path.getmtime(d) <= os.path.getmtime(out) for d in deps):
        return out
    import sysconfig
    import torch
    from torch.utils import cpp_extension as ce
    inc = ce.include_paths(device_type="cuda") if "device_type" in ce.include_paths.__code__.co_varnames \
        else ce.include_paths(cuda=True)
    libdirs = ce.library_paths(device_type="cuda") if "device_type" in ce.library_paths.__code__.co_varnames \
        else ce.library_paths(cuda=True)
    cxx = os.environ.get("CXX", "g++")
    cmd = [cxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-w",
           f"-DTORCH_EXTENSION_NAME={EXT_NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           "-I" + sysconfig.get_path("include")]
    cmd += ["-I" + p for p in inc]
    cmd += [EXT_SOURCE, "-o", out, "-L" + LIB_DIR, "-lttt_mlp_b200", "-Wl,-rpath,$ORIGIN"]
    cmd += ["-L" + p for p in libdirs] + ["-Wl,-rpath," + p for p in libdirs if "torch" in p]
    cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("building the test_time_training extension failed")
    return out


def load_extension():
    """Import and return the `test_time_training` module (building it if needed)."""
    import importlib.util
    import torch  # noqa: F401  (libtorch must be loaded before the extension)
    path = build_extension()
    spec = importlib.util.spec_from_file_location(EXT_NAME, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules.setdefault(EXT_NAME, mod)
    return mod
