"""Build the C-ABI library libgct_b200.so for sm_100a with nvcc (in-tree, next to this file)."""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCES = ["csrc/gct_attn_sm100.cu", "csrc/gct_elementwise.cu", "csrc/gct_manager.cu", "csrc/gct_static_scratch.cu",
           "csrc/gct_exchange.cu", "csrc/gct_decode.cu", "csrc/gct_render.cu"]
HEADERS = ["csrc/gct_common.h", "../include/gct_b200.h"]
LIB = os.path.join(HERE, "libgct_b200.so")


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put the CUDA toolkit on PATH")


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(os.path.join(HERE, s)) > t for s in SOURCES + HEADERS)


def build(force=False, verbose=False):
    """Compile every CUDA source of the package into libgct_b200.so.  Returns the library path."""
    if not force and not needs_build():
        return LIB
    cmd = [_nvcc(), "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
           "-Xcompiler", "-fPIC", "-shared", "-cudart", "static", "-o", LIB] + SOURCES
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    r = subprocess.run(cmd, cwd=HERE, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + r.stdout + r.stderr)
    if verbose:
        print(r.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
