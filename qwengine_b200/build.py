"""Builds libq38b200.so (the CUDA kernels and the C ABI) in-tree for sm_100a with nvcc.

    python -m qwengine_b200.build [--verbose]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libq38b200.so")
SOURCES = ["q38b_api.cu", "q38b_plan.cu", "q38b_prefill.cu", "q38b_static.cu", "q38b_gguf.cpp"]


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "q38b200.h")]
    return any(os.path.getmtime(d) > t for d in deps if os.path.isfile(d))


def build(verbose=False, force=False):
    if not force and not _stale():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
           "-Xcompiler", "-fPIC,-O2", "-shared", "-ccbin", "g++",
           "-o", LIB] + [os.path.join(CSRC, s) for s in SOURCES] + ["-lcudart", "-ldl"]
    if verbose:
        cmd.insert(1, "-Xptxas=-v,-warn-spills")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode:
        raise RuntimeError("nvcc failed")
    return LIB


if __name__ == "__main__":
    build(verbose="--verbose" in sys.argv, force=True)
    print(LIB)
