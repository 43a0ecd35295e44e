"""Builds the CUDA library in-tree: niutensor_b200/libntb_gemm.so (sm_100a only).

    python -m niutensor_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU. The library links the CUDA runtime statically and
looks up the one driver entry point it needs (the tensor-map encoder) at run time, so it
has no load-time dependency beyond libstdc++.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libntb_gemm.so")
SOURCES = ["ntb_api.cu", "ntb_tc.cu", "ntb_simt.cu", "ntb_noalloc.cu", "ntb_attn.cu", "ntb_logsoftmax.cu"]
HEADERS = [os.path.join(CSRC, "ntb_internal.h"), os.path.join(CSRC, "ntb_ptx.cuh"),
           os.path.join(os.path.dirname(HERE), "include", "ntb_gemm.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall", "--shared", "-cudart", "static"]


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES] + HEADERS + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    if not force and not needs_build():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + \
        ["-o", LIB] + [os.path.join(CSRC, s) for s in SOURCES]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(LIB)
