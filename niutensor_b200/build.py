"""Builds the CUDA library in-tree: niutensor_b200/libntb_gemm.so (sm_100a only).

    python -m niutensor_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU. Every source is compiled to an object of its own, in
parallel, and only sources newer than their object (or older than a header) are compiled
again; the objects live in niutensor_b200/build/. The library links the CUDA runtime
statically and looks up the one driver entry point it needs (the tensor-map encoder) at
run time, so it has no load-time dependency beyond libstdc++.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libntb_gemm.so")
SOURCES = ["ntb_api.cu", "ntb_tc.cu", "ntb_tc_pair.cu", "ntb_tc_split.cu", "ntb_tc_pairsplit.cu", "ntb_tc_f32pair.cu", "ntb_tc_ldg.cu", "ntb_repack.cu",
           "ntb_simt.cu", "ntb_noalloc.cu", "ntb_attn.cu", "ntb_logsoftmax.cu", "ntb_sharded.cu", "ntb_grouped.cu"]
HEADERS = [os.path.join(CSRC, "ntb_internal.h"), os.path.join(CSRC, "ntb_ptx.cuh"),
           os.path.join(CSRC, "ntb_tc_common.cuh"), os.path.join(CSRC, "ntb_tc_single.cuh"),
           os.path.join(os.path.dirname(HERE), "include", "ntb_gemm.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall", "-cudart", "static"]


def _sources():
    return [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _obj(src):
    return os.path.join(OBJ_DIR, os.path.splitext(src)[0] + ".o")


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def needs_build():
    deps = [os.path.join(CSRC, s) for s in _sources()] + HEADERS + [os.path.abspath(__file__)]
    return _stale(LIB, deps)


def build(force=False, verbose=False):
    if not force and not needs_build():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    extra = os.environ.get("NTB_NVCC_EXTRA", "").split()
    os.makedirs(OBJ_DIR, exist_ok=True)
    common = HEADERS + [os.path.abspath(__file__)]

    def compile_one(src):
        path, obj = os.path.join(CSRC, src), _obj(src)
        if not force and not _stale(obj, [path] + common):
            return
        cmd = [nvcc] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", path, "-o", obj]
        subprocess.check_call(cmd)

    srcs = _sources()
    with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 1)) as pool:
        list(pool.map(compile_one, srcs))
    subprocess.check_call([nvcc] + NVCC_FLAGS + ["--shared", "-o", LIB] + [_obj(s) for s in srcs])
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(LIB)
