"""Builds libhpspmm.so (the C-ABI library) for sm_100a with nvcc, in-tree.

    python hp-spmm-sddmm_b200/build.py [--force] [--verbose]

The library lands in hp-spmm-sddmm_b200/lib/libhpspmm.so.  nvcc cross-compiles, so no
GPU is needed to build.
"""
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_DIR = os.path.join(PKG_DIR, "lib")
OBJ_DIR = os.path.join(PKG_DIR, "build")
LIB_PATH = os.path.join(LIB_DIR, "libhpspmm.so")
TEST_ALL_PATH = os.path.join(LIB_DIR, "test_all")

SOURCES = [
    "capi_runtime.cu",
    "spmm_kernels.cu",
    "sddmm_kernels.cu",
    "structure_kernels.cu",
    "graph_layer.cu",
    "probe_kernels.cu",
    "sharded_product.cu",
    "host_side.cpp",
]

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-lineinfo", "-std=c++17", "-I", os.path.join(ROOT, "include"), "-I", CSRC,
          "-Xcompiler", "-fPIC,-fopenmp,-fvisibility=hidden,-O3", "-diag-suppress", "63"]


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build libhpspmm.so")
    return exe


def _newest_source_mtime():
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    paths.append(os.path.join(ROOT, "include", "hpspmm.h"))
    paths.append(os.path.abspath(__file__))
    return max(os.path.getmtime(p) for p in paths)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError("command failed: %s\n%s" % (" ".join(cmd), res.stdout))
    if verbose and res.stdout.strip():
        print(res.stdout)
    return res.stdout


def build(force=False, verbose=False, ptxas_info=False):
    """Compiles every CUDA source for sm_100a and links the shared library."""
    os.makedirs(LIB_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    if (not force and os.path.exists(LIB_PATH)
            and os.path.getmtime(LIB_PATH) >= _newest_source_mtime()):
        return LIB_PATH
    nvcc = _nvcc()
    extra = ["-Xptxas", "-v"] if ptxas_info else []

    def compile_one(src):
        obj = os.path.join(OBJ_DIR, os.path.splitext(src)[0] + ".o")
        cmd = [nvcc] + ARCH + COMMON + extra + ["-c", os.path.join(CSRC, src), "-o", obj]
        return obj, _run(cmd, verbose)

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        results = list(pool.map(compile_one, SOURCES))
    objs = [r[0] for r in results]
    if ptxas_info:
        for _, out in results:
            print(out)
    _run([nvcc] + ARCH + ["-shared", "-o", LIB_PATH] + objs + ["-Xcompiler", "-fopenmp", "-lgomp", "-ldl"],
         verbose)
    return LIB_PATH


def build_test_all(force=False, verbose=False):
    """Builds the C++ bench driver (successor of the reference's test/test_all.cpp)."""
    src = os.path.join(PKG_DIR, "host", "test_all.cpp")
    if not os.path.exists(src):
        return None
    build(force=force, verbose=verbose)
    if (not force and os.path.exists(TEST_ALL_PATH)
            and os.path.getmtime(TEST_ALL_PATH) >= max(os.path.getmtime(src), os.path.getmtime(LIB_PATH))):
        return TEST_ALL_PATH
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else (shutil.which("g++") or "g++")
    _run([cxx, "-O3", "-mavx2", "-mfma", "-std=c++17", "-fopenmp", "-I", os.path.join(ROOT, "include"), src, "-o",
          TEST_ALL_PATH, "-L", LIB_DIR, "-lhpspmm", "-Wl,-rpath,$ORIGIN"], verbose)
    return TEST_ALL_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv,
                 ptxas_info="--ptxas-info" in sys.argv)
    print(path)
    t = build_test_all(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    if t:
        print(t)
