"""The library's host-side code (generators, readers, partitioner, needed-rows planner) built with
-fsanitize=address,undefined and run through tests/host_sanitize/main.cpp.  No GPU: host_side.cpp needs
only the CUDA headers for the types of the shared internal header."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cuda_include():
    for base in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if base and os.path.exists(os.path.join(base, "include", "cuda_runtime.h")):
            return os.path.join(base, "include")
    nvcc = shutil.which("nvcc")
    if nvcc:
        inc = os.path.join(os.path.dirname(os.path.dirname(os.path.realpath(nvcc))), "include")
        if os.path.exists(os.path.join(inc, "cuda_runtime.h")):
            return inc
    return None


def test_host_side_under_asan_and_ubsan(tmp_path):
    inc = _cuda_include()
    if inc is None:
        pytest.skip("CUDA headers not found")
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else (shutil.which("g++") or "g++")
    exe = str(tmp_path / "host_sanitize")
    cmd = [cxx, "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=address,undefined",
           "-fno-sanitize-recover=undefined", "-fopenmp", "-I", os.path.join(ROOT, "include"),
           "-I", os.path.join(ROOT, "hp-spmm-sddmm_b200", "csrc"), "-I", inc,
           os.path.join(ROOT, "tests", "host_sanitize", "main.cpp"),
           os.path.join(ROOT, "hp-spmm-sddmm_b200", "csrc", "host_side.cpp"), "-o", exe]
    build = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert build.returncode == 0, build.stdout[-3000:]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1",
               OMP_NUM_THREADS="4")
    run = subprocess.run([exe, str(tmp_path)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env,
                         timeout=300)
    assert run.returncode == 0, run.stdout[-4000:]
    assert "host sanitizer run: ok" in run.stdout
    assert "runtime error" not in run.stdout and "AddressSanitizer" not in run.stdout
