"""Builds checkers_b200/lib/libcheckers_b200.so in-tree with nvcc for sm_100a."""
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
# CHECKERS_B200_LIB points the package at a library built elsewhere (it is then never rebuilt here)
LIB = os.environ.get("CHECKERS_B200_LIB") or os.path.join(LIB_DIR, "libcheckers_b200.so")
SOURCES = ["engine.cu", "repair.cu"]
HEADERS = ["kernels.cuh", "rans_kernels.cuh", "table_kernels.cuh", "stats_kernels.cuh", "plane_kernels.cuh", "study_kernels.cuh", "format_v3.inc", "sort_replica.hpp", "host_stream.inc", "tables.hpp", "clusters.hpp",
           os.path.join("..", "..", "include", "checkers_b200.h")]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared"]


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(CSRC, h) for h in HEADERS]
    return any(os.path.getmtime(f) > t for f in deps)


def build(force=False, verbose=False):
    """Compile the library if a source is newer than it.  Returns the library path."""
    if os.environ.get("CHECKERS_B200_LIB") or (not force and not needs_build()):
        return LIB
    os.makedirs(LIB_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + \
          [os.path.join(CSRC, s) for s in SOURCES] + ["-o", LIB]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
