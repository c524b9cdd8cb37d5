"""Build recipe: compiles the CUDA engine (sm_100a only) into lyapunovfractalwasm_b200/liblyap_b200.so.

nvcc cross-compiles without a GPU.  -fmad=false keeps nvcc from fusing a*b+c on its own: the exact
kernels fuse only where an fma is written out (see csrc/lyap_math.h).
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "liblyap_b200.so")

NVCC_FLAGS = [
    "-std=c++20", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-fmad=false",
    "-Xcompiler", "-fPIC,-ffp-contract=off,-Wall",
    "-shared", "-cudart", "shared",
]


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def lib_sources():
    names = ["lyap_abi.cu", "lyap_kernels.cu", "lyap_kernels_fast.cuh", "lyap_engine.h", "lyap_math.h",
             "lyap_tables.h"]
    return [os.path.join(CSRC, n) for n in names] + [os.path.join(ROOT, "include", "lyap_b200.h")]


def build_library(force=False, verbose=False):
    srcs = lib_sources()
    if not force and not _newer(LIB, srcs):
        return LIB
    cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + [
        "-o", LIB, os.path.join(CSRC, "lyap_abi.cu"), os.path.join(CSRC, "lyap_kernels.cu")]
    env = dict(os.environ)
    subprocess.run(cmd, check=True, env=env)
    return LIB


CLI = os.path.join(HERE, "lyap_cli")


def build_cli(force=False):
    """The C++23 command-line driver (host code only; links the engine library)."""
    src = os.path.join(CSRC, "lyap_cli.cpp")
    if not force and not _newer(CLI, [src, os.path.join(ROOT, "include", "lyap_b200.h"), LIB]):
        return CLI
    subprocess.run(["g++", "-std=c++23", "-O2", "-Wall", "-o", CLI, src, "-L", HERE, "-llyap_b200",
                    "-Wl,-rpath,$ORIGIN"], check=True)
    return CLI


def build_oracle():
    """Compile the CPU checkers (test infrastructure).  Uses the reference sources only where present."""
    subprocess.run(["make", "-s", "-C", os.path.join(ROOT, "oracle")], check=True)


if __name__ == "__main__":
    build_library(force="--force" in sys.argv, verbose="-v" in sys.argv)
    build_cli(force="--force" in sys.argv)
    build_oracle()
    print(LIB)
