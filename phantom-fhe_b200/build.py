"""Builds libb200fhe.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc", "b200fhe.cu")
OUT = os.path.join(HERE, "libb200fhe.so")
DEPS = [SRC] + [os.path.join(HERE, "csrc", f) for f in ("ntt_kernels.cuh", "modarith.cuh", "bconv_tc.cuh", "bconv_tc_plan.h", "sampler.cuh", "encoder.cuh")] + [
        os.path.join(os.path.dirname(HERE), "include", "b200fhe.h")]
FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
         "-Xcompiler", "-fPIC,-fopenmp", "-shared", "-lgomp"]


def build_native(force=False, verbose=False):
    if not force and os.path.exists(OUT) and all(os.path.getmtime(OUT) >= os.path.getmtime(d) for d in DEPS):
        return OUT
    cmd = ["nvcc"] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", OUT, SRC]
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build_native(force="--force" in sys.argv, verbose="-v" in sys.argv))
