"""Builds the CUDA backend (libphoenix_core_b200.so) for sm_100a, in-tree, with nvcc.

Usage: python -m phoenix_core_b200.csrc.build [--force] [--verbose]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libphoenix_core_b200.so")
SOURCES = ["api.cu", "simt_qgemm.cu", "tensor_path.cu", "pointwise_tc.cu", "conv_tc.cu", "narrow_tc.cu", "conv_tf32.cu", "aux_bn.cu"]
HEADERS = ["common.cuh", "tensor_path.cuh", "umma.cuh", "tc_common.cuh", os.path.join("..", "..", "include", "phoenix_core_b200.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall", "-shared",
]


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    for f in SOURCES + HEADERS + ["build.py"]:
        path = os.path.join(HERE, f)
        if os.path.exists(path) and os.path.getmtime(path) > t:
            return True
    return False


def build(force=False, verbose=False):
    """Compiles every CUDA source of the backend into one shared library next to the sources."""
    if not force and not _stale():
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB] + SOURCES
    res = subprocess.run(cmd, cwd=HERE, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building libphoenix_core_b200.so")
    if verbose:
        sys.stderr.write(res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
