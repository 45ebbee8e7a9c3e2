"""Builds the CUDA backend (libphoenix_core_b200.so) for sm_100a, in-tree, with nvcc.

Every source is compiled to an object file of its own (in parallel, and only when it or a header is newer than
the object), then the objects are linked into one shared library next to the sources.

Usage: python -m phoenix_core_b200.csrc.build [--force] [--verbose]
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libphoenix_core_b200.so")
OBJ_DIR = os.path.join(HERE, "build")
SOURCES = ["api.cu", "simt_qgemm.cu", "tensor_path.cu", "pointwise_tc.cu", "pointwise2_tc.cu", "pointwise8_tc.cu", "conv_tc.cu", "narrow_tc.cu",
           "conv_tf32.cu", "aux_bn.cu", "probe.cu"]
HEADERS = ["common.cuh", "tensor_path.cuh", "umma.cuh", "tc_common.cuh", os.path.join("..", "..", "include", "phoenix_core_b200.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall",
]


def _mtime(path):
    return os.path.getmtime(path) if os.path.exists(path) else 0.0


def _sources():
    return [s for s in SOURCES if os.path.exists(os.path.join(HERE, s))]


def _compile(nvcc, src, obj, verbose):
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", "-o", obj, src]
    return src, subprocess.run(cmd, cwd=HERE, capture_output=True, text=True)


def build(force=False, verbose=False):
    """Compiles every CUDA source of the backend into one shared library next to the sources."""
    nvcc = os.environ.get("NVCC", "nvcc")
    os.makedirs(OBJ_DIR, exist_ok=True)
    newest_header = max([_mtime(os.path.join(HERE, h)) for h in HEADERS] + [_mtime(os.path.join(HERE, "build.py"))])
    todo = []
    objs = []
    for src in _sources():
        obj = os.path.join(OBJ_DIR, src[:-3] + ".o")
        objs.append(obj)
        if force or _mtime(obj) < max(_mtime(os.path.join(HERE, src)), newest_header):
            todo.append((src, obj))
    if todo:
        with ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 1)) as pool:
            results = list(pool.map(lambda so: _compile(nvcc, so[0], so[1], verbose), todo))
        failed = [(s, r) for s, r in results if r.returncode != 0]
        for s, r in results:
            if r.returncode != 0 or verbose:
                sys.stderr.write("== %s\n%s%s" % (s, r.stdout, r.stderr))
        if failed:
            raise RuntimeError("nvcc failed building " + ", ".join(s for s, _ in failed))
    if todo or not os.path.exists(LIB) or any(_mtime(o) > _mtime(LIB) for o in objs):
        res = subprocess.run([nvcc, "-shared", "-o", LIB] + objs, cwd=HERE, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("linking libphoenix_core_b200.so failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
