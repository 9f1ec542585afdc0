"""Build libknet_sm100.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python knet.jl_b200/build.py [--force]

Objects go to knet.jl_b200/build/, the library to knet.jl_b200/libknet_sm100.so.
Flags that matter for results: -fmad=false (the kernels fuse multiply-adds only where they
say fma), IEEE division and square root (nvcc defaults), no fast-math.
"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libknet_sm100.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-fmad=false", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-I", INCLUDE,
]


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _newest_header():
    t = os.path.getmtime(os.path.join(INCLUDE, "knet_sm100.h"))
    for f in os.listdir(CSRC):
        if f.endswith((".cuh", ".inc", ".h")):
            t = max(t, os.path.getmtime(os.path.join(CSRC, f)))
    return t


def _compile(src, force, hdr_time):
    obj = os.path.join(OBJ, src[:-3] + ".o")
    path = os.path.join(CSRC, src)
    if not force and os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(path), hdr_time):
        return obj, False
    subprocess.check_call([NVCC] + FLAGS + ["-c", path, "-o", obj])
    return obj, True


def build(force=False, verbose=True):
    os.makedirs(OBJ, exist_ok=True)
    hdr_time = _newest_header()
    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        results = list(ex.map(lambda s: _compile(s, force, hdr_time), _sources()))
    objs = [o for o, _ in results]
    if force or any(c for _, c in results) or not os.path.exists(LIB):
        subprocess.check_call([NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
                               "-o", LIB] + objs + ["-lcudart_static", "-ldl", "-lrt", "-lpthread"])
        if verbose:
            print(f"built {LIB}")
    elif verbose:
        print(f"{LIB} is up to date")
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv)
