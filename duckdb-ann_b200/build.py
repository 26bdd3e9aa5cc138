"""Builds the CUDA library in-tree with nvcc for sm_100a (and nothing else).

    python duckdb-ann_b200/build.py            # or: __graft_entry__.build()
    python duckdb-ann_b200/build.py --measure  # profiling build, see below

Outputs, beside the sources (git-ignored, but they travel with the working tree):
    duckdb-ann_b200/libann_cuda.so        the search library (C ABI of include/*.h)
    duckdb-ann_b200/backend_driver        C++ driver that exercises the GpuBackend classes
    duckdb-ann_b200/libann_cuda_measure.so  (--measure only) the same library compiled with
        -DANN_CUDA_MEASURE: the flat kernel then carries its cycle counters and stage switches
        (environment variables ANN_CUDA_TC_STATS, ANN_CUDA_TC_DEBUG).  The product library has
        none of that code; load the profiling build with ANN_CUDA_LIB=<path>.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(ROOT, "include")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libann_cuda.so")
DRIVER = os.path.join(HERE, "backend_driver")

LIB_SOURCES = ["prep.cu", "scan.cu", "merge.cu", "flat_tc.cu", "flat_tc_bk32.cu", "flat_tc_h16.cu", "index.cu", "sharded.cu",
               "cuda_diskann_bridge.cu", "disk_search.cu", "gpu_backend_cuda.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
# /usr/bin/g++ is the system compiler; the image's $CXX points at a gcc without OpenMP support files
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-I", INCLUDE, "-I", CSRC,
          "-ccbin", "/usr/bin/g++"]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found")
    return exe


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, measure: bool = False) -> str:
    global OBJ, LIB
    if measure:
        OBJ = os.path.join(HERE, "build_measure")
        LIB = os.path.join(HERE, "libann_cuda_measure.so")
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh", ".hpp"))]
    headers.append(os.path.join(CSRC, "flat_tc.cu"))  # flat_tc_bk32.cu and flat_tc_h16.cu include it
    headers += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    headers += [os.path.join(INCLUDE, "faiss", f) for f in os.listdir(os.path.join(INCLUDE, "faiss"))]
    headers.append(os.path.abspath(__file__))
    objs = []
    procs = []
    for src in LIB_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _newer(o, [s] + headers):
            cmd = ([nvcc()] + ARCH + COMMON + (["-DANN_CUDA_MEASURE"] if measure else []) +
                   (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o])
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"--- {src}\n{out}\n")
        elif verbose and out:
            sys.stderr.write(f"--- {src}\n{out}\n")
    if failed:
        raise RuntimeError("nvcc failed")
    if force or _newer(LIB, objs):
        subprocess.check_call([nvcc()] + ARCH + ["-shared", "-o", LIB] + objs + ["-ccbin", "/usr/bin/g++", "-lcudart", "-lpthread"])
    drv_src = os.path.join(CSRC, "backend_driver.cpp")
    if not measure and (force or _newer(DRIVER, [drv_src, LIB] + headers)):
        subprocess.check_call(["/usr/bin/g++", "-O2", "-std=c++17", "-DFAISS_AVAILABLE", "-DFAISS_CUDA_ENABLED",
                               "-I", INCLUDE, "-I", CSRC, drv_src, "-o", DRIVER, "-L", HERE, "-lann_cuda",
                               "-Wl,-rpath,$ORIGIN"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, measure="--measure" in sys.argv))
