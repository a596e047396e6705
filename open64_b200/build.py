"""Builds libo64gemm.so in-tree with nvcc for sm_100a (cross-compiles without a GPU) and the
host-only tools o64nest (source rewriter) and o64whirl (WHIRL dump matcher) with g++.

Usage:  python -m open64_b200.build [--force] [--verbose] [--tuning]

--tuning builds a second library, libo64gemm_tuning.so, with -DO64_TUNING: the kernels then carry
the pipeline probes (O64_PROBE) and the cycle counters behind O64_TRACE=pipe, which the shipped
library does not.  Point O64_LIBRARY at it to load it instead of the shipped one.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libo64gemm.so")
OBJ_DIR = os.path.join(HERE, "build")
NEST_SRC = os.path.join(HERE, "nest2c", "nest2c.cpp")
NEST_OUT = os.path.join(HERE, "nest2c", "o64nest")
WHIRL_SRC = os.path.join(HERE, "whirl", "o64whirl.cpp")
WHIRL_OUT = os.path.join(HERE, "whirl", "o64whirl")

SOURCES = ["api.cu", "umma_gemm.cu", "umma_gemm_2cta.cu", "umma_gemm_wide.cu", "umma_gemm_skinny.cu", "simt_kernels.cu", "simt_generic.cu", "plan.cpp", "no_alloc.cu", "dotprod.cu"]
HEADERS = ["ptx_sm100.cuh", "umma_gemm.cuh", "umma_common.cuh", "simt_kernels.cuh", "../../include/o64gemm.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _nvcc():
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _sources():
    return [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force=False, verbose=False, tuning=False):
    """Compile every source to an object (in parallel) and link the shared library."""
    OBJ_DIR = os.path.join(HERE, "build", "tuning") if tuning else globals()["OBJ_DIR"]
    OUT = os.path.join(HERE, "libo64gemm_tuning.so") if tuning else globals()["OUT"]
    NVCC_FLAGS = globals()["NVCC_FLAGS"] + (["-DO64_TUNING"] if tuning else [])
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdrs = [os.path.join(CSRC, h) for h in HEADERS] + [os.path.abspath(__file__)]
    jobs = []
    objs = []
    for s in _sources():
        src = os.path.join(CSRC, s)
        obj = os.path.join(OBJ_DIR, os.path.splitext(s)[0] + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + hdrs):
            jobs.append([_nvcc(), *NVCC_FLAGS, "-x", "cu", "-c", src, "-o", obj])

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    logs = []
    with ThreadPoolExecutor(max_workers=4) as ex:
        for cmd, r in ex.map(run, jobs):
            logs.append(r.stderr)
            if verbose:
                sys.stderr.write(" ".join(cmd) + "\n" + r.stderr)
            if r.returncode != 0:
                raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    if jobs or force or _stale(OUT, objs):
        cmd = [_nvcc(), "-shared", "-o", OUT, *objs, "-ldl", "-Xcompiler", "-fPIC"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    with open(os.path.join(OBJ_DIR, "ptxas.log"), "a") as f:
        f.write("".join(logs))
    if os.path.exists(NEST_SRC) and (force or _stale(NEST_OUT, [NEST_SRC])):
        r = subprocess.run(["g++", "-O2", "-std=c++17", "-Wall", "-o", NEST_OUT, NEST_SRC], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("g++ failed on o64nest:\n" + r.stdout + r.stderr)
        if verbose:
            sys.stderr.write(r.stderr)
    if os.path.exists(WHIRL_SRC) and (force or _stale(WHIRL_OUT, [WHIRL_SRC])):
        r = subprocess.run(["g++", "-O2", "-std=c++17", "-Wall", "-o", WHIRL_OUT, WHIRL_SRC], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("g++ failed on o64whirl:\n" + r.stdout + r.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, tuning="--tuning" in sys.argv))
