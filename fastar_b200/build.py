"""Builds the native libraries in-tree for sm_100a.

  python -m fastar_b200.build          # libfst_cuda_mla.so + libfst_engine.so

nvcc cross-compiles without a GPU.  The CUDA runtime is linked statically and the driver is
reached through cudaGetDriverEntryPoint, so the libraries load (but refuse to create a
context) on a machine without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
HOST = os.path.join(PKG, "host")
LIB_CUDA = os.path.join(PKG, "libfst_cuda_mla.so")
LIB_ENGINE = os.path.join(PKG, "libfst_engine.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-cudart", "static"]
CUDA_SOURCES = ["mla_ctx.cu", "kernels_simt.cu", "gemm_tc.cu", "attn_stream.cu", "no_alloc.cu"]


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("build failed: " + " ".join(cmd))


def build(force: bool = False, verbose: bool = False) -> None:
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    srcs = [os.path.join(CSRC, s) for s in CUDA_SOURCES]
    hdrs = [os.path.join(CSRC, h) for h in os.listdir(CSRC) if h.endswith(".cuh")]
    hdrs.append(os.path.join(ROOT, "include", "fst_cuda_mla.h"))
    objdir = os.path.join(ROOT, "build")
    os.makedirs(objdir, exist_ok=True)
    objs = []
    for s in srcs:
        o = os.path.join(objdir, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or _newer(o, [s] + hdrs):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            _run(cmd)
    if force or _newer(LIB_CUDA, objs):
        _run([nvcc, "-shared", "-cudart", "static", "-o", LIB_CUDA] + objs + ["-ldl"])
    host_srcs = [os.path.join(HOST, f) for f in ("fst_engine.cpp", "fst_engine_capi.cpp", "fst_file.cpp")]
    host_hdrs = [os.path.join(HOST, "fst_engine.h"), os.path.join(HOST, "fst_file.h"), os.path.join(ROOT, "include", "fst_cuda_mla.h")]
    if all(os.path.exists(s) for s in host_srcs) and (force or _newer(LIB_ENGINE, host_srcs + host_hdrs + [LIB_CUDA])):
        _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-I", os.path.join(ROOT, "include"),
              "-o", LIB_ENGINE] + host_srcs + ["-L", PKG, "-l:libfst_cuda_mla.so", "-Wl,-rpath,$ORIGIN"])


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built", LIB_CUDA)
