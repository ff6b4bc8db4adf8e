"""Builds ``insignia_b200/lib/libinsignia_b200.so`` in-tree with nvcc for sm_100a.

One shared library holds the CUDA kernels, their C ABI (include/insignia_b200.h)
and the C++ host classes (include/insignia_*.hpp).  nvcc cross-compiles without a
GPU, so the build also runs on CPU-only hosts.
"""
from __future__ import annotations

import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "insignia_b200")
LIB_DIR = os.path.join(PKG, "lib")
LIB = os.path.join(LIB_DIR, "libinsignia_b200.so")
OBJ_DIR = os.path.join(LIB_DIR, "obj")

SOURCES = [
    "csrc/mxfp4_gemv.cu", "csrc/gemv_fused.cu", "csrc/umma_gemv.cu", "csrc/umma_gemm.cu", "csrc/persistent.cu", "csrc/deltanet.cu", "csrc/attention.cu", "csrc/elementwise.cu", "csrc/allreduce.cu", "csrc/compat_kernels.cu", "csrc/capi_util.cu",
    "host/model_file.cpp", "host/storage.cpp", "host/qwen35.cpp", "host/decode.cpp", "host/batch_decode.cpp", "host/engine_capi.cpp",
]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler",
         "-fPIC,-fvisibility=hidden", "-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(PKG, "csrc")]


def _deps_mtime() -> float:
    m = 0.0
    for d in (os.path.join(ROOT, "include"), os.path.join(PKG, "csrc"), os.path.join(PKG, "host")):
        for f in os.listdir(d):
            m = max(m, os.path.getmtime(os.path.join(d, f)))
    return m


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    srcs = [s for s in SOURCES if os.path.exists(os.path.join(PKG, s))]
    newest = _deps_mtime()
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= newest:
        return LIB
    procs, objs = [], []
    for s in srcs:
        obj = os.path.join(OBJ_DIR, os.path.basename(s) + ".o")
        objs.append(obj)
        src = os.path.join(PKG, s)
        hdr_m = max(os.path.getmtime(os.path.join(ROOT, "include", f)) for f in os.listdir(os.path.join(ROOT, "include")))
        com_m = max(os.path.getmtime(os.path.join(PKG, "csrc", f)) for f in os.listdir(os.path.join(PKG, "csrc"))
                    if f.endswith((".h", ".cuh")))
        if not force and os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(src), hdr_m, com_m):
            continue
        cmd = ["nvcc", *FLAGS, "-x", "cu", "-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for s, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- {s}\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.check_call(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB, *objs, "-lcudart"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
