"""Builds libbunker_cuda.so in-tree with nvcc for sm_100a.

    python -m bunker_b200.build [--force] [--verbose]

The library has no Python or torch dependency; it links the static CUDA runtime.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libbunker_cuda.so")
TOK_LIB = os.path.join(HERE, "libbunker_tok.so")
TOK_SRC = os.path.join(CSRC, "bk_tokenizer.cpp")
SOURCES = ["bk_runtime.cu", "bk_gemv.cu", "bk_gemv_mma.cu", "bk_ops.cu", "bk_attn.cu", "bk_launch.cu", "bk_model.cu", "bk_comm.cu", "bk_persist.cu", "bk_quantize.cu", "bk_gemv_umma.cu", "bk_sample.cu"]
HEADERS = ["bk_common.cuh", "bk_internal.h", "bk_gemv_shared.cuh", "bk_gemv_dp4a.cuh", "bk_gdn.cuh",
           os.path.join("..", "..", "include", "bunker_cuda.h"), os.path.join("..", "..", "include", "bunker_cuda_diag.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-fmad=false",            # no implicit fma contraction: fused multiply-adds are spelled fmaf
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build_tokenizer(force: bool = False) -> str:
    """libbunker_tok.so: plain C++ (g++), no CUDA."""
    if not force and os.path.exists(TOK_LIB) and os.path.getmtime(TOK_LIB) >= os.path.getmtime(TOK_SRC):
        return TOK_LIB
    cxx = os.environ.get("CXX_FOR_BUNKER", "g++")
    subprocess.check_call([cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-pthread", "-Wall", "-o", TOK_LIB, TOK_SRC])
    return TOK_LIB


def build_library(force: bool = False, verbose: bool = False) -> str:
    build_tokenizer(force)
    if not force and not needs_build():
        return LIB
    objs = []
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    procs = []
    for s in SOURCES:
        obj = os.path.join(CSRC, s.replace(".cu", ".o"))
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", os.path.join(CSRC, s), "-o", obj]
        procs.append((s, cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env, text=True)))
        objs.append(obj)
    for s, cmd, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0:
            sys.stderr.write(out)
            raise RuntimeError(f"nvcc failed on {s}: {' '.join(cmd)}")
        if verbose:
            sys.stderr.write(out)
    link = [_nvcc(), "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
    subprocess.check_call(link, env=env)
    return LIB


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
