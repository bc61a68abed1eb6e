"""Build libhlq_b200.so (CUDA kernels + C ABI) in-tree for sm_100a.

    python -m elutq_b200.build

nvcc cross-compiles without a GPU.  The library is placed next to the sources so that it
travels with the tree; nothing is installed into site-packages.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(CSRC, "libhlq_b200.so")
SOURCES = ["hlq_host.cpp", "hlq_layout.cu", "hlq_gemv.cu", "hlq_batch.cu", "hlq_batch_umma.cu", "hlq_batch_tmem.cu", "hlq_gemm.cu", "hlq_gemm_pair.cu", "hlq_glue.cu", "hlq_chain.cu", "hlq_sparse.cu", "hlq_fit.cu", "hlq_api.cu"]
HEADERS = ["hlq_layout.h", "hlq_internal.h", "hlq_gemv_dev.cuh", "hlq_gemv_args.cuh", "hlq_batch_dev.cuh", "hlq_gemm_dev.cuh", "hlq_attn_dev.cuh", os.path.join("..", "..", "include", "hlq_b200.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    headers = [os.path.join(CSRC, h) for h in HEADERS]
    objs = []
    procs = []
    for src in SOURCES:
        path = os.path.join(CSRC, src)
        obj = os.path.join(CSRC, os.path.splitext(src)[0] + ".o")
        objs.append(obj)
        if force or _stale(obj, [path] + headers):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", path, "-o", obj]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(out.decode(errors="replace"))
        if p.returncode != 0:
            failed = True
    if failed:
        raise RuntimeError("nvcc failed")
    if force or procs or _stale(LIB, objs):
        subprocess.run([nvcc, "-shared", "-o", LIB] + objs + ["-lcuda"], check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
