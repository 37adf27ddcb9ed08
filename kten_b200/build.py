"""Build recipe for libkten_cuda.so (sm_100a only).

`python -m kten_b200.build` compiles every translation unit under
`kten_b200/csrc` with nvcc for compute_100a/sm_100a and links them into
`kten_b200/libkten_cuda.so`, next to this file, so the library travels with the
source tree.  nvcc cross-compiles: no GPU is needed to build.

Flags that matter for result parity with kten-jvm:
  -fmad=false      a*b+c is never contracted; fused multiply-adds appear only
                   where fmaf() is written (IEEE + - * / must round per op)
  -prec-div=true, -prec-sqrt=true, -ftz=false   (nvcc defaults, stated)
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "csrc", "build")
LIB = os.path.join(HERE, "libkten_cuda.so")

SOURCES = ["ktc_runtime.cu", "ktc_api.cu", "ktc_elementwise.cu", "ktc_reduce.cu", "ktc_comm.cu", "ktc_noalloc.cu", "ktc_expr.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false", "-prec-div=true", "-prec-sqrt=true", "-ftz=false",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-O2",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("KTC_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; libkten_cuda.so cannot be built")


def _deps_mtime() -> float:
    t = 0.0
    for root in (CSRC, os.path.join(HERE, "..", "include")):
        for name in os.listdir(root):
            if name.endswith((".cu", ".cuh", ".hpp", ".h")):
                t = max(t, os.path.getmtime(os.path.join(root, name)))
    return max(t, os.path.getmtime(__file__))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile and link the library if any source is newer than it; return its path."""
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _deps_mtime():
        return LIB
    nvcc = _nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    env = dict(os.environ)
    # nvcc's host compiler is the system gcc; an inherited CC/CXX may point elsewhere
    ccbin = shutil.which("g++") or "g++"

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        cmd = [nvcc, "-ccbin", ccbin, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True, env=env)
        log = os.path.join(OBJ_DIR, src.replace(".cu", ".ptxas.log"))
        with open(log, "w") as fh:
            fh.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    link = [nvcc, "-ccbin", ccbin, "-shared", "-o", LIB, *objs, "-cudart", "static", "-ldl", "-lpthread"]
    r = subprocess.run(link, capture_output=True, text=True, env=env)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
