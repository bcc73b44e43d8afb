"""Compile csrc/*.cu for sm_100a into libglm53f_b200.so, in-tree, with nvcc.

Each source becomes an object under csrc/_obj (rebuilt only when it or a header is newer), then
everything is linked into one shared library beside this file. nvcc cross-compiles without a GPU.
Run as a script, or call build(). Set G5B_PTXAS_V=1 to print register / spill / shared-memory use.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(SRC, "_obj")
OUT = os.path.join(HERE, "libglm53f_b200.so")

NVCC = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
HOST_CXX = shutil.which("g++", path="/usr/bin:/bin") or "g++"
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-ccbin", HOST_CXX, "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    sources = sorted(glob.glob(os.path.join(SRC, "*.cu")))
    headers = (glob.glob(os.path.join(SRC, "*.cuh")) + glob.glob(os.path.join(SRC, "*.h")) +
               glob.glob(os.path.join(HERE, "..", "include", "*.h")) + [os.path.abspath(__file__)])
    flags = list(FLAGS)
    if os.environ.get("G5B_PTXAS_V"):
        flags += ["-Xptxas", "-v"]
    flags += os.environ.get("G5B_NVCC_FLAGS", "").split()      # e.g. -DG5B_STAGE_TIMERS for kernel timers

    def compile_one(src):
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        if _stale(obj, [src] + headers):
            cmd = [NVCC] + flags + ["-c", src, "-o", obj]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
            if verbose or os.environ.get("G5B_PTXAS_V"):
                sys.stderr.write(r.stderr)
        return obj

    with cf.ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(compile_one, sources))
    if _stale(OUT, objs):
        cmd = [NVCC, "-shared", "-ccbin", HOST_CXX, "-o", OUT] + objs + ["-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return OUT


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
