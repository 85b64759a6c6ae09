"""Compile the CUDA kernels of lsa_b200 into one in-tree shared library for sm_100a.

    python latent-sparse-attention_b200/build.py [--force] [--verbose]

Every `csrc/*.cu` is compiled with nvcc (`-gencode arch=compute_100a,code=sm_100a -lineinfo`) and linked into
`lsa_b200/liblsa_b200.so` beside the Python package, so the library travels with the source tree. nvcc
cross-compiles without a GPU.
"""

from __future__ import annotations

import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "build")
LIB_PATH = os.path.join(HERE, "lsa_b200", "liblsa_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math=false",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "-I", os.path.join(ROOT, "include"), "-I", CSRC,
]
FLAGS.remove("--use_fast_math=false")  # fast math stays off: the parity tests need IEEE fp32


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    when = os.path.getmtime(target)
    return any(os.path.getmtime(src) > when for src in sources)


def build(force: bool = False, verbose: bool = False) -> str:
    """Build the library if any source is newer than it; return its path."""
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = sorted(glob.glob(os.path.join(CSRC, "*.cuh"))) + sorted(glob.glob(os.path.join(ROOT, "include", "*.h")))
    os.makedirs(OBJ_DIR, exist_ok=True)
    jobs = []
    for src in sources:
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        if force or _stale(obj, [src, *headers]):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [NVCC, *FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c", src, "-o", obj]
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{done.stdout}\n{done.stderr}")
        return src, done.stderr

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for src, log in pool.map(compile_one, jobs):
            if verbose:
                print(f"== {os.path.basename(src)}\n{log}")
    objects = [os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o") for src in sources]
    if force or jobs or _stale(LIB_PATH, objects):
        cmd = [NVCC, "-shared", "-o", LIB_PATH, *objects, "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xcompiler", "-fPIC", "-lcudart"]
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode != 0:
            raise RuntimeError(f"link failed:\n{done.stdout}\n{done.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
