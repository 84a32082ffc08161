"""Builds ``libfmb200.so`` in-tree with nvcc for sm_100a (``python -m fastmace_b200.build``).

The tensor-product bodies are regenerated from the coupling tables first. Objects are rebuilt only when a source or
header is newer than them.
"""

from __future__ import annotations

import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

from . import codegen

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libfmb200.so")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
         "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found: the fmb200 CUDA library cannot be built")
    return found


def _newest_header() -> float:
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "generated", "*.cuh"))
    headers.append(os.path.join(os.path.dirname(HERE), "include", "fmb200.h"))
    return max(os.path.getmtime(h) for h in headers)


def _compile(source: str, verbose: bool) -> str:
    obj = os.path.join(BUILD, os.path.basename(source)[:-3] + ".o")
    if os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(source), _newest_header()):
        return obj
    cmd = [_nvcc(), *ARCH, *FLAGS, "-c", source, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    result = subprocess.run(cmd, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed for {source}:\n{result.stdout}\n{result.stderr}")
    if verbose:
        print(result.stderr)
    return obj


def build(verbose: bool = False, force: bool = False) -> str:
    codegen.main()
    os.makedirs(BUILD, exist_ok=True)
    if force:
        for obj in glob.glob(os.path.join(BUILD, "*.o")):
            os.remove(obj)
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objects = list(pool.map(lambda s: _compile(s, verbose), sources))
    if (not os.path.exists(LIB)) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objects):
        cmd = [_nvcc(), *ARCH, "-shared", "-o", LIB, *objects, "-lcudart"]
        result = subprocess.run(cmd, capture_output=True, text=True)
        if result.returncode != 0:
            raise RuntimeError(f"link failed:\n{result.stdout}\n{result.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
