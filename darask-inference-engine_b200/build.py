"""Builds libdarask_moe_b200.so (and the drop-in cubins) for sm_100a with nvcc, in-tree.

    python darask-inference-engine_b200/build.py [--force]

Every translation unit under csrc/ is compiled with
``-gencode arch=compute_100a,code=sm_100a -lineinfo``; ``hayate.cu`` additionally with
``--use_fast_math`` (the reference builds its GLM kernels that way and the router selection
has to round the same way).
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "build"
LIB = HERE / "libdarask_moe_b200.so"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
EXTRA = {"hayate.cu": ["--use_fast_math"]}


def _nvcc() -> str:
    for c in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if c and (os.path.isabs(c) and os.path.exists(c) or not os.path.isabs(c)):
            return c
    return "nvcc"


def _newest(paths) -> float:
    return max((p.stat().st_mtime for p in paths if p.exists()), default=0.0)


def build(force: bool = False, verbose: bool = True) -> Path:
    sources = sorted(CSRC.glob("*.cu"))
    headers = list(CSRC.glob("*.cuh")) + list((HERE.parent / "include").glob("*.h"))
    OBJ.mkdir(exist_ok=True)
    jobs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, _newest(headers)):
            jobs.append([_nvcc(), *ARCH, *COMMON, *EXTRA.get(src.name, []), "-c", str(src), "-o", str(obj)])

    def run(cmd):
        if verbose:
            print("+", " ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        list(pool.map(run, jobs))
    objs = [OBJ / (s.stem + ".o") for s in sources]
    if jobs or not LIB.exists() or LIB.stat().st_mtime < _newest(objs):
        run([_nvcc(), *ARCH, "-shared", "-o", str(LIB), *map(str, objs), "-lcudart"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
