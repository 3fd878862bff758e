"""Build recipe for the checker libraries.  TEST INFRASTRUCTURE ONLY.

* ``oracle/libcpu_moe.so`` : this project's C restatement (``cpu_moe.c``), always built.
* ``oracle/_ref/libref_math.so`` : the reference engine's own host-compilable arithmetic
  headers behind ``ref_shim.cpp``.
* ``oracle/_ref/*.cubin`` / ``libhayate_ref.so`` : the reference engine's MoE CUDA kernels
  compiled unmodified for sm_100a, used on a GPU as a second opinion.

The ``_ref`` outputs are only built when a reference checkout is present (path in the
``DARASK_REFERENCE`` environment variable, with a default for the build container); sources are compiled
from where they lie and never copied.  Machines without the checkout use the prebuilt files.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
# the reference checkout: $DARASK_REFERENCE, else a directory named "reference" beside this repository
REF = Path(os.environ["DARASK_REFERENCE"]) if os.environ.get("DARASK_REFERENCE") else HERE.parent.parent / "reference"
OUT = HERE / "_ref"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _run(cmd):
    print("+", " ".join(str(c) for c in cmd), flush=True)
    subprocess.run([str(c) for c in cmd], check=True)


def _stale(target: Path, *sources: Path) -> bool:
    return not target.exists() or any(s.exists() and s.stat().st_mtime > target.stat().st_mtime for s in sources)


def build_cpu() -> Path:
    src, out = HERE / "cpu_moe.c", HERE / "libcpu_moe.so"
    if _stale(out, src):
        # x86-64-v3 (AVX2, FMA, BMI2) rather than the build host's own instruction set: the library is built in one
        # place and loaded on another machine
        _run(["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-ffp-contract=off", "-shared", "-fPIC",
              "-o", out, src, "-lm"])
    return out


def build_ref(cuda: bool = True) -> bool:
    if not REF.exists():
        return False
    OUT.mkdir(exist_ok=True)
    glm = REF / "engines/hayate/crates/kernels/cu/glm53"
    out = OUT / "libref_math.so"
    if _stale(out, HERE / "ref_shim.cpp"):
        _run(["g++", "-O2", "-std=c++20", "-shared", "-fPIC", f"-I{glm}", "-o", out, HERE / "ref_shim.cpp"])
    if not cuda or shutil.which("nvcc") is None:
        return True
    tsj = REF / "engines/tsumuji/kernels"
    jobs = [
        (OUT / "kogarashi_native.cubin", REF / "engines/kogarashi/kernels/native.cu", []),
        (OUT / "tsumuji_gemv.cubin", tsj / "decode/gemv.cu", [f"-I{tsj / 'include'}"]),
        (OUT / "tsumuji_ops.cubin", tsj / "decode/ops.cu", [f"-I{tsj / 'include'}"]),
        (OUT / "tsumuji_quant.cubin", tsj / "decode/quant.cu", [f"-I{tsj / 'include'}"]),
    ]
    for target, src, inc in jobs:
        if _stale(target, src):
            _run(["nvcc", "-cubin", "-O3", "-std=c++20", *ARCH, *inc, "-o", target, src])
    lib = OUT / "libhayate_ref.so"
    srcs = [glm / n for n in ("ops.cu", "decode.cu", "packed_grouped.cu", "lowbit.cu")]
    if _stale(lib, *srcs):
        # same flags as the reference build (fast math), only the architecture differs
        _run(["nvcc", "-shared", "-O3", "-std=c++20", "--use_fast_math", *ARCH, "-Xcompiler", "-fPIC",
              f"-I{glm}", "-o", lib, *srcs])
    return True


if __name__ == "__main__":
    build_cpu()
    print("reference libraries:", "built" if build_ref("--no-cuda" not in sys.argv) else "no reference checkout")
