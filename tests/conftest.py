import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def cpu_lib():
    """The C restatement (oracle/cpu_moe.c), built on demand."""
    import ctypes
    from oracle import build_ref
    return ctypes.CDLL(str(build_ref.build_cpu()))


@pytest.fixture(scope="session")
def ref_math():
    """The reference engine's host arithmetic behind oracle/ref_shim.cpp, or skip."""
    import ctypes
    from oracle import build_ref
    try:
        build_ref.build_ref(cuda=False)
    except Exception:
        pass
    path = os.path.join(ROOT, "oracle", "_ref", "libref_math.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref/libref_math.so not built (no reference checkout)")
    lib = ctypes.CDLL(path)
    for name in ("ref_fp8", "ref_bf16", "ref_sigmoid", "ref_swiglu", "ref_expert_add", "ref_scaled_fp8", "ref_nvfp4"):
        getattr(lib, name).restype = ctypes.c_float
    lib.ref_storage.restype = ctypes.c_ulonglong
    lib.ref_stride.restype = ctypes.c_ulonglong
    return lib
