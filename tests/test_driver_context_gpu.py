"""The library inside a Driver-API host, as the reference's engines are.

The reference's hosts never touch the runtime API: they retain the primary context with `cuDevicePrimaryCtxRetain`,
allocate with `cuMemAlloc`, create `CU_STREAM_NON_BLOCKING` streams and launch cubin functions with `cuLaunchKernelEx`
(common/cuda/src/lib.rs:57-76, 130-145, 351-380, 395-402). This library is runtime-API code in a shared object; the
test runs it in a fresh process that set up its context, memory and stream that way, on driver-allocated pointers."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_runs_in_a_driver_api_context():
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    res = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "driver_context_child.py")], capture_output=True, text=True, cwd=ROOT, env=env,
                         timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    report = json.loads(res.stdout.strip().splitlines()[-1])
    for tokens in ("1", "3"):            # one token: the single persistent launch; three: the staged launches
        assert report[tokens]["status"] == 0
        assert report[tokens]["ids_equal"]
        assert report[tokens]["rel_l2"] <= 1e-3
