"""Expert-parallel exchange logic (`ep_forward`) with two gloo ranks on CPU and a numpy backend."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_workers(mode, world, tmp_path, port):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "ep_worker.py"), mode, str(tmp_path)]
    res = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    rows = [open(os.path.join(tmp_path, f"ok.{r}")).read().split() for r in range(world)]
    return [[int(v) for v in r] for r in rows]


@pytest.mark.parametrize("mode", ["cpu", "cpu_packed"])
@pytest.mark.parametrize("world", [2, 4])
def test_ep_forward_gloo(world, mode, tmp_path):
    rows = run_workers(mode, world, tmp_path, 29611 + world + (10 if mode == "cpu_packed" else 0))
    # every routed row is received by exactly one rank
    assert sum(r[0] for r in rows) == sum(r[1] for r in rows)
    assert any(r[2] > 0 for r in rows)          # and some rows did cross ranks
