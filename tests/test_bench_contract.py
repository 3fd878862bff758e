"""The reference arm of bench.py (`--impl reference`): runs on the host cores only, so its JSON line can be checked here."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_bench(args, env=None):
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, cwd=ROOT, timeout=900,
                         env=dict(os.environ, **(env or {})))
    assert res.returncode == 0, res.stderr[-2000:]
    return res.stdout


@pytest.mark.parametrize("workload,steps", [("qwen35moe_decode_t1", "4"), ("fp8_prefill", "1"), ("hayate_decode_t8", "3"), ("tsumuji_verify", "1")])
def test_reference_arm_line(workload, steps):
    out = run_bench(["--impl", "reference", "--workload", workload, "--steps", steps, "--warmup", "1"])
    line = json.loads(out.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "MoE layer tokens/s" and line["unit"] == "tokens/s"
    assert line["value"] > 0 and line["higher_is_better"] is True and line["n_gpus"] == 1 and line["vs_baseline"] is None
    assert line["config"]["workload"] == workload
    assert line["steps"] == int(steps) and line["warmup"] == 1          # exactly the steps asked for are timed
    base = line["cpu_baseline"]
    assert base["kind"] == "port" and base["cores"] >= 1 and base["value"] == line["value"] and "oracle/cpu_moe.c" in base["sample"]
    assert {c["cores"] for c in base["thread_counts"]} <= {base["cores"], min(8, base["cores"]), *[c["cores"] for c in base["thread_counts"]]}
    assert line["e2e"] == dict(value=line["value"], unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0)


def test_reference_arm_other_ranks_do_no_work():
    out = run_bench(["--impl", "reference", "--gpus", "2", "--steps", "1"], env=dict(RANK="1", WORLD_SIZE="2", LOCAL_RANK="1"))
    assert out.strip() == ""
