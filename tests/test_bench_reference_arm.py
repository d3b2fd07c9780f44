"""The benchmark's reference arm on CPU: `bench.py --impl reference` times the oracle on a bounded sample and prints one
JSON line with the keys the measurement contract names; under a multi-rank launch only rank 0 prints."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KEYS = {"impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
        "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e", "gpu_launches"}


def _run(extra, env=None):
    cmd = [sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0",
           "--cpu-sample-elements", "300000"] + extra
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    return [json.loads(line) for line in r.stdout.splitlines() if line.startswith("{")]


def _check(line, n_gpus):
    assert KEYS <= set(line), sorted(KEYS - set(line))
    assert line["impl"] == "reference" and line["metric"] == "folded_weight_GBps" and line["unit"] == "GB/s"
    assert line["n_gpus"] == n_gpus and line["higher_is_better"] is True and line["gpu_launches"] == 0
    assert line["value"] > 0 and line["ms_per_step"] > 0 and line["vs_baseline"] is None
    cpu = line["cpu_baseline"]
    assert cpu["kind"] == "port" and cpu["cores"] >= 1 and cpu["value"] == line["value"] and cpu["sample"]
    e2e = line["e2e"]
    assert e2e["value"] == line["value"] and e2e["unit"] == "GB/s" and e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0
    assert "workload" in line["config"] and "model" not in line["config"]


def test_reference_arm_prints_the_contract_line():
    lines = _run(["--layers", "1"])
    assert len(lines) == 1
    _check(lines[0], 1)
    small = _run(["--workload", "cfg3", "--instances", "1"])
    assert len(small) == 1
    _check(small[0], 1)


def test_reference_arm_under_a_two_rank_launch_prints_once(tmp_path):
    out = []
    procs = []
    for rank in (0, 1):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29631")
        cmd = [sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0",
               "--cpu-sample-elements", "300000", "--layers", "1"]
        procs.append(subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, cwd=ROOT, env=env))
    for p in procs:
        so, se = p.communicate(timeout=300)
        assert p.returncode == 0, se[-2000:]
        out.append([json.loads(line) for line in so.splitlines() if line.startswith("{")])
    assert len(out[0]) == 1 and out[1] == []
    _check(out[0][0], 2)
