"""The benchmark's contract, as far as it can be checked without a GPU: the reference arm (the CPU restatement of the
reference's attention on the host cores) prints one JSON line with the keys the driver reads, and the GPU arm fails
loudly -- it does not fall back to the CPU -- when there is no GPU."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, timeout=600):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], cwd=ROOT, capture_output=True, text=True,
                          timeout=timeout)


def test_reference_arm_prints_the_contract_line():
    r = _run("--impl", "reference", "--steps", "1", "--warmup", "0")
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "e2e", "cpu_baseline"):
        assert key in line, key
    assert line["metric"] == "prefill_attn_tflops" and line["unit"] == "TFLOP/s" and line["value"] > 0
    assert line["e2e"]["value"] == line["value"] and line["e2e"]["h2d_bytes_per_step"] == 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert "workload" in line["config"] and "model" not in line["config"]


def test_unknown_leg_is_refused():
    r = _run("--legs", "prefill,nonsense", timeout=120)
    assert r.returncode != 0 and "unknown legs" in r.stderr


def test_gpu_arm_fails_loudly_without_a_gpu():
    try:
        import ctypes
        ctypes.CDLL("libcuda.so.1")
        pytest.skip("a CUDA driver is present: the GPU arm would run")
    except OSError:
        pass
    r = _run("--legs", "prefill", "--steps", "1", "--warmup", "0", timeout=300)
    assert r.returncode != 0
    assert r.stdout.strip() == "" or "value" not in r.stdout        # no benchmark line is printed from a CPU fallback
