"""The reference arm of bench.py runs without a GPU (ruy's own CPU path, built from the reference sources into
oracle/_ref): its JSON line is checked here against the keys and meanings the benchmark contract gives it."""
import json
import os
import subprocess
import sys

import pytest

import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(oracle.reference() is None, reason="the compiled reference is not built here")
def test_reference_arm_prints_one_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1, lines
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "int8_gemm_tops" and d["unit"] == "TOP/s"
    assert d["n_gpus"] == 1 and d["steps"] == 1 and d["warmup"] == 1 and d["higher_is_better"] is True
    assert d["vs_baseline"] is None and d["dtype"] == "int8" and d["data"] == "synthetic"
    # the whole 4096 x 4096 x 8192 mul per step: value = ops / time
    assert d["config"]["workload"] == "c3_i8" and d["config"]["same_config"] is True
    assert d["value"] == pytest.approx(2.0 * 4096 * 4096 * 8192 / (d["ms_per_step"] * 1e-3) / 1e12, rel=1e-6)
    assert d["e2e"] == {"value": d["value"], "unit": "TOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    cb = d["cpu_baseline"]
    assert cb["kind"] == "reference" and cb["value"] == d["value"] and cb["cores"] >= 1 and cb["sample"]


def test_reference_arm_stays_silent_on_other_ranks():
    """Under torch.distributed.run only rank 0 times ruy on the host cores; the other ranks exit 0 without work."""
    env = dict(os.environ, RANK="1", LOCAL_RANK="1", WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29599")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                          "--warmup", "1"], capture_output=True, text=True, timeout=300, cwd=ROOT, env=env)
    assert out.returncode == 0 and out.stdout.strip() == "", (out.stdout[-500:], out.stderr[-500:])


def test_gpu_arm_refuses_to_run_without_a_gpu():
    """No CPU fallback: on a machine without a CUDA device the GPU arm ends with an error instead of a number."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "1", "--warmup", "1"],
                         capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert out.returncode != 0 and out.stdout.strip() == ""
    assert "no CUDA device" in out.stderr and "no CPU fallback" in out.stderr
