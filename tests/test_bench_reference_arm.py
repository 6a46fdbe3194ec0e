"""The reference arm of bench.py runs on host cores only, so its contract is checked here without a GPU: one JSON
line per workload with the keys the driver reads."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KEYS = {"impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
        "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e", "gpu_launches"}


@pytest.mark.parametrize("workload,metric,unit", [
    ("q4k_gemv_4096", "q4k_gemv_gbs", "GB/s"),
    ("q4k_gemm_prefill", "q4k_gemm_tflops", "TFLOP/s"),
    ("q8_0_batch32", "q8_0_batch32_gbs", "GB/s"),
    ("mxfp4_moe_gptoss", "mxfp4_moe_layers_per_s", "layers/s"),
    ("llama8b_q4k_decode", "decode_tok_s", "tok/s"),
])
def test_reference_arm_prints_the_contract_line(workload, metric, unit):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", workload,
                          "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert KEYS <= set(line), KEYS - set(line)
    assert line["impl"] == "reference" and line["metric"] == metric and line["unit"] == unit
    assert line["value"] > 0 and line["gpu_launches"] == 0 and line["vs_baseline"] is None
    cb = line["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["sample"] and cb["value"] == line["value"]
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["config"]["workload"] == workload


def test_reference_arm_is_silent_on_other_ranks():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, timeout=120, cwd=ROOT, env=env)
    assert out.returncode == 0 and not [l for l in out.stdout.splitlines() if l.startswith("{")]
