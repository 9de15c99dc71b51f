"""bench.py prints ONE JSON line with the keys the measurement contract names (CPU arm here, GPU arm under -m gpu)."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
BASE_KEYS = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
             "vs_baseline", "dtype", "data", "config", "e2e", "gpu_launches", "cpu_baseline"}


def _one_json_line(cmd, timeout):
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), *cmd], capture_output=True, text=True, timeout=timeout, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1, r.stdout[-2000:]
    return json.loads(lines[0])


def test_reference_arm_line():
    d = _one_json_line(["--impl", "reference", "--steps", "1", "--warmup", "3"], 600)
    assert d["impl"] == "reference" and d["metric"] == "decode_tokens_per_s" and d["unit"] == "tokens/s"
    assert BASE_KEYS <= set(d)
    assert d["value"] > 0 and d["cpu_baseline"]["kind"] in ("reference", "port") and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["value"] == d["value"] and d["e2e"]["h2d_bytes_per_step"] == 0 and d["gpu_launches"] == 0
    assert "workload" in d["config"]


@pytest.mark.gpu
def test_gpu_arm_line(cuda):
    d = _one_json_line(["--steps", "3", "--warmup", "3", "--no-cpu-baseline"], 900)
    assert (BASE_KEYS - {"cpu_baseline"}) | {"clocks", "roofline"} <= set(d)
    assert d["metric"] == "decode_tokens_per_s" and d["n_gpus"] == 1 and d["higher_is_better"] is True and d["scaling"] == "weak"
    assert d["value"] > 1000 and d["gpu_launches"] > 0
    assert d["e2e"]["h2d_bytes_per_step"] > 0 and d["e2e"]["d2h_bytes_per_step"] > 0 and d["e2e"]["value"] != d["value"]
    rf = d["roofline"]
    assert rf["bound"] == "hbm" and rf["unit"] == "GB/s" and abs(rf["frac"] - rf["achieved"] / rf["peak"]) < 1e-9 and rf["traffic"] > 0
    assert set(d["clocks"]) >= {"sm_mhz", "sm_max_mhz", "reasons"}
    # sub-records of the default line: the 512-request job (strong scaling) and the reference's CPU-runnable case
    assert d["dp512"]["scaling"] == "strong" and d["dp512"]["value"] > 1000 and d["dp512"]["config"]["job_seconds"] > 0
    assert d["gpt2_fp32"]["value"] > 100 and d["gpt2_fp32"]["launches_per_token"] > 0 and d["gpt2_fp32"]["roofline"]["frac"] > 0
