"""The benchmark script's contract, as far as it can be checked without a GPU: the
reference arm (OpenBLAS on the host cores, a bounded sample of the workload) prints one JSON
line with the agreed keys, and the library arm refuses to run without a GPU instead of
falling back to the CPU."""
import json
import pathlib
import subprocess
import sys

import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent


def _have_gpu() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def test_reference_arm_prints_the_contract_line():
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step",
                "higher_is_better", "scaling", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["unit"] == "TFLOP/s" and line["dtype"] == "f64" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["cpu_baseline"]["value"] == line["value"] == line["e2e"]["value"]
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert "workload" in line["config"] and "sample" in line["cpu_baseline"]
    assert line.get("gpu_launches", 0) == 0


@pytest.mark.skipif(_have_gpu(), reason="checks the behaviour on a box without a GPU")
def test_library_arm_has_no_cpu_fallback():
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--steps", "1", "--warmup", "0", "--no-cpu"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode != 0
    assert not any(l.startswith("{") for l in res.stdout.splitlines())   # no result line at all
