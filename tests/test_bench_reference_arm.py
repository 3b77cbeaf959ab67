"""`bench.py --impl reference` (the CPU oracle timed on the host cores) prints one well-formed JSON line for
both workloads without touching a GPU."""
import json
import subprocess
import sys

import pytest

from tests.conftest import ROOT


@pytest.mark.parametrize("workload", [None, "llama8b", "qwen3moe"])
def test_reference_arm_line(workload):
    cmd = [sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"]
    if workload:
        cmd += ["--workload", workload]
    else:
        workload = "qwen3moe"      # the default line is the expert-sharded model's
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=str(ROOT))
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "decode_tok_s" and line["unit"] == "tok/s"
    assert line["value"] > 0 and line["higher_is_better"] is True and line["extrapolated"] is True
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["config"]["workload"].startswith(workload.replace("llama8b", "llama8b_q4k"))
