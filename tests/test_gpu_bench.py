"""bench.py end to end on one GPU at reduced sizes: one JSON line with the contract's keys."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*flags):
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *flags], capture_output=True, text=True,
                         timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, res.stdout[-2000:]
    return json.loads(lines[0])


def test_layer_line_has_the_contract_keys_and_a_passing_self_check():
    d = _run("--batch", "4096", "--steps", "3", "--warmup", "3", "--no-baselines", "--cpu-rows", "64",
             "--cpu-ref-rows", "64")
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "roofline", "cpu_baseline", "e2e", "gpu_launches", "clocks",
                "per_rank", "dp_check"):
        assert key in d, key
    assert d["value"] > 0 and d["gpu_launches"] == 4 * 3 and d["dp_check"]["ok"]
    assert d["roofline"]["bound"] == "fp32_issue" and 0 < d["roofline"]["frac"] < 2
    assert d["e2e"]["h2d_bytes_per_step"] == 4096 * 256 * 4 * 2 and d["e2e"]["value"] > 0
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["cpu_baseline"]["value"] > 0
    assert len(d["per_rank"]["rows"]) == 1


@pytest.mark.parametrize("config,flags", [("mnist", ["--steps", "5"]),
                                          ("hqkan", ["--steps", "3", "--hqkan-layers", "2"]),
                                          ("bf16_sweep", ["--steps", "3", "--sweep-widths", "512", "--sweep-reps", "1"])])
def test_other_workloads_print_one_line(config, flags):
    d = _run("--config", config, *flags)
    assert d["value"] > 0 and d["ms_per_step"] > 0 and d["gpu_launches"] > 0
    assert config.split("_")[0] in d["config"]["workload"].lower().replace("-", "_") or config == "hqkan"
