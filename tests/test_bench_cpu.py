"""The CPU arm of bench.py (``--impl reference``: the oracle port of the reference's PyTorch path
timed on the host cores) keeps the JSON contract; ranks other than 0 print nothing."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
SMALL = ["--steps", "1", "--warmup", "0", "--ctx", "1024", "--batch", "2", "--heads", "2", "--kv-heads", "2",
         "--token-budget", "256", "--layers", "4"]


def _run(extra_env=None, args=()):
    env = dict(os.environ)
    env.update(extra_env or {})
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", *SMALL, *args],
                          capture_output=True, text=True, env=env, timeout=300)


def test_reference_arm_prints_the_contract_line():
    r = _run()
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "tokens/s" and d["higher_is_better"] is True
    assert d["metric"].startswith("sparse decode attn tokens/s/GPU")
    assert d["value"] > 0 and d["steps"] == 1 and d["gpu_launches"] == 0
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"] and "layer passes" in cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in d["config"] and "model" not in d["config"]
    # tokens/s = sequences / (pass time x layers)
    assert abs(d["value"] - 2 / (d["ms_per_step"] * 1e-3 * 4)) <= 1e-6 * d["value"]


def test_reference_arm_other_ranks_do_no_work():
    r = _run({"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"}, ["--gpus", "2"])
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_presets_select_the_other_configurations():
    r = _run(args=["--preset", "config2", "--ctx", "512"])   # no selector, top-p 0.9
    assert r.returncode == 0, r.stderr[-2000:]
    d = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][0])
    assert "top-p 0.9" in d["config"]["workload"]
