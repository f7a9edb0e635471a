"""The bench's reference arm runs on CPU; its line and the config it shares with the product arm are checked here."""
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench_module():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_arm_prints_one_line_with_the_shared_config():
    env = dict(os.environ, SAREK_BENCH_TARGET_S="0.2")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stderr
    lines = [ln for ln in res.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    bench = _bench_module()

    class Args:
        pass

    assert d["config"] == bench.make_config(Args())          # the same dict the product arm prints
    assert d["impl"] == "reference" and d["metric"] == bench.METRIC and d["unit"] == "TFLOP/s" and d["higher_is_better"] is True
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] == d["arm"]["threads"] >= 1
    assert "extrapolated" in d["arm"]["note"] and "extrapolated" in d["cpu_baseline"]["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    # ms_per_step is the time of a full 8192^3 step at the measured rate
    full = 2.0 * 8192 ** 3 / (d["value"] * 1e12) * 1e3
    assert abs(d["ms_per_step"] - full) / full < 1e-6
    assert "3xTF32" not in d["config"]["workload"]


def test_other_ranks_of_the_reference_arm_print_nothing():
    env = dict(os.environ, RANK="1", LOCAL_RANK="1", WORLD_SIZE="2")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, timeout=120, env=env)
    assert res.returncode == 0 and res.stdout.strip() == ""
