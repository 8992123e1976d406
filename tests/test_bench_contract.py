"""The benchmark's reference arm runs anywhere (it times the CPU port of the reference's expert path): its JSON line must
carry the contract's keys, and the GPU arm must refuse to run without a GPU instead of falling back."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_contract_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                       cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["impl"] == "reference" and d["metric"] == "moe_expert_ffn_tokens_per_s_per_layer" and d["unit"] == "tokens/s"
    assert d["config"]["workload"] == "decode16" and d["value"] > 0 and d["higher_is_better"] is True and d["vs_baseline"] is None
    assert set(d["cpu_baseline"]) >= {"value", "unit", "cores", "kind", "sample"} and d["cpu_baseline"]["kind"] == "port"
    assert d["e2e"] == dict(value=d["value"], unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0)


def test_gpu_arm_refuses_to_run_without_a_gpu():
    import torch

    if torch.cuda.is_available():
        return
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "1", "--warmup", "3"], cwd=ROOT,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode != 0 and "no CPU path" in (r.stderr + r.stdout)


def test_clock_record_summary_from_fake_samples():
    """The clock record of the JSON line: median SM clock, the maximum, and every throttle reason seen in any sample."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    argv, sys.argv = sys.argv, ["bench.py"]
    try:
        spec.loader.exec_module(bench)
    finally:
        sys.argv = argv
    c = bench.ClockSampler(0)
    assert c.summary()["samples"] == 0 and c.summary()["sm_mhz"] is None
    quiet = ["Not Active"] * 4
    c.rows = [["1965", "1965", "0"] + quiet, ["1410", "1965", "0"] + quiet[:3] + ["Active"], ["1350", "1965", "0"] + quiet,
              ["garbage"]]
    s = c.summary()
    assert s["samples"] == 3 and s["sm_mhz"] == 1410.0 and s["sm_max_mhz"] == 1965.0 and s["reasons"] == ["sw_power_cap"]
