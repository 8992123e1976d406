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


def _load_bench():
    import importlib.util

    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    argv, sys.argv = sys.argv, ["bench.py"]
    try:
        spec.loader.exec_module(bench)
    finally:
        sys.argv = argv
    return bench


def test_config_statistics_and_traffic_record():
    """`config` names the workload only and is what both arms print; a sample set is reported as median / min / max /
    mean; the traffic of the roofline is read from the record next to the profiler summaries, not typed into the script."""
    bench = _load_bench()
    for name in ("decode16", "verify128", "prefill8k", "prefill64k"):
        c = bench.workload_config(name)
        assert c["workload"] == name and c["tokens"] == bench.WORKLOADS[name]["tokens"] and c["top_k"] == 8
        assert "parallelism" not in c and "model" not in c
    assert bench.workload_config("verify128")["routing"] == "zipf1.2" and bench.workload_config("decode16")["routing"] == "uniform"
    s = bench.stats([3.0, 1.0, 2.0, 10.0, 4.0])
    assert s == dict(median=3.0, min=1.0, max=10.0, mean=4.0, samples=5)
    t = bench.profiled_traffic()
    assert t["decode16"]["fc1_dram_bytes"] > 9e8 and "profiles/" in t["decode16"]["source"] and t["prefill8k"]["fc1_dram_bytes"] > 2e9
    src = open(os.path.join(ROOT, "bench.py")).read()
    assert "915809536" not in src and "2774330624" not in src
    assert bench.identity(type("A", (), {})())["seed"] == "0x26afd"


def _ranks_worker(rank, world, port, q):
    import torch
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    bench = _load_bench()
    ctx = object.__new__(bench.Ctx)
    ctx.dev, ctx.rank, ctx.world = torch.device("cpu"), rank, world
    per, spread = ctx.over_ranks([1.0 + rank, 5.0 - 2 * rank, 2.0])          # rank 0: 1, 5, 2; rank 1: 2, 3, 2
    ok_all = ctx.all_true(True)
    ok_one = ctx.all_true(rank == 0)
    q.put((rank, per, spread, ok_all, ok_one))
    dist.barrier()
    dist.destroy_process_group()


def test_sample_time_is_the_maximum_over_ranks_and_parity_needs_every_rank():
    """Two gloo ranks: a sample's time is the slowest rank's, the spread is the median difference between ranks, and a
    parity flag is true only when every rank says so."""
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_ranks_worker, args=(r, 2, 29731, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=300) for _ in range(2))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, per, spread, ok_all, ok_one in got:
        assert per == [2.0, 5.0, 2.0] and spread == 1.0 and ok_all is True and ok_one is False
