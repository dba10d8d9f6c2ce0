"""bench.py on the host: the JSON line of the host-core arm (`--impl reference`) on the small workload, what the ranks
other than 0 do under a multi-process launch, and the clock sampler's summary of nvidia-smi rows.  No GPU needed."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(extra_env=None, *args):
    env = dict(os.environ, **(extra_env or {}))
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], cwd=ROOT, env=env, capture_output=True,
                         text=True, timeout=600)
    return out


def test_reference_arm_prints_one_contract_line():
    out = _run(None, "--impl", "reference", "--workload", "tiny", "--steps", "2", "--warmup", "3")
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "decode_tok_per_s" and d["unit"] == "tok/s"
    assert d["n_gpus"] == 1 and d["steps"] == 2 and d["warmup"] == 3 and d["higher_is_better"] is True
    assert d["scaling"] == "weak" and d["vs_baseline"] is None and d["data"] == "synthetic" and d["dtype"] == "bf16"
    assert d["config"]["workload"] == "tiny" and "model" not in d["config"]
    assert d["value"] > 0 and abs(d["value"] - d["config"]["cpu_sample_batch"] / (d["ms_per_step"] * 1e-3)) < 1e-6 * d["value"]
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"] and "requests per step" in cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["gpu_launches"] == 0


def test_reference_arm_runs_on_rank_zero_only():
    """Under a multi-process launch the other ranks leave at once, without output."""
    out = _run({"RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2"}, "--impl", "reference", "--workload", "tiny",
               "--gpus", "2", "--steps", "2", "--warmup", "3")
    assert out.returncode == 0, out.stderr[-2000:]
    assert not [l for l in out.stdout.splitlines() if l.startswith("{")]


def test_clock_summary_parses_rows_and_windows():
    sys.path.insert(0, ROOT)
    import bench
    cs = bench.ClockSampler(0)
    cs.rows = [(10.0, ["1965", "1965", "Not Active", "Not Active", "Not Active", "Not Active"]),
               (10.1, ["1800", "1965", "Not Active", "Not Active", "Not Active", "Active"]),
               (10.2, ["[N/A]", "1965", "Not Active", "Not Active", "Not Active", "Not Active"]),     # skipped
               (10.3, ["1200", "1965", "Not Active", "Active", "Not Active", "Not Active"]),
               (11.0, ["1965", "1965", "Not Active", "Not Active", "Not Active", "Not Active"])]
    every = cs.summary()
    assert every == {"sm_mhz": 1965, "sm_max_mhz": 1965, "reasons": ["hw_thermal_slowdown", "sw_power_cap"], "samples": 4}
    window = cs.summary(10.05, 10.15)
    assert window == {"sm_mhz": 1800, "sm_max_mhz": 1965, "reasons": ["sw_power_cap"], "samples": 1}
    assert cs.summary(20.0, 21.0) == {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}


import pytest  # noqa: E402


@pytest.mark.gpu
def test_native_arm_line_on_the_small_workload():
    """The whole default flow on a small model: one JSON line with the keys the contract names."""
    out = _run(None, "--workload", "tiny", "--steps", "8", "--warmup", "3", "--cpu-steps", "2")
    assert out.returncode == 0, out.stderr[-3000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["metric"] == "decode_tok_per_s" and d["unit"] == "tok/s" and d["n_gpus"] == 1 and d["steps"] == 8
    assert d["higher_is_better"] is True and d["scaling"] == "weak" and d["data"] == "synthetic" and d["dtype"] == "bf16"
    assert d["config"]["workload"] == "tiny" and d["value"] > 0 and d["gpu_launches"] > 0
    r = d["roofline"]
    assert r["bound"] == "hbm" and r["unit"] == "GB/s" and r["peak"] > 0 and abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-9
    e = d["e2e"]
    assert e["value"] > 0 and e["h2d_bytes_per_step"] > 0 and e["d2h_bytes_per_step"] > 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["value"] > 0
    assert d["evict"] is not None and d["evict"]["frac"] > 0          # an eviction falls inside the window
    assert d["evict_micro"]["frac"] > 0 and d["append"]["frac"] > 0
    assert set(d["clocks"]) >= {"sm_mhz", "sm_max_mhz", "reasons", "samples"}


@pytest.mark.gpu
@pytest.mark.parametrize("argv", [
    ["--micro", "evict", "--nseg", "16", "--M", "256", "--no-cpu-baseline"],
    ["--micro", "evict", "--nseg", "16", "--M", "256", "--ctas", "4", "--no-cpu-baseline"],
    ["--micro", "append", "--nseg", "64", "--M", "256", "--no-cpu-baseline"],
    ["--micro", "steady", "--nseg", "64", "--M", "256", "--ctas", "4"],
    ["--micro", "attn", "--nseg", "64"],
    ["--micro", "attn", "--nseg", "64", "--token-bound"],
    ["--micro", "attn", "--nseg", "64", "--packed"],
    ["--micro", "attn", "--attn-shape", "config2", "--nseg", "32"],
    ["--micro", "multi", "--nseg", "16", "--M", "256", "--q-tokens", "16"],
    ["--micro", "prefill", "--nseg", "8", "--M", "512"],
])
def test_every_microbenchmark_runs_and_prints_a_line(argv, capsys):
    """Small sizes: what is checked is that each microbenchmark of bench.py still runs and prints one JSON line."""
    sys.path.insert(0, ROOT)
    import bench
    bench.run_micro(bench.parse_args(argv + ["--steps", "3", "--warmup", "3"]))
    lines = [l for l in capsys.readouterr().out.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["micro"] == argv[1]
    times = [v for k, v in d.items() if k in ("avg_ms", "avg_ms_per_step", "query_resident_ms")]
    assert times and all(t > 0 for t in times)
