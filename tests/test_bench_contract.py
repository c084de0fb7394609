"""The parts of bench.py that need no GPU: the workload table against BASELINE.json's configurations, the partitioning
of cfg5 over ranks, the `config` object (identical for the b200 arm and the reference arm, so that the two lines
describe one workload), and the reference arm's JSON line."""
import importlib.util
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def bench(built_libs):
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_workloads_are_the_baseline_configurations(bench):
    w = bench.WORKLOADS
    assert bench.DEFAULT_WORKLOAD == "cfg5"
    assert (w["cfg2"]["m"], w["cfg2"]["n"], w["cfg2"]["k"], w["cfg2"]["k_split"]) == (4096, 4096, 4160, 4096)
    assert (w["cfg3"]["m"], w["cfg3"]["n"], w["cfg3"]["k"]) == (16, 14336, 4096)
    assert (w["cfg4"]["m"], w["cfg4"]["dtype"], w["cfg4"]["scales"]) == (8192, "fp8", True)
    for name in ("cfg5", "cfg5_nshard", "cfg5_kshard", "cfg5_kshard_fused", "cfg5_kshard_fused_bf16"):
        assert (w[name]["m"], w[name]["n"], w[name]["k"], w[name]["seed"]) == (16384, 28672, 8192, 4)
    assert set(bench.ALSO_ONE_GPU) == {"cfg2", "cfg3", "cfg4"}
    assert set(bench.ALSO_MULTI_GPU) == {"cfg5_kshard", "cfg5_kshard_fused", "cfg5_kshard_fused_bf16"}


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_cfg5_partitions_cover_the_problem(bench, world):
    w = bench.WORKLOADS["cfg5"]
    cols = [bench.shard_shape("cfg5", w, r, world) for r in range(world)]
    assert sum(s["n"] for s in cols) == w["n"] and all(s["n"] % 256 == 0 and s["m"] == w["m"] and s["k"] == w["k"] for s in cols)
    assert all(s["scaling"] == "strong" and s["job_flops"] == 2.0 * w["m"] * w["n"] * w["k"] for s in cols)
    ks = [bench.shard_shape("cfg5_kshard_fused", bench.WORKLOADS["cfg5_kshard_fused"], r, world) for r in range(world)]
    assert sum(s["k"] for s in ks) == w["k"] * (1 if world > 1 else 1) and all(s["n"] == w["n"] for s in ks)
    if world > 1:
        assert [s["lo"] for s in cols] == [sum(c["n"] for c in cols[:r]) for r in range(world)]
        assert bench.partition("cfg5", world) == "n" and bench.partition("cfg5_kshard", world) == "k"
        assert bench.partition("cfg2", world) == "panel" and bench.shard_shape("cfg2", bench.WORKLOADS["cfg2"], 0, world)["scaling"] == "weak"


def test_rows_to_check_hold_the_edges(bench):
    rows = bench.rows_to_check(16384, 256, 64, 17)
    assert rows[0] == 0 and rows[-1] == 16383 and 255 in rows and 256 in rows and len(rows) <= 64
    assert bench.rows_to_check(16, 128, 8, 1) == sorted(set(bench.rows_to_check(16, 128, 8, 1)))  # clipped, no duplicates
    assert max(bench.rows_to_check(16, 128, 8, 1)) == 15


def test_config_object_needs_no_gpu_and_names_the_kernel(bench):
    c1 = bench.config_dict("cfg5", bench.WORKLOADS["cfg5"], 1)
    assert c1["per_gpu"] == [16384, 28672, 8192] and c1["parallelism"] == "single GPU" and "pair=1" in c1["kernel"]
    c8 = bench.config_dict("cfg5", bench.WORKLOADS["cfg5"], 8)
    assert c8["per_gpu"] == [16384, 3584, 8192] and "n-sharded x8" in c8["parallelism"] and set(c8) == set(c1)
    c2 = bench.config_dict("cfg2", bench.WORKLOADS["cfg2"], 1)
    assert c2["loop_split"]["tail_iters"] == 1 and c2["loop_split"]["main_iters"] * 64 in (4096, 2048)  # main [0, 4096), one remainder block


def test_reference_arm_line(bench):
    """`--impl reference` on the smallest workload: one JSON line, the contract's keys, the same config object."""
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "cfg3",
                          "--steps", "1", "--warmup", "1"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "impl", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["value"] > 0 and line["vs_baseline"] is None
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["config"] == bench.config_dict("cfg3", bench.WORKLOADS["cfg3"], 1)
