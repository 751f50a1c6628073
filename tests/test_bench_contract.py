"""bench.py prints one JSON line with the agreed keys: the CPU arm runs anywhere, the GPU arm on a B200."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
COMMON = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
          "vs_baseline", "dtype", "data", "config", "e2e", "gpu_launches"}


def _run(*args, timeout=600):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, r.stdout[-2000:]
    return json.loads(lines[0])


def test_reference_arm_line():
    d = _run("--impl", "reference", "--config", "cfg1", "--steps", "2", "--warmup", "1")
    assert COMMON <= set(d) and d["impl"] == "reference"
    assert d["unit"] == "edges/s" and d["value"] > 0 and d["higher_is_better"] is True
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["cpu_baseline"]["cores"] == 1
    assert d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["config"]["workload"].startswith("cfg1") and d["gpu_launches"] == 0


def test_both_arms_describe_the_workload_identically():
    """The `config` object is built by one function from the workload alone (knobs and the partition are
    reported under other keys), so the two arms' lines can be compared key for key."""
    import ast
    src = open(os.path.join(ROOT, "bench.py")).read()
    calls = [n for n in ast.walk(ast.parse(src)) if isinstance(n, ast.Call) and getattr(n.func, "id", "") == "workload_config"]
    assert len(calls) == 2 and all(len(c.args) == 7 and not c.keywords for c in calls)
    sys.path.insert(0, ROOT)
    import bench
    a = type("A", (), {"config": "cfg2", "scale": 1.0})()
    c = bench.workload_config(a, 10, 20, {"kind": "x"}, 602, 16, 41)
    assert set(c) == {"workload", "nodes", "edges", "in_dim", "aggregated_width", "classes", "graph", "partition", "l2_policy"}


def test_reference_arm_sets_its_thread_count_at_run_time(monkeypatch):
    """Under torchrun every rank inherits OMP_NUM_THREADS=1; the CPU arm must still use the cores it
    reports: the oracle's thread count is set through the OpenMP runtime and read back."""
    env = dict(os.environ, OMP_NUM_THREADS="1", WORLD_SIZE="2", RANK="0", LOCAL_RANK="0")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--config", "cfg1", "--gpus", "2",
                        "--steps", "1", "--warmup", "1"], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    d = json.loads([ln for ln in r.stdout.splitlines() if ln.startswith("{")][0])
    cores = len(os.sched_getaffinity(0))
    assert d["cpu_baseline"]["omp_threads_dense_softmax"] == cores
    # the other ranks print nothing and exit 0
    env["RANK"] = "1"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--config", "cfg1", "--gpus", "2"],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_gpu_arm_needs_a_gpu_or_runs():
    import torch
    if torch.cuda.is_available():
        pytest.skip("covered by the gpu-marked test")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--config", "cfg1"], capture_output=True, text=True, timeout=300)
    assert r.returncode != 0 and "no CPU path" in (r.stdout + r.stderr)


@pytest.mark.gpu
def test_gpu_arm_line():
    d = _run("--config", "cfg1", "--steps", "5", "--warmup", "3")
    assert COMMON | {"roofline", "cpu_baseline", "clocks"} <= set(d) and "impl" not in d
    assert d["n_gpus"] == 1 and d["warmup"] >= 3 and d["steps"] == 5 and d["data"] == "synthetic" and d["dtype"] == "f32"
    rf = d["roofline"]
    assert rf["bound"] in ("hbm", "l1tex", "nvlink") and rf["unit"] == "GB/s" and rf["peak"] > 1000 and abs(rf["frac"] - rf["achieved"] / rf["peak"]) < 1e-9
    assert d["e2e"]["h2d_bytes_per_step"] == d["config"]["nodes"] * 16 * 4 and d["e2e"]["d2h_bytes_per_step"] > 0
    assert d["e2e"]["value"] != d["value"] and d["gpu_launches"] == 5 * 1      # no row of this graph reaches the hub threshold: one kernel per pass
    assert d["check"]["pass"] is True and d["check"]["rows"] == d["config"]["nodes"] and d["check"]["worst_over_tol"] <= 1.0
    assert d["repeats"] == 5 and d["roofline"]["bound_kind"] and d["roofline"]["frac_dram"] > 0
    assert d["cpu_baseline"]["value"] > 0 and "sample" in d["cpu_baseline"]
    assert d["clocks"]["sm_max_mhz"] and isinstance(d["clocks"]["reasons"], list)


@pytest.mark.gpu
def test_config5_shard_local_path_small():
    """Config 5's code path (shard-local graph, 64-bit row pointers, 128-16-172 GCN) at 1/16384 scale."""
    d = _run("--config", "cfg5", "--scale", "0.00006", "--steps", "3", "--warmup", "3")
    assert d["config"]["workload"].startswith("cfg5") and d["config"]["nodes"] == 111_000_000 >> 15
    assert d["config"]["classes"] == 172 and d["value"] > 0 and "cpu_baseline" not in d
    assert d["check"]["pass"] is True and d["check"]["rows"] > 0 and "stage by stage" in d["check"]["kind"]


def test_no_collective_is_called_by_rank_zero_alone():
    """A collective inside an ``if rank == 0:`` block deadlocks every multi-GPU run (the other ranks
    never join it).  Checked on the source: bench.py's collective helpers and torch.distributed calls
    must not appear under a rank test."""
    import ast
    src = open(os.path.join(ROOT, "bench.py")).read()
    collectives = {"sum_over_ranks", "max_over_ranks", "reduce_over_ranks", "sync_all", "all_reduce", "all_gather", "barrier", "broadcast",
                   "all_gather_object", "all_gather_into_tensor", "forward", "forward_host", "sampled_stage_check_gcn2", "status",
                   "SymmetricBuffer", "ReplicaBuffer", "FlagBarrier", "close"}

    def mentions_rank(test):
        return any(isinstance(n, ast.Name) and n.id in ("rank", "local_rank") for n in ast.walk(test))

    bad = []
    for node in ast.walk(ast.parse(src)):
        if isinstance(node, ast.If) and mentions_rank(node.test):
            for sub in node.body + node.orelse:
                for call in ast.walk(sub):
                    if isinstance(call, ast.Call):
                        f = call.func
                        name = f.id if isinstance(f, ast.Name) else f.attr if isinstance(f, ast.Attribute) else ""
                        if name in collectives:
                            bad.append((name, call.lineno))
    assert not bad, f"collective under a rank test: {bad}"
