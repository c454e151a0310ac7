"""bench.py's reference arm needs no GPU (it times the CPU restatement on the host cores),
so its line is checked here: the keys the driver reads, the same `config` the product arm
prints, rank 0 alone doing the work under a multi-rank launch, and no product library in
the process."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args, env_extra=None):
    env = dict(os.environ)
    env.update(env_extra or {})
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args],
                          capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)


def test_reference_arm_line(oracle):
    res = _run(["--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1"])
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["n_gpus"] == 1 and d["steps"] == 2
    assert d["unit"] == "params/s" and d["higher_is_better"] is True and d["vs_baseline"] is None
    assert d["value"] > 0 and abs(d["value"] - d["config"]["n_params"] / (d["ms_per_step"] * 1e-3)) \
        <= 1e-6 * d["value"]
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": "params/s", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0}
    # warmed by time as well as by count
    assert d["warmup"] >= 10
    # the same workload description as the product arm prints
    sys.path.insert(0, ROOT)
    import bench
    assert d["metric"] == bench.METRIC
    assert d["config"] == bench.base_config(d["config"]["n_params"], d["config"]["tensors"])
    assert d["config"]["n_params"] == 25601168 and d["config"]["tensors"] == 160


def test_reference_arm_other_ranks_do_nothing():
    res = _run(["--impl", "reference", "--gpus", "2", "--steps", "2", "--warmup", "1"],
               {"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"})
    assert res.returncode == 0 and res.stdout.strip() == ""


def test_reference_arm_source_keeps_the_product_out():
    """The arm may execute the oracle, never the product: its function imports neither the
    package nor torch (the workload generators are loaded by file path)."""
    src = open(os.path.join(ROOT, "bench.py")).read()
    start = src.index("def run_reference_arm(args):")
    body = src[start:src.index("\ndef ", start + 10)]
    assert "import torch" not in body and "saga_b200 import" not in body and "capi" not in body
    assert "from oracle import oracle" in body and "workload_module()" in body
