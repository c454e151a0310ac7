"""A whole Saga training run, unmodified library against the library with the b200opt
optimizer op: same injected initial tensors, same inputs, 20 steps of a small
mixed-precision classifier (three fc layers, fp16 with fp32 master copies) on one GPU.  The loss-scale trajectory must be identical bit
for bit and every trained tensor (read back through Saga's own host tensor access and
tensor files) must agree within 1e-5.  Skipped where the two programs were not built
(they need the Saga checkout at build time: saga_b200/host/e2e/build_saga_e2e.py)."""
import json
import os
import subprocess

import numpy as np
import pytest

from saga_b200 import optimizer as opt

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BUILD = os.path.join(ROOT, "saga_b200", "host", "e2e", "_build")
REF, B200 = os.path.join(BUILD, "saga_parity_ref"), os.path.join(BUILD, "saga_parity_b200")


def _run(exe, *args, gpus=1, **extra_env):
    env = dict(os.environ, SAGA_CUDA_CONTEXTS=str(gpus),
               CUDA_VISIBLE_DEVICES=",".join(map(str, range(gpus))))
    env.update({k: str(v) for k, v in extra_env.items()})
    res = subprocess.run([exe, *map(str, args)], capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith('{"parity"')]
    assert lines, res.stdout[-2000:]
    out = json.loads(lines[-1])
    # what the integrated build reports about itself on stderr (one JSON object per line)
    for ln in res.stderr.splitlines():
        if ln.startswith('{"b200_'):
            for key, val in json.loads(ln).items():
                if val.get("rank", 0) == 0:
                    out[key] = val
    return out


def _same_tensors(dir_a, dir_b, names):
    for name in names:
        a, b = opt.tensor_load(dir_a / name), opt.tensor_load(dir_b / name)
        assert a.shape == b.shape and a.tobytes() == b.tobytes(), f"{name} differs"


@pytest.mark.skipif(not (os.path.exists(REF) and os.path.exists(B200)),
                    reason="end-to-end programs not built (no Saga checkout at build time)")
def test_integrated_build_trains_like_the_unmodified_one(tmp_path):
    steps = 20
    init, out_ref, out_b200 = tmp_path / "init", tmp_path / "ref", tmp_path / "b200"
    _run(REF, "init", init)
    names = sorted(os.listdir(init))
    assert {"fc1-w", "fc2-w", "fc3-w"} <= set(names)
    a = _run(REF, "train", init, out_ref, steps)
    b = _run(B200, "train", init, out_b200, steps)
    assert a["steps"] == b["steps"] == steps
    assert a["scale_bits"] == b["scale_bits"], "loss-scale trajectories differ"
    # the scale moved (x1.02 per clean step from the batch size), i.e. the policy ran
    assert len(set(a["scale_bits"])) == steps
    assert abs(a["loss_mean"] - b["loss_mean"]) <= 1e-4 * max(1.0, abs(a["loss_mean"]))
    assert sorted(os.listdir(out_ref)) == sorted(os.listdir(out_b200)) == names
    moved = []
    for name in names:
        x0 = opt.tensor_load(init / name).astype(np.float64)
        xr = opt.tensor_load(out_ref / name).astype(np.float64)
        xb = opt.tensor_load(out_b200 / name).astype(np.float64)
        assert xr.shape == xb.shape == x0.shape, name
        fin = np.isfinite(xr)
        assert np.array_equal(fin, np.isfinite(xb)), name
        if fin.any():
            rms = np.sqrt(np.mean(xr[fin] ** 2))
            err = np.max(np.abs(xb[fin] - xr[fin]) / (np.abs(xr[fin]) + rms + 1e-30))
            assert err <= 1e-5, (name, err)
        if np.any(xr[fin] != x0[fin]):
            moved.append(name)
    # training changed the weights of every layer
    assert {"fc1-w", "fc2-w", "fc3-w"} <= set(moved), f"training changed only {moved} of {names}"


BUILT = pytest.mark.skipif(not os.path.exists(B200),
                           reason="end-to-end programs not built (no Saga checkout at build time)")


@BUILT
def test_loss_scale_on_the_device_follows_the_host_policy_build(tmp_path):
    """The integrated build with the loss scale kept on the device (the loss-gradient
    kernel reads it through a device pointer, the step kernel applies the policy, and
    CudaProgram::step no longer waits for the stream) against the same build with the
    reference's host-side policy block: 800 batches in ONE Program::run without a single
    tensor read in between, against 800 single-batch runs with the scale read after each.
    The run is long enough for the scale to climb into fp16 overflow and be halved.  The
    per-step log the device keeps must equal the host trajectory bit for bit, and so must
    every trained tensor."""
    steps = 800
    init, out_host, out_dev = tmp_path / "init", tmp_path / "host", tmp_path / "dev"
    _run(B200, "init", init)
    names = sorted(os.listdir(init))
    host = _run(B200, "train", init, out_host, steps)
    dev = _run(B200, "train", init, out_dev, steps, "oneshot", B200OPT_DEVICE_SCALE=1,
               B200OPT_SCALE_LOG=1024, B200OPT_PRINT_SCALE_LOG=1, E2E_LOSS_EVERY=0)
    log = dev["b200_scale_log"]
    assert log["steps"] == steps and len(host["scale_bits"]) == steps
    assert log["scale_bits"] == host["scale_bits"], "device-side scale trajectory differs"
    assert dev["scale_bits"] == host["scale_bits"][-1:]          # Program::getMPS reads it back
    # the policy had something to decide: overflow steps halved the scale
    overflow = [k for k, f in enumerate(log["flags"]) if f[1] or f[2]]
    assert overflow, "no overflow step in the run: the trajectory is a plain x1.02 ramp"
    _same_tensors(out_host, out_dev, names)


@BUILT
@pytest.mark.parametrize("buckets,layout", [(3, "graph"), (2, "reference"), (16, "graph")])
def test_buckets_behind_backward_train_like_the_whole_step(tmp_path, buckets, layout):
    """The optimizer step issued as buckets between the backward ops (side stream, gated
    by events) against the same build with one op behind all of backward: same scale
    trajectory and bit-identical trained tensors, with the flat layout in backward order
    and in the reference's order."""
    steps = 60
    init, out_whole, out_b = tmp_path / "init", tmp_path / "whole", tmp_path / "buckets"
    _run(B200, "init", init)
    names = sorted(os.listdir(init))
    whole = _run(B200, "train", init, out_whole, steps)
    bucketed = _run(B200, "train", init, out_b, steps, B200OPT_BUCKETS=buckets,
                    B200OPT_LAYOUT=layout, B200OPT_PRINT_PLAN=1)
    plan = bucketed["b200_bucket_plan"]["buckets"]
    assert 2 <= len(plan) <= min(buckets, 6)       # six trainable tensors in this model
    # consecutive ranges that cover the fp16 buffer; issue points never move backwards
    at = 0
    for b in plan:
        assert b["half"][0] == at
        at += b["half"][1]
    assert [b["after_op"] for b in plan] == sorted(b["after_op"] for b in plan)
    if layout == "graph":       # the first bucket goes out well before backward ends
        assert plan[0]["after_op"] < bucketed["b200_bucket_plan"]["ops"] - 1
    assert bucketed["scale_bits"] == whole["scale_bits"]
    _same_tensors(out_whole, out_b, names)


@BUILT
@pytest.mark.multigpu
def test_buckets_on_two_gpus_train_like_the_whole_step(tmp_path):
    """Two ranks (one host thread per GPU, Saga's threading model): every bucket's kernel
    waits for the peer's same bucket, reduces both ranks' gradients and writes the weights
    into both ranks' buffers while the rest of backward is still running.  Same layout,
    so the shards and with them the per-shard flags are the same: bit-identical result."""
    steps = 40
    init, out_whole, out_b = tmp_path / "init", tmp_path / "whole", tmp_path / "buckets"
    _run(B200, "init", init)
    names = sorted(os.listdir(init))
    whole = _run(B200, "train", init, out_whole, steps, gpus=2)
    bucketed = _run(B200, "train", init, out_b, steps, gpus=2, B200OPT_BUCKETS=3,
                    B200OPT_LAYOUT="reference")
    assert whole["ranks"] == bucketed["ranks"] == 2
    assert bucketed["scale_bits"] == whole["scale_bits"]
    _same_tensors(out_whole, out_b, names)
    # backward order moves tensors between the two shards; results stay the same as long
    # as no range flag is raised (the x0.9 rule counts shards), which 40 steps do not reach
    graph = _run(B200, "train", init, tmp_path / "graph", steps, gpus=2, B200OPT_BUCKETS=3)
    assert graph["scale_bits"] == whole["scale_bits"]
    _same_tensors(out_whole, tmp_path / "graph", names)


@BUILT
@pytest.mark.multigpu
def test_loss_scale_on_the_device_two_gpus(tmp_path):
    steps = 300
    init, out_host, out_dev = tmp_path / "init", tmp_path / "host", tmp_path / "dev"
    _run(B200, "init", init)
    names = sorted(os.listdir(init))
    host = _run(B200, "train", init, out_host, steps, gpus=2)
    dev = _run(B200, "train", init, out_dev, steps, "oneshot", gpus=2, B200OPT_DEVICE_SCALE=1,
               B200OPT_SCALE_LOG=512, B200OPT_PRINT_SCALE_LOG=1, E2E_LOSS_EVERY=0)
    assert dev["b200_scale_log"]["scale_bits"] == host["scale_bits"]
    _same_tensors(out_host, out_dev, names)


@pytest.mark.skipif(not (os.path.exists(REF) and os.path.exists(B200)),
                    reason="end-to-end programs not built (no Saga checkout at build time)")
@pytest.mark.multigpu
def test_two_gpu_integrated_build_tracks_the_unmodified_one(tmp_path):
    """Two ranks, unmodified library (NCCL reduce-scatter / all-gather, fp16 ring sum)
    against the integrated one (rank-ordered fp32 sum, one rounding).  The sums differ in
    the last fp16 bit here and there, so this is a tolerance check: no overflow step in
    either build (identical scale trajectory), the same mean loss and trained tensors
    within 1e-2 of each other."""
    steps = 40
    init, out_ref, out_b200 = tmp_path / "init", tmp_path / "ref", tmp_path / "b200"
    _run(REF, "init", init)
    names = sorted(os.listdir(init))
    a = _run(REF, "train", init, out_ref, steps, gpus=2)
    b = _run(B200, "train", init, out_b200, steps, gpus=2)
    assert a["ranks"] == b["ranks"] == 2
    assert a["scale_bits"] == b["scale_bits"] and len(set(a["scale_bits"])) == steps
    assert abs(a["loss_mean"] - b["loss_mean"]) <= 2e-3 * max(1.0, abs(a["loss_mean"]))
    for name in names:
        xr = opt.tensor_load(out_ref / name).astype(np.float64)
        xb = opt.tensor_load(out_b200 / name).astype(np.float64)
        assert np.isfinite(xr).all() and np.isfinite(xb).all(), name
        rms = np.sqrt(np.mean(xr ** 2))
        assert np.max(np.abs(xb - xr)) <= 1e-2 * (np.max(np.abs(xr)) + rms), name
