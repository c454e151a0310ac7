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


def _run(exe, *args):
    env = dict(os.environ, SAGA_CUDA_CONTEXTS="1", CUDA_VISIBLE_DEVICES="0")
    res = subprocess.run([exe, *map(str, args)], capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith('{"parity"')]
    assert lines, res.stdout[-2000:]
    return json.loads(lines[-1])


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
