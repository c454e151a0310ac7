"""Pins the CPU oracle to the golden fixtures: outputs of the reference's own
adam_mixed / adam_float kernels (compiled unmodified for sm_100a, run on a
B200 by tests/golden/make_golden.py) for seeded inputs.

The fused-multiply-add model of the oracle (model 1) must reproduce them bit
for bit; the uncontracted model (model 0) within the per-step tolerance."""
import glob
import os

import numpy as np
import pytest

from tests import synth

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
MIXED = sorted(glob.glob(os.path.join(GOLDEN, "adam_mixed_*.npz")))
FLOAT = sorted(glob.glob(os.path.join(GOLDEN, "adam_float_*.npz")))


def test_fixtures_are_present():
    assert len(MIXED) >= 3 and len(FLOAT) >= 1


@pytest.mark.parametrize("path", MIXED, ids=os.path.basename)
def test_oracle_reproduces_reference_adam_mixed(oracle, path):
    z = np.load(path)
    n, steps = int(z["n"]), int(z["steps"])
    lr, l2 = float(z["lr"]), float(z["l2"])
    st = {}
    for model in (0, 1):
        w = z["w0"].copy()
        st[model] = dict(w=w, c=oracle.master_init(w), m=np.zeros(n, np.float32),
                         v=np.zeros(n, np.float32))
    seen_flags = set()
    for step in range(1, steps + 1):
        b1t, b2t = oracle.bias_corrections(step)
        al = oracle.alpha(z[f"scale{step}"])
        want_flags = tuple(int(x) for x in z[f"flags{step}"])
        seen_flags.add(want_flags)
        for model, s in st.items():
            fl = oracle.adam_mixed(s["w"], z[f"g{step}"].copy(), s["m"], s["v"], s["c"], al,
                                   b1t, b2t, lr, l2, model=model)
            assert tuple(fl) == want_flags
        for key in "mvc":
            assert np.array_equal(st[1][key].view(np.uint32), z[f"{key}{step}"].view(np.uint32)), \
                (step, key)
            assert synth.rel_err(st[0][key], z[f"{key}{step}"]) <= 1e-6 * step
        assert np.array_equal(st[1]["w"], z[f"w{step}"])
        # the loss scale the generator fed the next step follows the policy
        if step < steps:
            assert oracle.policy_reference(z[f"scale{step}"], z[f"flags{step}"]) == z[f"scale{step + 1}"]
    assert len(seen_flags) >= 1


@pytest.mark.parametrize("path", FLOAT, ids=os.path.basename)
def test_oracle_reproduces_reference_adam_float(oracle, path):
    z = np.load(path)
    n, steps = int(z["n"]), int(z["steps"])
    w = z["w0"].copy()
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    flagged = False
    for step in range(1, steps + 1):
        b1t, b2t = oracle.bias_corrections(step)
        fl = oracle.adam_f32(w, z[f"g{step}"].copy(), m, v, b1t, b2t, float(z["lr"]),
                             float(z["l2"]), model=1)
        assert tuple(fl) == tuple(int(x) for x in z[f"flags{step}"])
        flagged |= bool(fl[1] and fl[2])
        for arr, key in ((w, "w"), (m, "m"), (v, "v")):
            assert np.array_equal(arr.view(np.uint32), z[f"{key}{step}"].view(np.uint32)), (step, key)
    assert flagged  # the fixture exercises inf and nan
