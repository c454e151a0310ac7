"""Generates the golden fixtures of tests/golden/ from the REFERENCE's own
kernels (oracle/_ref/libsaga_ref_kernels.so = the reference's unmodified
src/cuda/cuda_kernels.cu compiled for sm_100a).  Needs a GPU.

    python tests/golden/make_golden.py <output-dir>

Inputs come from tests/synth.py (seeded); outputs are whatever the reference's
saga::adam_mixed / saga::adam_float produced for them.  The .npz files written
here are committed; tests/test_golden_cpu.py holds the CPU oracle to them and
tests/test_step_gpu.py holds the CUDA path to them.
"""
import ctypes as C
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as orc  # noqa: E402
from tests import synth  # noqa: E402

DEV = torch.device("cuda", 0)


def dev_u16(a):
    return torch.from_numpy(a.view(np.int16).copy()).to(DEV)


def dev_f32(a):
    return torch.from_numpy(a.copy()).to(DEV)


def host_u16(t):
    return t.cpu().numpy().view(np.uint16).copy()


def run_mixed(name, n, steps, lr, l2, scale0, special_step, seed):
    R = orc.ref()
    w = synth.weights_half(n, seed=seed)
    c = orc.master_init(w)
    d = dict(w=dev_u16(w), c=dev_f32(c), m=torch.zeros(n, device=DEV), v=torch.zeros(n, device=DEV))
    aux = torch.zeros(4, dtype=torch.int32, device=DEV)
    out = {"n": n, "lr": np.float32(lr), "l2": np.float32(l2), "w0": w}
    scale = np.float32(scale0)
    for step in range(1, steps + 1):
        g = synth.grads_half(n, scale, step, seed=seed)
        if step == special_step:
            for k, bits in enumerate(synth.SPECIAL_HALF.values()):
                g[(k * 7) % n] = bits
            g[n - 1] = 0x7C00
        gd = dev_u16(g)
        b1t, b2t = orc.bias_corrections(step)
        al = orc.alpha(scale)
        aux.zero_()
        rc = R.sagaref_adam_mixed(n, al, d["w"].data_ptr(), gd.data_ptr(), d["m"].data_ptr(),
                                  d["v"].data_ptr(), d["c"].data_ptr(), b1t, b2t, lr, l2,
                                  aux.data_ptr(), None)
        assert rc == 0
        torch.cuda.synchronize()
        fl = aux.cpu().numpy().astype(np.uint32)[:3]
        out[f"g{step}"] = g
        out[f"scale{step}"] = scale
        out[f"flags{step}"] = fl
        out[f"w{step}"] = host_u16(d["w"])
        out[f"m{step}"] = d["m"].cpu().numpy()
        out[f"v{step}"] = d["v"].cpu().numpy()
        out[f"c{step}"] = d["c"].cpu().numpy()
        scale = orc.policy_reference(scale, fl)
    out["steps"] = steps
    return name, out


def run_float(name, n, steps, lr, l2, seed):
    R = orc.ref()
    w = synth.weights_float(n, seed=seed)
    d = dict(w=dev_f32(w), m=torch.zeros(n, device=DEV), v=torch.zeros(n, device=DEV))
    aux = torch.zeros(4, dtype=torch.int32, device=DEV)
    out = {"n": n, "lr": np.float32(lr), "l2": np.float32(l2), "w0": w, "steps": steps}
    for step in range(1, steps + 1):
        g = synth.grads_float(n, 64.0, step, seed=seed)
        if step == 2:
            g[0], g[n // 2], g[n - 1], g[5] = np.inf, -np.inf, np.nan, 1e15
        gd = dev_f32(g)
        b1t, b2t = orc.bias_corrections(step)
        aux.zero_()
        rc = R.sagaref_adam_float(n, d["w"].data_ptr(), gd.data_ptr(), d["m"].data_ptr(),
                                  d["v"].data_ptr(), b1t, b2t, lr, l2, aux.data_ptr(), None)
        assert rc == 0
        torch.cuda.synchronize()
        out[f"g{step}"] = g
        out[f"flags{step}"] = aux.cpu().numpy().astype(np.uint32)[:3]
        out[f"w{step}"] = d["w"].cpu().numpy()
        out[f"m{step}"] = d["m"].cpu().numpy()
        out[f"v{step}"] = d["v"].cpu().numpy()
    return name, out


def compare_with_oracle(out, model):
    """How far the CPU oracle is from what the reference kernel produced."""
    n, steps = int(out["n"]), int(out["steps"])
    w = out["w0"].copy()
    c = orc.master_init(w)
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    worst = {"m": 0.0, "v": 0.0, "c": 0.0}
    exact = True
    for step in range(1, steps + 1):
        b1t, b2t = orc.bias_corrections(step)
        fl = orc.adam_mixed(w, out[f"g{step}"].copy(), m, v, c, orc.alpha(out[f"scale{step}"]),
                            b1t, b2t, float(out["lr"]), float(out["l2"]), model=model)
        assert tuple(fl) == tuple(out[f"flags{step}"])
        for key, arr in (("m", m), ("v", v), ("c", c)):
            worst[key] = max(worst[key], synth.rel_err(arr, out[f"{key}{step}"]))
            exact &= np.array_equal(arr.view(np.uint32), out[f"{key}{step}"].view(np.uint32))
        exact &= np.array_equal(w, out[f"w{step}"])
    return {"bit_exact": bool(exact), **worst}


def main():
    outdir = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "golden_out")
    os.makedirs(outdir, exist_ok=True)
    report = {"gpu": torch.cuda.get_device_name(0)}
    for name, out in (
        run_mixed("adam_mixed_n4112", 4112, 6, 1e-3, 0.01, 1024.0, 3, seed=11),
        run_mixed("adam_mixed_n272_l2zero", 272, 4, 1e-2, 0.0, 64.0, 2, seed=12),
        run_mixed("adam_mixed_n16", 16, 3, 1e-3, 0.01, 256.0, 0, seed=13),
        run_mixed("adam_mixed_n1040_big_decay", 1040, 4, 0.05, 0.5, 64.0, 2, seed=15),
    ):
        np.savez_compressed(os.path.join(outdir, name + ".npz"), **out)
        report[name] = {f"oracle_model{k}": compare_with_oracle(out, k) for k in (0, 1)}
    for name, out in (run_float("adam_float_n1040", 1040, 4, 1e-3, 0.01, seed=14),
                      run_float("adam_float_n528_big_decay", 528, 4, 0.05, 0.5, seed=16)):
        np.savez_compressed(os.path.join(outdir, name + ".npz"), **out)
    with open(os.path.join(outdir, "report.json"), "w") as f:
        json.dump(report, f, indent=1)
    print(json.dumps(report, indent=1))


if __name__ == "__main__":
    main()
