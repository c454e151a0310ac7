"""GPU parity tests of the CUDA path, all through the C ABI.

Checked against (a) the CPU oracle on the same seeded inputs, (b) the golden
fixtures produced by the reference's own kernels, (c) the reference's compiled
kernels run side by side when oracle/_ref is present, and (d) size-independent
properties at the benchmark's full size.

Tolerances (from the task statement): flags and the loss-scale trajectory bit
for bit; fp32 master / m / v within 1e-6 relative per step and 1e-5 after 100
steps; fp16 weights exactly half_rn(master).  "Relative" is synth.rel_err.
"""
import ctypes as C
import glob
import os

import numpy as np
import pytest
import torch

from saga_b200 import AdamGroup, LossScaler, TrainingStepTail, capi
from saga_b200 import optimizer as opt
from tests import synth
from tests.gpu_util import Program, dev_f32, dev_u16, host_u16, stream_ptr

pytestmark = pytest.mark.gpu

TOL_STEP = 1e-6
TOL_100 = 1e-5
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _bits_equal(a, b):
    return np.array_equal(np.asarray(a).view(np.uint32), np.asarray(b).view(np.uint32))


# ------------------------------------------------------------------ kernel seam

def _seam_mixed(n, w, g, m, v, c, alpha, b1t, b2t, lr, l2, offset_elems=0):
    """b200opt_adam_mixed on torch-owned memory; offset_elems shifts every pointer
    to exercise the unaligned (element-wise) path."""
    o = offset_elems
    dw = dev_u16(np.concatenate([np.zeros(o, np.uint16), w]))
    dg = dev_u16(np.concatenate([np.zeros(o, np.uint16), g]))
    dm, dv, dc = (dev_f32(np.concatenate([np.zeros(o, np.float32), x])) for x in (m, v, c))
    aux = torch.zeros(4, dtype=torch.int32, device="cuda")
    opt.adam_mixed(n, alpha, dw.data_ptr() + 2 * o, dg.data_ptr() + 2 * o, dm.data_ptr() + 4 * o,
                   dv.data_ptr() + 4 * o, dc.data_ptr() + 4 * o, b1t, b2t, lr, l2, aux.data_ptr(),
                   stream_ptr())
    torch.cuda.synchronize()
    fl = tuple(int(x) for x in aux.cpu().numpy()[:3])
    return (host_u16(dw)[o:], dm.cpu().numpy()[o:], dv.cpu().numpy()[o:], dc.cpu().numpy()[o:], fl)


@pytest.mark.parametrize("n", [16, 272, 4112, 100003])
@pytest.mark.parametrize("offset", [0, 3])
def test_seam_adam_mixed_vs_oracle(oracle, n, offset):
    w = synth.weights_half(n, seed=21)
    c = oracle.master_init(w)
    rng = np.random.default_rng(n)
    m = (rng.standard_normal(n) * 1e-3).astype(np.float32)
    v = (rng.standard_normal(n) ** 2 * 1e-6).astype(np.float32)
    g = synth.grads_half(n, 1024.0, 7, seed=21)
    for k, bits in enumerate(synth.SPECIAL_HALF.values()):
        g[(k * 5) % n] = bits
    g[n - 1] = 0xFC00
    b1t, b2t = oracle.bias_corrections(7)
    al = oracle.alpha(1024.0)
    gw, gm, gv, gc, gfl = _seam_mixed(n, w, g, m, v, c, al, b1t, b2t, 1e-3, 0.01, offset)
    ow, om, ov, oc = w.copy(), m.copy(), v.copy(), c.copy()
    ofl = oracle.adam_mixed(ow, g, om, ov, oc, al, b1t, b2t, 1e-3, 0.01, model=1)
    assert gfl == tuple(ofl)
    assert synth.rel_err(gm, om) <= TOL_STEP
    assert synth.rel_err(gv, ov) <= TOL_STEP
    assert synth.rel_err(gc, oc) <= TOL_STEP
    # fp16 weights are exactly the rounding of the master the kernel itself wrote
    with np.errstate(over="ignore"):
        assert np.array_equal(gw, gc.astype(np.float16).view(np.uint16))
    # skipped elements: nothing moved
    skipped = (g & 0x7C00) == 0x7C00
    assert skipped.sum() >= 4
    assert np.array_equal(gw[skipped], w[skipped])
    assert _bits_equal(gm[skipped], m[skipped]) and _bits_equal(gc[skipped], c[skipped])


def test_seam_matches_reference_kernel_bit_for_bit(oracle):
    """Side by side with the reference's own compiled adam_mixed / adam_float."""
    if not oracle.ref_available():
        pytest.skip("oracle/_ref not built (reference checkout was absent at build time)")
    R = oracle.ref()
    for n in (16, 4112, 1 << 20):
        w = synth.weights_half(n, seed=31)
        c = oracle.master_init(w)
        ours = dict(w=dev_u16(w), c=dev_f32(c), m=torch.zeros(n, device="cuda"),
                    v=torch.zeros(n, device="cuda"))
        refs = {k: t.clone() for k, t in ours.items()}
        aux_o = torch.zeros(4, dtype=torch.int32, device="cuda")
        aux_r = torch.zeros(4, dtype=torch.int32, device="cuda")
        scale = np.float32(1024.0)
        for step in range(1, 11):
            g = synth.grads_half(n, scale, step, seed=31, inject_inf_every=5)
            gd = dev_u16(g)
            b1t, b2t = oracle.bias_corrections(step)
            al = oracle.alpha(scale)
            aux_o.zero_()
            aux_r.zero_()
            opt.adam_mixed(n, al, ours["w"].data_ptr(), gd.data_ptr(), ours["m"].data_ptr(),
                           ours["v"].data_ptr(), ours["c"].data_ptr(), b1t, b2t, 1e-3, 0.01,
                           aux_o.data_ptr(), stream_ptr())
            assert R.sagaref_adam_mixed(n, al, refs["w"].data_ptr(), gd.data_ptr(),
                                        refs["m"].data_ptr(), refs["v"].data_ptr(),
                                        refs["c"].data_ptr(), b1t, b2t, 1e-3, 0.01,
                                        aux_r.data_ptr(), stream_ptr()) == 0
            torch.cuda.synchronize()
            assert torch.equal(aux_o[:3], aux_r[:3])
            for k in ours:
                assert torch.equal(ours[k].view(torch.int32) if ours[k].dtype == torch.float32
                                   else ours[k], refs[k].view(torch.int32)
                                   if refs[k].dtype == torch.float32 else refs[k]), (n, step, k)
            scale = oracle.policy_reference(scale, aux_r.cpu().numpy()[:3].astype(np.uint32))
    # fp32 kernel
    n = 70001
    w = synth.weights_float(n, seed=32)
    ours = dict(w=dev_f32(w), m=torch.zeros(n, device="cuda"), v=torch.zeros(n, device="cuda"))
    refs = {k: t.clone() for k, t in ours.items()}
    for step in range(1, 6):
        g = synth.grads_float(n, 64.0, step, seed=32)
        if step == 3:
            g[0], g[n - 1], g[77] = np.inf, np.nan, -np.inf
        gd = dev_f32(g)
        b1t, b2t = oracle.bias_corrections(step)
        aux_o = torch.zeros(4, dtype=torch.int32, device="cuda")
        aux_r = torch.zeros(4, dtype=torch.int32, device="cuda")
        opt.adam_float(n, ours["w"].data_ptr(), gd.data_ptr(), ours["m"].data_ptr(),
                       ours["v"].data_ptr(), b1t, b2t, 1e-3, 0.01, aux_o.data_ptr(), stream_ptr())
        assert R.sagaref_adam_float(n, refs["w"].data_ptr(), gd.data_ptr(), refs["m"].data_ptr(),
                                    refs["v"].data_ptr(), b1t, b2t, 1e-3, 0.01, aux_r.data_ptr(),
                                    stream_ptr()) == 0
        torch.cuda.synchronize()
        assert torch.equal(aux_o[:3], aux_r[:3])
        for k in ours:
            assert torch.equal(ours[k].view(torch.int32), refs[k].view(torch.int32)), (step, k)


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "adam_mixed_*.npz"))))
def test_seam_reproduces_golden_fixtures(path):
    """Outputs the reference's kernel produced on a B200, committed as fixtures."""
    z = np.load(path)
    n, steps = int(z["n"]), int(z["steps"])
    w = z["w0"].copy()
    from oracle import oracle as orc
    c = orc.master_init(w)
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    for step in range(1, steps + 1):
        b1t, b2t = orc.bias_corrections(step)
        w, m, v, c, fl = _seam_mixed(n, w, z[f"g{step}"], m, v, c, orc.alpha(z[f"scale{step}"]),
                                     b1t, b2t, float(z["lr"]), float(z["l2"]))
        assert fl == tuple(int(x) for x in z[f"flags{step}"])
        assert np.array_equal(w, z[f"w{step}"])
        assert _bits_equal(m, z[f"m{step}"]) and _bits_equal(v, z[f"v{step}"])
        assert _bits_equal(c, z[f"c{step}"])


# ------------------------------------------------------------- handle API, 1 rank

VARIANTS = [capi.KERNEL_DIRECT, capi.KERNEL_STAGED]


def _run_trajectory(oracle, nranks, n_half, n_float, steps, lr, l2, scale0, seed,
                    inject_every=0, check_every=1, tol_final=TOL_100, variant=None, devices=None,
                    path=None, create_flags=0):
    W0 = synth.weights_half(n_half, seed=seed) if n_half else None
    Wf0 = synth.weights_float(n_float, seed=seed) if n_float else None
    prog = Program(nranks, n_half, n_float, variant=variant, devices=devices, path=path,
                   create_flags=create_flags)
    prog.set_weights([W0] * nranks if n_half else None, [Wf0] * nranks if n_float else None)
    ost = oracle.MultiRankState(nranks, [W0] * nranks if n_half else None,
                                [Wf0] * nranks if n_float else None)
    gs = LossScaler(scale0)
    oscale = np.float32(scale0)
    try:
        for step in range(1, steps + 1):
            G = [synth.grads_half(n_half, gs.scale, step, rank=r, seed=seed,
                                  inject_inf_every=inject_every if r == 0 else 0)
                 for r in range(nranks)] if n_half else None
            Gf = [synth.grads_float(n_float, gs.scale, step, rank=r, seed=seed)
                  for r in range(nranks)] if n_float else None
            prog.set_grads(G, Gf)
            flags = prog.step(lr, l2, gs.scale)
            oflags = ost.step([g.copy() for g in G] if G else None,
                              [g.copy() for g in Gf] if Gf else None, oscale, lr, l2, model=1)
            assert flags == oflags, (step, flags, oflags)
            gs.update(flags)
            oscale = oracle.policy_reference(oscale, oflags)
            assert gs.scale == oscale and gs.scale.tobytes() == oscale.tobytes(), step
            if step % check_every == 0 or step == steps:
                tol = TOL_STEP * min(step, 10) if step < 100 else tol_final
                for r in range(nranks):
                    if n_half:
                        for which, ref in ((0, ost.m[r]), (1, ost.v[r]), (2, ost.c[r])):
                            assert synth.rel_err(prog.state(r, capi.HALF, which), ref) <= tol, \
                                (step, r, which)
                    if n_float:
                        for which, ref in ((0, ost.mf[r]), (1, ost.vf[r])):
                            assert synth.rel_err(prog.state(r, capi.FLOAT, which), ref) <= tol
                        assert synth.rel_err(prog.weights_float(r), ost.Wf[r]) <= tol
        # fp16 weights: every rank holds the same buffer, equal to half_rn(master) of the owners
        if n_half:
            sh = n_half // nranks
            w0 = prog.weights_half(0)
            for r in range(nranks):
                assert np.array_equal(prog.weights_half(r), w0)
                with np.errstate(over="ignore"):
                    mine = prog.state(r, capi.HALF, 2).astype(np.float16).view(np.uint16)
                assert np.array_equal(w0[r * sh:(r + 1) * sh], mine)
            # and the oracle's fp16 weights differ from ours at most where the masters
            # round differently (never by more than one fp16 ulp)
            diff = w0.astype(np.int32) - ost.W[0].astype(np.int32)
            assert np.abs(diff).max() <= 1
            assert (diff != 0).mean() < 1e-3
        return gs.scale
    finally:
        prog.close()


@pytest.mark.parametrize("variant", VARIANTS)
def test_single_rank_100_steps_config2_distribution(oracle, variant):
    """n = 2^20, 100 steps, gradients N(0,1e-3)*scale, an inf every 50th step."""
    _run_trajectory(oracle, 1, 1 << 20, 0, 100, 1e-3, 0.01, 1024.0, seed=41,
                    inject_every=50, check_every=25, variant=variant)


@pytest.mark.parametrize("variant", VARIANTS)
def test_single_rank_both_groups_small(oracle, variant):
    for n_half, n_float in ((16, 16), (272, 48), (4112, 1040), (0, 528), (100000 - 16, 0),
                            (5, 3), (2048 * 9 + 8, 0)):
        _run_trajectory(oracle, 1, n_half, n_float, 6, 1e-2, 0.01, 64.0, seed=42, inject_every=4,
                        variant=variant)


def test_iteration_counter_advances_on_overflow_steps(oracle):
    n = 64
    prog = Program(1, n)
    try:
        prog.set_weights([synth.weights_half(n, seed=1)])
        g = synth.grads_half(n, 64.0, 1, seed=1)
        g[3] = 0x7C00
        prog.set_grads([g])
        assert prog.step(1e-3, 0.0, 64.0) == (1, 1, 0)
        assert prog.groups[0].iter == 1
        prog.step(1e-3, 0.0, 64.0)
        assert prog.groups[0].iter == 2
    finally:
        prog.close()


def test_step_tail_runs_like_program_step(oracle):
    """TrainingStepTail = exec + flag read + policy, the reference's step tail."""
    n = 4096
    g = AdamGroup.create(0, 1, 0, n, 0)
    try:
        w, gr = g.buffers(capi.HALF)
        w.view(torch.int16).copy_(dev_u16(synth.weights_half(n, seed=3)))
        g.init_master(stream_ptr())
        tail = TrainingStepTail(g, LossScaler(128.0), 1e-3, 0.01)
        scales = []
        for step in range(1, 8):
            bits = synth.grads_half(n, tail.scaler.scale, step, seed=3)
            if step == 4:
                bits[100] = 0x7E00
            gr.view(torch.int16).copy_(dev_u16(bits))
            tail.step(stream_ptr())
            scales.append(tail.scaler.scale)
        want = np.float32(128.0)
        for step in range(1, 8):
            want = oracle.policy_reference(want, (1, 0, 1) if step == 4 else (0, 0, 0))
            assert scales[step - 1] == want
    finally:
        g.destroy()


def test_step_host_takes_host_gradients(oracle):
    n_half, n_float = 8192, 256
    g = AdamGroup.create(0, 1, 0, n_half, n_float)
    try:
        W0, Wf0 = synth.weights_half(n_half, seed=6), synth.weights_float(n_float, seed=6)
        w, _ = g.buffers(capi.HALF)
        wf, _ = g.buffers(capi.FLOAT)
        w.view(torch.int16).copy_(dev_u16(W0))
        wf.copy_(dev_f32(Wf0))
        g.init_master(stream_ptr())
        ost = oracle.MultiRankState(1, [W0], [Wf0])
        for step in range(1, 4):
            G = synth.grads_half(n_half, 64.0, step, seed=6, inject_inf_every=2)
            Gf = synth.grads_float(n_float, 64.0, step, seed=6)
            hg = torch.from_numpy(G.view(np.int16).copy()).pin_memory()
            hf = torch.from_numpy(Gf.copy()).pin_memory()
            flags = g.step_host(hg.data_ptr(), hf.data_ptr(), 1e-3, 0.01, 64.0, stream_ptr())
            assert flags == ost.step([G.copy()], [Gf.copy()], 64.0, 1e-3, 0.01)
        assert synth.rel_err(g.export_state(capi.HALF, 2), ost.c[0]) <= 3 * TOL_STEP
    finally:
        g.destroy()


def test_step_host_pipelines_large_buffers_bit_for_bit(oracle):
    """Above 2^22 fp16 elements b200opt_step_host cuts the gradient copy into chunks on a
    copy stream and issues the step as one bucket per chunk behind it.  Same gradients
    through that call and through a plain device step: flags, m, v, master (both groups)
    and fp16 weights must come out bit for bit the same, also when the same host buffer
    is refilled and sent again right away."""
    n_half, n_float = (1 << 22) + 4112, 528
    W0, Wf0 = synth.weights_half(n_half, seed=16), synth.weights_float(n_float, seed=16)
    groups = [AdamGroup.create(0, 1, 0, n_half, n_float) for _ in range(2)]
    try:
        for g in groups:
            w, _ = g.buffers(capi.HALF)
            wf, _ = g.buffers(capi.FLOAT)
            w.view(torch.int16).copy_(dev_u16(W0))
            wf.copy_(dev_f32(Wf0))
            g.init_master(stream_ptr())
        a, b = groups
        _, ga = a.buffers(capi.HALF)
        _, gaf = a.buffers(capi.FLOAT)
        hg = torch.empty(n_half, dtype=torch.int16).pin_memory()
        hf = torch.empty(n_float, dtype=torch.float32).pin_memory()
        scale = np.float32(64.0)
        for step in range(1, 5):
            G = synth.grads_half(n_half, scale, step, seed=16)
            Gf = synth.grads_float(n_float, scale, step, seed=16)
            if step == 2:
                G[n_half - 77] = 0x7C00          # +inf in the last chunk
                G[5] = 0x7800                    # 32768 in the first
            if step == 3:
                G[n_half // 2 + 1] = 0x7E00      # NaN in the middle
            hg.copy_(torch.from_numpy(G.view(np.int16)))
            hf.copy_(torch.from_numpy(Gf))
            ga.view(torch.int16).copy_(hg, non_blocking=True)
            gaf.copy_(hf, non_blocking=True)
            a.exec(1e-3, 0.01, scale, stream_ptr())
            fa = a.flags(stream_ptr())
            fb = b.step_host(hg.data_ptr(), hf.data_ptr(), 1e-3, 0.01, scale, stream_ptr())
            assert fa == fb == {2: (1, 1, 0), 3: (1, 0, 1)}.get(step, (0, 0, 0))
            scale = oracle.policy_reference(scale, fa)
        assert a.iter == b.iter == 4
        for dtype in (capi.HALF, capi.FLOAT):
            for which in range(3 if dtype == capi.HALF else 2):
                x, y = a.export_state(dtype, which), b.export_state(dtype, which)
                assert x.tobytes() == y.tobytes(), (dtype, which)
            wa, _ = a.buffers(dtype)
            wb, _ = b.buffers(dtype)
            assert torch.equal(wa.view(torch.int16 if dtype == capi.HALF else torch.int32),
                               wb.view(torch.int16 if dtype == capi.HALF else torch.int32))
    finally:
        for g in groups:
            g.destroy()


def test_export_import_state_resumes_exactly(oracle):
    n = 4112
    W0 = synth.weights_half(n, seed=8)

    def run(groups_steps, resume_from=None):
        g = AdamGroup.create(0, 1, 0, n, 0)
        w, gr = g.buffers(capi.HALF)
        if resume_from is None:
            w.view(torch.int16).copy_(dev_u16(W0))
            g.init_master(stream_ptr())
        else:
            w.view(torch.int16).copy_(dev_u16(resume_from["w"]))
            g.init_master(stream_ptr())
            torch.cuda.synchronize()
            for which, key in enumerate("mvc"):
                g.import_state(capi.HALF, which, resume_from[key])
            g.iter = resume_from["iter"]
        for step in groups_steps:
            gr.view(torch.int16).copy_(dev_u16(synth.grads_half(n, 64.0, step, seed=8)))
            g.exec(1e-3, 0.01, 64.0, stream_ptr())
            g.flags(stream_ptr())
        out = dict(w=host_u16(w), m=g.export_state(capi.HALF, 0), v=g.export_state(capi.HALF, 1),
                   c=g.export_state(capi.HALF, 2), iter=g.iter)
        g.destroy()
        return out

    straight = run(range(1, 9))
    half = run(range(1, 5))
    resumed = run(range(5, 9), resume_from=half)
    for key in "wmvc":
        assert np.array_equal(straight[key], resumed[key])


def test_checkpoint_files_resume_exactly(oracle, tmp_path):
    """m, v, master, iteration counter and loss scale through Saga tensor files: a run
    resumed from the files continues bit for bit; files of another layout are refused."""
    from saga_b200 import optimizer as optmod
    n_half, n_float = 4112, 528
    W0, Wf0 = synth.weights_half(n_half, seed=12), synth.weights_float(n_float, seed=12)

    def fresh(weights=None, wf=None):
        g = AdamGroup.create(0, 1, 0, n_half, n_float)
        w, gr = g.buffers(capi.HALF)
        wf_, gf = g.buffers(capi.FLOAT)
        w.view(torch.int16).copy_(dev_u16(W0 if weights is None else weights))
        wf_.copy_(dev_f32(Wf0 if wf is None else wf))
        g.init_master(stream_ptr())
        torch.cuda.synchronize()
        return g, w, gr, wf_, gf

    def steps(g, gr, gf, scaler, rng):
        for step in rng:
            bits = synth.grads_half(n_half, scaler.scale, step, seed=12, inject_inf_every=3)
            gr.view(torch.int16).copy_(dev_u16(bits))
            gf.copy_(dev_f32(synth.grads_float(n_float, scaler.scale, step, seed=12)))
            g.exec(1e-3, 0.01, scaler.scale, stream_ptr())
            scaler.update(g.flags(stream_ptr()))

    g, w, gr, wf, gf = fresh()
    sc = LossScaler(128.0)
    steps(g, gr, gf, sc, range(1, 9))
    straight = (host_u16(w), wf.cpu().numpy().copy(), [g.export_state(capi.HALF, k) for k in range(3)],
                [g.export_state(capi.FLOAT, k) for k in range(2)], g.iter, sc.scale)
    g.destroy()

    g, w, gr, wf, gf = fresh()
    sc = LossScaler(128.0)
    steps(g, gr, gf, sc, range(1, 5))
    g.checkpoint_save(tmp_path, sc.scale, 7)
    saved_w, saved_wf = host_u16(w), wf.cpu().numpy().copy()
    g.destroy()
    names = sorted(os.listdir(tmp_path))
    assert names == ["adam.r0of1.float.m.saga", "adam.r0of1.float.v.saga", "adam.r0of1.half.m.saga",
                     "adam.r0of1.half.master.saga", "adam.r0of1.half.v.saga", "adam.r0of1.meta.saga"]
    m_file = optmod.tensor_load(tmp_path / "adam.r0of1.half.m.saga")
    assert m_file.dtype == np.float32 and m_file.shape == (n_half,)

    g, w, gr, wf, gf = fresh(saved_w, saved_wf)     # weights come from Saga's own save
    scale, pstate = g.checkpoint_load(tmp_path)
    assert pstate == 7 and g.iter == 4
    sc = LossScaler(scale)
    steps(g, gr, gf, sc, range(5, 9))
    assert np.array_equal(host_u16(w), straight[0])
    assert np.array_equal(wf.cpu().numpy().view(np.uint32), straight[1].view(np.uint32))
    for k in range(3):
        assert _bits_equal(g.export_state(capi.HALF, k), straight[2][k])
    for k in range(2):
        assert _bits_equal(g.export_state(capi.FLOAT, k), straight[3][k])
    assert g.iter == straight[4] and sc.scale.tobytes() == straight[5].tobytes()
    g.destroy()

    other = AdamGroup.create(0, 1, 0, n_half + 16, n_float)
    try:
        with pytest.raises(capi.B200OptError):
            other.checkpoint_load(tmp_path)
    finally:
        other.destroy()


# ------------------------------------------- several ranks on one GPU (serial mode)

@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("nranks", [2, 3, 4, 5, 6, 7, 8])
def test_multirank_serial_matches_oracle(oracle, nranks, variant):
    # sizes chosen to hit: shard edges off the 8-element grid (16/8 = 2 per rank),
    # a tail nobody owns (n % nranks != 0), sizes with full vector groups, and
    # shards of several 2048-element tiles with a ragged last tile
    for n_half, n_float in ((16, 16), (272, 48), (8208, 528), (2048 * 3 * nranks + 80, 0)):
        _run_trajectory(oracle, nranks, n_half, n_float, 5, 1e-2, 0.01, 64.0, seed=50 + nranks,
                        inject_every=3, variant=variant)


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("nranks", [2, 4, 8])
def test_special_values_at_shard_edges(oracle, nranks, variant):
    n = 64 * nranks
    s = n // nranks
    W0 = synth.weights_half(n, seed=60)
    prog = Program(nranks, n, variant=variant)
    ost = oracle.MultiRankState(nranks, [W0] * nranks)
    try:
        prog.set_weights([W0] * nranks)
        G = [np.zeros(n, np.uint16) for _ in range(nranks)]
        base = synth.grads_half(n, 64.0, 1, seed=60)
        G[0][:] = base
        specials = list(synth.SPECIAL_HALF.values())
        for r in range(nranks):
            # first and last element of every shard, delivered by different ranks
            G[r][r * s] = specials[r % len(specials)]
            G[(r + 1) % nranks][(r + 1) * s - 1] = specials[(r + 5) % len(specials)]
        before = prog.weights_half(0)
        prog.set_grads(G)
        flags = prog.step(1e-3, 0.01, 64.0)
        assert flags == ost.step([g.copy() for g in G], None, 64.0, 1e-3, 0.01)
        after = prog.weights_half(0)
        assert np.array_equal(after, ost.W[0]) or np.abs(
            after.astype(np.int32) - ost.W[0].astype(np.int32)).max() <= 1
        # elements whose reduced gradient is inf/nan keep their fp16 weight on every rank
        red = np.zeros(n, np.float32)
        with np.errstate(invalid="ignore", over="ignore"):
            for r in range(nranks):
                red = red + G[r].view(np.float16).astype(np.float32)
            red16 = red.astype(np.float16)
        skipped = ~np.isfinite(red16)
        assert skipped.any()
        for r in range(nranks):
            assert np.array_equal(prog.weights_half(r)[skipped], before[skipped])
    finally:
        prog.close()


@pytest.mark.parametrize("nranks", [2, 4, 8])
def test_range_flag_on_one_vs_two_shards_drives_the_scale(oracle, nranks):
    n = 32 * nranks
    s = n // nranks
    for shards_hit, factor in ((1, 1.02), (2, 0.9)):
        prog = Program(nranks, n)
        try:
            prog.set_weights([synth.weights_half(n, seed=61)] * nranks)
            G = [np.zeros(n, np.uint16) for _ in range(nranks)]
            for k in range(shards_hit):
                G[nranks - 1][k * s + 3] = 0x7800  # 32768 lands in shard k
            prog.set_grads(G)
            flags = prog.step(1e-3, 0.0, 64.0)
            assert flags == (shards_hit, 0, 0)
            sc = LossScaler(64.0)
            sc.update(flags)
            assert sc.scale == np.float32(np.float64(np.float32(64.0)) * factor)
        finally:
            prog.close()


def test_partial_sums_that_would_overflow_in_fp16_do_not(oracle):
    """60000 + 60000 - 60000 - 60000 + 1: any fp16 partial sum overflows, the fp32 sum is 1."""
    nranks, n = 4, 64
    prog = Program(nranks, n)
    try:
        prog.set_weights([synth.weights_half(n, seed=62)] * nranks)
        vals = [60000.0, 60000.0, -60000.0, -59999.0]
        G = [np.full(n, np.float16(x)).view(np.uint16).copy() for x in vals]
        prog.set_grads(G)
        flags = prog.step(1e-3, 0.0, 1.0)
        ost = oracle.MultiRankState(nranks, [synth.weights_half(n, seed=62)] * nranks)
        assert flags == ost.step([g.copy() for g in G], None, 1.0, 1e-3, 0.0) == (0, 0, 0)
    finally:
        prog.close()


# ------------------------------------------------------------- full-size properties

def test_full_size_layout_properties(oracle):
    """25.6 M parameters in 160 padded tensors: padding stays exactly zero, fp16
    weights equal half_rn(master), flags as injected, after several steps."""
    from saga_b200 import FlatLayout
    sizes = synth.tensor_sizes()
    lay = FlatLayout(sizes)
    offs, total = oracle.flat_layout(sizes)
    assert lay.offsets == offs and lay.total == total
    n = lay.total
    dev = torch.device("cuda", 0)
    g = AdamGroup.create(0, 1, 0, n, 0)
    try:
        w, gr = g.buffers(capi.HALF)
        mask = torch.zeros(n, dtype=torch.bool, device=dev)  # True on real elements
        for sl in lay.slices():
            mask[sl] = True
        gen = torch.Generator(device=dev).manual_seed(1234)
        w.copy_((torch.randn(n, device=dev, generator=gen) * 0.02).half() * mask)
        g.init_master(stream_ptr())
        scale = LossScaler(1024.0)
        for step in range(1, 6):
            grad = (torch.randn(n, device=dev, generator=gen) * 1e-3 * float(scale.scale)).half() * mask
            if step == 3:
                grad[lay.offsets[17] + 5] = float("inf")
            gr.copy_(grad)
            g.exec(1e-3, 0.01, scale.scale, stream_ptr())
            flags = g.flags(stream_ptr())
            assert flags == ((1, 1, 0) if step == 3 else (0, 0, 0))
            scale.update(flags)
        c = torch.from_numpy(g.export_state(capi.HALF, 2)).to(dev)
        m = torch.from_numpy(g.export_state(capi.HALF, 0)).to(dev)
        v = torch.from_numpy(g.export_state(capi.HALF, 1)).to(dev)
        assert torch.equal(w, c.half())
        assert not w[~mask].any() and not c[~mask].any() and not m[~mask].any() and not v[~mask].any()
        assert torch.isfinite(c).all() and (v >= 0).all()
    finally:
        g.destroy()


def test_full_size_config2_bit_equal_to_reference_kernel(oracle):
    """The benchmark's workload at full size (25.6 M fp16 parameters in 160 padded tensors),
    six steps through the handle API with an injected +inf, a 32768 and a NaN: m, v, master
    and fp16 weights bit for bit equal to the reference's own compiled adam_mixed run side
    by side on the same gradients; flags and loss scale equal to the oracle's; and m, v,
    master within 1e-6 element-wise relative of the CPU oracle over the whole buffer."""
    from saga_b200 import FlatLayout
    sizes = synth.tensor_sizes()
    lay = FlatLayout(sizes)
    n = lay.total
    assert n > 25_600_000
    dev = torch.device("cuda", 0)
    W0 = synth.scatter_into_flat(lay.offsets, lay.sizes, n, synth.weights_half(sum(sizes), seed=91))
    R = oracle.ref() if oracle.ref_available() else None
    g = AdamGroup.create(0, 1, 0, n, 0)
    try:
        w, gr = g.buffers(capi.HALF)
        w.view(torch.int16).copy_(dev_u16(W0))
        g.init_master(stream_ptr())
        if R is not None:
            ref = dict(w=dev_u16(W0), c=dev_f32(oracle.master_init(W0)),
                       m=torch.zeros(n, device=dev), v=torch.zeros(n, device=dev))
            aux = torch.zeros(4, dtype=torch.int32, device=dev)
        ow, oc = W0.copy(), oracle.master_init(W0)
        om, ov = np.zeros(n, np.float32), np.zeros(n, np.float32)
        oracle.use_all_host_threads()
        scaler = LossScaler(1024.0)
        oscale = np.float32(1024.0)
        want_flags = {2: (1, 1, 0), 3: (1, 0, 0), 5: (1, 0, 1)}
        for step in range(1, 7):
            bits = synth.scatter_into_flat(
                lay.offsets, lay.sizes, n, synth.grads_half(sum(sizes), scaler.scale, step, seed=91))
            if step == 2:
                bits[lay.offsets[40] + 7] = 0x7C00      # +inf: element skipped
            if step == 3:
                bits[lay.offsets[99]] = 0x7800          # 32768: range flag, element updated
                bits[n - 17] = 0xF800                   # -32768 in the last tensor
            if step == 5:
                bits[lay.offsets[3] + 1] = 0x7E01       # NaN
            gd = dev_u16(bits)
            gr.view(torch.int16).copy_(gd)
            g.exec(1e-3, 0.01, scaler.scale, stream_ptr())
            flags = g.flags(stream_ptr())
            b1t, b2t = oracle.bias_corrections(step)
            al = oracle.alpha(oscale)
            oflags = tuple(int(x) for x in
                           oracle.adam_mixed(ow, bits, om, ov, oc, al, b1t, b2t, 1e-3, 0.01,
                                             model=1, threads=True))
            assert flags == oflags == want_flags.get(step, (0, 0, 0)), (step, flags, oflags)
            if R is not None:
                aux.zero_()
                assert R.sagaref_adam_mixed(n, al, ref["w"].data_ptr(), gd.data_ptr(),
                                            ref["m"].data_ptr(), ref["v"].data_ptr(),
                                            ref["c"].data_ptr(), b1t, b2t, 1e-3, 0.01,
                                            aux.data_ptr(), stream_ptr()) == 0
                torch.cuda.synchronize()
                assert tuple(int(x) for x in aux.cpu()[:3]) == flags
                for which, key in enumerate("mvc"):
                    ours = torch.from_numpy(g.export_state(capi.HALF, which)).to(dev)
                    assert torch.equal(ours.view(torch.int32), ref[key].view(torch.int32)), (step, key)
                    del ours
                assert torch.equal(w.view(torch.int16), ref["w"]), step
            scaler.update(flags)
            oscale = oracle.policy_reference(oscale, oflags)
            assert scaler.scale.tobytes() == oscale.tobytes(), step
        for which, o in enumerate((om, ov, oc)):
            assert synth.strict_rel_err(g.export_state(capi.HALF, which), o) <= TOL_STEP, which
        assert np.array_equal(host_u16(w), ow)
    finally:
        w = gr = None
        g.destroy()


def test_linearity_in_the_loss_scale(oracle):
    """Scaling gradients and the loss scale by the same power of two changes nothing."""
    n = 1 << 16
    outs = []
    for k in (1.0, 16.0):
        g = AdamGroup.create(0, 1, 0, n, 0)
        w, gr = g.buffers(capi.HALF)
        w.view(torch.int16).copy_(dev_u16(synth.weights_half(n, seed=70)))
        g.init_master(stream_ptr())
        for step in range(1, 4):
            base = synth.grads_half(n, 8.0, step, seed=70).view(np.float16).astype(np.float32)
            gr.view(torch.int16).copy_(dev_u16((base * np.float32(k)).astype(np.float16).view(np.uint16)))
            g.exec(1e-3, 0.01, 8.0 * k, stream_ptr())
            assert g.flags(stream_ptr()) == (0, 0, 0)
        outs.append((host_u16(w), g.export_state(capi.HALF, 0), g.export_state(capi.HALF, 2)))
        g.destroy()
    for a, b in zip(outs[0], outs[1]):
        assert np.array_equal(a, b)


# --------------------------------------------------- long trajectories, big buffers

@pytest.mark.parametrize("policy", ["reference", "interval"])
def test_2100_steps_flags_and_scale_bit_exact(oracle, policy):
    """2100 steps with an inf injected every 50th step.  Under the reference policy the
    scale climbs x1.02 per clean step until gradients overflow on their own, then
    saw-tooths; under the interval policy it halves on overflow and doubles after
    2000 clean steps.  Every step's flag tuple and scale must equal the oracle's."""
    n, steps = 1 << 14, 2100
    W0 = synth.weights_half(n, seed=71)
    prog = Program(1, n)
    try:
        prog.set_weights([W0])
        ost = oracle.MultiRankState(1, [W0])
        pol = capi.POLICY_REFERENCE if policy == "reference" else capi.POLICY_INTERVAL
        gs = LossScaler(1024.0, policy=pol, interval=2000)
        oscale, oclean = np.float32(1024.0), 0
        seen = set()
        halvings = doublings = 0
        for step in range(1, steps + 1):
            G = synth.grads_half(n, gs.scale, step, seed=71, inject_inf_every=50)
            if policy == "interval" and step > 60:
                G = synth.grads_half(n, gs.scale, step, seed=71)  # 2000 clean steps in a row
            prog.set_grads([G])
            flags = prog.step(1e-3, 0.0, gs.scale)
            oflags = ost.step([G.copy()], None, oscale, 1e-3, 0.0)
            assert flags == oflags, (step, flags, oflags)
            seen.add(flags)
            prev = gs.scale
            gs.update(flags)
            if policy == "reference":
                oscale = oracle.policy_reference(oscale, oflags)
            else:
                oscale, oclean = oracle.policy_interval(oscale, oclean, oflags, 2000)
            assert gs.scale.tobytes() == oscale.tobytes(), step
            halvings += gs.scale < prev
            doublings += gs.scale == np.float32(2) * prev
        if policy == "reference":
            # injected infs, natural overflows near the top of the saw-tooth, range-only steps
            assert (1, 1, 0) in seen and (0, 0, 0) in seen and (1, 0, 0) in seen
            assert halvings > 42      # more than the 42 injected ones: natural overflows too
        else:
            assert halvings == 1 and doublings == 1
        assert synth.rel_err(prog.state(0, capi.HALF, 2), ost.c[0]) <= 1e-5
    finally:
        prog.close()


def test_padding_stays_zero_across_eight_ranks(oracle):
    """160 tensors padded to 16 elements, eight ranks: padding is zero in the weights of
    every rank and in every rank's m, v and master after several steps."""
    from saga_b200 import FlatLayout
    nranks = 8
    sizes = synth.tensor_sizes(1_000_000, 160, lo=8, hi=60000, seed=3)
    lay = FlatLayout(sizes)
    n = lay.total
    real = np.zeros(n, dtype=bool)
    for sl in lay.slices():
        real[sl] = True
    assert (~real).sum() > 500
    W0 = synth.weights_half(n, seed=72)
    W0[~real] = 0
    prog = Program(nranks, n)
    try:
        prog.set_weights([W0] * nranks)
        for step in range(1, 4):
            G = []
            for r in range(nranks):
                g = synth.grads_half(n, 64.0, step, rank=r, seed=72)
                g[~real] = 0
                G.append(g)
            prog.set_grads(G)
            prog.step(1e-2, 0.01, 64.0)
        s = n // nranks
        for r in range(nranks):
            assert not prog.weights_half(r)[~real].any()
            pad = ~real[r * s:(r + 1) * s]
            for which in range(3):
                assert not prog.state(r, capi.HALF, which)[pad].any()
        assert prog.weights_half(0)[real].any()
    finally:
        prog.close()


def test_flat_buffer_of_2_30_elements(oracle):
    """The largest size of the bandwidth sweep: 2^30 fp16 elements on one GPU (the
    reference indexes with int; this path with size_t).  Checked through properties:
    slices at the start, middle and end against the oracle, fp16 weights equal to the
    rounded master everywhere, flags from an inf planted in the last element."""
    n = 1 << 30
    free, _ = torch.cuda.mem_get_info(0)
    if free < 40 * (1 << 30):
        pytest.skip("needs 40 GB of free device memory")
    dev = torch.device("cuda", 0)
    g = AdamGroup.create(0, 1, 0, n, 0)
    try:
        w, gr = g.buffers(capi.HALF)
        chunk = 1 << 27
        gen = torch.Generator(device=dev).manual_seed(5)
        for c0 in range(0, n, chunk):
            w[c0:c0 + chunk] = (torch.randn(chunk, device=dev, generator=gen) * 0.02).half()
            gr[c0:c0 + chunk] = (torch.randn(chunk, device=dev, generator=gen) * 0.5).half()
        gr[n - 1] = float("inf")
        g.init_master(stream_ptr())
        torch.cuda.synchronize()
        slices = [(0, 1 << 16), (n // 2 - 12345, 1 << 16), (n - (1 << 16), 1 << 16)]
        before = [(host_u16(w[a:a + k]), host_u16(gr[a:a + k])) for a, k in slices]
        g.exec(1e-3, 0.01, 512.0, stream_ptr())
        assert g.flags(stream_ptr()) == (1, 1, 0)
        b1t, b2t = oracle.bias_corrections(1)
        for (a, k), (w0, g0) in zip(slices, before):
            ow, om, ov = w0.copy(), np.zeros(k, np.float32), np.zeros(k, np.float32)
            oc = oracle.master_init(w0)
            oracle.adam_mixed(ow, g0, om, ov, oc, oracle.alpha(512.0), b1t, b2t, 1e-3, 0.01)
            assert np.array_equal(host_u16(w[a:a + k]), ow), a
        # the planted inf: last element untouched
        assert host_u16(w[n - 1:])[0] == before[2][0][-1]
        # weights == half(master) over the whole buffer, chunk by chunk through the state export
        c = g.export_state(capi.HALF, 2)
        assert c.size == n
        for c0 in range(0, n, chunk):
            cc = torch.from_numpy(c[c0:c0 + chunk]).to(dev)
            assert torch.equal(w[c0:c0 + chunk], cc.half())
    finally:
        w = gr = None
        g.destroy()
