"""A step issued as several buckets (so that reduction and update can start
while backward still runs) must give bit for bit what one whole step gives:
same flags, same optimizer state, same weights on every rank."""
import numpy as np
import pytest
import torch

from saga_b200 import AdamGroup, capi
from saga_b200.capi import B200OptError
from tests import synth
from tests.gpu_util import Program, stream_ptr

pytestmark = pytest.mark.gpu


def _buckets(n, k, rng):
    """k contiguous buckets covering [0, n) with ragged (odd) boundaries, one empty."""
    if n == 0:
        return [(0, 0)] * k
    cuts = sorted(int(x) for x in rng.integers(0, n + 1, size=k - 1))
    cuts[len(cuts) // 2] = cuts[len(cuts) // 2 - 1] if len(cuts) > 1 else cuts[0]  # an empty bucket
    cuts = sorted(cuts)
    edges = [0] + cuts + [n]
    return [(edges[i], edges[i + 1] - edges[i]) for i in range(k)]


def _run(nranks, n_half, n_float, bucketed, variant, devices=None, steps=4, seed=33):
    rng = np.random.default_rng(seed)
    prog = Program(nranks, n_half, n_float, variant=variant, devices=devices)
    W0 = synth.weights_half(n_half, seed=seed) if n_half else None
    Wf0 = synth.weights_float(n_float, seed=seed) if n_float else None
    prog.set_weights([W0] * nranks if n_half else None, [Wf0] * nranks if n_float else None)
    flags_seen = []
    try:
        for step in range(1, steps + 1):
            G = [synth.grads_half(n_half, 64.0, step, rank=r, seed=seed,
                                  inject_inf_every=2 if r == 0 else 0)
                 for r in range(nranks)] if n_half else None
            Gf = [synth.grads_float(n_float, 64.0, step, rank=r, seed=seed)
                  for r in range(nranks)] if n_float else None
            if Gf is not None and step == 3:
                Gf[nranks - 1][n_float // 2] = np.nan
            prog.set_grads(G, Gf)
            hb = _buckets(n_half, 5, rng)
            fb = _buckets(n_float, 5, rng)
            if not bucketed:
                flags_seen.append(prog.step(1e-2, 0.01, 64.0))
                continue
            order = list(rng.permutation(5))          # buckets need not come in index order
            for g in prog.groups:
                g.step_begin()
            for pos, b in enumerate(order):
                for r, g in enumerate(prog.groups):
                    g.exec_bucket(hb[b], fb[b], 1e-2, 0.01, 64.0,
                                  stream_ptr(prog.devices[r]), last=(pos == 4))
            fl = [g.flags(stream_ptr(prog.devices[r])) for r, g in enumerate(prog.groups)]
            assert all(f == fl[0] for f in fl)
            flags_seen.append(fl[0])
        out = {"flags": flags_seen, "iter": prog.groups[0].iter}
        for r in range(nranks):
            out[f"w{r}"] = prog.weights_half(r) if n_half else None
            out[f"wf{r}"] = prog.weights_float(r) if n_float else None
            for which in range(3):
                out[f"h{r}{which}"] = prog.state(r, capi.HALF, which) if n_half else None
            for which in range(2):
                out[f"f{r}{which}"] = prog.state(r, capi.FLOAT, which) if n_float else None
        return out
    finally:
        prog.close()


def _same(a, b):
    assert a["flags"] == b["flags"] and a["iter"] == b["iter"]
    assert any(f != (0, 0, 0) for f in a["flags"])
    for k in a:
        if k in ("flags", "iter") or a[k] is None:
            continue
        assert np.array_equal(a[k].view(np.uint8), b[k].view(np.uint8)), k


@pytest.mark.parametrize("variant", [None, 1, 2])
@pytest.mark.parametrize("nranks", [1, 2, 4])
def test_bucketed_step_equals_whole_step(nranks, variant):
    for n_half, n_float in ((2048 * 5 * nranks + 48, 1040), (272, 0)):
        _same(_run(nranks, n_half, n_float, False, variant),
              _run(nranks, n_half, n_float, True, variant))


@pytest.mark.multigpu
def test_bucketed_step_two_gpus():
    n_half, n_float = 2048 * 9 + 80, 528
    _same(_run(2, n_half, n_float, False, None, devices=[0, 1]),
          _run(2, n_half, n_float, True, None, devices=[0, 1]))


def test_bucket_call_order_is_checked():
    g = AdamGroup.create(0, 1, 0, 4096, 0)
    try:
        g.init_master(stream_ptr())
        with pytest.raises(B200OptError) as e:
            g.exec_bucket((0, 16), (0, 0), 1e-3, 0.0, 1.0, stream_ptr(), last=True)
        assert e.value.status == capi.ESTATE
        g.step_begin()
        with pytest.raises(B200OptError) as e:
            g.exec(1e-3, 0.0, 1.0, stream_ptr())        # a bucketed step is open
        assert e.value.status == capi.ESTATE
        with pytest.raises(B200OptError) as e:
            g.exec_bucket((4000, 200), (0, 0), 1e-3, 0.0, 1.0, stream_ptr())
        assert e.value.status == capi.EINVAL
        g.exec_bucket((0, 4096), (0, 0), 1e-3, 0.0, 1.0, stream_ptr(), last=True)
        assert g.flags(stream_ptr()) == (0, 0, 0) and g.iter == 1
        g.exec(1e-3, 0.0, 1.0, stream_ptr())
        assert g.flags(stream_ptr()) == (0, 0, 0) and g.iter == 2
    finally:
        g.destroy()
