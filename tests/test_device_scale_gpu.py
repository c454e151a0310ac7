"""The loss scale kept on the device: steps are enqueued back to back with no
host synchronise in between; flags, the scale trajectory and the optimizer
state must equal what the step-by-step host loop of the reference gives
(CudaProgram::step, src/cuda/cuda_program.cpp:293-302 of the Saga tree)."""
import numpy as np
import pytest
import torch

from saga_b200 import AdamGroup, capi
from saga_b200.capi import B200OptError
from tests import synth
from tests.gpu_util import dev_u16, stream_ptr

pytestmark = pytest.mark.gpu


def _oracle_run(oracle, nranks, n, steps, scale0, policy, interval, seed):
    """Step-by-step host loop: returns per-step gradients, flags, scales and the final state."""
    W0 = synth.weights_half(n, seed=seed)
    st = oracle.MultiRankState(nranks, [W0] * nranks)
    scale, clean = np.float32(scale0), 0
    grads, flags, scales = [], [], []
    for step in range(1, steps + 1):
        G = [synth.grads_half(n, scale, step, rank=r, seed=seed,
                              inject_inf_every=7 if r == 0 else 0) for r in range(nranks)]
        if step % 11 == 0:  # a range flag in two shards (or one, with a single rank)
            s = n // nranks
            for r in range(min(2, nranks)):
                G[r][r * s + 5] = 0x7800
        grads.append(G)
        fl = st.step([g.copy() for g in G], None, scale, 1e-3, 0.01)
        if policy == capi.POLICY_REFERENCE:
            scale = oracle.policy_reference(scale, fl)
        else:
            scale, clean = oracle.policy_interval(scale, clean, fl, interval)
        flags.append(fl)
        scales.append(scale)
    return W0, st, grads, flags, scales


@pytest.mark.parametrize("policy,interval", [(capi.POLICY_REFERENCE, 0), (capi.POLICY_INTERVAL, 5)])
def test_device_scale_matches_host_loop(oracle, policy, interval):
    n, steps = 1 << 16, 40
    W0, ost, grads, flags, scales = _oracle_run(oracle, 1, n, steps, 1024.0, policy,
                                                max(interval, 1), seed=91)
    g = AdamGroup.create(0, 1, 0, n, 0)
    try:
        w, gr = g.buffers(capi.HALF)
        w.view(torch.int16).copy_(dev_u16(W0))
        g.init_master(stream_ptr())
        g.device_scale_enable(1024.0, policy, max(interval, 1), log_capacity=64)
        stack = [dev_u16(G[0]) for G in grads]
        torch.cuda.synchronize()
        # before any step: the initial scale, step 0
        assert g.device_scale_peek() == (np.float32(1024.0), 0)
        seen = []
        for step in range(steps):        # no host synchronise inside this loop
            gr.view(torch.int16).copy_(stack[step], non_blocking=True)
            g.exec_device_scale(1e-3, 0.01, stream_ptr())
            seen.append(g.device_scale_peek())   # does not wait: any finished step's value
        scale, log = g.device_scale_read(stream_ptr(), capacity=64)
        # every peek saw the scale that belongs to the step number it came with
        # (or the initial one), and after the wait it is the last step's
        for s, k in seen:
            assert 0 <= k <= steps
        peek_scale, peek_step = g.device_scale_peek()
        assert peek_step == steps and peek_scale.tobytes() == scales[-1].tobytes()
        assert len(log) == steps
        for k in range(steps):
            assert log[k][:3] == flags[k], (k, log[k], flags[k])
            assert log[k][3].tobytes() == scales[k].tobytes(), (k, log[k][3], scales[k])
        assert scale.tobytes() == scales[-1].tobytes()
        assert g.iter == steps
        for which, ref in ((0, ost.m[0]), (1, ost.v[0]), (2, ost.c[0])):
            assert synth.rel_err(g.export_state(capi.HALF, which), ref) <= 1e-5
        # the live scale is readable by other kernels through its device address
        p = g.device_scale_ptr()
        assert p and p % 4 == 0
    finally:
        g.destroy()


def test_device_scale_log_is_a_ring_and_needs_enabling(oracle):
    n = 4096
    g = AdamGroup.create(0, 1, 0, n, 0)
    try:
        with pytest.raises(B200OptError) as err:
            g.exec_device_scale(1e-3, 0.0, stream_ptr())
        assert err.value.status == capi.ESTATE
        w, gr = g.buffers(capi.HALF)
        g.init_master(stream_ptr())
        g.device_scale_enable(8.0, log_capacity=4)
        for _ in range(10):
            g.exec_device_scale(1e-3, 0.0, stream_ptr())
        scale, log = g.device_scale_read(stream_ptr(), capacity=8)
        want = np.float32(8.0)
        seq = []
        for _ in range(10):
            want = np.float32(np.float64(want) * 1.02)
            seq.append(want)
        assert len(log) == 4 and [x[3] for x in log] == seq[-4:]
        assert scale == seq[-1]
    finally:
        g.destroy()


@pytest.mark.multigpu
def test_device_scale_two_gpus_agree(oracle):
    n, steps = 2048 * 6 + 16, 25
    W0, ost, grads, flags, scales = _oracle_run(oracle, 2, n, steps, 256.0, capi.POLICY_REFERENCE,
                                                1, seed=92)
    groups = AdamGroup.create_group([0, 1], n, 0)
    try:
        bufs = []
        for r, g in enumerate(groups):
            w, gr = g.buffers(capi.HALF)
            w.view(torch.int16).copy_(dev_u16(W0, r))
            g.init_master(stream_ptr(r))
            g.device_scale_enable(256.0, log_capacity=64)
            bufs.append((gr, [dev_u16(G[r], r) for G in grads]))
        torch.cuda.synchronize(0)
        torch.cuda.synchronize(1)
        for step in range(steps):
            for r, g in enumerate(groups):
                with torch.cuda.device(r):
                    bufs[r][0].view(torch.int16).copy_(bufs[r][1][step], non_blocking=True)
                g.exec_device_scale(1e-3, 0.01, stream_ptr(r))
        for r, g in enumerate(groups):
            scale, log = g.device_scale_read(stream_ptr(r), capacity=64)
            assert [x[:3] for x in log] == flags
            assert [x[3].tobytes() for x in log] == [s.tobytes() for s in scales]
            assert synth.rel_err(g.export_state(capi.HALF, 2), ost.c[r]) <= 1e-5
        assert (11 <= steps) and (2, 0, 0) in flags  # the x0.9 branch was exercised
    finally:
        for g in groups:
            g.destroy()
