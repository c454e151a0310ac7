"""The allocation-free entry point, b200opt_adam_mixed_static, through the C ABI.

Some users of this library may not allocate device memory once they are
running: their memory is planned once at start-up (as Saga itself does with its
tensor arena), or an allocation's implicit device synchronisation would stall
their step loop, or they live inside a fixed memory reservation.  For them the
library keeps the step kernel's scratch in a fixed array inside its own image.

This file is collected last on purpose: if it fails, a run that stops at the
first failure has already run every other test.  It passes on its own in a fresh
process and after the rest of the suite: the entry point shares one scratch
array per GPU with every earlier call and must not depend on what they left.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from saga_b200 import capi
from saga_b200 import optimizer as opt
from tests import synth
from tests.gpu_util import dev_f32, dev_u16, host_u16, stream_ptr

pytestmark = pytest.mark.gpu


def _call_static(n, alpha, t, g, b1t, b2t, lr, l2, flags):
    vp = C.c_void_p
    rc = capi.lib().b200opt_adam_mixed_static(
        n, alpha, vp(t["w"].data_ptr()), vp(g.data_ptr()), vp(t["m"].data_ptr()),
        vp(t["v"].data_ptr()), vp(t["c"].data_ptr()), b1t, b2t, lr, l2,
        vp(flags.data_ptr()), vp(stream_ptr()))
    assert rc == capi.OK, capi.lib().b200opt_strerror(rc)


@pytest.mark.parametrize("n", [16, 4112, (1 << 20) + 8])
def test_static_entry_point_matches_adam_mixed_on_two_calls_in_a_row(oracle, n):
    w0 = synth.weights_half(n, seed=77)
    c0 = oracle.master_init(w0)
    make = lambda: dict(w=dev_u16(w0), c=dev_f32(c0), m=torch.zeros(n, device="cuda"),
                        v=torch.zeros(n, device="cuda"))
    a, b = make(), make()
    aux = torch.zeros(4, dtype=torch.int32, device="cuda")
    # poison the output words: the entry point overwrites, it does not accumulate
    flags = torch.full((3,), 7, dtype=torch.int32, device="cuda")
    scale = np.float32(1024.0)
    for step in (1, 2):          # two calls in a row, the second builds on the first
        bits = synth.grads_half(n, scale, step, seed=77)
        if step == 2:
            bits[n // 2] = 0x7C00        # +inf: skipped element, inf and range flags
            bits[3] = 0x7800             # 32768: range flag, element still updated
        g = dev_u16(bits)
        b1t, b2t = oracle.bias_corrections(step)
        al = oracle.alpha(scale)
        aux.zero_()
        opt.adam_mixed(n, al, a["w"].data_ptr(), g.data_ptr(), a["m"].data_ptr(),
                       a["v"].data_ptr(), a["c"].data_ptr(), b1t, b2t, 1e-3, 0.01,
                       aux.data_ptr(), stream_ptr())
        _call_static(n, al, b, g, b1t, b2t, 1e-3, 0.01, flags)
        torch.cuda.synchronize()
        want = tuple(int(x) for x in aux.cpu()[:3])
        got = tuple(int(x) for x in flags.cpu())
        assert got == want == ((1, 1, 0) if step == 2 else (0, 0, 0))
        for key in "wmvc":     # same kernel, same arithmetic: bit for bit
            x, y = a[key], b[key]
            if x.dtype == torch.float32:
                x, y = x.view(torch.int32), y.view(torch.int32)
            assert torch.equal(x, y), (step, key)
        scale = oracle.policy_reference(scale, want)
    # and both agree with the oracle within the per-step tolerance
    ow, om, ov, oc = w0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32), c0.copy()
    scale = np.float32(1024.0)
    for step in (1, 2):
        bits = synth.grads_half(n, scale, step, seed=77)
        if step == 2:
            bits[n // 2] = 0x7C00
            bits[3] = 0x7800
        b1t, b2t = oracle.bias_corrections(step)
        fl = oracle.adam_mixed(ow, bits, om, ov, oc, oracle.alpha(scale), b1t, b2t, 1e-3, 0.01)
        scale = oracle.policy_reference(scale, fl)
    assert synth.rel_err(b["c"].cpu().numpy(), oc) <= 2e-6
    assert synth.rel_err(b["m"].cpu().numpy(), om) <= 2e-6
    assert np.array_equal(host_u16(b["w"]), ow)


def test_static_entry_point_allocates_nothing_and_accepts_an_empty_buffer(oracle):
    """After the first call on the device (which looks up the scratch array and opts the
    kernel in to its shared-memory size), further calls leave the amount of free device
    memory exactly where it was; n = 0 still reports (zero) flags; and a clean call after
    a flagged one does not inherit its flags from the shared scratch."""
    n = 1 << 16
    w0 = synth.weights_half(n, seed=78)
    t = dict(w=dev_u16(w0), c=dev_f32(oracle.master_init(w0)), m=torch.zeros(n, device="cuda"),
             v=torch.zeros(n, device="cuda"))
    flags = torch.full((3,), 9, dtype=torch.int32, device="cuda")
    clean = dev_u16(synth.grads_half(n, 64.0, 1, seed=78))
    bad_bits = synth.grads_half(n, 64.0, 2, seed=78)
    bad_bits[11] = 0x7E01          # NaN
    bad = dev_u16(bad_bits)
    b1t, b2t = oracle.bias_corrections(1)
    _call_static(n, oracle.alpha(64.0), t, clean, b1t, b2t, 1e-3, 0.0, flags)   # set-up call
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    _call_static(n, oracle.alpha(64.0), t, bad, b1t, b2t, 1e-3, 0.0, flags)
    torch.cuda.synchronize()
    assert tuple(int(x) for x in flags.cpu()) == (1, 0, 1)
    _call_static(n, oracle.alpha(64.0), t, clean, b1t, b2t, 1e-3, 0.0, flags)
    torch.cuda.synchronize()
    assert tuple(int(x) for x in flags.cpu()) == (0, 0, 0)      # nothing left over
    flags.fill_(9)
    _call_static(0, oracle.alpha(64.0), t, clean, b1t, b2t, 1e-3, 0.0, flags)
    torch.cuda.synchronize()
    assert tuple(int(x) for x in flags.cpu()) == (0, 0, 0)      # written also for n = 0
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, "the allocation-free entry point changed the free device memory"


def test_static_entry_point_rejects_sizes_beyond_its_scratch():
    vp = C.c_void_p
    flags = torch.zeros(3, dtype=torch.int32, device="cuda")
    x = torch.zeros(16, device="cuda")
    rc = capi.lib().b200opt_adam_mixed_static(
        capi.STATIC_MAX_ELEMS + 1, 1.0, vp(x.data_ptr()), vp(x.data_ptr()), vp(x.data_ptr()),
        vp(x.data_ptr()), vp(x.data_ptr()), 1.0, 1.0, 1e-3, 0.0, vp(flags.data_ptr()),
        vp(stream_ptr()))
    assert rc == capi.ETOOBIG
    assert b"scratch" in capi.lib().b200opt_strerror(rc)
    # nothing was launched: the output words are untouched
    torch.cuda.synchronize()
    assert int(flags.sum()) == 0
    # unaligned caller memory is refused rather than handled by an allocation
    rc = capi.lib().b200opt_adam_mixed_static(
        8, 1.0, vp(x.data_ptr() + 2), vp(x.data_ptr()), vp(x.data_ptr()), vp(x.data_ptr()),
        vp(x.data_ptr()), 1.0, 1.0, 1e-3, 0.0, vp(flags.data_ptr()), vp(stream_ptr()))
    assert rc == capi.EINVAL
