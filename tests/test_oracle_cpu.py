"""CPU checks of the oracle itself (no GPU): conversions, scalars, the policy,
the Adam restatement against an independent numpy evaluation, the flat layout
and the multi-rank step's bookkeeping."""
import numpy as np
import pytest

from tests import synth


def test_fp16_conversions_match_cpu_instructions(oracle):
    # 2^24 float patterns spread over the whole range plus all 65536 half patterns
    assert oracle.lib().orc_selfcheck_fp16(0, 257, 1 << 24) == 0
    # dense sweep across the half-precision boundaries: subnormal edge, 65504/inf edge
    for start in (0x33000000, 0x38000000, 0x477FE000 - 4096, 0x7F7FF000):
        assert oracle.lib().orc_selfcheck_fp16(start, 1, 1 << 16) == 0


def test_fp16_conversions_match_numpy(oracle):
    rng = np.random.default_rng(1)
    bits = rng.integers(0, 1 << 32, size=20000, dtype=np.uint64).astype(np.uint32)
    f = bits.view(np.float32)
    f = f[np.isfinite(f)]
    with np.errstate(over="ignore"):
        want = f.astype(np.float16).view(np.uint16)
    got = np.array([oracle.f2h(x) for x in f], dtype=np.uint16)
    assert np.array_equal(got, want)
    h = np.arange(65536, dtype=np.uint16)
    back = np.array([oracle.h2f(int(x)) for x in h], dtype=np.float32)
    ref = h.view(np.float16).astype(np.float32)
    ok = (back.view(np.uint32) == ref.view(np.uint32)) | (np.isnan(back) & np.isnan(ref))
    assert ok.all()


def test_f2h_ties_and_edges(oracle):
    assert oracle.f2h(65504.0) == 0x7BFF
    assert oracle.f2h(65519.996) == 0x7BFF      # below the tie: stays finite
    assert oracle.f2h(65520.0) == 0x7C00        # tie rounds to even = inf
    assert oracle.f2h(-65520.0) == 0xFC00
    assert oracle.f2h(2.0 ** -25) == 0x0000     # tie to even -> 0
    assert oracle.f2h(np.nextafter(np.float32(2.0 ** -25), np.float32(1))) == 0x0001
    assert oracle.f2h(2.0 ** -24) == 0x0001
    assert oracle.f2h(float("nan")) == 0x7FFF
    assert oracle.f2h(-0.0) == 0x8000


def test_bias_corrections_are_double_then_float(oracle):
    for it in (1, 2, 10, 100, 1000, 5000, 100000):
        b1t, b2t = oracle.bias_corrections(it)
        assert b1t == np.float32(1.0 / (1.0 - 0.9 ** it))
        assert b2t == np.float32(1.0 / (1.0 - 0.999 ** it))
    assert oracle.bias_corrections(1)[0] == np.float32(10.000000000000002)


def test_policy_reference_uses_double_factors(oracle):
    s = np.float32(64.0)
    mine = np.float32(64.0)
    rng = np.random.default_rng(3)
    differs_from_float_factor = False
    sf = np.float32(64.0)
    for step in range(3000):
        r = rng.random()
        flags = (0, 0, 0)
        if r < 0.03:
            flags = (1, 1, 0)
        elif r < 0.04:
            flags = (1, 0, 2)
        elif r < 0.10:
            flags = (2, 0, 0)
        elif r < 0.2:
            flags = (1, 0, 0)       # range on one rank only: still x1.02
        s = oracle.policy_reference(s, flags)
        k = 0.5 if (flags[1] or flags[2]) else (0.9 if flags[0] > 1 else 1.02)
        mine = np.float32(np.float64(mine) * k)
        sf = np.float32(sf * np.float32(k))
        differs_from_float_factor |= sf != s
        assert s == mine, step
    assert differs_from_float_factor  # the double literal is load-bearing


def test_policy_interval(oracle):
    s, clean = np.float32(1024.0), 0
    for step in range(1, 4101):
        flags = (1, 1, 0) if step == 50 else (0, 0, 0)
        s, clean = oracle.policy_interval(s, clean, flags, 2000)
    # halved at 50, doubled after 2000 and 4000 clean steps
    assert s == np.float32(2048.0)


def _numpy_adam_mixed(w, g, m, v, c, alpha, b1t, b2t, lr, l2):
    """Independent restatement, every operation rounded to float32 (no fusing)."""
    f32 = np.float32
    b1, b2, e = f32(0.9), f32(0.999), f32(1e-8)
    flags = [0, 0, 0]
    rng_mask = (g & 0x7800) == 0x7800
    infnan = (g & 0x7C00) == 0x7C00
    nan = infnan & ((g & 0x3FF) != 0)
    flags[0] = int(rng_mask.any())
    flags[1] = int((infnan & ~nan).any())
    flags[2] = int(nan.any())
    keep = ~infnan
    with np.errstate(invalid="ignore", over="ignore"):
        dw = g.view(np.float16).astype(f32) * f32(alpha)
        m2 = b1 * m + (f32(1.0) - b1) * dw
        v2 = b2 * v + ((f32(1.0) - b2) * dw) * dw
        mh = m2 * f32(b1t)
        vh = v2 * f32(b2t)
        rs = (1.0 / np.sqrt((vh + e).astype(np.float64))).astype(f32)
        w2 = (c - (f32(lr) * mh) * rs) - (f32(lr) * f32(l2)) * c
    m[keep], v[keep], c[keep] = m2[keep], v2[keep], w2[keep]
    w[keep] = w2[keep].astype(np.float16).view(np.uint16)
    return tuple(flags)


@pytest.mark.parametrize("n", [16, 272, 4112])
def test_adam_mixed_uncontracted_model_equals_numpy(oracle, n):
    w = synth.weights_half(n, seed=5)
    c = oracle.master_init(w)
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    w2, c2, m2, v2 = w.copy(), c.copy(), m.copy(), v.copy()
    scale = np.float32(1024.0)
    for step in range(1, 6):
        g = synth.grads_half(n, scale, step, seed=5)
        if step == 3:
            for k, bits in enumerate(synth.SPECIAL_HALF.values()):
                g[(k * 7) % n] = bits
        b1t, b2t = oracle.bias_corrections(step)
        al = oracle.alpha(scale)
        fl = oracle.adam_mixed(w, g, m, v, c, al, b1t, b2t, 1e-3, 0.01, model=0)
        fl2 = _numpy_adam_mixed(w2, g, m2, v2, c2, al, b1t, b2t, 1e-3, 0.01)
        assert tuple(fl) == fl2
        assert np.array_equal(m.view(np.uint32), m2.view(np.uint32))
        assert np.array_equal(v.view(np.uint32), v2.view(np.uint32))
        assert np.array_equal(c.view(np.uint32), c2.view(np.uint32))
        assert np.array_equal(w, w2)
        scale = oracle.policy_reference(scale, fl)


def test_adam_mixed_models_agree_within_tolerance(oracle):
    n = 1 << 16
    w = synth.weights_half(n, seed=9)
    st = [dict(w=w.copy(), c=oracle.master_init(w), m=np.zeros(n, np.float32),
               v=np.zeros(n, np.float32)) for _ in range(3)]
    scale = np.float32(1024.0)
    for step in range(1, 21):
        g = synth.grads_half(n, scale, step, seed=9)
        b1t, b2t = oracle.bias_corrections(step)
        al = oracle.alpha(scale)
        flags = []
        for k, s in enumerate(st):
            flags.append(tuple(oracle.adam_mixed(s["w"], g, s["m"], s["v"], s["c"], al, b1t, b2t,
                                                 1e-3, 0.01, model=min(k, 1), threads=(k == 2))))
        assert flags[0] == flags[1] == flags[2]
        scale = oracle.policy_reference(scale, flags[0])
    # the multi-threaded timing variant is the fused model, bit for bit
    for key in "wcmv":
        assert np.array_equal(st[1][key], st[2][key])
    # fused vs unfused stay within the per-step budget accumulated over 20 steps
    for key in "cmv":
        assert synth.rel_err(st[0][key], st[1][key]) < 1e-5


def test_skipped_elements_keep_everything(oracle):
    n = 64
    w = synth.weights_half(n, seed=2)
    c = oracle.master_init(w)
    m = np.full(n, 0.25, np.float32)
    v = np.full(n, 0.5, np.float32)
    g = synth.grads_half(n, 1024.0, 1, seed=2)
    g[0], g[17], g[63] = 0x7C00, 0xFC00, 0x7E01
    g[5] = 0x7800  # 32768: range flag, but updated
    w0, c0 = w.copy(), c.copy()
    fl = oracle.adam_mixed(w, g, m, v, c, oracle.alpha(1024.0), 10.0, 1000.0, 1e-3, 0.01)
    assert tuple(fl) == (1, 1, 1)
    for i in (0, 17, 63):
        assert (w[i], c[i], m[i], v[i]) == (w0[i], c0[i], np.float32(0.25), np.float32(0.5))
    assert c[5] != c0[5] and m[5] != np.float32(0.25)
    assert c[1] != c0[1]


def test_adam_f32_flags_and_no_range(oracle):
    n = 40
    w = synth.weights_float(n)
    g = synth.grads_float(n, 64.0, 1)
    g[3], g[9], g[20] = np.inf, np.nan, 1e15  # huge but finite: no flag at all
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    w0 = w.copy()
    fl = oracle.adam_f32(w, g, m, v, 10.0, 1000.0, 1e-3, 0.0)
    assert tuple(fl) == (0, 1, 1)
    assert w[3] == w0[3] and w[9] == w0[9] and m[3] == 0 and v[9] == 0
    assert w[20] != w0[20]


def test_flat_layout_pads_each_tensor_to_16(oracle):
    sizes = [1, 16, 17, 100, 4096, 5]
    offs, total = oracle.flat_layout(sizes)
    assert offs == [0, 16, 32, 64, 176, 4272]
    assert total == 4288 and total % 16 == 0
    sizes = synth.tensor_sizes()
    offs, total = oracle.flat_layout(sizes)
    assert len(sizes) == 160 and abs(sum(sizes) - 25_600_000) < 200
    assert total % 16 == 0 and total - sum(sizes) < 16 * 160


def test_reduction_is_rank_ordered_fp32_then_one_rounding(oracle):
    # 2048 + 1 + 1: fp16 pairwise sums lose both ones (2048+1 ties to 2048), the
    # fp32 sum keeps them: 2050
    N, n = 3, 48
    W = [np.zeros(n, np.uint16) for _ in range(N)]
    st = oracle.MultiRankState(N, W)
    vals = [2048.0, 1.0, 1.0]
    G = [np.full(n, np.float16(x)).view(np.uint16).copy() for x in vals]
    st.step(G, None, 1.0, 0.0, 0.0)
    s = n // N
    for r in range(N):
        shard = G[r][r * s:(r + 1) * s].view(np.float16)
        assert (shard == np.float16(2050.0)).all()


def test_multirank_flag_sums_are_per_shard(oracle):
    N, n = 4, 64
    W = [synth.weights_half(n, seed=1) for _ in range(N)]
    st = oracle.MultiRankState(N, W)
    G = [np.zeros(n, np.uint16) for _ in range(N)]
    G[0][1] = 0x7800      # shard 0 (elements 0..15): range
    G[2][20] = 0x7800     # shard 1: range (contributed by rank 2's gradient)
    G[1][40] = 0x7C00     # shard 2: inf (also range)
    flags = st.step(G, None, 64.0, 1e-3, 0.01)
    assert flags == (3, 1, 0)
    # all ranks hold identical weights after the gather
    for r in range(1, N):
        assert np.array_equal(st.W[0], st.W[r])


def test_multirank_tail_beyond_divisible_part_untouched(oracle):
    N, n = 3, 16  # 16/3 = 5, element 15 belongs to nobody
    W = [synth.weights_half(n, seed=4) for _ in range(N)]
    st = oracle.MultiRankState(N, W)
    before = st.W[0].copy()
    G = [synth.grads_half(n, 64.0, 1, rank=r, seed=4) for r in range(N)]
    st.step(G, None, 64.0, 1e-2, 0.0)
    assert st.W[0][15] == before[15]
    assert (st.W[0][:15] != before[:15]).any()


def test_n_rank_step_with_one_contributing_rank_equals_one_rank_step(oracle):
    """x + 0 + ... + 0 is exact in fp32 and rounds back to x: with only rank 2 holding
    gradients, the N-rank oracle must reproduce the one-rank oracle bit for bit."""
    n, N = 4096, 4
    W0 = synth.weights_half(n, seed=8)
    one = oracle.MultiRankState(1, [W0])
    many = oracle.MultiRankState(N, [W0] * N)
    for step in range(1, 5):
        g = synth.grads_half(n, 128.0, step, seed=8, inject_inf_every=3)
        f1 = one.step([g.copy()], None, 128.0, 1e-2, 0.01)
        G = [np.zeros(n, np.uint16) for _ in range(N)]
        G[2] = g.copy()
        fN = many.step(G, None, 128.0, 1e-2, 0.01)
        # flags: the one-rank tuple is 0/1; the N-rank one counts shards that saw the class
        assert tuple(int(x > 0) for x in fN) == f1
    s = n // N
    assert np.array_equal(many.W[0], one.W[0])
    for r in range(N):
        assert np.array_equal(many.c[r].view(np.uint32), one.c[0][r * s:(r + 1) * s].view(np.uint32))
        assert np.array_equal(many.m[r].view(np.uint32), one.m[0][r * s:(r + 1) * s].view(np.uint32))


def test_two_rank_sum_is_symmetric(oracle):
    """A two-term fp32 sum commutes: swapping the two ranks' gradients changes nothing."""
    n = 2048
    W0 = synth.weights_half(n, seed=9)
    a = oracle.MultiRankState(2, [W0, W0])
    b = oracle.MultiRankState(2, [W0, W0])
    for step in range(1, 4):
        g0 = synth.grads_half(n, 64.0, step, rank=0, seed=9)
        g1 = synth.grads_half(n, 64.0, step, rank=1, seed=9, inject_inf_every=2)
        fa = a.step([g0.copy(), g1.copy()], None, 64.0, 1e-2, 0.0)
        fb = b.step([g1.copy(), g0.copy()], None, 64.0, 1e-2, 0.0)
        assert fa == fb
    assert np.array_equal(a.W[0], b.W[1])
    for r in range(2):
        assert np.array_equal(a.c[r].view(np.uint32), b.c[r].view(np.uint32))


def test_adam_update_is_invariant_under_power_of_two_loss_scale(oracle):
    """Multiplying gradients and the loss scale by 2^k is exact in fp16 (away from
    subnormals and overflow) and must leave the update unchanged bit for bit."""
    n = 4096
    w = synth.weights_half(n, seed=10)
    outs = []
    for k in (1.0, 32.0):
        g = (synth.grads_half(n, 16.0, 1, seed=10).view(np.float16).astype(np.float32)
             * np.float32(k)).astype(np.float16).view(np.uint16)
        ww, c = w.copy(), oracle.master_init(w)
        m, v = np.zeros(n, np.float32), np.zeros(n, np.float32)
        b1t, b2t = oracle.bias_corrections(1)
        fl = oracle.adam_mixed(ww, g, m, v, c, oracle.alpha(16.0 * k), b1t, b2t, 1e-3, 0.01)
        assert tuple(fl) == (0, 0, 0)
        outs.append((ww, m.copy(), v.copy(), c.copy()))
    for x, y in zip(outs[0], outs[1]):
        assert np.array_equal(x.view(np.uint8), y.view(np.uint8))
