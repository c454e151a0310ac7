"""Seeded synthetic inputs of the benchmark configurations (numpy only).

They stand in for real training state with the shapes and value distributions
of the benchmark configurations: fp32 master weights N(0, 0.02) held as their
fp16 rounding, fp16 gradients N(0, 1e-3) times the loss scale, 160 tensors with
log-uniform sizes in 64..4M renormalised to 25.6 M elements, one +inf injected
every 50th step.  Every draw is keyed by (seed, rank, step) through a
counter-based generator, so CPU and GPU sides see identical bits.
"""
import numpy as np

SEED = 0x5A6A


def _rng(*key):
    k = np.zeros(2, dtype=np.uint64)
    k[0] = np.uint64(SEED)
    mix = 0
    for x in key:
        mix = (mix * 1000003 + int(x) + 1) & 0xFFFFFFFFFFFFFFFF
    k[1] = np.uint64(mix)
    return np.random.Generator(np.random.Philox(key=k))


def tensor_sizes(total=25_600_000, k=160, lo=64, hi=4 * 2 ** 20, seed=0):
    """k sizes, log-uniform in [lo, hi], renormalised so that they sum to ~total."""
    r = _rng(seed, 0xA11)
    sizes = np.exp(r.uniform(np.log(lo), np.log(hi), size=k))
    sizes = np.maximum(1, np.round(sizes * (total / sizes.sum()))).astype(np.int64)
    return [int(s) for s in sizes]


def weights_half(n, seed=0, rank=0):
    """Initial fp16 weights: N(0, 0.02) rounded to fp16 (bit patterns, uint16)."""
    r = _rng(seed, 0xBEE, rank)
    return (r.standard_normal(n, dtype=np.float32) * np.float32(0.02)).astype(np.float16).view(np.uint16)


def weights_float(n, seed=0):
    r = _rng(seed, 0xF10)
    return (r.standard_normal(n, dtype=np.float32) * np.float32(0.5) + np.float32(1.0)).astype(np.float32)


def grads_half(n, scale, step, rank=0, seed=0, inject_inf_every=0):
    """fp16 gradient bits: N(0, 1e-3) * scale, rounded to fp16 (may overflow to inf)."""
    r = _rng(seed, 0x6AD, rank, step)
    g = r.standard_normal(n, dtype=np.float32) * np.float32(1e-3) * np.float32(scale)
    with np.errstate(over="ignore"):
        h = g.astype(np.float16)
    if inject_inf_every and n and step % inject_inf_every == 0:
        h[int(r.integers(0, n))] = np.float16(np.inf)
    return h.view(np.uint16)


def grads_float(n, scale, step, rank=0, seed=0):
    r = _rng(seed, 0xF6A, rank, step)
    return (r.standard_normal(n, dtype=np.float32) * np.float32(1e-3) * np.float32(scale)).astype(np.float32)


def scatter_into_flat(layout_offsets, sizes, total, values):
    """Places a dense value stream into the padded flat buffer (padding stays 0)."""
    flat = np.zeros(total, dtype=values.dtype)
    pos = 0
    for o, s in zip(layout_offsets, sizes):
        flat[o:o + s] = values[pos:pos + s]
        pos += s
    return flat
