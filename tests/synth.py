"""Seeded synthetic inputs for the tests: the benchmark workload generators
(saga_b200.workload) plus the special values and error measures only tests need."""
import numpy as np

from saga_b200.workload import (SEED, grads_float, grads_half, scatter_into_flat,  # noqa: F401
                                tensor_sizes, weights_float, weights_half)


# fp16 bit patterns that exercise every branch of the overflow classification
SPECIAL_HALF = {
    "+inf": 0x7C00, "-inf": 0xFC00, "nan": 0x7E01, "-nan": 0xFD55,
    "+32768": 0x7800, "-32768": 0xF800, "65504": 0x7BFF, "32752": 0x77FF,
    "subnormal": 0x0001, "-subnormal": 0x83FF, "+0": 0x0000, "-0": 0x8000,
    "one": 0x3C00,
}


def rel_err(a, b):
    """Largest |a-b| relative to the element's magnitude plus the tensor's RMS.

    m and the master weights pass through zero (the terms of their sums cancel),
    where a purely element-wise ratio is unbounded; the RMS term keeps the measure
    finite there while staying a per-element relative error everywhere else."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    if a.size == 0:
        return 0.0
    rms = np.sqrt(np.mean(b * b))
    denom = np.abs(b) + rms
    denom[denom == 0] = 1.0
    return float(np.max(np.abs(a - b) / denom))


def strict_rel_err(a, b):
    """Largest |a-b| / |b| over the elements with b != 0; where b == 0, a must be 0 too
    (returns inf otherwise).  The element-wise reading of "1e-6 relative"."""
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    if a.size == 0:
        return 0.0
    nz = b != 0
    if np.any(a[~nz] != 0):
        return float("inf")
    if not nz.any():
        return 0.0
    return float(np.max(np.abs(a[nz] - b[nz]) / np.abs(b[nz])))
