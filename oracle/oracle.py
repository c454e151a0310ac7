"""ctypes access to the CPU oracle (oracle/liboracle.so) and, when present, to
the reference's own compiled Adam kernels (oracle/_ref/libsaga_ref_kernels.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by
bench.py's CPU-baseline leg, never by the saga_b200 package.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liboracle.so")
REF_LIB = os.path.join(HERE, "_ref", "libsaga_ref_kernels.so")

_u16p = np.ctypeslib.ndpointer(dtype=np.uint16, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(dtype=np.uint32, flags="C_CONTIGUOUS")
_szp = np.ctypeslib.ndpointer(dtype=np.uintp, flags="C_CONTIGUOUS")

_lib = None
_ref = None


def build():
    """(Re)builds liboracle.so, and oracle/_ref when the reference checkout exists."""
    subprocess.run(["make", "-s", "-C", HERE], check=True)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            build()
        L = C.CDLL(LIB)
        L.orc_h2f.restype = C.c_float
        L.orc_h2f.argtypes = [C.c_uint16]
        L.orc_f2h.restype = C.c_uint16
        L.orc_f2h.argtypes = [C.c_float]
        L.orc_selfcheck_fp16.restype = C.c_uint64
        L.orc_selfcheck_fp16.argtypes = [C.c_uint32, C.c_uint32, C.c_uint64]
        L.orc_bias_corrections.argtypes = [C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_float)]
        L.orc_alpha.restype = C.c_float
        L.orc_alpha.argtypes = [C.c_float]
        L.orc_rsqrt_rn.restype = C.c_float
        L.orc_rsqrt_rn.argtypes = [C.c_float]
        L.orc_adam_mixed.argtypes = [C.c_size_t, C.c_float, _u16p, _u16p, _f32p, _f32p, _f32p,
                                     C.c_float, C.c_float, C.c_float, C.c_float, _u32p, C.c_int]
        L.orc_adam_mixed_mt.argtypes = L.orc_adam_mixed.argtypes[:-1]
        L.orc_adam_f32.argtypes = [C.c_size_t, _f32p, _f32p, _f32p, _f32p, C.c_float, C.c_float,
                                   C.c_float, C.c_float, _u32p, C.c_int]
        L.orc_master_init.argtypes = [C.c_size_t, _u16p, _f32p]
        L.orc_flat_layout.restype = C.c_size_t
        L.orc_flat_layout.argtypes = [_szp, C.c_size_t, _szp]
        L.orc_policy_reference.argtypes = [C.POINTER(C.c_float), _u32p]
        L.orc_policy_interval.argtypes = [C.POINTER(C.c_float), C.POINTER(C.c_int), _u32p, C.c_int]
        L.orc_num_threads.restype = C.c_int
        L.orc_set_num_threads.argtypes = [C.c_int]
        L.orc_reduce_half_mt.argtypes = [C.c_int, C.POINTER(C.c_void_p), C.c_size_t, _u16p]
        pp = C.POINTER(C.c_void_p)
        L.orc_step_multi.argtypes = [C.c_int, C.c_size_t, pp, pp, pp, pp, pp, C.c_size_t, pp, pp,
                                     pp, pp, C.c_int, C.c_float, C.c_float, C.c_float, _u32p,
                                     C.c_int]
        _lib = L
    return _lib


# ------------------------------------------------------------------ scalars

def h2f(bits):
    return np.float32(lib().orc_h2f(int(bits)))


def f2h(value):
    return int(lib().orc_f2h(float(np.float32(value))))


def bias_corrections(it):
    a, b = C.c_float(), C.c_float()
    lib().orc_bias_corrections(int(it), C.byref(a), C.byref(b))
    return np.float32(a.value), np.float32(b.value)


def alpha(scale):
    return np.float32(lib().orc_alpha(float(np.float32(scale))))


def policy_reference(scale, flags):
    s = C.c_float(float(np.float32(scale)))
    lib().orc_policy_reference(C.byref(s), np.asarray(flags, dtype=np.uint32))
    return np.float32(s.value)


def policy_interval(scale, clean, flags, interval=2000):
    s = C.c_float(float(np.float32(scale)))
    c = C.c_int(int(clean))
    lib().orc_policy_interval(C.byref(s), C.byref(c), np.asarray(flags, dtype=np.uint32), interval)
    return np.float32(s.value), c.value


def flat_layout(sizes):
    sizes = np.asarray(sizes, dtype=np.uintp)
    offs = np.zeros(max(len(sizes), 1), dtype=np.uintp)
    total = lib().orc_flat_layout(sizes if len(sizes) else np.zeros(1, np.uintp), len(sizes), offs)
    return [int(o) for o in offs[:len(sizes)]], int(total)


# ------------------------------------------------------------------- kernels

def adam_mixed(w, g, m, v, c, alpha_, b1t, b2t, lr, l2, flags=None, model=1, threads=False):
    """In place on uint16 w/g (bit patterns) and float32 m/v/c; returns flags[3]."""
    if flags is None:
        flags = np.zeros(3, dtype=np.uint32)
    if threads:
        lib().orc_adam_mixed_mt(w.size, alpha_, w, g, m, v, c, b1t, b2t, lr, l2, flags)
    else:
        lib().orc_adam_mixed(w.size, alpha_, w, g, m, v, c, b1t, b2t, lr, l2, flags, model)
    return flags


def adam_f32(w, g, m, v, b1t, b2t, lr, l2, flags=None, model=1):
    if flags is None:
        flags = np.zeros(3, dtype=np.uint32)
    lib().orc_adam_f32(w.size, w, g, m, v, b1t, b2t, lr, l2, flags, model)
    return flags


def master_init(w_shard):
    c = np.empty(w_shard.size, dtype=np.float32)
    lib().orc_master_init(w_shard.size, np.ascontiguousarray(w_shard), c)
    return c


def num_threads():
    return int(lib().orc_num_threads())


def use_all_host_threads():
    """Makes the timed variants use every core this process may run on (launchers
    such as torchrun export OMP_NUM_THREADS=1)."""
    import os
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().orc_set_num_threads(n)
    return num_threads()


def reduce_half_threads(grads, out):
    """Rank-ordered fp32 sum of whole fp16 gradient buffers, all host threads."""
    arr = (C.c_void_p * len(grads))(*[g.ctypes.data for g in grads])
    lib().orc_reduce_half_mt(len(grads), arr, out.size, out)
    return out


class MultiRankState:
    """All ranks' buffers of one program, stepped by orc_step_multi.

    W, G: lists (per rank) of uint16 arrays (n_half); Wf, Gf: float32 (n_float).
    Shard state is created the reference way: m = v = 0, master = float(W shard).
    """

    def __init__(self, nranks, W, Wf=None):
        self.N = nranks
        self.n_half = W[0].size if W is not None else 0
        self.W = [np.ascontiguousarray(w, dtype=np.uint16).copy() for w in W] if W else []
        self.n_f32 = Wf[0].size if Wf else 0
        self.Wf = [np.ascontiguousarray(w, dtype=np.float32).copy() for w in Wf] if Wf else []
        sh, sf = self.n_half // nranks, self.n_f32 // nranks
        self.sh, self.sf = sh, sf
        self.m = [np.zeros(sh, np.float32) for _ in range(nranks)]
        self.v = [np.zeros(sh, np.float32) for _ in range(nranks)]
        self.c = [master_init(self.W[r][r * sh:(r + 1) * sh]) if sh else np.zeros(0, np.float32)
                  for r in range(nranks)]
        self.mf = [np.zeros(sf, np.float32) for _ in range(nranks)]
        self.vf = [np.zeros(sf, np.float32) for _ in range(nranks)]
        self.iter = 0

    @staticmethod
    def _pp(arrays, n):
        arr = (C.c_void_p * max(n, 1))()
        for i, a in enumerate(arrays):
            arr[i] = a.ctypes.data
        return arr

    def step(self, G, Gf, scale, lr, l2, model=1):
        """G / Gf: per-rank gradient arrays (modified in place like ncclReduceScatter).
        Returns the flag sums {range, inf, nan}."""
        N = self.N
        self.iter += 1
        G = [np.ascontiguousarray(g, dtype=np.uint16) for g in G] if self.n_half else []
        Gf = [np.ascontiguousarray(g, dtype=np.float32) for g in Gf] if self.n_f32 else []
        sums = np.zeros(3, dtype=np.uint32)
        empty = [np.zeros(1, np.float32)] * N
        lib().orc_step_multi(
            N, self.n_half,
            self._pp(self.W or empty, N), self._pp(G or empty, N), self._pp(self.m, N),
            self._pp(self.v, N), self._pp(self.c, N),
            self.n_f32,
            self._pp(self.Wf or empty, N), self._pp(Gf or empty, N), self._pp(self.mf, N),
            self._pp(self.vf, N),
            self.iter, float(np.float32(scale)), float(np.float32(lr)), float(np.float32(l2)),
            sums, model)
        return tuple(int(x) for x in sums)


def half_ulp_distance(a_bits, b_bits):
    """Distance between fp16 bit patterns in units in the last place, element-wise (finite
    values on a sign-magnitude number line; +0 and -0 coincide).  Where either value is inf
    or NaN the distance is 0 if both have the same class and sign, else a large number."""
    a = np.asarray(a_bits, dtype=np.uint16).astype(np.int64)
    b = np.asarray(b_bits, dtype=np.uint16).astype(np.int64)

    def line(x):
        mag = x & 0x7FFF
        return np.where(x & 0x8000, -mag, mag)
    d = np.abs(line(a) - line(b))
    special = ((a & 0x7C00) == 0x7C00) | ((b & 0x7C00) == 0x7C00)
    same = ((a & 0xFC00) == (b & 0xFC00)) & (((a & 0x3FF) != 0) == ((b & 0x3FF) != 0))
    return np.where(special, np.where(same, 0, 1 << 20), d)


def rank_ordered_sum_half(grads):
    """fp32 sum of the ranks' fp16 buffers in rank order, one rounding to fp16."""
    out = np.empty(grads[0].size, np.uint16)
    return reduce_half_threads([np.ascontiguousarray(g, dtype=np.uint16) for g in grads], out)


# ------------------------------------------------- reference kernels (GPU only)

def ref_available():
    return os.path.exists(REF_LIB)


def ref():
    """The reference's own adam_mixed / adam_float launchers (needs a GPU to run)."""
    global _ref
    if _ref is None:
        R = C.CDLL(REF_LIB)
        vp, f = C.c_void_p, C.c_float
        R.sagaref_adam_mixed.argtypes = [C.c_int, f, vp, vp, vp, vp, vp, f, f, f, f, vp, vp]
        R.sagaref_adam_float.argtypes = [C.c_int, vp, vp, vp, vp, f, f, f, f, vp, vp]
        _ref = R
    return _ref
