"""CPU checks of the C-ABI library: it loads, exports every symbol the header
declares, and its host-only entry points agree with the oracle.  No GPU call."""
import ctypes as C
import os
import re

import numpy as np

from tests import synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "b200opt.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"B200OPT_API\s+[\w\s\*]*?\b(b200opt_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(built_library):
    names = _declared()
    assert len(names) >= 28
    handle = C.CDLL(built_library)
    for name in names:
        assert hasattr(handle, name), f"{name} declared in include/b200opt.h but not exported"
    from saga_b200 import capi
    assert sorted(capi.SIGNATURES) == names
    assert b"sm_100a" in capi.lib().b200opt_version()
    assert capi.lib().b200opt_strerror(capi.ETIMEOUT) != capi.lib().b200opt_strerror(capi.OK)


def test_missing_library_fails_loudly(built_library, monkeypatch):
    from saga_b200 import capi
    monkeypatch.setattr(capi, "_lib", None)
    monkeypatch.setattr(capi, "LIB_PATH", "/nonexistent/libb200opt.so")
    try:
        capi.lib()
    except ImportError as e:
        assert "no CPU or PyTorch fallback" in str(e)
    else:
        raise AssertionError("loading a missing library must raise")


def test_policy_update_matches_oracle_bit_for_bit(oracle):
    from saga_b200 import policy_update, capi
    rng = np.random.default_rng(7)
    a = b = np.float32(256.0)
    for step in range(5000):
        r = rng.random()
        flags = (0, 0, 0) if r > 0.2 else (int(rng.integers(0, 4)), int(rng.integers(0, 2)),
                                           int(rng.integers(0, 2)))
        a, _ = policy_update(a, flags)
        b = oracle.policy_reference(b, flags)
        assert a.tobytes() == b.tobytes(), step
    a = b = np.float32(1024.0)
    sa = sb = 0
    for step in range(1, 6001):
        flags = (1, 1, 0) if step % 50 == 0 and step < 2500 else (0, 0, 0)
        a, sa = policy_update(a, flags, capi.POLICY_INTERVAL, sa, 2000)
        b, sb = oracle.policy_interval(b, sb, flags, 2000)
        assert (a.tobytes(), sa) == (b.tobytes(), sb), step


def test_bias_corrections_and_layout_match_oracle(oracle):
    from saga_b200 import bias_corrections, FlatLayout, capi
    for it in (1, 2, 3, 17, 100, 2100, 100000):
        assert bias_corrections(it) == oracle.bias_corrections(it)
    sizes = synth.tensor_sizes()
    lay = FlatLayout(sizes)
    offs, total = oracle.flat_layout(sizes)
    assert (lay.offsets, lay.total) == (offs, total)
    assert FlatLayout([]).total == 0
    b1, b2 = C.c_float(), C.c_float()
    assert capi.lib().b200opt_bias_corrections(0, C.byref(b1), C.byref(b2)) == capi.EINVAL


def test_argument_checks_without_a_gpu(built_library):
    from saga_b200 import capi
    L = capi.lib()
    h = C.c_void_p()
    assert L.b200opt_create(C.byref(h), 0, 0, 0, 16, 0) == capi.EINVAL      # nranks < 1
    assert L.b200opt_create(C.byref(h), 2, 2, 0, 16, 0) == capi.EINVAL      # rank out of range
    assert L.b200opt_create(C.byref(h), 0, 9, 0, 16, 0) == capi.EINVAL      # more than MAX_RANKS
    assert L.b200opt_destroy(None) == capi.EINVAL
    assert L.b200opt_step(None, 1e-3, 0.0, 1.0, None) == capi.EINVAL
    s = C.c_float(1.0)
    fl = (C.c_uint32 * 3)(0, 0, 0)
    assert L.b200opt_policy_update(C.byref(s), fl, 7, None, 0) == capi.EINVAL
    assert L.b200opt_policy_update(C.byref(s), fl, capi.POLICY_INTERVAL, None, 2000) == capi.EINVAL


def test_header_is_plain_c(tmp_path):
    """include/b200opt.h must compile as C99 on its own: it is what foreign hosts bind."""
    import subprocess
    src = tmp_path / "use_header.c"
    src.write_text('#include "b200opt.h"\n'
                   'int main(void) { b200opt_t *h = 0; (void)h; return B200OPT_MAX_RANKS == 8 ? 0 : 1; }\n')
    res = subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", "-fsyntax-only",
                          "-I", os.path.join(ROOT, "include"), str(src)],
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stderr


def test_path_rule(built_library):
    """Which collective path a step takes, including the fallback to NCCL when the
    GPUs cannot reach one another's memory (no GPU needed: the rule is host-only)."""
    from saga_b200 import capi
    L = capi.lib()

    def choose(req, nranks=8, serial=0, reach=1, nccl=0, mc=0, n=1 << 20, cross=0):
        out = C.c_int(-1)
        rc = L.b200opt_choose_path(req, nranks, serial, reach, nccl, mc, n, cross, C.byref(out))
        return rc, out.value

    A, P, N, M = capi.PATH_AUTO, capi.PATH_PEER, capi.PATH_NCCL, capi.PATH_NVLS
    # default: the bit-exact peer kernel, never the multicast path by itself
    assert choose(A) == (capi.OK, P)
    assert choose(A, nccl=1, mc=1) == (capi.OK, P)
    # no peer access: NCCL by itself; nothing usable without a communicator
    assert choose(A, reach=0, nccl=1) == (capi.OK, N)
    assert choose(A, reach=0, nccl=0)[0] == capi.EUNSUPPORTED
    assert choose(P, reach=0, nccl=1)[0] == capi.EUNSUPPORTED
    # measured crossover: NCCL only below it and only with a communicator
    assert choose(A, nccl=1, n=1000, cross=4096) == (capi.OK, N)
    assert choose(A, nccl=0, n=1000, cross=4096) == (capi.OK, P)
    assert choose(A, nccl=1, n=8192, cross=4096) == (capi.OK, P)
    # explicit requests need what they run on
    assert choose(N, nccl=0)[0] == capi.ESTATE
    assert choose(N, nccl=1) == (capi.OK, N)
    assert choose(M, mc=0)[0] == capi.ESTATE
    assert choose(M, mc=1) == (capi.OK, M)
    # one rank, or ranks stepped serially on one GPU: always the peer-pointer kernel
    assert choose(N, nranks=1, nccl=1) == (capi.OK, P)
    assert choose(A, nranks=4, serial=1, reach=0) == (capi.OK, P)
    assert choose(M, nranks=4, serial=1, mc=1)[0] == capi.EUNSUPPORTED
    assert choose(7)[0] == capi.EINVAL
    assert L.b200opt_choose_path(A, 2, 0, 1, 0, 0, 16, 0, None) == capi.EINVAL
