"""Tests that need two or more GPUs: the in-kernel cross-GPU waits, peer loads
and stores over NVLink, CUDA-IPC wiring between processes, the NCCL path and the
bounded wait when a rank never arrives.  Skipped on a single-GPU machine, where
tests/test_step_gpu.py covers the same arithmetic in serial mode."""
import json
import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

from saga_b200 import AdamGroup, LossScaler, capi
from saga_b200.capi import B200OptError
from tests import synth
from tests.gpu_util import Program, dev_u16, host_u16, stream_ptr
from tests.test_step_gpu import _run_trajectory

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ngpu():
    return torch.cuda.device_count()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("variant", [capi.KERNEL_DIRECT, capi.KERNEL_STAGED])
def test_two_gpus_one_process_matches_oracle(oracle, variant):
    """Both ranks in this process (Saga's model), kernels waiting for one another."""
    for n_half, n_float in ((16, 16), (8208, 528), (2048 * 7 * 2 + 80, 0)):
        _run_trajectory(oracle, 2, n_half, n_float, 6, 1e-2, 0.01, 64.0, seed=81,
                        inject_every=3, variant=variant, devices=[0, 1])


def test_two_gpus_fabric_arena_matches_oracle(oracle):
    """Arenas from the virtual-memory API (shareable by file descriptor), peer path."""
    _run_trajectory(oracle, 2, 2048 * 7 * 2 + 80, 528, 6, 1e-2, 0.01, 64.0, seed=84,
                    inject_every=3, devices=[0, 1], create_flags=capi.CREATE_FABRIC)


def _multicast_or_skip(ndev):
    if not all(AdamGroup.multicast_supported(d) for d in range(ndev)):
        pytest.skip("these GPUs do not support NVSwitch multicast")


def _run_multicast_trajectory(oracle, nranks, n_half, n_float, steps, seed):
    """The multicast path against the oracle, the way its arithmetic allows:

    * the switch's fp16 sum lands within one fp16 ulp of the correctly rounded
      rank-ordered sum (measured property of multimem.ld_reduce on f16x2; NCCL's own NVLS
      reduce-scatter, which Saga would use here, has the same arithmetic);
    * GIVEN that sum (the kernel leaves it in the gradient buffer, as ncclReduceScatter
      does in place), flags, loss scale, m, v, master and fp16 weights equal the oracle's
      bit for bit on every rank."""
    devices = list(range(nranks))
    W0 = synth.weights_half(n_half, seed=seed)
    Wf0 = synth.weights_float(n_float, seed=seed) if n_float else None
    prog = Program(nranks, n_half, n_float, devices=devices, path=capi.PATH_NVLS,
                   create_flags=capi.CREATE_MULTICAST)
    for g in prog.groups:
        g.set_option(capi.OPT_KEEP_REDUCED, 1)
    prog.set_weights([W0] * nranks, [Wf0] * nranks if n_float else None)
    ost = oracle.MultiRankState(nranks, [W0] * nranks, [Wf0] * nranks if n_float else None)
    gs = LossScaler(64.0)
    s = n_half // nranks
    worst_ulp, off_by_one = 0, 0
    try:
        for step in range(1, steps + 1):
            G = [synth.grads_half(n_half, gs.scale, step, rank=r, seed=seed,
                                  inject_inf_every=3 if r == 0 else 0) for r in range(nranks)]
            if step == 2:
                G[nranks - 1][min(7, s - 1)] = 0x7800  # 32768 in shard 0
                G[0][(nranks - 1) * s + min(8, s - 1)] = 0xF800  # -32768 in the last shard
            Gf = [synth.grads_float(n_float, gs.scale, step, rank=r, seed=seed)
                  for r in range(nranks)] if n_float else None
            prog.set_grads(G, Gf)
            flags = prog.step(1e-2, 0.01, gs.scale)
            reduced = G[0].copy()
            for r in range(nranks):
                reduced[r * s:(r + 1) * s] = host_u16(prog.Gh[r][r * s:(r + 1) * s])
            want = oracle.rank_ordered_sum_half(G)
            d = oracle.half_ulp_distance(reduced[:nranks * s], want[:nranks * s])
            worst_ulp = max(worst_ulp, int(d.max()))
            off_by_one += int((d != 0).sum())
            # the oracle fed with the switch's sums: rank 0 brings them, the others -0
            G2 = [reduced] + [np.full(n_half, 0x8000, np.uint16) for _ in range(nranks - 1)]
            oflags = ost.step(G2, [x.copy() for x in Gf] if Gf else None, gs.scale, 1e-2, 0.01)
            assert flags == oflags, (step, flags, oflags)
            gs.update(flags)
            for r in range(nranks):
                for which, ref in ((0, ost.m[r]), (1, ost.v[r]), (2, ost.c[r])):
                    got = prog.state(r, capi.HALF, which)
                    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32)), (step, r, which)
                assert np.array_equal(prog.weights_half(r), ost.W[0]), (step, r)
                if n_float:
                    assert np.array_equal(prog.weights_float(r).view(np.uint32),
                                          ost.Wf[0].view(np.uint32))
        assert worst_ulp <= 1, worst_ulp
        return off_by_one
    finally:
        prog.close()


def test_two_gpus_multicast_path(oracle):
    """Switch-reduced gradient loads and switch-replicated weight stores, two ranks."""
    _multicast_or_skip(2)
    for n_half, n_float in ((16, 16), (8208, 528), (2048 * 7 * 2 + 80, 0)):
        _run_multicast_trajectory(oracle, 2, n_half, n_float, 6, seed=85)
    _run_multicast_trajectory(oracle, 2, 2048 * 40 * 2 + 80, 0, 4, seed=88)


def test_what_the_switch_computes(tmp_path):
    """The measured properties of multimem.ld_reduce that the multicast path's parity rule
    rests on (tests/nvls_probe.cu): on f16x2 the switch's sum is deterministic, the same with
    and without .acc::f32, never more than one fp16 ulp from the correctly rounded sum -- but
    one ulp off for a good part of the values; on f32 it is the correctly rounded sum."""
    n = _ngpu()
    n = 8 if n >= 8 else (4 if n >= 4 else 2)
    _multicast_or_skip(n)
    exe = tmp_path / "nvls_probe"
    res = subprocess.run(["nvcc", "-std=c++17", "-O2", "-gencode", "arch=compute_100a,code=sm_100a",
                          "-I", os.path.join(ROOT, "include"),
                          os.path.join(ROOT, "tests", "nvls_probe.cu"),
                          os.path.join(ROOT, "saga_b200", "csrc", "fabric.cpp"), "-o", str(exe)],
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-3000:]
    res = subprocess.run([str(exe), str(n)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    rows = [json.loads(ln) for ln in res.stdout.splitlines() if ln.startswith("{")]
    print("\n".join(json.dumps(r) for r in rows))          # shown with pytest -s / on failure
    by = {r["form"]: r for r in rows}
    plain, acc, f32 = by["f16x2"], by["f16x2 acc::f32"], by["f32"]
    for r in (plain, acc):
        assert r["differ_between_runs"] == 0 and r["beyond"] == 0
        h = r["ulps_minus4_to_plus4"]
        assert sum(h[:3]) == 0 and sum(h[6:]) == 0          # never more than one ulp
        assert 0.05 * r["values"] < h[3] + h[5] < 0.5 * r["values"]   # but often one
    assert plain["ulps_minus4_to_plus4"] == acc["ulps_minus4_to_plus4"]
    assert f32["differ_from_correctly_rounded_sum"] == 0


def test_multicast_path_needs_its_object(oracle):
    prog = Program(2, 4096, devices=[0, 1], path=capi.PATH_NVLS)
    try:
        prog.set_weights([synth.weights_half(4096, seed=1)] * 2)
        with pytest.raises(B200OptError) as err:
            prog.groups[0].exec(1e-3, 0.0, 1.0, stream_ptr(0))
        assert err.value.status == capi.ESTATE
        assert prog.groups[0].iter == 0      # a refused step moves no counter
    finally:
        prog.close()


def test_all_gpus_multicast_path(oracle):
    """Four or eight ranks through the multicast path (same rule as with two)."""
    n = _ngpu()
    if n < 4:
        pytest.skip("needs >= 4 GPUs")
    n = 8 if n >= 8 else 4
    _multicast_or_skip(n)
    _run_multicast_trajectory(oracle, n, 2048 * 5 * n + 16, 528, 6, seed=86)
    _run_multicast_trajectory(oracle, n, 2048 * 40 * n + 16, 0, 3, seed=89)


def test_all_gpus_one_process_matches_oracle(oracle):
    n = _ngpu()
    if n < 4:
        pytest.skip("needs >= 4 GPUs")
    n = 8 if n >= 8 else 4
    _run_trajectory(oracle, n, 2048 * 5 * n + 16, 528, 6, 1e-2, 0.01, 64.0, seed=82,
                    inject_every=3, devices=list(range(n)))


def test_auto_path_falls_back_to_nccl_without_peer_access(oracle):
    """Wired as on a machine whose GPUs cannot reach one another's memory: the peer
    path is refused, AUTO steps through NCCL by itself."""
    n = 2048 * 4 + 16
    W0 = synth.weights_half(n, seed=87)
    groups = [AdamGroup.create(r, 2, r, n, 0) for r in range(2)]
    try:
        for g in groups:
            g.set_option(capi.OPT_ASSUME_NO_PEER_ACCESS, 1)
        for r, g in enumerate(groups):
            rc = capi.lib().b200opt_attach_local(g.handle, 1 - r, groups[1 - r].handle)
            assert rc == capi.OK
        for r, g in enumerate(groups):
            w, _ = g.buffers(capi.HALF)
            w.view(torch.int16).copy_(dev_u16(W0, r))
            g.init_master(stream_ptr(r))
        # no NCCL communicator yet: nothing can step this group
        with pytest.raises(B200OptError) as err:
            groups[0].exec(1e-3, 0.0, 64.0, stream_ptr(0))
        assert err.value.status == capi.EUNSUPPORTED and groups[0].iter == 0
        groups[0].set_option(capi.OPT_PATH, capi.PATH_PEER)
        with pytest.raises(B200OptError) as err:
            groups[0].exec(1e-3, 0.0, 64.0, stream_ptr(0))
        assert err.value.status == capi.EUNSUPPORTED
        groups[0].set_option(capi.OPT_PATH, capi.PATH_AUTO)
        # communicators are created from one thread per rank, as NCCL requires
        import threading
        uid = AdamGroup.nccl_unique_id()
        errs = []

        def init(g):
            try:
                torch.cuda.set_device(g.device)
                g.nccl_init(uid)
            except Exception as e:   # noqa: BLE001
                errs.append(e)
        ts = [threading.Thread(target=init, args=(g,)) for g in groups]
        [t.start() for t in ts]
        [t.join() for t in ts]
        assert not errs, errs
        ost = oracle.MultiRankState(2, [W0] * 2)
        G = [synth.grads_half(n, 64.0, 1, rank=r, seed=87) for r in range(2)]
        G[1][5] = 0x7C00
        for r, g in enumerate(groups):
            _, gr = g.buffers(capi.HALF)
            gr.view(torch.int16).copy_(dev_u16(G[r], r))

        def step(g):
            torch.cuda.set_device(g.device)
            g.exec(1e-2, 0.01, 64.0, stream_ptr(g.device))
        ts = [threading.Thread(target=step, args=(g,)) for g in groups]
        [t.start() for t in ts]
        [t.join() for t in ts]
        flags = [g.flags(stream_ptr(g.device)) for g in groups]
        oflags = ost.step([x.copy() for x in G], None, 64.0, 1e-2, 0.01)
        assert flags[0] == flags[1] == oflags      # two summands: fp16 and fp32 sums agree
        for r, g in enumerate(groups):
            assert synth.rel_err(g.export_state(capi.HALF, 2), ost.c[r]) <= 1e-6
    finally:
        for g in groups:
            g.destroy()


def test_driver_in_sagas_threading_model():
    """host/mt_driver: one std::thread per GPU, no host barrier inside the loop."""
    from saga_b200.build import build_driver
    drv = build_driver()
    nranks = 2
    res = subprocess.run([drv, str(nranks), str(1 << 20), "30"], capture_output=True, text=True,
                         timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    out = json.loads(res.stdout.strip().splitlines()[-1])
    assert out["ok"] and out["weights_identical"], out
    assert out["status"] == [0] * nranks
    # gradients are uniform in (-2, 2) at scale 1024: no overflow, scale grows x1.02 per step
    assert out["flags"] == [0, 0, 0] * 30
    want = np.float32(1024.0)
    for s in out["scales"]:
        want = np.float32(np.float64(want) * 1.02)
        assert np.float32(s) == want


def test_rank_that_never_steps_times_out_cleanly():
    """Host-side fault: rank 1 simply never calls step.  Rank 0's kernel gives up
    after the wait limit, the status reaches the host, the context stays usable."""
    n = 1 << 16
    groups = AdamGroup.create_group([0, 1], n, 0)
    try:
        for g in groups:
            g.set_option(capi.OPT_TIMEOUT_MS, 300)
            g.init_master(stream_ptr(g.device))
        torch.cuda.synchronize(0)
        torch.cuda.synchronize(1)
        groups[0].exec(1e-3, 0.0, 64.0, stream_ptr(0))
        with pytest.raises(B200OptError) as err:
            groups[0].flags(stream_ptr(0))
        assert err.value.status == capi.ETIMEOUT
        assert "rank 1" in str(err.value)
        # the handle refuses further steps instead of running on inconsistent state
        with pytest.raises(B200OptError) as err:
            groups[0].exec(1e-3, 0.0, 64.0, stream_ptr(0))
        assert err.value.status == capi.ESTATE
    finally:
        for g in groups:
            g.destroy()
    # the device context is intact: a fresh one-rank step runs and checks out
    prog = Program(1, 4096)
    try:
        prog.set_weights([synth.weights_half(4096, seed=1)])
        prog.set_grads([synth.grads_half(4096, 64.0, 1, seed=1)])
        assert prog.step(1e-3, 0.0, 64.0) == (0, 0, 0)
    finally:
        prog.close()


def test_mismatched_sizes_are_refused_at_wiring():
    a = AdamGroup.create(0, 2, 0, 4096, 0)
    b = AdamGroup.create(1, 2, 1, 8192, 0)
    try:
        rc = capi.lib().b200opt_attach_local(a.handle, 1, b.handle)
        assert rc == capi.EINVAL
        with pytest.raises(B200OptError) as err:   # peers not wired: no step
            a.exec(1e-3, 0.0, 1.0, stream_ptr(0))
        assert err.value.status == capi.ESTATE
    finally:
        a.destroy()
        b.destroy()


@pytest.mark.parametrize("path", ["peer", "fabric", "nvls", "nccl"])
def test_one_process_per_gpu(tmp_path, path):
    """torchrun-style launch: peers attached through b200opt_ipc_export/attach, or, for
    arenas from the virtual-memory API, through file descriptors ("fabric": peer path on
    such arenas; "nvls": the multicast path, skipped by the worker where unsupported)."""
    nproc = _ngpu() if _ngpu() in (4, 8) else 2
    out = tmp_path / f"mp_{path}.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node",
           str(nproc), "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "tests", "mp_worker.py"), "gpu", str(out), path]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-6000:]
    got = json.loads(out.read_text())
    assert got["ok"] and len(got["ranks"]) == nproc
    if got.get("skipped"):
        pytest.skip(got["skipped"])
    if path != "nccl":
        assert all(r["worst_rel_err"] <= 1e-5 and r["w_ulp_diff_max"] <= 1 for r in got["ranks"])
