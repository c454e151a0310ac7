"""Worker of the multi-process tests; started once per rank by
torch.distributed.run (see tests/test_multigpu.py and tests/test_gloo_cpu.py).

mode "gloo":  CPU only.  Checks the launcher plumbing (handle exchange order,
              max-over-ranks) and that two ranks which each hold only their own
              gradients reach bit-identical flag sums and loss scales through the
              oracle's rank-ordered reduction.
mode "gpu":   one GPU per rank.  Every rank steps the CUDA path through the C ABI
              with peers attached over CUDA IPC and checks flags, loss scale and
              its shard's state against the oracle.
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from oracle import oracle as orc  # noqa: E402
from saga_b200 import launch  # noqa: E402
from tests import synth  # noqa: E402


class FakeGroup:
    """Stands in for AdamGroup where there is no GPU: records what it is given."""

    def __init__(self, rank, nranks):
        self.rank, self.nranks, self.attached = rank, nranks, {}

    def ipc_export(self):
        return bytes([self.rank]) * 64

    def ipc_attach(self, q, hb):
        self.attached[q] = hb


def run_gloo(out_path):
    dist.init_process_group("gloo")
    rank, world, _ = launch.env_rank()
    fg = FakeGroup(rank, world)
    launch.wire_process_group(fg)
    assert sorted(fg.attached) == [q for q in range(world) if q != rank]
    assert all(hb == bytes([q]) * 64 for q, hb in fg.attached.items())
    assert launch.max_over_ranks([1.0 + rank, 5.0 - rank]) == [float(world), 5.0]
    assert launch.broadcast_bytes(b"id-from-0" if rank == 0 else b"", 0) == b"id-from-0"

    # file descriptors between ranks: every rank sends the write end of a pipe to every
    # other rank, which writes its own rank number into it
    ex = launch.FdExchange(rank, world)
    rd, wr = os.pipe()
    for q in range(world):
        if q != rank:
            ex.send(q, wr, 40 + rank)
    os.close(wr)
    for src, tag, fd in ex.recv(world - 1):
        assert tag == 40 + src
        os.write(fd, bytes([rank]))
        os.close(fd)
    dist.barrier()
    assert sorted(os.read(rd, 64)) == [q for q in range(world) if q != rank]
    os.close(rd)
    ex.close()

    # each rank owns only its gradients; the reduction needs everyone's
    n, steps = 4096, 12
    W0 = synth.weights_half(n, seed=5)
    st = orc.MultiRankState(world, [W0] * world)
    scale = np.float32(256.0)
    scales = []
    for step in range(1, steps + 1):
        mine = synth.grads_half(n, scale, step, rank=rank, seed=5,
                                inject_inf_every=5 if rank == 1 else 0)
        if step == 7:
            mine[rank * (n // world) + 3] = 0x7800  # a range flag in every rank's shard
        gathered = [torch.zeros(n, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(mine.astype(np.int32)))
        G = [g.numpy().astype(np.uint16) for g in gathered]
        flags = st.step(G, None, scale, 1e-3, 0.01)
        scale = orc.policy_reference(scale, flags)
        scales.append(float(scale))
    all_scales = [None] * world
    dist.all_gather_object(all_scales, scales)
    assert all(s == all_scales[0] for s in all_scales)
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump({"ok": True, "scales": scales, "world": world}, f)
    dist.destroy_process_group()


def run_gpu(out_path, path="peer"):
    from saga_b200 import AdamGroup, LossScaler, capi
    rank, world, local = launch.env_rank()
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("cpu:gloo,cuda:nccl", device_id=dev)
    n_half, n_float, steps = 2048 * 6 * world + 80, 528, 8
    flags = {"fabric": capi.CREATE_FABRIC, "nvls": capi.CREATE_MULTICAST}.get(path, 0)
    grp = AdamGroup.create(rank, world, local, n_half, n_float, flags)
    grp.set_option(capi.OPT_TIMEOUT_MS, 20000)
    info = launch.wire_process_group(grp, with_nccl=(path == "nccl"))
    if path == "nvls" and not info["multicast"]:
        if rank == 0:
            with open(out_path, "w") as f:
                json.dump({"ok": True, "path": path, "ranks": [],
                           "skipped": "these GPUs do not support NVSwitch multicast"}, f)
        dist.barrier()
        grp.destroy()
        dist.destroy_process_group()
        return
    grp.set_option(capi.OPT_PATH, {"nccl": capi.PATH_NCCL, "nvls": capi.PATH_NVLS}.get(path, capi.PATH_PEER))
    if path == "nvls":
        grp.set_option(capi.OPT_KEEP_REDUCED, 1)
    sp = torch.cuda.current_stream(dev).cuda_stream
    W0, Wf0 = synth.weights_half(n_half, seed=9), synth.weights_float(n_float, seed=9)
    w, g = grp.buffers(capi.HALF)
    wf, gf = grp.buffers(capi.FLOAT)
    w.view(torch.int16).copy_(torch.from_numpy(W0.view(np.int16).copy()))
    wf.copy_(torch.from_numpy(Wf0.copy()))
    grp.init_master(sp)
    torch.cuda.synchronize(dev)
    dist.barrier()
    ost = orc.MultiRankState(world, [W0] * world, [Wf0] * world)
    scaler = LossScaler(64.0)
    worst = 0.0
    for step in range(1, steps + 1):
        G = [synth.grads_half(n_half, scaler.scale, step, rank=r, seed=9,
                              inject_inf_every=3 if r == 0 else 0) for r in range(world)]
        Gf = [synth.grads_float(n_float, scaler.scale, step, rank=r, seed=9) for r in range(world)]
        g.view(torch.int16).copy_(torch.from_numpy(G[rank].view(np.int16).copy()))
        gf.copy_(torch.from_numpy(Gf[rank].copy()))
        grp.exec(1e-2, 0.01, scaler.scale, sp)
        flags = grp.flags(sp)
        if path == "nvls":
            # the oracle is fed with the switch's sums, which every rank left in its own
            # shard of the gradient buffer: within one fp16 ulp of the rank-ordered sum
            sh = n_half // world
            parts = [None] * world
            dist.all_gather_object(parts, g[rank * sh:(rank + 1) * sh].view(torch.int16).cpu()
                                   .numpy().view(np.uint16).tobytes())
            reduced = G[0].copy()
            reduced[:world * sh] = np.frombuffer(b"".join(parts), dtype=np.uint16)
            d = orc.half_ulp_distance(reduced, orc.rank_ordered_sum_half(G))
            assert int(d[:world * sh].max()) <= 1, (rank, step, int(d.max()))
            G = [reduced] + [np.full(n_half, 0x8000, np.uint16) for _ in range(world - 1)]
        oflags = ost.step([x.copy() for x in G], [x.copy() for x in Gf], scaler.scale, 1e-2, 0.01)
        if path != "nccl":
            assert flags == oflags, (rank, step, flags, oflags)
        scaler.update(oflags if path == "nccl" else flags)
        for which, ref in ((0, ost.m[rank]), (1, ost.v[rank]), (2, ost.c[rank])):
            worst = max(worst, synth.rel_err(grp.export_state(capi.HALF, which), ref))
        worst = max(worst, synth.rel_err(grp.export_state(capi.FLOAT, 0), ost.mf[rank]))
    torch.cuda.synchronize(dev)
    dist.barrier()
    mine = w.view(torch.int16).cpu().numpy().view(np.uint16)
    diff = np.abs(mine.astype(np.int32) - ost.W[0].astype(np.int32))
    # NCCL sums fp16 in fp16 in its own order: only the peer path is held to the
    # rank-ordered oracle; the NCCL path is reported
    tol = 1e-5 if path != "nccl" else 5e-2
    assert worst <= tol, (rank, worst)
    if path != "nccl":
        assert diff.max() <= 1
    gathered = [None] * world
    dist.all_gather_object(gathered, mine.tobytes())
    assert all(x == gathered[0] for x in gathered), "ranks hold different weights"
    res = [None] * world
    dist.all_gather_object(res, {"rank": rank, "worst_rel_err": worst,
                                 "w_ulp_diff_max": int(diff.max()), "scale": float(scaler.scale)})
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump({"ok": True, "path": path, "ranks": res}, f)
    dist.barrier()   # every rank has finished stepping before any arena is released
    grp.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    mode, out = sys.argv[1], sys.argv[2]
    if mode == "gloo":
        run_gloo(out)
    else:
        run_gpu(out, sys.argv[3] if len(sys.argv) > 3 else "peer")
