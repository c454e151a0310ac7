#!/usr/bin/env python
"""Benchmark of the fused gradient reduce-scatter + mixed-precision Adam +
weight all-gather step (the data-parallel parameter update of Saga) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N > 1 is launched as one process per GPU by torch.distributed.run; rank 0
prints ONE JSON line.  A "step" is one optimizer step over the whole flat
parameter buffer: at N ranks every rank contributes its own gradient buffer,
updates its 1/N shard and receives all updated weights.

Workload at every N: 25.6 M fp16 parameters in 160 tensors (sizes log-uniform
in 64..4 M, renormalised, each padded to 16 elements), fp32 master N(0, 0.02),
gradients N(0, 1e-3) x loss scale 1024, lr 1e-3, lambda 0.01.  Synthetic,
seeded; per-step state touched (717 MB at N=1) is larger than L2, so no flush
is needed between steps.
"""
import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

TOTAL_PARAMS = 25_600_000
LR, L2, SCALE0 = 1e-3, 0.01, 1024.0
NVLINK_MEASURED_GBS = 770.0   # peer copy per direction measured on this pool
NVLINK_NOMINAL_GBS = 900.0
HBM_FALLBACK_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the default one-rank
# kernel on this workload, from the ncu capture summarised in
# profiles/staged_step_kernel_n1_config2.md
NCU_TRAFFIC_N1_BYTES = 660_591_104


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return HBM_FALLBACK_GBS, "fallback"


def workload():
    from tests import synth
    from saga_b200 import FlatLayout
    sizes = synth.tensor_sizes(TOTAL_PARAMS, 160)
    return sizes, FlatLayout(sizes)


# ------------------------------------------------------------------ clocks

class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) from a
    thread while the timed regions run."""

    def __init__(self, device_index):
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80): "hw_power_brake",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.004)

    def start(self):
        if self.nv:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join()
        return {
            "sm_mhz": float(np.median(self.samples)) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


# ----------------------------------------------------------- CPU baseline leg

def cpu_baseline(n, budget_s=12.0, max_steps=5000):
    """The CPU restatement of the reference's adam_kernel_mp (the reference has
    no CPU implementation of this path), all host threads, on the full buffer."""
    from oracle import oracle as orc
    from tests import synth
    orc.use_all_host_threads()
    w = synth.weights_half(n, seed=1)
    c = orc.master_init(w)
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    g = synth.grads_half(n, SCALE0, 1, seed=1)
    b1t, b2t = orc.bias_corrections(1)
    al = orc.alpha(SCALE0)
    for _ in range(2):
        orc.adam_mixed(w, g, m, v, c, al, b1t, b2t, LR, L2, threads=True)
    t0 = time.perf_counter()
    steps = 0
    while steps < max_steps and (time.perf_counter() - t0 < budget_s or steps < 3):
        orc.adam_mixed(w, g, m, v, c, al, b1t, b2t, LR, L2, threads=True)
        steps += 1
    dt = time.perf_counter() - t0
    return {
        "value": n * steps / dt, "unit": "params/s", "cores": orc.num_threads(),
        "kind": "port",
        "sample": f"{steps} full steps over all {n} parameters "
                  f"({dt:.1f} s, OpenMP over elements, 28 B/param)",
        "ms_per_step": dt / steps * 1e3,
    }


def run_reference_arm(args):
    """--impl reference: the reference has no CPU (or buildable dnnl) training
    path, so this arm times the CPU restatement of its path on all host cores:
    per step the rank-ordered sum of the N ranks' gradient buffers (N > 1) and
    the mixed-precision Adam update of the same 25.6 M-parameter buffer."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as orc
    from tests import synth
    cores = orc.use_all_host_threads()
    world = max(args.gpus, 1)
    sizes, lay = workload()
    n = lay.total
    w = synth.weights_half(n, seed=1)
    c = orc.master_init(w)
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    grads = [synth.grads_half(n, SCALE0, 1, rank=r, seed=1) for r in range(world)]
    gsum = np.empty(n, np.uint16)
    al = orc.alpha(SCALE0)
    steps = min(args.steps, 200)

    def one_step(it):
        b1t, b2t = orc.bias_corrections(it)
        g = orc.reduce_half_threads(grads, gsum) if world > 1 else grads[0]
        orc.adam_mixed(w, g, m, v, c, al, b1t, b2t, LR, L2, threads=True)

    for it in range(1, args.warmup + 1):
        one_step(it)
    t0 = time.perf_counter()
    for it in range(args.warmup + 1, args.warmup + steps + 1):
        one_step(it)
    dt = time.perf_counter() - t0
    value = world * n * steps / dt
    sample = (f"{steps} full steps over all {n} parameters"
              + (f", each summing {world} gradient buffers first" if world > 1 else "")
              + f" ({dt:.1f} s; CPU restatement of src/cuda adam_kernel_mp, OpenMP over elements; "
                "the reference ships no CPU training path)")
    line = {
        "impl": "reference", "metric": "fused grad-reduce+Adam params/sec", "value": value,
        "unit": "params/s", "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup,
        "ms_per_step": dt / steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "config2: 25.6M fp16 params in 160 tensors, 1 optimizer step",
                   "n_params": n, "tensors": len(sizes)},
        "cpu_baseline": {"value": value, "unit": "params/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "params/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------- N-rank kernel on one GPU (ncu aid)

def run_serial_ranks(args):
    """All N ranks live on GPU 0 and are stepped in turn, so the N-rank instance
    of the step kernel can be captured by ncu (which never wraps a multi-rank
    command here).  Peer loads and stores hit local HBM: the line reports the
    SM-side cost of one rank's launch, not an NVLink figure, and is not a
    benchmark value."""
    import torch
    from saga_b200 import AdamGroup, capi
    N = args.serial_ranks
    sizes, lay = workload()
    n = args.params or lay.total
    dev = torch.device("cuda", 0)
    groups = AdamGroup.create_group([0] * N, n, 0)
    stream = torch.cuda.current_stream(dev)
    sp = stream.cuda_stream
    gen = torch.Generator(device=dev).manual_seed(0x5A6A)
    w0 = (torch.randn(n, device=dev, generator=gen) * 0.02).half()
    for r, g in enumerate(groups):
        if args.variant >= 0:
            g.set_option(capi.OPT_KERNEL_VARIANT, args.variant)
        if args.ctas_per_sm:
            g.set_option(capi.OPT_CTAS_PER_SM, args.ctas_per_sm)
        w, gr = g.buffers(capi.HALF)
        w.copy_(w0)
        gr.copy_((torch.randn(n, device=dev, generator=gen) * (1e-3 * SCALE0)).half())
        g.init_master(sp)
    torch.cuda.synchronize(dev)

    def one_round():
        for g in groups:
            g.exec(LR, L2, SCALE0, sp)

    for _ in range(max(args.warmup, 3)):
        one_round()
    torch.cuda.synchronize(dev)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for _ in range(args.steps):
        one_round()
    b.record(stream)
    torch.cuda.synchronize(dev)
    flags = groups[0].flags(sp)
    us = a.elapsed_time(b) / (args.steps * N) * 1e3
    # one rank's launch: N gradient shards in, m/v/master in and out, N weight shards out
    alg = (4 * n + 24 * n / N) / 1.0
    print(json.dumps({
        "mode": "serial-ranks (profiling aid, not a benchmark value)", "ranks_on_one_gpu": N,
        "n_params": n, "us_per_rank_launch": us, "local_hbm_gbs": alg / (us * 1e-6) / 1e9,
        "algorithmic_bytes_per_launch": alg, "flags": list(flags)}), flush=True)
    for g in groups:
        g.destroy()


# ------------------------------------------------------------------- our arm

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--params", type=int, default=0,
                    help="flat fp16 buffer of this many elements instead of the 160-tensor workload")
    ap.add_argument("--fp32-group", action="store_true",
                    help="put the parameters in the fp32 group (the reference's AdamF32 path: "
                         "fp32 weights and gradients, no master copy) instead of the fp16 group")
    ap.add_argument("--e2e-steps", type=int, default=0, help="default: min(steps, 50)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--with-ref-gpu", action="store_true",
                    help="also time the reference's own compiled Adam kernel (oracle/_ref) as a "
                         "GPU baseline beside the CPU one; off by default")
    ap.add_argument("--ctas-per-sm", type=int, default=0)
    ap.add_argument("--variant", type=int, default=-1)
    ap.add_argument("--stages", type=int, default=0)
    ap.add_argument("--grid", type=int, default=0)
    ap.add_argument("--path", default="auto", choices=["auto", "peer", "push", "nccl"])
    ap.add_argument("--with-allreduce-baseline", action="store_true",
                    help="N > 1: also time NCCL all-reduce of the whole fp16 gradient buffer followed "
                         "by the one-GPU Adam kernel over all parameters on every rank")
    ap.add_argument("--serial-ranks", type=int, default=0,
                    help="profiling aid: N ranks on ONE GPU, stepped one after the other "
                         "(no cross-GPU waits); times the N-rank kernel against local HBM only")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.serial_ranks:
        return run_serial_ranks(args)
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist
    from saga_b200 import AdamGroup, LossScaler, capi

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch N>1 through torch.distributed.run (one process per GPU)")
        args.gpus = world
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world,
                                device_id=dev)

    if args.params:
        sizes, n = [args.params], (args.params + 15) // 16 * 16
        wl = f"flat fp16 buffer of {n} elements, 1 optimizer step"
    else:
        sizes, lay = workload()
        n = lay.total
        wl = "config2: 25.6M fp16 params in 160 tensors, 1 optimizer step"

    f32 = args.fp32_group
    if f32:
        wl = wl.replace("fp16", "fp32") + " (fp32 group)"
    grp = AdamGroup.create(rank, world, local, 0 if f32 else n, n if f32 else 0)
    if world > 1:
        from saga_b200 import launch
        launch.wire_process_group(grp, with_nccl=True)
        grp.set_option(capi.OPT_PATH, {"auto": capi.PATH_AUTO, "peer": capi.PATH_PEER,
                                       "push": capi.PATH_PUSH, "nccl": capi.PATH_NCCL}[args.path])
    if args.ctas_per_sm:
        grp.set_option(capi.OPT_CTAS_PER_SM, args.ctas_per_sm)
    if args.variant >= 0:
        grp.set_option(capi.OPT_KERNEL_VARIANT, args.variant)
    if args.stages:
        grp.set_option(capi.OPT_STAGES, args.stages)
    if args.grid:
        grp.set_option(capi.OPT_GRID, args.grid)

    stream = torch.cuda.current_stream(dev)
    sp = stream.cuda_stream
    w, g = grp.buffers(capi.FLOAT if f32 else capi.HALF)
    gen = torch.Generator(device=dev).manual_seed(0x5A6A)          # same weights on every rank
    w.copy_((torch.randn(n, device=dev, generator=gen) * 0.02).to(w.dtype))
    gen_g = torch.Generator(device=dev).manual_seed(0x5A6A + 1 + rank)  # own gradients per rank
    g.copy_((torch.randn(n, device=dev, generator=gen_g) * (1e-3 * SCALE0)).to(g.dtype))
    grp.init_master(sp)
    host_g = torch.empty(n, dtype=g.dtype).pin_memory()
    host_g.copy_(g)
    host_ptrs = (0, host_g.data_ptr()) if f32 else (host_g.data_ptr(), 0)
    torch.cuda.synchronize(dev)

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local])
        torch.cuda.synchronize(dev)

    sampler = ClockSampler(local) if rank == 0 else None
    scaler = LossScaler(SCALE0)

    def timed_steps(k):
        """k steps back to back on one stream; device time in ms (this rank)."""
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(k):
            grp.exec(LR, L2, scaler.scale, sp)
        b.record(stream)
        torch.cuda.synchronize(dev)
        return a.elapsed_time(b)

    # ---- device-resident throughput: K steps back to back on one stream
    for _ in range(args.warmup):
        grp.exec(LR, L2, scaler.scale, sp)
    flags = grp.flags(sp)
    barrier()
    launches0 = grp.launch_count
    if sampler:
        sampler.start()
    ms = timed_steps(args.steps)
    barrier()
    launches = grp.launch_count - launches0
    flags = grp.flags(sp)

    # ---- N > 1: the reference's own sequence (ncclReduceScatter, Adam on the shard,
    # ncclAllGather, 3-word all-reduce) on the same buffers, for comparison
    nccl_ms = None
    if world > 1 and args.path != "nccl":
        grp.set_option(capi.OPT_PATH, capi.PATH_NCCL)
        k = min(args.steps, 200)
        for _ in range(5):
            grp.exec(LR, L2, scaler.scale, sp)
        grp.flags(sp)
        barrier()
        nccl_ms = timed_steps(k) / k
        grp.flags(sp)
        barrier()
        grp.set_option(capi.OPT_PATH, {"auto": capi.PATH_AUTO, "peer": capi.PATH_PEER,
                                       "push": capi.PATH_PUSH}[args.path])

    # ---- N > 1, on request: the other classic arrangement -- all-reduce the whole
    # gradient buffer (NCCL, fp16), then every rank updates ALL parameters with the
    # one-GPU kernel (unsharded optimizer state)
    allreduce_ms = None
    if world > 1 and args.with_allreduce_baseline and not f32:
        from saga_b200 import optimizer as opt_mod
        from saga_b200 import bias_corrections
        aw, ag = w.clone(), g.clone()
        am, av = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        ac = aw.float()
        aux = torch.zeros(4, dtype=torch.int32, device=dev)
        b1t, b2t = bias_corrections(1)

        def ar_step():
            dist.all_reduce(ag, op=dist.ReduceOp.AVG)   # AVG keeps the values bounded over many steps
            opt_mod.adam_mixed(n, 1.0 / SCALE0, aw.data_ptr(), ag.data_ptr(), am.data_ptr(),
                               av.data_ptr(), ac.data_ptr(), float(b1t), float(b2t), LR, L2,
                               aux.data_ptr(), sp)
        for _ in range(5):
            ar_step()
        barrier()
        k = min(args.steps, 200)
        ea, eb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ea.record(stream)
        for _ in range(k):
            ar_step()
        eb.record(stream)
        torch.cuda.synchronize(dev)
        allreduce_ms = ea.elapsed_time(eb) / k
        barrier()
        del aw, ag, am, av, ac

    # ---- N = 1, on request: a second baseline beside cpu_baseline -- the reference's own
    # kernel (src/cuda/cuda_kernels.cu compiled unmodified for sm_100a, oracle/_ref) on
    # buffers of the same size
    ref_gpu = None
    if world == 1 and rank == 0 and args.with_ref_gpu:
        from oracle import oracle as orc
        if orc.ref_available():
            R = orc.ref()
            rw, rg = w.clone(), g.clone()
            rm, rv = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
            rc_ = rw.float()
            aux = torch.zeros(4, dtype=torch.int32, device=dev)
            b1t, b2t = orc.bias_corrections(1)

            def ref_step():
                R.sagaref_adam_mixed(n, float(orc.alpha(SCALE0)), rw.data_ptr(), rg.data_ptr(),
                                     rm.data_ptr(), rv.data_ptr(), rc_.data_ptr(), float(b1t),
                                     float(b2t), LR, L2, aux.data_ptr(), sp)
            for _ in range(5):
                ref_step()
            torch.cuda.synchronize(dev)
            k = min(args.steps, 200)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for _ in range(k):
                ref_step()
            b.record(stream)
            torch.cuda.synchronize(dev)
            rms = a.elapsed_time(b) / k
            ref_gpu = {"kernel": "saga::adam_mixed, the reference's src/cuda/cuda_kernels.cu "
                                 "compiled unmodified for sm_100a",
                       "ms_per_step": rms, "value": n / (rms * 1e-3), "unit": "params/s",
                       "hbm_gbs": 28 * n / (rms * 1e-3) / 1e9, "steps": k}
            del rw, rg, rm, rv, rc_

    # ---- end to end through the C ABI: gradients start in pinned host memory,
    # every step copies them in, steps, waits, reads the flag sums back and
    # updates the loss scale on the host (what Saga's step tail does)
    e2e_steps = args.e2e_steps or min(args.steps, 50)
    for _ in range(3):
        grp.step_host(host_ptrs[0], host_ptrs[1], LR, L2, scaler.scale, sp)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        fl = grp.step_host(host_ptrs[0], host_ptrs[1], LR, L2, scaler.scale, sp)
        scaler.update(fl)
    torch.cuda.synchronize(dev)
    e2e_s = time.perf_counter() - t0
    barrier()
    clocks = sampler.stop() if sampler else None

    if world > 1:
        t = torch.tensor([ms, e2e_s, nccl_ms or 0.0, allreduce_ms or 0.0], dtype=torch.float64,
                         device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s, nccl_ms = float(t[0]), float(t[1]), float(t[2]) or None
        allreduce_ms = float(t[3]) or None

    if rank == 0:
        per_step_ms = ms / args.steps
        hbm_peak, peak_kind = measured_peaks()
        # algorithmic bytes of one launch on one rank: read g of every rank's
        # shard copy (2n in total over self+peers), read+write m/v/master of the
        # shard (24n/N), write the fp16 weights of the whole buffer (2n)
        alg_bytes = 4 * n + 24 * n / world
        if f32:  # gradients 4 B read per rank copy, weights 4 B written per rank copy, w/m/v of the shard
            alg_bytes = 8 * n + 20 * n / world
        achieved = alg_bytes / (per_step_ms * 1e-3) / 1e9
        line = {
            "metric": "fused grad-reduce+Adam params/sec",
            "value": world * n / (per_step_ms * 1e-3),
            "unit": "params/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": per_step_ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {
                "workload": wl, "n_params": n, "tensors": len(sizes),
                "value_counts": "gradient parameters reduced and applied per second summed over "
                                "ranks (every rank brings its own n-element gradient buffer)",
                "unique_params_per_s": n / (per_step_ms * 1e-3),
                "l2": "inputs larger than L2: each step streams "
                      f"{alg_bytes / 1e6:.0f} MB per GPU against 126 MB of L2; no flush",
                "lr": LR, "l2_lambda": L2, "loss_scale": SCALE0, "path": args.path,
            },
            "roofline": {
                "bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                "frac": achieved / hbm_peak,
                "traffic": NCU_TRAFFIC_N1_BYTES if (world == 1 and not args.params and not f32) else None,
                "peak_kind": f"of {peak_kind}", "algorithmic_bytes_per_launch": alg_bytes,
                "frac_of_8000_nominal": achieved / 8000.0,
            },
            "e2e": {
                "value": world * n * e2e_steps / e2e_s, "unit": "params/s",
                "h2d_bytes_per_step": (4 if f32 else 2) * n, "d2h_bytes_per_step": 32,
                "ms_per_step": e2e_s / e2e_steps * 1e3, "steps": e2e_steps,
            },
            "gpu_launches": int(launches),
            "clocks": clocks,
            "flags_last_step": list(flags),
        }
        if world > 1:
            nv_bytes = (8 if f32 else 4) * n * (world - 1) / world
            nv = nv_bytes / (per_step_ms * 1e-3) / 1e9
            line["roofline_nvlink"] = {
                "bound": "nvlink", "achieved": nv, "peak": NVLINK_MEASURED_GBS, "unit": "GB/s",
                "frac": nv / NVLINK_MEASURED_GBS, "frac_of_900_nominal": nv / NVLINK_NOMINAL_GBS,
                "bytes_per_direction_per_launch": nv_bytes,
                "note": "with several ranks the step is bound by NVLink, not HBM: this is the "
                        "binding roofline, `roofline` above is the HBM side of the same launch",
            }
            if nccl_ms:
                line["nccl_sequence"] = {
                    "what": "ncclReduceScatter + Adam kernel on the shard + ncclAllGather + "
                            "3-word ncclAllReduce, the reference's call sequence, same buffers",
                    "ms_per_step": nccl_ms, "speedup_of_fused_kernel": nccl_ms / per_step_ms}
        if allreduce_ms:
            line["allreduce_sequence"] = {
                "what": "NCCL all-reduce of the whole fp16 gradient buffer + one-GPU Adam kernel over "
                        "all parameters on every rank (unsharded state)",
                "ms_per_step": allreduce_ms, "speedup_of_fused_kernel": allreduce_ms / per_step_ms}
        if ref_gpu:
            ref_gpu["speedup_of_fused_kernel"] = ref_gpu["ms_per_step"] / per_step_ms
            line["ref_gpu"] = ref_gpu
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(n)
        print(json.dumps(line), flush=True)

    grp.destroy()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
