#!/usr/bin/env python
"""Benchmark of the fused gradient reduce-scatter + mixed-precision Adam +
weight all-gather step (the data-parallel parameter update of Saga) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --gpus N --sweep          (under torch.distributed.run)

N > 1 is launched as one process per GPU by torch.distributed.run; rank 0
prints ONE JSON line.  A "step" is one optimizer step over the whole flat
parameter buffer: at N ranks every rank contributes its own gradient buffer,
updates its 1/N shard and receives all updated weights.

Workload at every N: 25.6 M fp16 parameters in 160 tensors (sizes log-uniform
in 64..4 M, renormalised, each padded to 16 elements), fp32 master N(0, 0.02),
gradients N(0, 1e-3) x loss scale 1024, lr 1e-3, lambda 0.01.  Synthetic,
seeded; per-step state touched (717 MB at N=1) is larger than L2, so no flush
is needed between steps.

Legs of the default run (all on the same buffers):
  value / roofline   K steps back to back on one stream, one CUDA event between
                     every two steps (mean = ms_per_step, median, min)
  parity             a small buffer stepped through the SAME collective path at
                     this N and compared with the CPU oracle (outside all timed
                     regions; a mismatch makes the run exit non-zero)
  phases             where the step kernel's time goes (entry wait, body,
                     completion protocol), from its own %globaltimer stamps
  nccl_sequence      N > 1: the reference's call sequence on the same buffers
  peer_copy          N > 1: NVLink bandwidth per direction measured in this run
  config2_as_written N = 1: gradients regenerated every step from the live loss
                     scale under the reference policy, +inf every 50th step, L2
                     flushed before every step
  e2e                gradients in pinned host memory, copied in every step
  cpu_baseline       N = 1: the CPU restatement on all host cores
"""
import argparse
import importlib.util
import json
import os
import signal
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

TOTAL_PARAMS = 25_600_000
TENSORS = 160
LR, L2, SCALE0 = 1e-3, 0.01, 1024.0
NVLINK_NOMINAL_GBS = 900.0
HBM_FALLBACK_GBS = 6650.0
# DRAM bytes per parameter of the one-rank step kernel, from one ncu capture (--set full, two
# launches at 2^26 parameters: 1819.9 and 1820.4 MB read + written per launch)
NCU_DRAM_BYTES_PER_PARAM = 1820.15e6 / (1 << 26)
METRIC = ("fused grad-reduce+Adam params/sec (gradient elements reduced and applied per second, "
          "summed over ranks: N ranks x n parameters / step time)")
WORKLOAD = "config2: 25.6M fp16 params in 160 tensors, 1 optimizer step"


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return HBM_FALLBACK_GBS, "fallback"


def workload_module():
    """saga_b200/workload.py loaded by file path: numpy-only generators, usable by the
    reference arm without importing (or mapping the library of) the package."""
    spec = importlib.util.spec_from_file_location(
        "b200_workload", os.path.join(ROOT, "saga_b200", "workload.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def padded_layout(sizes):
    """The reference's flat layout (each tensor padded to 16 elements) in plain Python."""
    offs, at = [], 0
    for s in sizes:
        offs.append(at)
        at += (int(s) + 15) // 16 * 16
    return offs, at


def base_config(n, tensors, wl=WORKLOAD):
    """The part of `config` both arms print identically."""
    return {"workload": wl, "n_params": n, "tensors": tensors, "lr": LR, "l2_lambda": L2,
            "loss_scale": SCALE0,
            "l2": "inputs larger than L2: a step streams 4n + 24n/N bytes per GPU (717 MB at "
                  "N=1, 179 MB at N=8) against 126 MB of L2; no flush between steps"}


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


# ----------------------------------------------------------- CPU baseline legs

def cpu_baseline(n, budget_s=12.0, max_steps=5000):
    """The CPU restatement of the reference's adam_kernel_mp (the reference has
    no CPU implementation of this path), all host threads, on the full buffer."""
    from oracle import oracle as orc
    wl = workload_module()
    orc.use_all_host_threads()
    w = wl.weights_half(n, seed=1)
    c = orc.master_init(w)
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    g = wl.grads_half(n, SCALE0, 1, seed=1)
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
    the mixed-precision Adam update of the same 25.6 M-parameter buffer.  It
    imports nothing of the product: the oracle and the numpy workload only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as orc
    wl = workload_module()
    cores = orc.use_all_host_threads()
    world = max(args.gpus, 1)
    sizes = wl.tensor_sizes(TOTAL_PARAMS, TENSORS)
    _, n = padded_layout(sizes)
    w = wl.weights_half(n, seed=1)
    c = orc.master_init(w)
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    grads = [wl.grads_half(n, SCALE0, 1, rank=r, seed=1) for r in range(world)]
    gsum = np.empty(n, np.uint16)
    al = orc.alpha(SCALE0)
    steps = min(args.steps, 200)
    it = [0]

    def one_step():
        it[0] += 1
        b1t, b2t = orc.bias_corrections(it[0])
        g = orc.reduce_half_threads(grads, gsum) if world > 1 else grads[0]
        orc.adam_mixed(w, g, m, v, c, al, b1t, b2t, LR, L2, threads=True)

    # Warm by time as well as by count, and until the step time has stopped falling:
    # the thread pool, the page tables of 400 MB of state, the cores' clocks and (on a
    # two-socket host) the kernel's migration of pages towards the threads that use
    # them take seconds to settle, and this arm should be timed at its sustained rate.
    t_warm = time.perf_counter()
    k = 0
    best_block = None
    while True:
        tb = time.perf_counter()
        for _ in range(10):
            one_step()
        k += 10
        block = (time.perf_counter() - tb) / 10
        waited = time.perf_counter() - t_warm
        settled = best_block is not None and block >= 0.97 * best_block
        best_block = block if best_block is None else min(best_block, block)
        if k >= args.warmup and ((waited >= 2.5 and settled) or waited >= 25.0):
            break
    t0 = time.perf_counter()
    for _ in range(steps):
        one_step()
    dt = time.perf_counter() - t0
    value = world * n * steps / dt
    sample = (f"{steps} full steps over all {n} parameters"
              + (f", each summing {world} gradient buffers first" if world > 1 else "")
              + f" ({dt:.1f} s after {k} warm-up steps; CPU restatement of src/cuda adam_kernel_mp, "
                "OpenMP over elements; the reference ships no CPU training path)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value,
        "unit": "params/s", "n_gpus": args.gpus, "steps": steps, "warmup": k,
        "ms_per_step": dt / steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": base_config(n, len(sizes)),
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
    from saga_b200 import AdamGroup, FlatLayout, capi, workload
    N = args.serial_ranks
    n = args.params or FlatLayout(workload.tensor_sizes(TOTAL_PARAMS, TENSORS)).total
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


# ----------------------------------------------------------------- helpers

class Env:
    """Process-group facts and the helpers every leg needs."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus:
            if self.world == 1 and args.gpus > 1:
                raise SystemExit("launch N>1 through torch.distributed.run (one process per GPU)")
            args.gpus = self.world
        self.dev = torch.device("cuda", self.local)
        torch.cuda.set_device(self.dev)
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("cpu:gloo,cuda:nccl", rank=self.rank, world_size=self.world,
                                    device_id=self.dev)
        self.stream = torch.cuda.current_stream(self.dev)
        self.sp = self.stream.cuda_stream

    def barrier(self):
        if self.world > 1:
            self.dist.barrier(device_ids=[self.local])
        self.torch.cuda.synchronize(self.dev)

    def max_over_ranks(self, values):
        if self.world == 1:
            return [float(x) for x in values]
        t = self.torch.tensor([float(x) for x in values], dtype=self.torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(x) for x in t]

    def all_true(self, flag):
        if self.world == 1:
            return bool(flag)
        t = self.torch.tensor([1 if flag else 0], dtype=self.torch.int32, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return bool(int(t[0]))


def make_group(env, n_half, n_float, want_path):
    """One rank's optimizer wired to its peers; returns (group, path actually used).
    `want_path`: auto | peer | nvls | nccl.  "auto" is the benchmark's own choice: the
    multicast path where the GPUs offer it and it was measured faster than the peer path
    (eight ranks: 143 against 158 us per step; at four ranks the peer path wins, 137
    against 146 us, at two it moves fewer bytes to begin with), the peer path otherwise."""
    from saga_b200 import AdamGroup, capi, launch
    flags = 0
    if env.world > 1 and want_path in ("auto", "nvls"):
        flags = capi.CREATE_MULTICAST
    grp = None
    if flags:
        # every rank must end up with the same kind of arena: fall back together
        try:
            grp = AdamGroup.create(env.rank, env.world, env.local, n_half, n_float, flags)
        except capi.B200OptError:
            grp = None
        if not env.all_true(grp is not None):
            if grp is not None:
                grp.destroy()
            grp, flags = None, 0
    if grp is None:
        grp = AdamGroup.create(env.rank, env.world, env.local, n_half, n_float, 0)
    info = {"multicast": False}
    if env.world > 1:
        info = launch.wire_process_group(grp, with_nccl=True)
    path = want_path
    if want_path == "auto":
        path = "nvls" if (info["multicast"] and env.world >= 8) else "peer"
    elif want_path == "nvls" and not info["multicast"]:
        path = "peer"
    if env.world == 1:
        path = "peer"
    set_path(grp, path)
    return grp, path, info


def set_path(grp, path):
    from saga_b200 import capi
    if grp.nranks > 1:
        grp.set_option(capi.OPT_PATH, {"peer": capi.PATH_PEER, "nvls": capi.PATH_NVLS,
                                       "nccl": capi.PATH_NCCL}[path])


def timed_steps(env, fn, k, lead_in=3):
    """k calls of fn back to back on the stream with one event between every two;
    returns the per-step device times in ms (this rank) and their total.

    `lead_in` untimed calls are enqueued first, in the same burst: the ranks leave the
    host barrier tens of microseconds apart, and without work already queued on every
    GPU that host-side skew would sit inside the first timed step (the slowest rank's
    late launch stalls everyone in the step's entry wait).  The first event is recorded
    on the stream behind the lead-in, whose completion protocol aligns the GPUs."""
    torch = env.torch
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(k + 1)]
    for _ in range(lead_in if env.world > 1 else 0):
        fn()
    ev[0].record(env.stream)
    for i in range(k):
        fn()
        ev[i + 1].record(env.stream)
    torch.cuda.synchronize(env.dev)
    return [ev[i].elapsed_time(ev[i + 1]) for i in range(k)], ev[0].elapsed_time(ev[k])


def timed_block(env, fn, k, lead_in=3):
    """k calls of fn back to back between ONE pair of events (plus the untimed lead-in
    described in timed_steps); device time in ms (this rank)."""
    torch = env.torch
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(lead_in if env.world > 1 else 0):
        fn()
    a.record(env.stream)
    for _ in range(k):
        fn()
    b.record(env.stream)
    torch.cuda.synchronize(env.dev)
    return a.elapsed_time(b)


def summarize(per_step_ms):
    a = np.asarray(per_step_ms, dtype=np.float64) * 1e3
    return {"mean": float(a.mean()), "median": float(np.median(a)), "min": float(a.min()),
            "p95": float(np.percentile(a, 95)), "steps": int(a.size)}


# ------------------------------------------------------------------ parity leg

def parity_leg(env, path):
    """A small buffer stepped through the real collective path of this run at this N
    and compared with the CPU oracle (rank-ordered fp32 sum, one fp16 rounding, the
    reference's update): 2048*6*N+80 fp16 + 528 fp32 parameters, 4 steps, an inf from
    rank 0 on step 2, a 32768 in two shards on step 3.  Returns the block for the JSON line.

    Peer path: everything bit for bit (reported as relative error and bit differences).
    Multicast path: the switch forms the fp16 sum with its own arithmetic, so the check
    has two parts -- the sums it returned (the kernel leaves them in the gradient buffer,
    where ncclReduceScatter leaves them in Saga) lie within one fp16 ulp of the
    rank-ordered sums, and GIVEN those sums flags, loss scale, m, v, master and weights
    equal the oracle's bit for bit."""
    import torch
    from oracle import oracle as orc
    from saga_b200 import LossScaler, capi, workload
    N, rank = env.world, env.rank
    n_half, n_float, steps = 2048 * 6 * N + 80, 528, 4
    grp, used, _ = make_group(env, n_half, n_float, path)
    nvls = used == "nvls"
    out = {"n_ranks": N, "path": used, "n_half": n_half, "n_float": n_float, "steps": steps}
    try:
        if nvls:
            grp.set_option(capi.OPT_KEEP_REDUCED, 1)
        W0, Wf0 = workload.weights_half(n_half, seed=17), workload.weights_float(n_float, seed=17)
        w, g = grp.buffers(capi.HALF)
        wf, gf = grp.buffers(capi.FLOAT)
        w.view(torch.int16).copy_(torch.from_numpy(W0.view(np.int16).copy()))
        wf.copy_(torch.from_numpy(Wf0.copy()))
        grp.init_master(env.sp)
        env.barrier()
        ost = orc.MultiRankState(N, [W0] * N, [Wf0] * N)
        scaler, oscale = LossScaler(64.0), np.float32(64.0)
        sh = n_half // N
        flags_equal = scale_equal = True
        flag_log = []
        sum_ulp_max = sum_off = 0
        for step in range(1, steps + 1):
            G = [workload.grads_half(n_half, oscale, step, rank=r, seed=17) for r in range(N)]
            Gf = [workload.grads_float(n_float, oscale, step, rank=r, seed=17) for r in range(N)]
            if step == 2:
                G[0][n_half // 2 + 3] = 0x7C00
            if step == 3:
                G[N - 1][5] = 0x7800
                G[0][(N - 1) * sh + 9] = 0x7800
            g.view(torch.int16).copy_(torch.from_numpy(G[rank].view(np.int16).copy()))
            gf.copy_(torch.from_numpy(Gf[rank].copy()))
            env.barrier()
            grp.exec(1e-2, 0.01, scaler.scale, env.sp)
            flags = grp.flags(env.sp)
            if nvls:
                parts = [None] * N
                env.dist.all_gather_object(
                    parts, g[rank * sh:(rank + 1) * sh].view(torch.int16).cpu().numpy().tobytes())
                reduced = G[0].copy()
                reduced[:N * sh] = np.frombuffer(b"".join(parts), dtype=np.uint16)
                d = orc.half_ulp_distance(reduced[:N * sh], orc.rank_ordered_sum_half(G)[:N * sh])
                sum_ulp_max = max(sum_ulp_max, int(d.max()))
                sum_off += int(np.count_nonzero(d))
                G = [reduced] + [np.full(n_half, 0x8000, np.uint16) for _ in range(N - 1)]
            oflags = ost.step([x.copy() for x in G], [x.copy() for x in Gf], oscale, 1e-2, 0.01)
            flag_log.append(list(flags))
            flags_equal &= tuple(flags) == tuple(oflags)
            scaler.update(flags)
            oscale = orc.policy_reference(oscale, oflags)
            scale_equal &= scaler.scale.tobytes() == oscale.tobytes()
        env.barrier()

        def rel(a, b):      # |a-b| / (|b| + rms(b)): m and the master pass through zero
            a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
            if not a.size:
                return 0.0
            return float(np.max(np.abs(a - b) / (np.abs(b) + np.sqrt(np.mean(b * b)) + 1e-300)))
        worst = 0.0
        state_bit_diffs = 0
        for which, ref in ((0, ost.m[rank]), (1, ost.v[rank]), (2, ost.c[rank])):
            mine = grp.export_state(capi.HALF, which)
            worst = max(worst, rel(mine, ref))
            state_bit_diffs += int(np.count_nonzero(mine.view(np.uint32) != ref.view(np.uint32)))
        for which, ref in ((0, ost.mf[rank]), (1, ost.vf[rank])):
            worst = max(worst, rel(grp.export_state(capi.FLOAT, which), ref))
        mine_w = w.view(torch.int16).cpu().numpy().view(np.uint16)
        d = np.abs(mine_w.astype(np.int64) - ost.W[0].astype(np.int64))
        worst, ulp, wdiff, sdiff, sulp, soff = env.max_over_ranks(
            [worst, float(d.max()), float(np.count_nonzero(d)), float(state_bit_diffs),
             float(sum_ulp_max), float(sum_off)])
        all_flags = env.all_true(flags_equal)
        all_scale = env.all_true(scale_equal)
        out.update({"flags_equal": all_flags, "scale_bits_equal": all_scale,
                    "max_rel_err": worst, "w_ulp_max": int(ulp), "w_bit_diffs": int(wdiff),
                    "state_bit_diffs_max_rank": int(sdiff), "flags_per_step": flag_log})
        if nvls:
            out.update({
                "switch_sum_ulp_max": int(sulp), "switch_sums_off_by_one": int(soff),
                "switch_sums_checked": steps * N * sh,
                "against": "CPU oracle fed with the sums the switch returned (left in the gradient "
                           "buffer): everything bit for bit; the sums themselves against the "
                           "rank-ordered fp32 sum with one fp16 rounding: within one fp16 ulp"})
            out["ok"] = bool(all_flags and all_scale and worst == 0.0 and ulp == 0 and sulp <= 1)
        else:
            out["against"] = ("CPU oracle: rank-ordered fp32 sum, one fp16 rounding, reference "
                              "update; tolerance 1e-6 per step (bit differences reported)")
            out["ok"] = bool(all_flags and all_scale and worst <= 1e-6 * steps and ulp <= 1)
    finally:
        w = g = wf = gf = None
        env.barrier()
        grp.destroy()
    return out


# ------------------------------------------------------ config 2 as written

def config2_as_written(env, grp, n, steps):
    """Config 2 the way it is specified, on one GPU: gradients N(0, 1e-3) x the LIVE loss
    scale regenerated every step, the reference's policy (x1.02 per clean step, x0.5 on
    inf/NaN), one +inf injected every 50th step, the flag sums read back and the scale
    updated on the host every step as Saga's step tail does.  The scale climbs from 1024
    until gradients overflow by themselves (about 470 steps), then saw-tooths, so steps
    that take the per-element classification arm (|g| >= 32768) and skipped elements are
    inside the timed set.  Only the step kernel is between the two events of a step; the
    gradient generation and an L2 flush (a 256 MB memset) come before the first event."""
    import torch
    from saga_b200 import LossScaler, capi
    dev = env.dev
    w, g = grp.buffers(capi.HALF)
    gen = torch.Generator(device=dev).manual_seed(0xC0F2)
    base = torch.empty(n, dtype=torch.float32, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    scaler = LossScaler(SCALE0)
    times, kinds = [], []
    evs = []
    for step in range(1, steps + 1):
        base.normal_(0.0, 1e-3, generator=gen)
        torch.mul(base, float(scaler.scale), out=base)
        g.copy_(base)                       # fp32 -> fp16, overflows to inf by itself
        if step % 50 == 0:
            g[int(torch.randint(0, n, (1,), generator=gen, device=dev))] = float("inf")
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(env.stream)
        grp.exec(LR, L2, scaler.scale, env.sp)
        b.record(env.stream)
        flags = grp.flags(env.sp)           # stream sync, as in CudaProgram::step
        evs.append((a, b))
        kinds.append("overflow" if (flags[1] or flags[2]) else ("range" if flags[0] else "clean"))
        scaler.update(flags)
    times = np.array([a.elapsed_time(b) for a, b in evs]) * 1e3
    kinds = np.array(kinds)
    out = {"steps": steps, "us_per_step": summarize(times / 1e3),
           "final_scale": float(scaler.scale), "l2": "flushed before every step",
           "policy": "reference (x1.02 clean, x0.9 two range flags, x0.5 inf/NaN)"}
    for k in ("clean", "range", "overflow"):
        sel = times[kinds == k]
        out[k + "_steps"] = int(sel.size)
        if sel.size:
            out[k + "_us_median"] = float(np.median(sel))
    del base, flush
    return out


# ------------------------------------------------------- NVLink copy, this run

def peer_copy_leg(env, grp, nbytes):
    """NVLink copy rate per direction as this run sees it, between the arenas the step
    kernel uses: device-to-device copies of the fp16 weight buffer (identical on all
    ranks) with the copy engines -- rank 0 alone pulling from rank 1, and every rank
    pulling from the next one at the same time."""
    torch = env.torch
    nxt = (env.rank + 1) % env.world
    res = {}
    for name, active in (("one_pair", env.rank == 0), ("ring_all_ranks", True)):
        peer = 1 if name == "one_pair" else nxt
        for _ in range(2):
            if active:
                grp.peer_copy(peer, nbytes, env.sp)
        env.barrier()
        k = 20
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(env.stream)
        for _ in range(k):
            if active:
                grp.peer_copy(peer, nbytes, env.sp)
        b.record(env.stream)
        torch.cuda.synchronize(env.dev)
        ms = env.max_over_ranks([a.elapsed_time(b) / k])[0]
        env.barrier()
        res[name + "_gbs"] = nbytes / (ms * 1e-3) / 1e9
    res["what"] = (f"cudaMemcpyAsync of {nbytes / 1e6:.0f} MB from a peer's arena, GB/s per "
                   "direction per GPU, max over ranks")
    return res


# -------------------------------------------------------------- NCCL baselines

def nccl_sequence_leg(env, grp, restore_path, k):
    """The reference's own sequence (ncclReduceScatter, Adam on the shard, ncclAllGather,
    3-word all-reduce) on the same buffers."""
    set_path(grp, "nccl")
    for _ in range(5):
        grp.exec(LR, L2, SCALE0, env.sp)
    grp.flags(env.sp)
    env.barrier()
    total = timed_block(env, lambda: grp.exec(LR, L2, SCALE0, env.sp), k)
    grp.flags(env.sp)
    env.barrier()
    set_path(grp, restore_path)
    return env.max_over_ranks([total / k])[0]


def allreduce_sequence_leg(env, n, w, g, k):
    """The other classic arrangement: all-reduce the whole fp16 gradient buffer (NCCL),
    then every rank updates ALL parameters with the one-GPU kernel (unsharded state)."""
    torch, dist = env.torch, env.dist
    from saga_b200 import bias_corrections
    from saga_b200 import optimizer as opt_mod
    aw, ag = w.clone(), g.clone()
    am, av = torch.zeros(n, device=env.dev), torch.zeros(n, device=env.dev)
    ac = aw.float()
    aux = torch.zeros(4, dtype=torch.int32, device=env.dev)
    b1t, b2t = bias_corrections(1)

    def ar_step():
        dist.all_reduce(ag, op=dist.ReduceOp.AVG)   # AVG keeps the values bounded over many steps
        opt_mod.adam_mixed(n, 1.0 / SCALE0, aw.data_ptr(), ag.data_ptr(), am.data_ptr(),
                           av.data_ptr(), ac.data_ptr(), float(b1t), float(b2t), LR, L2,
                           aux.data_ptr(), env.sp)
    for _ in range(3):
        ar_step()
    env.barrier()
    total = timed_block(env, ar_step, k)
    env.barrier()
    del aw, ag, am, av, ac
    return env.max_over_ranks([total / k])[0]


# ---------------------------------------------------------------- sweep mode

def run_sweep(args):
    """BASELINE config 5: flat fp16 buffers of 2^20 .. 2^30 elements at this N; the fused
    kernel (peer path, and the multicast path where available) against NCCL
    reduce-scatter + Adam on the shard + all-gather (what the reference does) and NCCL
    all-reduce + Adam over the whole buffer on every rank.  One JSON line."""
    env = Env(args)
    torch = env.torch
    from saga_b200 import capi
    rows = []
    exps = [int(x) for x in args.sweep_exps.split(",")]
    for e in exps:
        n = 1 << e
        k = max(5, min(args.steps, 100 if e <= 26 else (30 if e <= 28 else 10)))
        grp, _, info = make_group(env, n, 0, "nvls" if env.world > 1 else "peer")
        w, g = grp.buffers(capi.HALF)
        gen = torch.Generator(device=env.dev).manual_seed(0x5A6A)
        chunk = 1 << 26
        for c0 in range(0, n, chunk):
            c1 = min(n, c0 + chunk)
            w[c0:c1] = (torch.randn(c1 - c0, device=env.dev, generator=gen) * 0.02).half()
        gen_g = torch.Generator(device=env.dev).manual_seed(0x5A6A + 1 + env.rank)
        for c0 in range(0, n, chunk):
            c1 = min(n, c0 + chunk)
            g[c0:c1] = (torch.randn(c1 - c0, device=env.dev, generator=gen_g) * (1e-3 * SCALE0)).half()
        grp.init_master(env.sp)
        env.barrier()
        row = {"log2_n": e, "n": n, "steps": k}
        paths = ["peer"] + (["nvls"] if info["multicast"] else [])
        for path in paths:
            set_path(grp, path)
            for _ in range(max(3, args.warmup // 4)):
                grp.exec(LR, L2, SCALE0, env.sp)
            grp.flags(env.sp)
            env.barrier()
            total = timed_block(env, lambda: grp.exec(LR, L2, SCALE0, env.sp), k)
            grp.flags(env.sp)
            env.barrier()
            us = env.max_over_ranks([total / k])[0] * 1e3
            row["fused_" + path + "_us"] = us
            if env.world > 1:
                row["fused_" + path + "_nvlink_gbs_algorithmic"] = \
                    4 * n * (env.world - 1) / env.world / (us * 1e-6) / 1e9
            else:
                row["hbm_gbs"] = 28 * n / (us * 1e-6) / 1e9
        if env.world > 1:
            row["nccl_rs_adam_ag_us"] = nccl_sequence_leg(env, grp, "peer", k) * 1e3
            row["nccl_allreduce_full_adam_us"] = allreduce_sequence_leg(env, n, w, g, k) * 1e3
        w = g = None
        env.barrier()
        grp.destroy()
        torch.cuda.empty_cache()
        rows.append(row)
    if env.rank == 0:
        print(json.dumps({"mode": "sweep (config 5)", "n_gpus": env.world,
                          "unit": "us per step, device time, max over ranks", "rows": rows}),
              flush=True)
    if env.world > 1:
        env.dist.destroy_process_group()


def run_tune(args):
    """Tuning aid: several launch settings of the step kernel on the benchmark workload in
    one process launch.  Not a benchmark value."""
    env = Env(args)
    torch = env.torch
    from saga_b200 import FlatLayout, capi, workload
    n = args.params or FlatLayout(workload.tensor_sizes(TOTAL_PARAMS, TENSORS)).total
    grp, _, info = make_group(env, n, 0, "nvls" if env.world > 1 else "peer")
    w, g = grp.buffers(capi.HALF)
    gen = torch.Generator(device=env.dev).manual_seed(0x5A6A)
    w.copy_((torch.randn(n, device=env.dev, generator=gen) * 0.02).half())
    gen_g = torch.Generator(device=env.dev).manual_seed(0x5A6A + 1 + env.rank)
    g.copy_((torch.randn(n, device=env.dev, generator=gen_g) * (1e-3 * SCALE0)).half())
    grp.init_master(env.sp)
    env.barrier()
    rows = []
    for spec in args.tune.split(","):
        parts = spec.split(":")
        path = parts[0]
        ctas = int(parts[1]) if len(parts) > 1 and parts[1] else 0
        variant = int(parts[2]) if len(parts) > 2 and parts[2] else 0
        grp.set_option(capi.OPT_GRID, int(parts[3]) if len(parts) > 3 and parts[3] else 0)
        if path == "nvls" and not info["multicast"]:
            continue
        set_path(grp, path)
        grp.set_option(capi.OPT_CTAS_PER_SM, ctas)
        grp.set_option(capi.OPT_KERNEL_VARIANT, variant)
        fn = lambda: grp.exec(LR, L2, SCALE0, env.sp)   # noqa: E731
        for _ in range(10):
            fn()
        grp.flags(env.sp)
        env.barrier()
        ms = env.max_over_ranks([timed_block(env, fn, args.steps)])[0]
        grp.flags(env.sp)
        env.barrier()
        grp.set_option(capi.OPT_PHASE_TIMERS, 1)
        ph = []
        for _ in range(6):
            for _ in range(20):
                fn()
            grp.flags(env.sp)
            ph.append(grp.phase_times())
            env.barrier()
        grp.set_option(capi.OPT_PHASE_TIMERS, 0)
        med = env.max_over_ranks(list(np.median(np.asarray(ph[1:], dtype=np.float64), axis=0) / 1e3))
        rows.append({"setting": spec, "us_per_step": ms / args.steps * 1e3,
                     "entry_wait_us": med[0], "body_end_us": med[1], "completion_us": med[2]})
    if env.rank == 0:
        print(json.dumps({"mode": "tune", "n_gpus": env.world, "n": n, "steps": args.steps,
                          "rows": rows}), flush=True)
    w = g = None
    env.barrier()
    grp.destroy()
    if env.world > 1:
        env.dist.destroy_process_group()


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
    ap.add_argument("--config2-steps", type=int, default=2400,
                    help="steps of the config-2-as-written leg (N = 1; 0 switches it off)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--only-timed", action="store_true",
                    help="tuning aid: the back-to-back timed loop and the phase timers only")
    ap.add_argument("--with-ref-gpu", action="store_true",
                    help="also time the reference's own compiled Adam kernel (oracle/_ref) as a "
                         "GPU baseline beside the CPU one; off by default")
    ap.add_argument("--ctas-per-sm", type=int, default=0)
    ap.add_argument("--variant", type=int, default=-1)
    ap.add_argument("--stages", type=int, default=0)
    ap.add_argument("--grid", type=int, default=0)
    ap.add_argument("--path", default="auto", choices=["auto", "peer", "nvls", "nccl"])
    ap.add_argument("--with-allreduce-baseline", action="store_true",
                    help="N > 1: also time NCCL all-reduce of the whole fp16 gradient buffer followed "
                         "by the one-GPU Adam kernel over all parameters on every rank")
    ap.add_argument("--serial-ranks", type=int, default=0,
                    help="profiling aid: N ranks on ONE GPU, stepped one after the other "
                         "(no cross-GPU waits); times the N-rank kernel against local HBM only")
    ap.add_argument("--tune", default="",
                    help="tuning aid: comma-separated path[:ctas_per_sm[:variant[:grid]]] settings, each "
                         "timed for --steps steps on the benchmark workload; prints one JSON line")
    ap.add_argument("--sweep", action="store_true", help="config 5: sizes 2^20..2^30 at this N")
    ap.add_argument("--sweep-exps", default="20,22,24,26,28,30")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.serial_ranks:
        return run_serial_ranks(args)
    if args.sweep:
        return run_sweep(args)
    if args.tune:
        return run_tune(args)
    args.warmup = max(args.warmup, 3)
    if args.only_timed:
        args.no_parity = args.no_cpu_baseline = True
        args.config2_steps = 0

    env = Env(args)
    torch, dist = env.torch, env.dist
    world, rank, dev, sp = env.world, env.rank, env.dev, env.sp
    from saga_b200 import FlatLayout, LossScaler, capi, workload

    # An orderly exit on SIGTERM (the launcher's way of stopping the other ranks when
    # one fails): a rank must release its multicast binding itself, not be torn down
    # while its peers may still address it.
    live = []

    def on_term(signum, frame):
        for gx in live:
            try:
                torch.cuda.synchronize(dev)
                gx.destroy()
            except Exception:
                pass
        os._exit(143)
    signal.signal(signal.SIGTERM, on_term)

    if args.params:
        sizes, n = [args.params], (args.params + 15) // 16 * 16
        wl = f"flat fp16 buffer of {n} elements, 1 optimizer step"
    else:
        sizes = workload.tensor_sizes(TOTAL_PARAMS, TENSORS)
        n = FlatLayout(sizes).total
        assert n == padded_layout(sizes)[1]
        wl = WORKLOAD

    f32 = args.fp32_group
    if f32:
        wl = wl.replace("fp16", "fp32") + " (fp32 group)"

    # ---- parity of this run's collective path at this N, before anything is timed
    parity = parity_peer = None
    if not args.no_parity:
        parity = parity_leg(env, args.path)
        if parity["path"] == "nvls":     # the bit-exact path at this N, for the record
            parity_peer = parity_leg(env, "peer")

    grp, path, info = make_group(env, 0 if f32 else n, n if f32 else 0, args.path)
    live.append(grp)
    if args.ctas_per_sm:
        grp.set_option(capi.OPT_CTAS_PER_SM, args.ctas_per_sm)
    if args.variant >= 0:
        grp.set_option(capi.OPT_KERNEL_VARIANT, args.variant)
    if args.stages:
        grp.set_option(capi.OPT_STAGES, args.stages)
    if args.grid:
        grp.set_option(capi.OPT_GRID, args.grid)

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

    sampler = ClockSampler(env.local) if rank == 0 else None
    scaler = LossScaler(SCALE0)
    step = lambda: grp.exec(LR, L2, scaler.scale, sp)   # noqa: E731

    # ---- device-resident throughput: K steps back to back on one stream
    for _ in range(args.warmup):
        step()
    flags = grp.flags(sp)
    env.barrier()
    launches0 = grp.launch_count
    if sampler:
        sampler.start()
    total_ms = timed_block(env, step, args.steps)
    env.barrier()
    launches = grp.launch_count - launches0
    flags = grp.flags(sp)
    ms = env.max_over_ranks([total_ms])[0]
    # the distribution over steps comes from a second pass with an event between every two
    # steps (the extra stream operations cost a few microseconds per step, so its mean sits
    # above ms_per_step); element-wise max over ranks = the slowest rank's view
    per_step, _ = timed_steps(env, step, min(args.steps, 300))
    per_step = env.max_over_ranks(per_step)
    env.barrier()

    # ---- where the kernel's time goes: its own timer stamps.  The stamps of a launch are
    # overwritten by the next one, so the last step of each back-to-back burst is read.
    phases = None
    if world > 1 and path != "nccl":
        grp.set_option(capi.OPT_PHASE_TIMERS, 1)
        rows = []
        for _ in range(12):
            for _ in range(20):
                step()
            grp.flags(sp)
            rows.append(grp.phase_times())
            env.barrier()
        grp.set_option(capi.OPT_PHASE_TIMERS, 0)
        med = np.median(np.asarray(rows[2:], dtype=np.float64), axis=0) / 1e3
        med = env.max_over_ranks(list(med))
        phases = {"entry_wait_us": med[0], "entry_to_last_cta_done_us": med[1],
                  "completion_protocol_us": med[2], "kernel_total_us": med[3],
                  "what": "the step kernel's own %globaltimer stamps: wait for the peers' "
                          "announcements (first CTA; the first trip's local loads are already in "
                          "flight), kernel entry until the last CTA finished its share, completion "
                          "protocol in the last CTA, and their sum; 20th step of back-to-back "
                          "bursts, median over 10 bursts, max over ranks"}
        env.barrier()

    # ---- N > 1: the reference's own sequence on the same buffers, for comparison
    nccl_ms = None
    if world > 1 and path != "nccl" and not args.only_timed:
        nccl_ms = nccl_sequence_leg(env, grp, path, min(args.steps, 200))

    allreduce_ms = None
    if world > 1 and args.with_allreduce_baseline and not f32:
        allreduce_ms = allreduce_sequence_leg(env, n, w, g, min(args.steps, 200))

    peer_copy = None
    if world > 1 and not args.only_timed and not f32 and path != "nccl":
        peer_copy = peer_copy_leg(env, grp, n * 2)

    # ---- N = 1, on request: a second baseline beside cpu_baseline -- the reference's own
    # kernel (src/cuda/cuda_kernels.cu compiled unmodified for sm_100a, oracle/_ref) on
    # buffers of the same size
    ref_gpu = None
    if world == 1 and rank == 0 and args.with_ref_gpu and not f32:
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
            rtotal = timed_block(env, ref_step, k)
            rms = rtotal / k
            ref_gpu = {"kernel": "saga::adam_mixed, the reference's src/cuda/cuda_kernels.cu "
                                 "compiled unmodified for sm_100a",
                       "ms_per_step": rms, "value": n / (rms * 1e-3), "unit": "params/s",
                       "hbm_gbs": 28 * n / (rms * 1e-3) / 1e9, "steps": k}
            del rw, rg, rm, rv, rc_

    # ---- end to end through the C ABI: gradients start in pinned host memory,
    # every step copies them in, steps, waits, reads the flag sums back and
    # updates the loss scale on the host (what Saga's step tail does)
    e2e_steps = 3 if args.only_timed else (args.e2e_steps or min(args.steps, 50))
    for _ in range(3):
        grp.step_host(host_ptrs[0], host_ptrs[1], LR, L2, scaler.scale, sp)
    env.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        fl = grp.step_host(host_ptrs[0], host_ptrs[1], LR, L2, scaler.scale, sp)
        scaler.update(fl)
    torch.cuda.synchronize(dev)
    e2e_s = time.perf_counter() - t0
    env.barrier()
    e2e_s = env.max_over_ranks([e2e_s])[0]
    clocks = sampler.stop() if sampler else None

    # ---- N = 1: config 2 as it is written (live scale, injected inf, cold L2)
    as_written = None
    if world == 1 and not f32 and not args.params and args.config2_steps > 0:
        grp.init_master(sp)       # fresh m, v, master for a clean trajectory
        torch.cuda.synchronize(dev)
        as_written = config2_as_written(env, grp, n, args.config2_steps)

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
        roof_hbm = {
            "bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
            "frac": achieved / hbm_peak,
            "traffic": NCU_DRAM_BYTES_PER_PARAM * n if world == 1 and not f32 else None,
            "peak_kind": f"of {peak_kind}", "algorithmic_bytes_per_launch": alg_bytes,
            "frac_of_8000_nominal": achieved / 8000.0,
            "traffic_note": "not measured by this run: dram__bytes_read.sum + dram__bytes_write.sum "
                            "of one launch of the one-rank kernel from an ncu capture at 2^26 "
                            "parameters (1820 MB), scaled to this launch in proportion to the "
                            "parameters (every array is passed over once); null for other kernels",
        }
        cfg = base_config(n, len(sizes), wl)
        run = {
            "value_counts": "gradient elements reduced and applied per second summed over ranks "
                            "(every rank brings its own n-element gradient buffer: weak scaling)",
            "unique_params_per_s": n / (per_step_ms * 1e-3),
            "bytes_streamed_per_gpu_per_step": alg_bytes,
            "path": path, "path_requested": args.path, "multicast": bool(info["multicast"]),
        }
        line = {
            "metric": METRIC,
            "value": world * n / (per_step_ms * 1e-3),
            "unit": "params/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": per_step_ms,
            "step_us": dict(summarize(per_step),
                            note="second pass with an event between every two steps, which "
                                 "adds a few us per step; ms_per_step is the one-event-pair mean"),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": cfg,
            "run": run,
            "e2e": {
                "value": world * n * e2e_steps / e2e_s, "unit": "params/s",
                "h2d_bytes_per_step": (4 if f32 else 2) * n, "d2h_bytes_per_step": 32,
                "ms_per_step": e2e_s / e2e_steps * 1e3, "steps": e2e_steps,
                "note": "per step: the gradients travel host to device, the flag sums device to "
                        "host; the updated weights stay on the device, where the next forward "
                        "pass reads them (Saga never copies them back during training)",
            },
            "gpu_launches": int(launches),
            "clocks": clocks,
            "flags_last_step": list(flags),
        }
        if world == 1:
            line["roofline"] = roof_hbm
        else:
            # algorithmic bytes per NVLink direction: reduce-scatter + all-gather of
            # fp16 (fp32) buffers = 4n(N-1)/N (8n(N-1)/N); what the path in use puts on the
            # links is reported beside it
            nv_alg = (8 if f32 else 4) * n * (world - 1) / world
            nv = nv_alg / (per_step_ms * 1e-3) / 1e9
            link = (2 * n + 2 * n / world) if (path == "nvls" and not f32) else nv_alg
            peak = max(peer_copy["one_pair_gbs"], peer_copy["ring_all_ranks_gbs"]) if peer_copy else None
            line["roofline"] = {
                "bound": "nvlink", "achieved": nv, "peak": peak or NVLINK_NOMINAL_GBS,
                "unit": "GB/s per direction per GPU",
                "frac": nv / (peak or NVLINK_NOMINAL_GBS),
                "peak_kind": "of measured (peer copies between the arenas in this run, the larger "
                             "of one pair and an all-rank ring)" if peak else "of nominal",
                "peak_nominal": NVLINK_NOMINAL_GBS, "frac_of_900_nominal": nv / NVLINK_NOMINAL_GBS,
                "algorithmic_bytes_per_direction_per_launch": nv_alg,
                "link_bytes_per_direction_of_this_path": link,
                "link_gbs_of_this_path": link / (per_step_ms * 1e-3) / 1e9,
                "traffic": None,
                "note": "achieved = reduce-scatter + all-gather bytes per direction (4n(N-1)/N) / "
                        "step time; the multicast path moves fewer bytes than that over the links "
                        "(2n + 2n/N: switch-reduced loads, switch-replicated stores), which is how "
                        "`frac` can pass the fraction of the link rate a peer-to-peer design reaches",
            }
            line["roofline_hbm"] = roof_hbm
            line["peer_copy"] = peer_copy
            if phases:
                line["phases"] = phases
            if nccl_ms:
                line["nccl_sequence"] = {
                    "what": "ncclReduceScatter + Adam kernel on the shard + ncclAllGather + "
                            "3-word ncclAllReduce, the reference's call sequence, same buffers",
                    "ms_per_step": nccl_ms, "speedup_of_fused_kernel": nccl_ms / per_step_ms}
        if parity is not None:
            line["parity"] = parity
        if parity_peer is not None:
            line["parity_peer_path"] = parity_peer
        if allreduce_ms:
            line["allreduce_sequence"] = {
                "what": "NCCL all-reduce of the whole fp16 gradient buffer + one-GPU Adam kernel over "
                        "all parameters on every rank (unsharded state)",
                "ms_per_step": allreduce_ms, "speedup_of_fused_kernel": allreduce_ms / per_step_ms}
        if ref_gpu:
            ref_gpu["speedup_of_fused_kernel"] = ref_gpu["ms_per_step"] / per_step_ms
            line["ref_gpu"] = ref_gpu
        if as_written:
            line["config2_as_written"] = as_written
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(n)
        print(json.dumps(line), flush=True)

    w = g = None
    env.barrier()      # every rank has stopped stepping before any arena is released
    live.clear()
    grp.destroy()
    if world > 1:
        dist.destroy_process_group()
    for blk in (parity, parity_peer):
        if blk is not None and not blk.get("ok", False):
            raise SystemExit("parity leg failed: " + json.dumps(blk))


if __name__ == "__main__":
    main()
