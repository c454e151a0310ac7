"""A/B of end-to-end training throughput on ONE box: the unmodified Saga library against
the library with the b200opt optimizer op, same program, alternating runs.

    python saga_b200/host/e2e/ab_compare.py --gpus N [--repeats 3] [--model cifar18|resnet-50]
                                            [--variants ref,b200,b200+buckets4,b200+dscale]

Variants: "ref" the unmodified library, "b200" the integrated one; "+buckets<k>" issues the
optimizer step as k buckets between the backward ops (B200OPT_BUCKETS), "+dscale" keeps the loss
scale on the device (B200OPT_DEVICE_SCALE: no stream synchronise per step), "+grid<c>" gives the
buckets that run beside backward c CTAs (B200OPT_BUCKET_GRID), "+layoutref" keeps the reference's
tensor order in the flat buffer (B200OPT_LAYOUT=reference), "+noloss" makes the
program read the per-batch loss never (E2E_LOSS_EVERY=0, CIFAR program only; reading a tensor
waits for the stream, which hides what "+dscale" removes).

Every run is a child process under a time limit (a run that exceeds it is reported as
"timeout" and the comparison goes on); the integrated build's runs also report the device
time of the optimizer op (B200OPT_TIME_OP=1), from which the update's share of a training
step and its fraction of the bytes-moved roofline follow.  Prints one JSON line.
"""
import argparse
import json
import os
import re
import statistics
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD = os.path.join(HERE, "_build")

# parameters of the fp16 group of the two models (padded flat size) for the roofline line
PARAMS = {"cifar18": 11_173_962, "resnet-50": 25_557_032}


def run(cmd, env, limit):
    try:
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=limit, env=env)
    except subprocess.TimeoutExpired:
        return None, None
    if res.returncode != 0:
        return None, None
    line = [ln for ln in res.stdout.splitlines() if ln.startswith('{"e2e"')]
    ops = []
    for ln in res.stderr.splitlines():       # one object per rank thread
        if ln.startswith('{"b200_adam_op"'):
            try:
                ops.append(json.loads(ln)["b200_adam_op"])
            except ValueError:
                pass                         # two ranks' lines ran into each other
    if not line:
        return None, ops
    # printf spells a non-finite mean loss "nan" / "inf", which is not JSON
    text = re.sub(r"-?\bnan\b", "NaN", re.sub(r"\binf\b", "Infinity", line[-1]))
    try:
        return json.loads(text), ops
    except ValueError:
        return None, ops


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--repeats", type=int, default=3)
    ap.add_argument("--model", default="cifar18", choices=["cifar18", "resnet-50"])
    ap.add_argument("--limit", type=int, default=150, help="seconds per run")
    ap.add_argument("--batches", type=int, default=60)
    ap.add_argument("--variants", default="ref,b200")
    args = ap.parse_args()
    base_env = dict(os.environ, SAGA_CUDA_CONTEXTS=str(args.gpus), E2E_GPUS=str(args.gpus),
                    B200OPT_TIME_OP="1")
    if args.model == "cifar18":
        batch = 256
        cmd = lambda lib: [os.path.join(BUILD, "saga_cifar18_" + lib), str(batch),   # noqa: E731
                           str(args.batches), "4"]
    else:
        batch = 128
        base_env.update(E2E_HW="224", E2E_LABELS="1000",
                        E2E_TRAIN_BATCHES=str(min(args.batches, 30)), E2E_EPOCHS="3")
        cmd = lambda lib: [os.path.join(BUILD, "saga_e2e_" + lib), "-m", "resnet-50", "-h",   # noqa: E731
                           "-c", "-b", str(batch), "-U"]
    variants = {}
    for name in args.variants.split(","):
        lib, *mods = name.split("+")
        env = dict(base_env)
        for m in mods:
            if m.startswith("buckets"):
                env["B200OPT_BUCKETS"] = m[len("buckets"):]
            elif m.startswith("grid"):
                env["B200OPT_BUCKET_GRID"] = m[len("grid"):]
            elif m == "layoutref":
                env["B200OPT_LAYOUT"] = "reference"
            elif m == "dscale":
                env["B200OPT_DEVICE_SCALE"] = "1"
            elif m == "noloss":
                env["E2E_LOSS_EVERY"] = "0"
            else:
                raise SystemExit("unknown variant modifier " + m)
        variants[name] = (cmd(lib), env)
    out = {"model": args.model, "gpus": args.gpus, "batch_per_gpu": batch, "repeats": args.repeats,
           "runs": {v: [] for v in variants}, "op_us": []}
    for _ in range(args.repeats):
        for v, (c, env) in variants.items():   # alternate, so that drift hits all alike
            r, ops = run(c, env, args.limit)
            out["runs"][v].append(r["img_per_s_mean"] if r else "timeout or failure")
            if r and "loss_mean_rank0" in r:   # the CIFAR program reports these
                out.setdefault("loss_mean", {}).setdefault(v, []).append(r["loss_mean_rank0"])
                out.setdefault("loss_scale", {}).setdefault(v, []).append(r["loss_scale_rank0"])
            if v == "b200" and ops:
                out["op_us"].append(max(o["mean_us"] for o in ops))
    for v in variants:
        ok = [x for x in out["runs"][v] if isinstance(x, float)]
        if ok:
            out[v + "_img_per_s"] = {"mean": statistics.mean(ok), "median": statistics.median(ok),
                                     "min": min(ok), "max": max(ok)}
    if out["op_us"] and "b200_img_per_s" in out:
        op_us = statistics.mean(out["op_us"])
        step_us = 1e6 * batch * args.gpus / out["b200_img_per_s"]["mean"]
        n, N = PARAMS[args.model], args.gpus
        # bytes-moved roofline of the update step: HBM on one GPU, NVLink per direction beyond
        floor_us = (28 * n / 8000e9 if N == 1 else 4 * n * (N - 1) / N / 900e9) * 1e6
        out["update"] = {"op_us_mean": op_us, "training_step_us": step_us,
                         "share_of_step": op_us / step_us,
                         "roofline_floor_us": floor_us, "fraction_of_roofline": floor_us / op_us,
                         "roofline": "28 B/param at 8 TB/s" if N == 1 else
                                     "4n(N-1)/N B per NVLink direction at 900 GB/s"}
    print(json.dumps(out))


if __name__ == "__main__":
    main()
