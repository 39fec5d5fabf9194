#!/usr/bin/env python
"""Benchmark of the approx-star verification path on B200.

    python bench.py --gpus N --steps K --warmup W            # CUDA engine
    python bench.py --impl reference --steps K --warmup W    # CPU restatement of the reference path

Workload: the 32x32x3 CNN robustness configuration (seeded synthetic images,
random-init FP64 weights): [conv3x3x32 -> BN -> ReLU]x2 -> avgpool2 ->
[conv3x3x64 -> BN -> ReLU]x2 -> avgpool2 -> FC256 -> ReLU -> FC10, L-inf
eps = 2/255 on all 3072 pixels, target = class of the centre image.

One step = one batch of B input sets pushed through reach + the output
halfspace test.  With N > 1 GPUs every rank verifies its own B sets per step
(independent queries, no data-path collective), so `value` is the whole-job
rate N*K*B / max-over-ranks time.

value   device-resident inputs (already uploaded), device time by CUDA events
        on the engine's stream.
e2e     the public call NN.verify_robustness_batch on host arrays: host staging,
        H2D copy, reach, halfspace test, D2H of the verdicts, wall clock between
        device synchronisations.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "verified ImageStar queries/sec"
UNIT = "queries/s"
WORKLOAD = "cnn32: 32x32x3 CNN, eps=2/255 on 3072 pixels, approx-star (estimated bounds) reach + halfspace verdict"
# Share of one image's dense contraction work done by the prefix conv1..conv2 (+BN, ReLU 1)
# that the CPU sample runs; columns per layer of seeded image 0: 3073, 4623, 7812, 10834, 20394.
CPU_PREFIX_LAYERS = 5


def dense_flops_per_layer(layers, in_shape, cols):
    """Algorithmic flops of every contraction layer given the column count entering it."""
    from nnv_b200.configs import out_shape
    out = []
    shape = in_shape
    ci = 0
    for i, L in enumerate(layers):
        nxt = out_shape([L], shape)
        if L["type"] == "conv2d":
            kh, kw, cin, cout = L["W"].shape
            out.append((i, 2.0 * nxt[0] * nxt[1] * cout * kh * kw * cin * cols[ci]))
        elif L["type"] == "fc":
            out.append((i, 2.0 * L["W"].shape[0] * L["W"].shape[1] * cols[ci]))
        elif L["type"] == "relu":
            ci += 1
        shape = nxt
    return out


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples every 200 ms while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc = None
        self.lines = []
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_sample(layers, query, n_layers):
    """Oracle (CPU restatement) on one image through the first n_layers layers."""
    from oracle import nnv_oracle as O
    t0 = time.perf_counter()
    S = O.reach(layers[:n_layers], O.star_from_query(query), keep_constraints=False)
    dt = time.perf_counter() - t0
    cols = [3073] + [t["P_out"] + 1 for t in S.trace]
    return dt, cols


def cpu_queries_per_s(cfg, reps=1):
    """Bounded CPU sample scaled to whole queries by dense contraction work."""
    layers = cfg["layers"]
    times = []
    for r in range(reps):
        dt, cols = cpu_sample(layers, cfg["queries"][0], CPU_PREFIX_LAYERS)
        times.append(dt)
    # whole-image column counts of seeded image 0 (from the engine; identical in the oracle)
    full_cols = [3073, 4623, 7812, 10834, 20394, 20650]
    fl = dense_flops_per_layer(layers, cfg["in_shape"], full_cols)
    total = sum(f for _, f in fl)
    prefix = sum(f for i, f in fl if i < CPU_PREFIX_LAYERS)
    frac = prefix / total
    t = float(np.median(times))
    return frac / t, t, frac


def run_reference(args):
    from nnv_b200.configs import make_config
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = make_config("cnn32", n_queries=1)
    cores = os.cpu_count()
    vals = []
    for _ in range(args.warmup):
        cpu_queries_per_s(cfg)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        v, t, frac = cpu_queries_per_s(cfg)
        vals.append(v)
    wall = time.perf_counter() - t0
    value = float(np.mean(vals))
    sample = ("1 image, layers 1-%d (conv1, BN, ReLU, conv2, BN: %.1f%% of the image's dense contraction flops), "
              "scaled to whole queries; reach only, NumPy/OpenBLAS FP64" % (CPU_PREFIX_LAYERS, 100 * frac))
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * wall / max(args.steps, 1),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": WORKLOAD, "batch_per_step": 1},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit(line)


def run_ours(args):
    import torch
    import torch.distributed as dist

    from nnv_b200 import nn
    from nnv_b200.configs import make_config
    from nnv_b200.engine import Batch, Context, Network

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    B, K, W = args.batch, args.steps, args.warmup

    # workload: distinct images per step and per rank, cycling through the 128 of the configuration
    n_distinct = min(K + W, max(1, 128 // (B * world)) if world * B <= 128 else 1)
    cfg = make_config("cnn32", n_queries=128)
    layers, shape = cfg["layers"], cfg["in_shape"]
    offs = rank * n_distinct * B
    step_queries = [[cfg["queries"][(offs + s * B + i) % 128] for i in range(B)] for s in range(n_distinct)]

    ctx = Context(local, args.arena_gb << 30)
    net = Network(ctx, layers, shape)
    stream = torch.cuda.ExternalStream(ctx.stream, device=dev)
    batches = []
    for qs in step_queries:
        b = Batch(net, qs)
        b.upload()
        batches.append((b, np.array([q["target"] for q in qs], dtype=np.int32)))

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def step(s):
        b, tg = batches[s % n_distinct]
        b.reach(keep_layer_bounds=True)
        return b.verify_robust(tg, "max")

    verdict_counts = {1: 0, 2: 0, -1: 0}
    # sizing pass: the context's working buffers grow to what the largest batch needs, so that no timed step
    # pays for a reallocation (the engine allocates nothing once its buffers have their size)
    for s in range(n_distinct):
        step(s)
    for s in range(W):
        step(s)
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    ctx.profile_enable(True)
    l0 = ctx.launch_count
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for s in range(K):
        v, _, _ = step(W + s)
        for x in v:
            verdict_counts[int(x)] += 1
    ev1.record(stream)
    barrier()
    dev_ms = ev0.elapsed_time(ev1)
    prof = ctx.profile_read()
    ctx.profile_enable(False)
    launches = ctx.launch_count - l0
    stats = batches[(W + K - 1) % n_distinct][0].relu_stats()

    # end to end through the public API on host arrays
    sets = [[nn.ImageStar(q["lb"], q["ub"]) for q in qs] for qs in step_queries]
    targets = [[q["target"] + 1 for q in qs] for qs in step_queries]
    model = nn.NN(layers, ctx=ctx)
    for s in range(min(W, 2)):
        model.verify_robustness_batch(sets[s % n_distinct], {"reachMethod": "approx-star"}, targets[s % n_distinct])
    barrier()
    t0 = time.perf_counter()
    for s in range(K):
        model.verify_robustness_batch(sets[(W + s) % n_distinct], {"reachMethod": "approx-star"},
                                      targets[(W + s) % n_distinct])
    torch.cuda.synchronize(dev)
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop() if sampler else None

    t = torch.tensor([dev_ms, e2e_s * 1e3, float(launches)], dtype=torch.float64, device=dev)
    if world > 1:
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        tsum = t.clone()
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        dev_ms, e2e_ms, launches = float(tmax[0]), float(tmax[1]), int(tsum[2])
    else:
        e2e_ms = e2e_s * 1e3

    if rank == 0:
        value = world * K * B / (dev_ms * 1e-3)
        e2e = world * K * B / (e2e_ms * 1e-3)
        # FP64 contraction roofline: cuBLAS DGEMM measured in this run (no FP64 figure is pre-measured)
        n = 6144
        a = torch.randn(n, n, dtype=torch.float64, device=dev)
        bb = torch.randn(n, n, dtype=torch.float64, device=dev)
        best = 1e9
        for _ in range(6):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch.matmul(a, bb)
            e1.record()
            torch.cuda.synchronize(dev)
            best = min(best, e0.elapsed_time(e1))
        dgemm_tflops = 2.0 * n ** 3 / (best * 1e-3) / 1e12
        del a, bb
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
        hbm_src = "MEASURED_PEAKS.json hbm_gbs" if peaks else "fallback 6650 GB/s"
        dgemm_src = "cuBLAS DGEMM 6144^3 measured in this run (burst, best of 6)"
        kernels = {"conv": "conv_win_kernel (windowed generator columns) + conv_f64_kernel (centres): FP64 DMMA "
                           "implicit GEMM, useful products only; the time includes the window-only copies written for "
                           "the bound reduction",
                   "fc": "fc_gather_kernel (windowed columns) + fc_f64_kernel / fc_skinny_kernel: FP64 DMMA GEMM",
                   "avgpool": "avgpool_windowed_kernel / avgpool_f64_kernel (bytes of the windows)",
                   "ranges": "range_windows_kernel + range_partial_* + range_finalize_kernel (Star.estimateRanges, "
                             "bytes of the windows)"}
        # DRAM bytes (read + write) of one image's convolution launches, from the ncu capture of the batch-1
        # run summarised in profiles/conv_win_kernel_cnn32_batch1.md; the launches of a batch of B images move
        # B times as much (every column is touched once per layer).  The capture's launch on the 1x1 windows of
        # the ReLU-2 columns (51 MB) is no longer made: those columns reach the convolution as unit vectors
        # the window-only copies written since for the bound reduction add their size, 257 MB (whole sectors)
        conv_dram_bytes_per_image = 530e6 + 257e6

        def roof(fam):
            f = prof[fam]
            tensor = fam in ("conv", "fc")
            ach = f["work"] / (f["ms"] * 1e-3) / (1e12 if tensor else 1e9) if f["ms"] > 0 else 0.0
            peak = dgemm_tflops if tensor else hbm_peak
            return {"bound": "tensor" if tensor else "hbm", "kernel": kernels[fam], "achieved": ach, "peak": peak,
                    "unit": "TFLOP/s" if tensor else "GB/s", "frac": ach / peak if peak else None,
                    "peak_source": dgemm_src if tensor else hbm_src, "launches": f["launches"],
                    "avg_launch_ms": f["ms"] / max(f["launches"], 1), "share_of_step": f["ms"] / dev_ms,
                    "traffic": (conv_dram_bytes_per_image * B * K / max(f["launches"], 1)) if fam == "conv" else None,
                    ("algorithmic_flops_per_launch" if tensor else "algorithmic_bytes_per_launch"):
                        f["work"] / max(f["launches"], 1)}

        # The same families against the dense algorithmic figures (every column a full image:
        # 2*Ho*Wo*Cout*kh*kw*Cin flop per column and convolution, 2*Out*In per column and FC layer).  The
        # engine skips the products with the structural zeros outside the columns' windows, so these
        # exceed the pipe's peak: they say how much dense work a step stands for, not how busy the pipe is.
        cols_seg = [B * (1 + 3072)] + [s_["cols_after"] for s_ in stats]
        per_layer = dense_flops_per_layer(layers, cfg["in_shape"], cols_seg)
        dense = {"conv": sum(f for i, f in per_layer if layers[i]["type"] == "conv2d"),
                 "fc": sum(f for i, f in per_layer if layers[i]["type"] == "fc")}

        def dense_equiv(fam):
            ms_step = prof[fam]["ms"] / K
            ach = dense[fam] / (ms_step * 1e-3) / 1e12 if ms_step > 0 else 0.0
            return {"achieved": ach, "unit": "TFLOP/s", "frac": ach / dgemm_tflops,
                    "note": "dense algorithmic flops of the step (columns counted as full images) over the family's "
                            "time; above 1 because products with structural zeros are skipped, not executed"}

        # ReLU step (Star.estimateRanges + classification + relaxation): bytes of the windows actually moved
        # over the time of the two families, and the dense-layout figure (V read once, cleared rows and new
        # one-hot columns written) that the windows and the work left to the next layer avoid
        relu_ms = (prof["ranges"]["ms"] + prof["relax"]["ms"]) / K
        # executed: the windows read by the bound reduction, lb/ub written and read back by the relaxation,
        # the predicate bounds of the new columns (rows are not cleared and one-hot columns not written here)
        relu_bytes = prof["ranges"]["work"] / K + sum(16.0 * s_["N"] * B + 16.0 * s_["n_cross"] for s_ in stats)
        dense_relu = 0.0
        for i, s_ in enumerate(stats):
            cin, n = cols_seg[i], s_["N"]
            dense_relu += 8.0 * n * cin + 16.0 * (cin - B) + 16.0 * n * B                      # estimateRanges
            dense_relu += 16.0 * n * B + 8.0 * (s_["n_dead"] + s_["n_cross"]) * cin / B + 8.0 * n * s_["n_cross"] \
                + 16.0 * s_["n_cross"]                                                          # relaxation
        relu_step = {"bound": "hbm", "achieved": relu_bytes / (relu_ms * 1e-3) / 1e9 if relu_ms > 0 else 0.0,
                     "peak": hbm_peak, "unit": "GB/s", "peak_source": hbm_src, "ms_per_step": relu_ms,
                     "dense_equivalent": {"achieved": dense_relu / (relu_ms * 1e-3) / 1e9 if relu_ms > 0 else 0.0,
                                          "unit": "GB/s",
                                          "note": "dense-layout bytes of the step over the same time; above the "
                                                  "copy rate because zero windows are skipped, cleared rows are "
                                                  "masked by the next layer and one-hot columns stay implicit"}}
        relu_step["frac"] = relu_step["achieved"] / hbm_peak
        relu_step["dense_equivalent"]["frac"] = relu_step["dense_equivalent"]["achieved"] / hbm_peak

        # the roofline entry is the kernel family with the largest share of the timed region
        dominant = max(kernels, key=lambda k: prof[k]["ms"])
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": dev_ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f64", "data": "synthetic",
            "config": {"workload": WORKLOAD, "batch_per_step": B, "distinct_batches": n_distinct,
                       "l2": "inputs larger than L2 (the column windows one layer reads: up to 0.16 GB per image)",
                       "verdicts": {"robust": verdict_counts[1], "unknown": verdict_counts[2],
                                    "undecided_on_device": verdict_counts[-1]},
                       "columns_after_relu": [s_["cols_after"] for s_ in stats]},
            "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": B * 2 * 3072 * 8,
                    "d2h_bytes_per_step": B * (4 + 9 * 4 + 9 * 8) + 5 * (B + 1) * 16},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": dict(roof(dominant), **({"dense_equivalent": dense_equiv(dominant)} if dominant in dense else {})),
            "roofline_other": {k: dict(roof(k), **({"dense_equivalent": dense_equiv(k)} if k in dense else {}))
                               for k in kernels if k != dominant},
            "relu_step": relu_step,
            "family_ms_per_step": {k: v["ms"] / K for k, v in prof.items()},
        }
        if world == 1 and not args.no_cpu_baseline:
            one = make_config("cnn32", n_queries=1)
            v, tcpu, frac = cpu_queries_per_s(one)
            line["cpu_baseline"] = {
                "value": v, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
                "sample": "1 image, layers 1-%d (%.1f%% of the image's dense contraction flops) in %.1f s, scaled to "
                          "whole queries; reach only, NumPy/OpenBLAS FP64" % (CPU_PREFIX_LAYERS, 100 * frac, tcpu)}
        emit(line)
    for b, _ in batches:
        b.close()
    net.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


_RESULT_FD = None


def emit(line):
    """The one JSON line goes to the process's original stdout; everything else printed while the bench
    runs (library banners such as NCCL's version line) was diverted to stderr in main()."""
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def main():
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=16, help="input sets per step and per GPU")
    ap.add_argument("--arena-gb", type=int, default=112)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
