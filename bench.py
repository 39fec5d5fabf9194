#!/usr/bin/env python
"""Benchmark of the approx-star verification path on B200.

    python bench.py --gpus N --steps K --warmup W                    # CUDA engine, all workloads
    python bench.py --workload cnn28 ...                             # one workload as the headline line
    python bench.py --workload vgg224 --shard generators --gpus 8    # one set sharded over the GPUs
    python bench.py --impl reference --steps K --warmup W            # CPU restatement of the reference path

Workloads (seeded synthetic images, random-init FP64 weights; nnv_b200/configs.py):

    cnn32     32x32x3 CNN [conv3x3x32-BN-ReLU]x2-pool-[conv3x3x64-BN-ReLU]x2-pool-FC256-ReLU-FC10,
              L-inf eps = 2/255 on all 3072 pixels, 128 images                    (the headline workload)
    cnn28     28x28x1 CNN conv3x3x8-ReLU-conv3x3x16/2-ReLU-FC128-ReLU-FC10, eps = 1/255, 256 images
    bright28  same network, one brightening predicate per image, 16384 images
    fc5       FC 5-[50 ReLU]x6-5, box of half width 0.01, 100 queries, "output 0 is minimal"
    vgg224    VGG16-shaped 224x224x3 network (average pools), 64 perturbed entries, 8 images

One step = one pass over the workload's whole query list: reach + the output halfspace test for every query,
in sub-batches that fit the arena.  With N > 1 GPUs every rank verifies its own copy of the list per step
(independent queries, no data-path collective), so `value` is N * K * queries / max-over-ranks time
(weak scaling); with --shard generators ONE set per step is split along its generator dimension over the
ranks and the partial bound sums are added over NVLink before every ReLU step (strong scaling).

value   inputs already uploaded; device time by CUDA events on the engine's stream around the K steps.
        Queries the device tests leave undecided are finished inside the timed region (second reach with
        constraint records, back-substitution bound, host LP), so every query counted has its verdict.
e2e     the public call NN.verify_robustness_batch on host arrays: host staging, H2D copy, reach,
        halfspace tests, D2H of the verdicts, wall clock between device synchronisations.
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

# name -> (queries of the configuration, queries per engine batch, description)
WORKLOADS = {
    "cnn32": (128, 64, "cnn32: 32x32x3 CNN, eps=2/255 on 3072 pixels, 128 images, approx-star (estimated bounds) "
                       "reach + halfspace verdict"),
    "cnn28": (256, 256, "cnn28: 28x28x1 CNN, eps=1/255 on 784 pixels, 256 images, reach + verdict"),
    "bright28": (16384, 4096, "bright28: 28x28x1 CNN, one brightening predicate per image, 16384 images, reach + verdict"),
    "fc5": (100, 100, "fc5: FC 5-[50 ReLU]x6-5, box half-width 0.01, 100 queries, reach + verdict (output 0 minimal)"),
    "vgg224": (8, 1, "vgg224: VGG16-shaped 224x224x3 network, 64 perturbed entries (eps=2/255), reach + verdict"),
}
# what the default line carries beside cnn32, with the steps they get (their steps are short)
EXTRAS = ("cnn28", "bright28", "fc5")          # plus vgg224, generator-sharded over the ranks


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
        # the median under load: samples taken while the SMs were clocked up
        busy = [x for x in sm if mx and x >= 0.5 * max(mx)] or sm
        return {"sm_mhz": float(np.median(busy)) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------ CPU arm


def _host_threads():
    info = {"cores": os.cpu_count()}
    try:
        import torch
        info["torch_threads"] = torch.get_num_threads()
    except Exception:
        pass
    try:
        from threadpoolctl import threadpool_info
        info["blas_threads"] = max([p.get("num_threads", 1) for p in threadpool_info()] or [1])
    except Exception:
        pass
    return info


def cpu_reference(name, budget_s=60.0):
    """The CPU restatement of the reference path (oracle/nnv_oracle.py: NumPy/OpenBLAS FP64, convolutions
    through torch's CPU FP64 conv2d, verdict LPs through HiGHS) on whole queries of the workload, as many as
    fit the time budget (at least one).  Returns (queries/s, description, oracle set of query 0)."""
    from nnv_b200.configs import make_config
    from oracle import nnv_oracle as O
    if name == "vgg224":
        return None, "not run: one dense 224x224 reach is hours of CPU work", None
    n_max = {"cnn32": 1, "cnn28": 8, "bright28": 64, "fc5": 100}[name]
    cfg = make_config(name, n_queries=n_max)
    with_lp = name != "cnn32"
    O.set_conv_backend("torch")
    first = None
    done = 0
    t0 = time.perf_counter()
    try:
        for qu in cfg["queries"]:
            S = O.reach(cfg["layers"], O.star_from_query(qu), keep_constraints=with_lp)
            if with_lp:
                G, g = O.robustness_set(S.mat().shape[0], qu["target"], qu.get("spec", "max"))
                O.verify_specification(S, G, g)
            if first is None:
                first = S
            done += 1
            if time.perf_counter() - t0 > budget_s:
                break
    finally:
        O.set_conv_backend("numpy")
    dt = time.perf_counter() - t0
    th = _host_threads()
    what = "reach + verdict (HiGHS feasibility LPs)" if with_lp else \
        ("reach only: the verdict LP of this size (about 20 650 variables, 52 700 rows, 34 M non-zeros, up to 9 "
         "solves) is not timed, so the figure is an upper bound of the CPU rate")
    sample = ("%d whole quer%s of the workload in %.1f s; %s; NumPy/OpenBLAS FP64 + torch CPU FP64 conv2d, %s"
              % (done, "y" if done == 1 else "ies", dt, what,
                 ", ".join("%s=%s" % kv for kv in sorted(th.items()))))
    return done / dt, sample, first


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    name = args.workload or "cnn32"
    nq, sub, desc = WORKLOADS[name]
    t0 = time.perf_counter()
    # whole queries, timed once (a query is deterministic: further steps would repeat the same computation);
    # each step then re-times a short prefix of query 0 (first affine layer + first ReLU step) as a stability check
    value, sample, _ = cpu_reference(name, budget_s=90.0 if name == "cnn32" else 45.0)
    from nnv_b200.configs import make_config
    from oracle import nnv_oracle as O
    cfg = make_config(name, n_queries=1)
    prefix = 1
    while prefix < len(cfg["layers"]) and cfg["layers"][prefix - 1]["type"] != "relu":
        prefix += 1
    O.set_conv_backend("torch")
    pre = []
    for s in range(args.warmup + args.steps):
        t1 = time.perf_counter()
        O.reach(cfg["layers"][:prefix], O.star_from_query(cfg["queries"][0]), keep_constraints=False)
        if s >= args.warmup:
            pre.append(time.perf_counter() - t1)
    O.set_conv_backend("numpy")
    wall = time.perf_counter() - t0
    if value is None:
        emit({"impl": "reference", "unavailable": sample})
        return
    sample += "; per step a re-timed prefix (layers 1-%d of query 0): median %.3f s, spread %.1f%%" % (
        prefix, float(np.median(pre)), 100.0 * (max(pre) - min(pre)) / max(np.median(pre), 1e-12))
    th = _host_threads()
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * wall / max(args.steps, 1),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": desc, "queries_per_step": nq, "batch_per_launch": sub},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": th["cores"], "kind": "port", "sample": sample,
                             "threads": th},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit(line)


# ------------------------------------------------------------------------------------------ GPU arm


def _sets_of(nn, queries):
    return [nn.ImageStar(q["lb"], q["ub"]) if "lb" in q else nn.ImageStar(q["V"], q["C"], q["d"], q["pl"], q["pu"])
            for q in queries]


def _bytes_in(q):
    if "lb" in q:
        return 2 * q["lb"].size * 8
    return q["V"].size * 8 + 16 * q["pl"].size


def run_workload(env, name, K, W, profile=False, keep_first=False):
    """Device-resident and end-to-end rates of one workload with query sharding; returns a dict."""
    import torch
    from nnv_b200 import _lib as L
    from nnv_b200 import nn
    from nnv_b200.configs import make_config
    from nnv_b200.engine import Batch, Network

    ctx, dev, stream, barrier, world, rank = (env[k] for k in ("ctx", "dev", "stream", "barrier", "world", "rank"))
    nq, sub, desc = WORKLOADS[name]
    if env["args"].batch and name == (env["args"].workload or "cnn32"):
        sub = env["args"].batch
    if env["args"].queries and name == (env["args"].workload or "cnn32"):
        nq = min(nq, env["args"].queries)          # a shorter list (profiling runs): not the benchmark's workload
        desc += " [first %d queries only]" % nq
    cfg = make_config(name, n_queries=nq)
    layers, shape = cfg["layers"], cfg["in_shape"]
    kind = cfg["queries"][0].get("spec", "max")
    # ranks start at different places of the list: every rank does the whole list per step
    order = np.roll(np.arange(nq), -(rank * nq) // max(world, 1))
    groups = [order[i:i + sub] for i in range(0, nq, sub)]
    net = Network(ctx, layers, shape)
    model = nn.NN(layers, ctx=ctx)
    model._nets[tuple(int(x) for x in shape)] = net
    sets_all = _sets_of(nn, cfg["queries"])
    batches = []
    for g in groups:
        b = Batch(net, [cfg["queries"][i] for i in g])
        b.upload()
        batches.append(b)
    targets0 = [np.array([cfg["queries"][i]["target"] for i in g], dtype=np.int32) for g in groups]
    opts = {"reachMethod": "approx-star"}
    counts = {"robust": 0, "unknown": 0, "second_pass": 0}
    first = {}

    def step(count):
        for gi, (b, g) in enumerate(zip(batches, groups)):
            b.reach(keep_layer_bounds=True)
            v, _, _ = b.verify_robust(targets0[gi], kind)
            if gi == len(groups) - 1:
                first["stats"] = b.relu_stats()            # before a second pass reuses the context's buffers
            if keep_first and gi == 0 and "cross" not in first:
                first["batch"] = b
                first["cross"] = [b.get_crossing(0, li)[0] for li in range(net.n_relu)]
                first["bounds"] = [b.get_layer_ranges(0, li, st["N"]) for li, st in enumerate(b.relu_stats())]
                first["ranges"] = b.get_ranges(0)
                first["query"] = int(g[0])
            und = int((v == L.UNDECIDED).sum())
            if und:
                res = model.finish_verdicts([sets_all[i] for i in g], opts, targets0[gi] + 1, v, kind)
            else:
                res = np.where(v == L.VERDICT_EMPTY, 1, 2)
            if count:
                counts["robust"] += int((res == 1).sum())
                counts["unknown"] += int((res == 2).sum())
                counts["second_pass"] += und

    step(False)                               # sizing pass: the context's working buffers reach their final size
    for _ in range(W):
        step(False)
    barrier()
    if profile:
        ctx.profile_enable(True)
    l0 = ctx.launch_count
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(K):
        step(True)
    ev1.record(stream)
    barrier()
    dev_ms = ev0.elapsed_time(ev1)
    launches = ctx.launch_count - l0
    prof = None
    if profile:
        prof = ctx.profile_read()
        ctx.profile_enable(False)
    stats = first["stats"]

    # end to end through the public API on host arrays
    tg1 = [t + 1 for t in targets0]
    for gi, g in enumerate(groups[:2]):
        model.verify_robustness_batch([sets_all[i] for i in g], opts, tg1[gi], kind)
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        for gi, g in enumerate(groups):
            model.verify_robustness_batch([sets_all[i] for i in g], opts, tg1[gi], kind)
    torch.cuda.synchronize(dev)
    e2e_ms = (time.perf_counter() - t0) * 1e3

    t = torch.tensor([dev_ms, e2e_ms, float(launches)], dtype=torch.float64, device=dev)
    if world > 1:
        import torch.distributed as dist
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        tsum = t.clone()
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        dev_ms, e2e_ms, launches = float(tmax[0]), float(tmax[1]), int(tsum[2])
    n_out = int(np.prod(net.out_shape))
    out = {"workload": desc, "value": world * K * nq / (dev_ms * 1e-3), "unit": UNIT, "steps": K,
           "ms_per_step": dev_ms / K, "queries_per_step": nq, "batch_per_launch": sub,
           "e2e": {"value": world * K * nq / (e2e_ms * 1e-3), "unit": UNIT,
                   "h2d_bytes_per_step": int(sum(_bytes_in(q) for q in cfg["queries"])),
                   "d2h_bytes_per_step": int(nq * (4 + (n_out - 1) * 12))},
           "gpu_launches": launches,
           "verdicts": {"robust": counts["robust"], "unknown": counts["unknown"], "violated": 0,
                        "finished_by_second_pass": counts["second_pass"]},
           "columns_after_relu": [s_["cols_after"] for s_ in stats]}
    res = {"line": out, "prof": prof, "stats": stats, "cfg": cfg, "first": first, "dev_ms": dev_ms, "sub": sub}
    if not keep_first:
        for b in batches:
            b.close()
        model._nets = {}
        net.close()
    else:
        res["cleanup"] = (batches, net, model)
    return res


def parity_check(first, S):
    """Engine results of the first query of the first timed batch against the CPU oracle's run of the same
    query: crossing sets, predicate columns, bounds per ReLU layer, output ranges."""
    from oracle import nnv_oracle as O
    same = all(np.array_equal(a, t["cross"]) for a, t in zip(first["cross"], S.trace))
    rel = 0.0
    for (lb, ub), t in zip(first["bounds"], S.trace):
        sc = max(np.abs(t["lb"]).max(), np.abs(t["ub"]).max())
        rel = max(rel, np.abs(lb - t["lb"]).max() / sc, np.abs(ub - t["ub"]).max() / sc)
    rl, ru = O.output_ranges(S)
    sc = max(np.abs(rl).max(), np.abs(ru).max())
    out_rel = max(np.abs(first["ranges"][0] - rl).max(), np.abs(first["ranges"][1] - ru).max()) / sc
    return {"query": first["query"], "relu_layers": len(S.trace), "crossing_sets_identical": bool(same),
            "columns_after_relu_oracle": [t["P_out"] + 1 for t in S.trace],
            "columns_after_relu_engine": [int(x) for x in
                                          np.cumsum([S.trace[0]["P_in"] + 1] + [len(a) for a in first["cross"]])[1:]],
            "max_rel_layer_bound_diff": float(rel), "max_rel_output_range_diff": float(out_rel),
            "tolerance": 1e-9, "ok": bool(same and rel < 1e-9 and out_rel < 1e-9)}


def measure_dgemm(torch, dev):
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
    return 2.0 * n ** 3 / (best * 1e-3) / 1e12


def rooflines(res, K, dgemm_tflops, hbm_peak, hbm_src):
    """Per kernel family: algorithmic work of its launches over their device time (event pairs around every
    launch group on the engine's stream), against the DGEMM rate / the copy bandwidth."""
    prof, stats, cfg, dev_ms, B = res["prof"], res["stats"], res["cfg"], res["dev_ms"], res["sub"]
    layers = cfg["layers"]
    dgemm_src = "cuBLAS DGEMM 6144^3 measured in this run (burst, best of 6); no FP64 figure is pre-measured"
    kernels = {"conv": "conv_win_kernel (windowed generator columns) + conv_f64_kernel (centres, dense columns): FP64 "
                       "DMMA implicit GEMM, products inside the columns' windows only; the time includes the "
                       "window-only copies written for the bound reduction",
               "fc": "fc_gather_kernel (windowed columns) + fc_f64_kernel / fc_skinny_kernel: FP64 DMMA GEMM",
               "avgpool": "avgpool_windowed_kernel / avgpool_f64_kernel (bytes of the windows)",
               "ranges": "range_windows_kernel + range_partial_* + range_finalize_kernel (Star.estimateRanges, "
                         "bytes of the windows)"}

    def roof(fam):
        f = prof[fam]
        tensor = fam in ("conv", "fc")
        ach = f["work"] / (f["ms"] * 1e-3) / (1e12 if tensor else 1e9) if f["ms"] > 0 else 0.0
        peak = dgemm_tflops if tensor else hbm_peak
        return {"bound": "tensor" if tensor else "hbm", "kernel": kernels[fam], "achieved": ach, "peak": peak,
                "unit": "TFLOP/s" if tensor else "GB/s", "frac": ach / peak if peak else None,
                "peak_source": dgemm_src if tensor else hbm_src, "launches": f["launches"],
                "avg_launch_ms": f["ms"] / max(f["launches"], 1), "share_of_step": f["ms"] / dev_ms,
                # DRAM bytes per launch come from an ncu capture, not from this run: see the profile summaries
                "traffic": None,
                ("algorithmic_flops_per_launch" if tensor else "algorithmic_bytes_per_launch"):
                    f["work"] / max(f["launches"], 1)}

    # The same families against the dense algorithmic figures (every column a full image).  The engine skips
    # the products with the structural zeros outside the columns' windows, so these exceed the pipe's peak:
    # they say how much dense work a step stands for, not how busy the pipe is.
    n_batches = len(range(0, res["line"]["queries_per_step"], B))
    q0 = cfg["queries"][0]
    p_in = int((q0["ub"] != q0["lb"]).sum()) if "lb" in q0 else int(q0["pl"].size)
    cols_seg = [B * (1 + p_in)] + [s_["cols_after"] for s_ in stats]
    per_layer = dense_flops_per_layer(layers, cfg["in_shape"], cols_seg)
    dense = {"conv": n_batches * sum(f for i, f in per_layer if layers[i]["type"] == "conv2d"),
             "fc": n_batches * sum(f for i, f in per_layer if layers[i]["type"] == "fc")}

    def dense_equiv(fam):
        ms_step = prof[fam]["ms"] / K
        ach = dense[fam] / (ms_step * 1e-3) / 1e12 if ms_step > 0 else 0.0
        return {"achieved": ach, "unit": "TFLOP/s", "frac": ach / dgemm_tflops,
                "note": "dense algorithmic flops of the step (columns counted as full images, the last batch's "
                        "column counts for every batch) over the family's time; above 1 because products with "
                        "structural zeros are skipped, not executed"}

    relu_ms = (prof["ranges"]["ms"] + prof["relax"]["ms"]) / K
    relu_bytes = prof["ranges"]["work"] / K + n_batches * sum(16.0 * s_["N"] * B + 16.0 * s_["n_cross"] for s_ in stats)
    dense_relu = 0.0
    for i, s_ in enumerate(stats):
        cin, n = cols_seg[i], s_["N"]
        dense_relu += 8.0 * n * cin + 16.0 * (cin - B) + 16.0 * n * B
        dense_relu += 16.0 * n * B + 8.0 * (s_["n_dead"] + s_["n_cross"]) * cin / B + 8.0 * n * s_["n_cross"] \
            + 16.0 * s_["n_cross"]
    dense_relu *= n_batches
    relu_step = {"bound": "hbm", "achieved": relu_bytes / (relu_ms * 1e-3) / 1e9 if relu_ms > 0 else 0.0,
                 "peak": hbm_peak, "unit": "GB/s", "peak_source": hbm_src, "ms_per_step": relu_ms,
                 "dense_equivalent": {"achieved": dense_relu / (relu_ms * 1e-3) / 1e9 if relu_ms > 0 else 0.0,
                                      "unit": "GB/s",
                                      "note": "dense-layout bytes of the step over the same time; above the copy "
                                              "rate because zero windows are skipped, cleared rows are masked by "
                                              "the next layer and one-hot columns stay implicit"}}
    relu_step["frac"] = relu_step["achieved"] / hbm_peak
    relu_step["dense_equivalent"]["frac"] = relu_step["dense_equivalent"]["achieved"] / hbm_peak
    dominant = max(kernels, key=lambda k: prof[k]["ms"])
    out_main = roof(dominant)
    if dominant == "conv" and cfg.get("name") == "cnn32" and not cfg.get("small"):
        # DRAM read + write of the convolution launches of one reach, from the committed ncu capture at 8 images per
        # batch (profiles/conv_win_ws_and_fc_gather_cnn32_batch8.md: 154.6 + 289.5 + 64.2 + 773.1 + 275.1 + 380.7 MB
        # for the six windowed launches of 8 images), scaled by the images a step processes: the columns, and with
        # them the bytes, grow in proportion to the images
        traffic_per_image = 1937.2e6 / 8.0
        out_main["traffic"] = traffic_per_image * res["line"]["queries_per_step"] * K / max(prof["conv"]["launches"], 1)
        out_main["traffic_source"] = ("dram__bytes (read + write) of conv_win_ws_kernel from an ncu capture at 8 images "
                                      "per batch, scaled to this step's images; per launch of the family "
                                      "(the family's launches include the small centre-column launches)")
    return {"roofline": dict(out_main, **({"dense_equivalent": dense_equiv(dominant)} if dominant in dense else {})),
            "roofline_other": {k: dict(roof(k), **({"dense_equivalent": dense_equiv(k)} if k in dense else {}))
                               for k in kernels if k != dominant},
            "relu_step": relu_step,
            "family_ms_per_step": {k: v["ms"] / K for k, v in prof.items()}}


def run_sharded(env, name, K, W):
    """One set per step, its generators split over the ranks (strong scaling); see nnv_b200/sharding.py."""
    import torch
    from nnv_b200 import _lib as L
    from nnv_b200.configs import make_config
    from nnv_b200.engine import Batch, Network

    ctx, dev, stream, barrier, world, rank = (env[k] for k in ("ctx", "dev", "stream", "barrier", "world", "rank"))
    nq, sub, desc = WORKLOADS[name]
    n_img = min(nq, max(1, env["args"].images))
    cfg = make_config(name, n_queries=n_img)
    net = Network(ctx, cfg["layers"], cfg["in_shape"])
    if world > 1:
        ctx.set_shard_nccl(rank, world, peer_memory=bool(env["args"].peer_memory))
    batches = []
    for qu in cfg["queries"]:
        b = Batch(net, [qu])
        b.upload()
        batches.append((b, np.array([qu["target"]], dtype=np.int32)))
    verdicts = []

    def step(s, keep):
        b, tg = batches[s % n_img]
        b.reach(keep_layer_bounds=True)
        v, _, _ = b.verify_robust(tg, "max")
        if keep:
            verdicts.append(int(v[0]))

    step(0, False)
    for s in range(W):
        step(s, False)
    barrier()
    ctx.profile_enable(True)
    l0 = ctx.launch_count
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for s in range(K):
        step(W + s, True)
    ev1.record(stream)
    barrier()
    dev_ms = ev0.elapsed_time(ev1)
    prof = ctx.profile_read()
    ctx.profile_enable(False)
    sh = prof["allreduce"]
    launches = ctx.launch_count - l0
    stats = batches[(W + K - 1) % n_img][0].relu_stats()
    t = torch.tensor([dev_ms, float(launches)], dtype=torch.float64, device=dev)
    if world > 1:
        import torch.distributed as dist
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        tsum = t.clone()
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        dev_ms, launches = float(tmax[0]), int(tsum[1])
    out = {"workload": desc, "value": K / (dev_ms * 1e-3), "unit": UNIT, "steps": K, "ms_per_step": dev_ms / K,
           "scaling": "strong", "shard": "generators", "images": n_img,
           "gpu_launches": launches,
           "verdicts": {"robust": verdicts.count(L.VERDICT_EMPTY), "unknown": verdicts.count(L.VERDICT_NONEMPTY),
                        "undecided_on_device": verdicts.count(L.UNDECIDED)},
           "columns_after_relu_this_rank": [s_["cols_after"] for s_ in stats],
           "crossing_per_relu": [s_["n_cross"] for s_ in stats],
           "family_ms_per_step": {k: v["ms"] / K for k, v in prof.items()},
           "allreduce": {"bytes_per_rank_per_step": sh["work"] / K, "ms_per_step": sh["ms"] / K,
                         "share_of_step": sh["ms"] / dev_ms if dev_ms else None,
                         "how": ("none: one rank" if world == 1 else
                                 "NCCL all-reduce inside the library (ncclDouble, ncclSum) per ReLU layer"
                                 if not env["args"].peer_memory else
                                 "peer memory: per ReLU layer the partial sums are written to a peer-mapped buffer and "
                                 "added inside the classification kernel (time = reduce + flag + classify kernels); "
                                 "NCCL for the small verdict reductions")}}
    for b, _ in batches:
        b.close()
    net.close()
    if world > 1:
        ctx.set_shard_nccl(0, 1)              # back to unsharded sets
    return out


def run_contexts(args, n_ctx):
    """``--contexts C``: the workload's query list split over C engine contexts of ONE GPU, each with its own stream
    and host thread (ctypes releases the GIL inside the library).  Small batches leave the GPU mostly idle between a
    reach's host round trips (one per ReLU layer, two in the verdict); a second context fills those gaps with the
    other batch's kernels.  Timing: wall clock between two device synchronisations around the K steps of all
    threads (the contexts' streams are independent, so no single stream's events cover the region)."""
    import threading

    import torch

    from nnv_b200 import _lib as L
    from nnv_b200 import nn
    from nnv_b200.configs import make_config
    from nnv_b200.engine import Batch, Context, Network

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    K, W = args.steps, args.warmup
    name = args.workload or "cnn32"
    nq, sub, desc = WORKLOADS[name]
    if args.batch:
        sub = args.batch
    if args.queries:
        nq = min(nq, args.queries)
        desc += " [first %d queries only]" % nq
    cfg = make_config(name, n_queries=nq)
    layers, shape = cfg["layers"], cfg["in_shape"]
    kind = cfg["queries"][0].get("spec", "max")
    groups = [np.arange(i, min(nq, i + sub)) for i in range(0, nq, sub)]
    opts = {"reachMethod": "approx-star"}
    sets_all = _sets_of(nn, cfg["queries"])
    gate = threading.Barrier(n_ctx + 1)
    counts = [dict(robust=0, unknown=0, second_pass=0, launches=0) for _ in range(n_ctx)]
    errors = []

    def worker(c):
        try:
            torch.cuda.set_device(local)
            ctx = Context(local, (args.arena_gb << 30) // n_ctx)
            net = Network(ctx, layers, shape)
            model = nn.NN(layers, ctx=ctx)
            model._nets[tuple(int(x) for x in shape)] = net
            mine = groups[c::n_ctx]
            batches = []
            for g in mine:
                b = Batch(net, [cfg["queries"][i] for i in g])
                b.upload()
                batches.append(b)
            targets0 = [np.array([cfg["queries"][i]["target"] for i in g], dtype=np.int32) for g in mine]

            def step(count):
                for b, g, t0 in zip(batches, mine, targets0):
                    b.reach(keep_layer_bounds=True)
                    v, _, _ = b.verify_robust(t0, kind)
                    und = int((v == L.UNDECIDED).sum())
                    res = (model.finish_verdicts([sets_all[i] for i in g], opts, t0 + 1, v, kind) if und
                           else np.where(v == L.VERDICT_EMPTY, 1, 2))
                    if count:
                        counts[c]["robust"] += int((res == 1).sum())
                        counts[c]["unknown"] += int((res == 2).sum())
                        counts[c]["second_pass"] += und

            for _ in range(W + 1):
                step(False)
            torch.cuda.synchronize(dev)
            gate.wait()                 # all contexts warm: the main thread starts the clock
            l0 = ctx.launch_count
            for _ in range(K):
                step(True)
            torch.cuda.synchronize(dev)
            counts[c]["launches"] = ctx.launch_count - l0
            gate.wait()
            for b in batches:           # handles go in the order batch, network, context
                b.close()
            net.close()
            ctx.close()
        except BaseException as exc:     # a failed worker must not leave the others at the gate
            errors.append(exc)
            gate.abort()

    threads = [threading.Thread(target=worker, args=(c,)) for c in range(n_ctx)]
    sampler = ClockSampler(local)
    for t in threads:
        t.start()
    try:
        gate.wait()
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        gate.wait()
        torch.cuda.synchronize(dev)
        wall = time.perf_counter() - t0
    except threading.BrokenBarrierError:
        wall = None
    for t in threads:
        t.join()
    clocks = sampler.stop()
    if errors or wall is None:
        raise errors[0] if errors else RuntimeError("a context thread failed")
    emit({"metric": METRIC, "value": K * nq / wall, "unit": UNIT, "n_gpus": 1, "steps": K, "warmup": W,
          "ms_per_step": wall * 1e3 / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
          "dtype": "f64", "data": "synthetic",
          "config": {"workload": desc, "queries_per_step": nq, "batch_per_launch": sub, "contexts": n_ctx,
                     "timing": "wall clock between device synchronisations around the K steps of all context threads",
                     "verdicts": {"robust": sum(x["robust"] for x in counts), "unknown": sum(x["unknown"] for x in counts),
                                  "finished_by_second_pass": sum(x["second_pass"] for x in counts)}},
          "gpu_launches": sum(x["launches"] for x in counts), "clocks": clocks})


def run_ours(args):
    import torch
    import torch.distributed as dist

    from nnv_b200.engine import Context

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    K, W = args.steps, args.warmup

    ctx = Context(local, args.arena_gb << 30)
    stream = torch.cuda.ExternalStream(ctx.stream, device=dev)

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    env = {"ctx": ctx, "dev": dev, "stream": stream, "barrier": barrier, "world": world, "rank": rank, "args": args}
    main = args.workload or "cnn32"

    if args.shard == "generators":
        sampler = ClockSampler(local) if rank == 0 else None
        out = run_sharded(env, main, K, W)
        clocks = sampler.stop() if sampler else None
        if rank == 0:
            line = {"metric": METRIC, "value": out["value"], "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
                    "ms_per_step": out["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                    "vs_baseline": None, "dtype": "f64", "data": "synthetic",
                    "config": {"workload": out["workload"], "shard": "generators", "images": out["images"],
                               "l2": "inputs larger than L2 (generator tensors of hundreds of MB per layer)"},
                    "gpu_launches": out["gpu_launches"], "clocks": clocks, "sharded": out}
            emit(line)
        ctx.close()
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    sampler = ClockSampler(local) if rank == 0 else None
    res = run_workload(env, main, K, W, profile=True, keep_first=(world == 1 and not args.no_cpu_baseline))
    clocks = sampler.stop() if sampler else None
    line = None
    if rank == 0:
        dgemm_tflops = measure_dgemm(torch, dev)
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
        hbm_src = "MEASURED_PEAKS.json hbm_gbs (measured copy bandwidth)" if peaks else "fallback 6650 GB/s"
        o = res["line"]
        line = {"metric": METRIC, "value": o["value"], "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
                "ms_per_step": o["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "f64", "data": "synthetic",
                "config": {"workload": o["workload"], "queries_per_step": o["queries_per_step"],
                           "batch_per_launch": o["batch_per_launch"],
                           "l2": "inputs larger than L2 (the column windows one layer reads: up to 0.16 GB per image)",
                           "verdicts": o["verdicts"], "columns_after_relu": o["columns_after_relu"]},
                "e2e": o["e2e"], "gpu_launches": o["gpu_launches"], "clocks": clocks}
        line.update(rooflines(res, K, dgemm_tflops, hbm_peak, hbm_src))
    # the other workloads of the configuration list ride along (their steps are short)
    extras = {}
    if not args.workload and not args.no_extras:
        for name in EXTRAS:
            k2 = max(2, min(K, 10))
            r2 = run_workload(env, name, k2, min(W, 3))
            extras[name] = r2["line"]
        # the fifth configuration: one 224x224 set per step, its generators split over the N ranks
        extras["vgg224"] = run_sharded(env, "vgg224", 3, 1)
    if rank == 0:
        if extras:
            line["extra"] = extras
        if world == 1 and not args.no_cpu_baseline:
            v, sample, S = cpu_reference(main)
            th = _host_threads()
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": th["cores"], "kind": "port", "sample": sample,
                                    "threads": th}
            if S is not None and "cross" in res["first"]:
                line["parity_check"] = parity_check(res["first"], S)
            for name in extras:
                if name == "vgg224":
                    extras[name]["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": th["cores"], "kind": "port",
                                                    "sample": cpu_reference(name)[1]}
                    continue
                v2, sample2, _ = cpu_reference(name, budget_s=20.0)
                extras[name]["cpu_baseline"] = {"value": v2, "unit": UNIT, "cores": th["cores"], "kind": "port",
                                                "sample": sample2}
        emit(line)
    if "cleanup" in res:
        batches, net, model = res["cleanup"]
        for b in batches:
            b.close()
        model._nets = {}
        net.close()
    ctx.close()
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
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS),
                    help="headline workload (default cnn32, with cnn28 / bright28 / fc5 carried under 'extra')")
    ap.add_argument("--shard", default="queries", choices=["queries", "generators"])
    ap.add_argument("--images", type=int, default=1, help="--shard generators: distinct images cycled through")
    ap.add_argument("--batch", type=int, default=0, help="input sets per engine batch (0: the workload's default)")
    ap.add_argument("--queries", type=int, default=0,
                    help="use only the first N queries of the headline workload (profiling captures)")
    ap.add_argument("--arena-gb", type=int, default=112)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--peer-memory", action="store_true",
                    help="--shard generators: the fused peer-memory classification instead of the NCCL all-reduce "
                         "(measured slower than NCCL at 2 and at 8 GPUs, so not the default)")
    ap.add_argument("--no-peer-memory", action="store_true", help="accepted for older command lines; the default now")
    ap.add_argument("--contexts", type=int, default=1,
                    help="one GPU: split the query list over this many engine contexts (own stream and host thread each)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.contexts > 1 and int(os.environ.get("WORLD_SIZE", "1")) == 1:
        run_contexts(args, args.contexts)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
