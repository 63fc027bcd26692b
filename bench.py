#!/usr/bin/env python
"""Headline benchmark: GQA backward TFLOP/s at B8 Hq12 Hkv4 S4096 D64 bf16 (non-causal).

    python bench.py --gpus N --steps K --warmup W            # N = 1
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...                      # the reference's CPU path (PyTorch SDPA autograd)

A step is one whole ``gqa_bwd`` call (Delta preprocess + tensor-core main kernel + dQ finalise) on one
batch of seeded synthetic inputs of the headline shape, through the C ABI.  The headline metric is weak
scaling: every rank owns a full headline-shaped batch (global batch 8*N), no data-path collective.
FLOPs use the reference's convention, backward = 4 x forward = 16*B*Hq*S^2*D
(precision/baseline_gqa.py:532-533, src/attention/GQA_bwd.cu:16090); the five GEMMs of the kernel execute
10*B*Hq*S^2*D, and the tensor roofline fraction is computed from those.

Rank 0 prints ONE JSON line.  Keys beyond the base contract:
  roofline     tensor-core roofline of the dominant kernel (the backward main kernel): executed-MMA
               TFLOP/s over its duration, measured live with CUDA events inside the library on the
               launching stream, against the measured cuBLAS bf16 peak
  sustained    the same step repeated back to back for >= 2 s (power-capped regime), with clocks
  parity       max-abs / relative-RMS of O, dQ, dK, dV against fp32 PyTorch SDPA autograd (the CPU-baseline
               sample acts as the checker, outside every timed region)
  cpu_baseline the reference's oracle path (fp32 PyTorch SDPA autograd) on the host cores, bounded sample
  e2e          same metric with host (pinned) buffers: H2D of Q,K,V,O,dO,LSE + gqa_bwd + D2H of dQ,dK,dV
  sharded      the split the (batch x KV-head) groups allow: ONE problem cut over the N ranks (strong
               scaling), headline shape and the long-context shape, outputs gathered over NCCL and compared
               with the unsharded run
  config.other the remaining benchmark configurations on one GPU (N = 1 runs only)
"""
from __future__ import annotations

import argparse
import datetime
import itertools
import json
import math
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HEADLINE = dict(B=8, Hq=12, Hkv=4, S=4096, D=64, causal=False)
LONG_CONTEXT = dict(B=1, Hq=64, Hkv=8, S=32768, D=128, causal=True)
METRIC = "GQA bwd TFLOP/s (B8 Hq12 Hkv4 S4096 D64 bf16)"
NOMINAL_BF16_TFLOPS = 2250.0
# dram__bytes_read.sum + dram__bytes_write.sum of the backward main kernel from one ncu capture at B=4
# (B4 Hq12 Hkv4 S4096 D64: 124.0 MB read + 26.9 MB written = 150.9 MB), scaled by 2 to the headline batch: the
# (batch, KV-head) groups are independent, so traffic grows in proportion to B.
MAIN_KERNEL_DRAM_BYTES_PER_LAUNCH = 2 * 150.9e6
# dram bytes of the forward kernel at B4 Hq12 Hkv4 S4096 D64 (42.0 MB read + 0.8 MB written), same scaling
FWD_KERNEL_DRAM_BYTES_PER_LAUNCH = 2 * 42.8e6


def fwd_flops(B, Hq, S, D, causal):
    f = 4.0 * B * Hq * S * S * D
    return f * 0.5 if causal else f


def bwd_flops(B, Hq, S, D, causal):
    return 4.0 * fwd_flops(B, Hq, S, D, causal)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"bf16_tflops": float(p["bf16_tflops"]), "bf16_tflops_sustained": float(p["bf16_tflops_sustained"]),
                "hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi for the whole run; every sample carries
    nvidia-smi's timestamp, so the samples that fall inside a timed region can be picked out afterwards."""

    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index: int):
        self.proc = None
        self.samples = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def wait_until_reporting(self, seconds: float = 1.5):
        """nvidia-smi needs a moment before its first sample; timed regions start after this."""
        if self.proc is not None:
            time.sleep(seconds)

    def stop(self):
        if self.proc is None or self.samples is not None:
            return
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        self.samples = []
        for line in out.splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                t = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                sm, mx, power = float(parts[1]), float(parts[2]), float(parts[3])
            except ValueError:
                continue
            reasons = [n for n, v in zip(self.NAMES, parts[4:8]) if v.lower().startswith("active")]
            self.samples.append((t, sm, mx, power, reasons))

    def window(self, t0: float, t1: float):
        """Median SM clock, power and the throttle reasons seen between two time.time() stamps."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvidia-smi unavailable"]}
        self.stop()
        inside = [s for s in self.samples if t0 <= s[0] <= t1]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": max((s[2] for s in self.samples), default=None), "samples": 0,
                    "reasons": []}
        return {"sm_mhz": statistics.median(s[1] for s in inside), "sm_max_mhz": max(s[2] for s in inside),
                "power_w_median": statistics.median(s[3] for s in inside), "samples": len(inside),
                "reasons": sorted({r for s in inside for r in s[4]})}


def host_inputs(B, Hq, Hkv, S, D, seed):
    """Q, K, V ~ N(0,1) from `seed`, dO ~ N(0,1) from `seed + 1` (torch CPU generator), rounded to bf16."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hq, S, D, generator=g).bfloat16()
    k = torch.randn(B, Hkv, S, D, generator=g).bfloat16()
    v = torch.randn(B, Hkv, S, D, generator=g).bfloat16()
    do = torch.randn(B, Hq, S, D, generator=torch.Generator().manual_seed(seed + 1)).bfloat16()
    return q, k, v, do


def cpu_sdpa_backward_sample(steps: int, warmup: int, sample_b: int, shape, seed=42):
    """The reference's oracle path on the host: fp32 SDPA + autograd (precision/baseline_gqa.py:64-66,
    :429-435; harness/run_gqa_bwd_v44_bench.py:108-118) on the first `sample_b` of the B batches of the seeded
    inputs.  Returns the median backward seconds, the thread count, the sample description and the fp32
    results (O, dQ, dK, dV) of the sample, which the caller may use as the parity checker."""
    import torch.nn.functional as F

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    Hq, Hkv, S, D, causal = shape["Hq"], shape["Hkv"], shape["S"], shape["D"], shape["causal"]
    q, k, v, do = (t[:sample_b].float() for t in host_inputs(shape["B"], Hq, Hkv, S, D, seed))
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    times, o = [], None
    for i in range(warmup + steps):
        q.grad = k.grad = v.grad = None
        o = F.scaled_dot_product_attention(q, k, v, scale=1.0 / math.sqrt(D), enable_gqa=True, is_causal=causal)
        t0 = time.perf_counter()
        o.backward(do)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    sample = (f"{sample_b} of {shape['B']} batches ({sample_b * Hkv} of {shape['B'] * Hkv} (batch,KV-head) groups), "
              f"fp32 torch SDPA autograd backward, {warmup} warm-up + {steps} timed")
    return statistics.median(times), threads, sample, (o.detach(), q.grad, k.grad, v.grad)


def run_reference_arm(args, rank):
    if rank != 0:
        return
    shape = HEADLINE
    sample_b = 2
    sec, threads, sample, _ = cpu_sdpa_backward_sample(max(1, args.steps), max(1, args.warmup), sample_b, shape)
    tflops = bwd_flops(sample_b, shape["Hq"], shape["S"], shape["D"], shape["causal"]) / sec / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "GQA non-causal backward, B8 Hq12 Hkv4 S4096 D64 (reference config)",
                   "sample": sample},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "reference", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def tensor_metrics(got, ref):
    d = got.double() - ref.double()
    return {"max_abs": float(d.abs().max()),
            "rel_rms": float(d.pow(2).sum().sqrt() / ref.double().pow(2).sum().sqrt().clamp_min(1e-30)),
            "gate_ok": bool((d.abs() <= 2e-2 + 2e-2 * ref.double().abs()).all())}


class Timer:
    """Median device time of a callable over L2-flushed repetitions (CUDA events on the current stream)."""

    def __init__(self, flush):
        self.flush = flush

    def __call__(self, fn, reps=10, warmup=3):
        for _ in range(warmup):
            fn()
        ms = []
        for _ in range(reps):
            self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            b.synchronize()
            ms.append(a.elapsed_time(b))
        return statistics.median(ms)


def rate(flops, ms, peaks, executed_ratio):
    """TFLOP/s in the reference's convention and as executed MMA work, with roofline fractions."""
    tf = flops / (ms * 1e-3) / 1e12
    ex = tf * executed_ratio
    return {"ms": round(ms, 4), "tflops": round(tf, 1), "tflops_executed_mma": round(ex, 1),
            "frac_nominal": round(tf / NOMINAL_BF16_TFLOPS, 3),
            "frac_executed_of_measured_burst": round(ex / peaks["bf16_tflops"], 3),
            "frac_executed_of_measured_sustained": round(ex / peaks["bf16_tflops_sustained"], 3)}


def device_inputs(B, Hq, Hkv, S, D, dev, seed, do_mul=1.0):
    g = torch.Generator(device=dev).manual_seed(seed)
    q = torch.randn(B, Hq, S, D, generator=g, device=dev).bfloat16()
    k = torch.randn(B, Hkv, S, D, generator=g, device=dev).bfloat16()
    v = torch.randn(B, Hkv, S, D, generator=g, device=dev).bfloat16()
    do = (torch.randn(B, Hq, S, D, generator=g, device=dev) * do_mul).bfloat16()
    return q, k, v, do


def other_configs(gqa, ops, dev, timer, peaks):
    """The remaining benchmark configurations on one GPU: forward at the headline shape, forward + backward at the
    causal D = 128 and the long-context shape, and the 16-point forward sweep.  Device-timed medians of 10
    L2-flushed repetitions after 3 warm-ups."""
    out = {}

    def fwd_bwd(name, B, Hq, Hkv, S, D, causal, do_mul=1.0, backward=True):
        q, k, v, do = device_inputs(B, Hq, Hkv, S, D, dev, 7, do_mul)
        sc = 1.0 / math.sqrt(D)
        o = torch.empty_like(q)
        lse = torch.empty(B, Hq, S, dtype=torch.float32, device=dev)
        f_ms = timer(lambda: gqa.gqa_forward(q, k, v, causal=causal, scale=sc, out=o, lse=lse))
        ops.check_status()
        entry = {"shape": f"B{B} Hq{Hq} Hkv{Hkv} S{S} D{D} {'causal' if causal else 'non-causal'}",
                 "fwd": rate(fwd_flops(B, Hq, S, D, causal), f_ms, peaks, 1.0)}
        if backward:
            ws = torch.empty(gqa.bwd_workspace_bytes(B, Hq, Hkv, S, D, causal), dtype=torch.uint8, device=dev)
            dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
            b_ms = timer(lambda: gqa.gqa_backward(q, k, v, o, do, lse, causal=causal, scale=sc, workspace=ws, dq=dq,
                                                  dk=dk, dv=dv))
            ops.check_status(ws)
            entry["bwd"] = rate(bwd_flops(B, Hq, S, D, causal), b_ms, peaks, 10.0 / 16.0)
        out[name] = entry

    fwd_bwd("headline_forward", 8, 12, 4, 4096, 64, False, backward=False)
    fwd_bwd("headline_shape_causal", 8, 12, 4, 4096, 64, True)
    fwd_bwd("causal_d128", 4, 32, 8, 8192, 128, True, do_mul=0.1)
    fwd_bwd("long_context", 1, 64, 8, 32768, 128, True)
    # a packed variable-length batch: 32 768 tokens in sequences of 128 .. 8 192 (two thirds of them short), causal
    lens = [8192, 4096, 4096, 2048, 2048, 2048, 1024, 1024, 1024, 1024] + [512] * 8 + [256] * 6 + [128] * 4
    T, Hq, Hkv, D = sum(lens), 32, 8, 128
    g = torch.Generator(device=dev).manual_seed(13)
    q = torch.randn(T, Hq, D, generator=g, device=dev).bfloat16()
    k = torch.randn(T, Hkv, D, generator=g, device=dev).bfloat16()
    v = torch.randn(T, Hkv, D, generator=g, device=dev).bfloat16()
    do = (torch.randn(T, Hq, D, generator=g, device=dev) * 0.1).bfloat16()
    cu = torch.tensor([0] + list(itertools.accumulate(lens)), dtype=torch.int32, device=dev)
    o, lse = torch.empty_like(q), torch.empty(Hq, T, dtype=torch.float32, device=dev)
    f_ms = timer(lambda: ops.gqa_forward_varlen(q, k, v, cu, max(lens), causal=True, out=o, lse=lse))
    ops.check_status()
    ws = torch.empty(ops.bwd_varlen_workspace_bytes(T, Hq, Hkv, D), dtype=torch.uint8, device=dev)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    b_ms = timer(lambda: ops.gqa_backward_varlen(q, k, v, o, do, lse, cu, max(lens), causal=True, workspace=ws, dq=dq,
                                                 dk=dk, dv=dv))
    ops.check_status(ws)
    f_fl = sum(fwd_flops(1, Hq, n, D, True) for n in lens)
    out["packed_varlen_causal_d128"] = {
        "shape": f"{len(lens)} sequences of 128..8192 tokens, {T} in all, Hq{Hq} Hkv{Hkv} D{D} causal, [T,H,D] + cu_seqlens",
        "fwd": rate(f_fl, f_ms, peaks, 1.0), "bwd": rate(4.0 * f_fl, b_ms, peaks, 10.0 / 16.0),
        "outputs_finite": bool(torch.isfinite(dq.float()).all() and torch.isfinite(dk.float()).all()
                               and torch.isfinite(dv.float()).all() and torch.isfinite(o.float()).all())}
    del q, k, v, do, o, lse, ws, dq, dk, dv
    sweep = {}
    for D in (64, 128):
        for S in (1024, 2048, 4096, 16384):
            for causal in (False, True):
                B, Hq, Hkv = 16, 16, 2
                q, k, v, _ = device_inputs(B, Hq, Hkv, S, D, dev, 11)
                o = torch.empty_like(q)
                lse = torch.empty(B, Hq, S, dtype=torch.float32, device=dev)
                ms = timer(lambda: gqa.gqa_forward(q, k, v, causal=causal, out=o, lse=lse))
                sweep[f"S{S}_D{D}_{'causal' if causal else 'noncausal'}"] = {
                    "ms": round(ms, 4), "tflops": round(fwd_flops(B, Hq, S, D, causal) / (ms * 1e-3) / 1e12, 1)}
                del q, k, v, o, lse
    ops.check_status()
    out["forward_sweep_B16_Hq16_Hkv2"] = sweep
    return out


def sharded_problem(name, shape, tensors, gqa, ops, sharding, timer, dist, rank, world, peaks, sdpa_sample=None,
                    sdpa_group_check=False):
    """ONE problem cut over the ranks by (batch x KV-head) groups (strong scaling): every rank holds the whole
    seeded problem, runs the unmodified forward/backward on zero-copy views of its group range, and its backward
    is device-timed (median of 5 L2-flushed repetitions).  Aggregate = total FLOPs / slowest rank.  Outside the
    timed region the shards of dQ/dK/dV are all-gathered over NCCL and compared on rank 0 with the unsharded
    run of the same problem, whose time is the N = 1 reference for the efficiency."""
    B, Hq, Hkv, S, D, causal = (shape[k] for k in ("B", "Hq", "Hkv", "S", "D", "causal"))
    G, n_groups, sc = Hq // Hkv, B * Hkv, 1.0 / math.sqrt(D)
    q, k, v, do = tensors
    dev = q.device
    begin, end = sharding.group_range(rank, world, n_groups)
    n = end - begin
    parts = [sharding.shard(t, Hkv, rank, world) for t in (q, k, v, do)]
    my_ms = 0.0
    if n > 0:
        sq, sk, sv, sdo = parts
        so, slse = gqa.gqa_forward(sq, sk, sv, causal=causal, scale=sc)
        # a shard may hold too few KV tiles to fill the GPU evenly: let the library split tiles by query head
        ws = torch.empty(gqa.bwd_workspace_bytes(n, G, 1, S, D, causal, split_heads=True), dtype=torch.uint8, device=dev)
        sdq, sdk, sdv = torch.empty_like(sq), torch.empty_like(sk), torch.empty_like(sv)
        my_ms = timer(lambda: gqa.gqa_backward(sq, sk, sv, so, sdo, slse, causal=causal, scale=sc, workspace=ws,
                                               dq=sdq, dk=sdk, dv=sdv, split_heads=True), reps=5, warmup=2)
        ops.check_status(ws)
        del ws
    else:
        sdq = q.new_zeros((0, G, S, D))
        sdk = sdv = k.new_zeros((0, 1, S, D))
    times = torch.tensor([my_ms], dtype=torch.float64, device=dev)
    if dist is not None:
        all_t = [torch.empty_like(times) for _ in range(world)]
        dist.all_gather(all_t, times)
        all_ms = [float(t.item()) for t in all_t]
        gathered = [sharding.gather_groups(t, n_groups, rank, world) for t in (sdq, sdk, sdv)]
    else:
        all_ms = [my_ms]
        gathered = [sdq, sdk, sdv]
    result = None
    if rank == 0:
        # the unsharded run of the same problem on this GPU: the N = 1 time and the values to compare with
        o, lse = gqa.gqa_forward(q, k, v, causal=causal, scale=sc)
        ws = torch.empty(gqa.bwd_workspace_bytes(B, Hq, Hkv, S, D, causal), dtype=torch.uint8, device=dev)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        if world > 1:
            one_ms = timer(lambda: gqa.gqa_backward(q, k, v, o, do, lse, causal=causal, scale=sc, workspace=ws, dq=dq,
                                                    dk=dk, dv=dv), reps=5, warmup=2)
        else:
            gqa.gqa_backward(q, k, v, o, do, lse, causal=causal, scale=sc, workspace=ws, dq=dq, dk=dk, dv=dv)
            one_ms = my_ms
        ops.check_status(ws)
        gdq, gdk, gdv = (g.reshape(t.shape) for g, t in zip(gathered, (dq, dk, dv)))
        dq_m, dk_m, dv_m = tensor_metrics(gdq, dq), tensor_metrics(gdk, dk), tensor_metrics(gdv, dv)
        bit_equal = bool(torch.equal(gdk, dk) and torch.equal(gdv, dv))
        # dK/dV are bit-equal to the unsharded run unless a shard used the head split (fp32 partial sums added in a
        # fixed order: same values up to the last bf16 bit)
        gather_ok = bool(dq_m["rel_rms"] <= 2e-3 and (bit_equal or max(dk_m["rel_rms"], dv_m["rel_rms"]) <= 2e-3))
        slow = max(all_ms)
        flops = bwd_flops(B, Hq, S, D, causal)
        result = {
            "shape": f"B{B} Hq{Hq} Hkv{Hkv} S{S} D{D} {'causal' if causal else 'non-causal'}, {n_groups} groups over "
                     f"{world} rank(s)",
            "rank_ms": [round(x, 4) for x in all_ms], "slowest_ms": round(slow, 4), "one_gpu_ms": round(one_ms, 4),
            "tflops_aggregate": round(flops / (slow * 1e-3) / 1e12, 1),
            "frac_executed_of_measured_burst_per_gpu": round(flops * 10 / 16 / (slow * 1e-3) / 1e12 / world
                                                             / peaks["bf16_tflops"], 3),
            "speedup_vs_one_gpu": round(one_ms / slow, 3), "efficiency": round(one_ms / slow / world, 3),
            "work_items_per_rank": int(math.ceil(S / 128) * max(e - b for b, e in
                                                                     (sharding.group_range(r, world, n_groups)
                                                                      for r in range(world)))),
            "gather": "NCCL all_gather of dQ/dK/dV shards" if dist is not None else "single rank (no gather)",
            "gather_ok": gather_ok, "dk_dv_bit_equal_to_unsharded": bit_equal,
            "dk_dv_rel_rms_vs_unsharded": max(dk_m["rel_rms"], dv_m["rel_rms"]),
            "dq_rel_rms_vs_unsharded": dq_m["rel_rms"],
            "head_split": "GQA_BWD_SPLIT_HEADS passed for the shards (the library splits only when a shard has too few "
                          "KV tiles to fill its GPU)",
        }
        if sdpa_sample is not None:  # fp32 SDPA autograd of the first batches (the CPU-baseline sample)
            _, rdq, rdk, rdv = sdpa_sample
            nb = rdq.shape[0]
            pm = {n_: tensor_metrics(g_[:nb].float().cpu(), r_) for n_, g_, r_ in
                  (("dQ", gdq, rdq), ("dK", gdk, rdk), ("dV", gdv, rdv))}
            result["gathered_vs_fp32_sdpa_sample"] = {
                "gate_ok": all(m["gate_ok"] and m["rel_rms"] <= 2e-2 for m in pm.values()),
                **{n_: {"max_abs": m["max_abs"], "rel_rms": m["rel_rms"]} for n_, m in pm.items()}}
        if sdpa_group_check:  # fp32 SDPA on this GPU for one (batch, KV-head) group of the gathered result
            from oracle import sdpa_ref

            hs = slice(0, G)
            _, _, rdq, rdk, rdv = sdpa_ref.sdpa_group(q[0, hs], k[0, 0], v[0, 0], do[0, hs], sc, causal, want_lse=False)
            pm = {"dQ": tensor_metrics(gdq[0, hs], rdq), "dK": tensor_metrics(gdk[0, 0], rdk),
                  "dV": tensor_metrics(gdv[0, 0], rdv)}
            result["gathered_vs_fp32_sdpa_group0"] = {
                "gate_ok": all(m["gate_ok"] and m["rel_rms"] <= 2e-2 for m in pm.values()),
                **{n_: {"max_abs": m["max_abs"], "rel_rms": m["rel_rms"]} for n_, m in pm.items()}}
    if dist is not None:
        dist.barrier()
    return result


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline and the parity block it feeds")
    ap.add_argument("--no-other", action="store_true", help="skip the other benchmark configurations (N = 1 only)")
    ap.add_argument("--no-sharded", action="store_true", help="skip the strong-scaling (sharded) block")
    ap.add_argument("--sustain-seconds", type=float, default=2.0)
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs WORLD_SIZE={args.gpus} (launch with torch.distributed.run); got {world}")
    if args.warmup < 3:
        args.warmup = 3

    import hopper_jeni_b200 as gqa
    from hopper_jeni_b200 import ops, sharding

    sampler = ClockSampler(local_rank) if rank == 0 else None
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)

    B, Hq, Hkv, S, D, causal = (HEADLINE[k] for k in ("B", "Hq", "Hkv", "S", "D", "causal"))
    scale = 1.0 / math.sqrt(D)
    # seeded on the host (rank r: seeds 42 + 2r / 43 + 2r) so that the CPU baseline sample sees the same values
    host_q, host_k, host_v, host_do = host_inputs(B, Hq, Hkv, S, D, 42 + 2 * rank)
    q, k, v, do = (t.to(dev) for t in (host_q, host_k, host_v, host_do))
    o, lse = gqa.gqa_forward(q, k, v, causal=causal, scale=scale)
    ops.check_status()
    ws = torch.empty(gqa.bwd_workspace_bytes(B, Hq, Hkv, S, D, causal), dtype=torch.uint8, device=dev)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    timer = Timer(flush)
    peaks = load_peaks()

    def step():
        gqa.gqa_backward(q, k, v, o, do, lse, causal=causal, scale=scale, workspace=ws, dq=dq, dk=dk, dv=dv)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    if sampler:
        sampler.wait_until_reporting()
    for _ in range(args.warmup):
        step()
    barrier()
    ops.check_status(ws)

    # ---- timed region: K steps, device-timed per step, L2 flushed before each ----
    launches0 = gqa.launch_count()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier()
    t_head0 = time.time()
    for i in range(args.steps):
        flush.zero_()
        starts[i].record()
        step()
        stops[i].record()
    barrier()
    t_head1 = time.time()
    launches = gqa.launch_count() - launches0
    step_ms = [a.elapsed_time(b) for a, b in zip(starts, stops)]
    total_ms = torch.tensor([sum(step_ms)], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
    total_ms = float(total_ms.item())
    ops.check_status(ws)

    # ---- dominant kernel alone (roofline): stage times measured inside the library ----
    stage_ms = [ops.bwd_stage_times(q, k, v, o, do, lse, causal, scale, ws, dq, dk, dv, flush) for _ in range(5)]
    main_ms = statistics.median(s[1] for s in stage_ms)
    pre_ms = statistics.median(s[0] for s in stage_ms)
    fin_ms = statistics.median(s[2] for s in stage_ms)
    fwd_ms = timer(lambda: gqa.gqa_forward(q, k, v, causal=causal, scale=scale, out=o, lse=lse)) if rank == 0 else None
    dev_o, dev_dq, dev_dk, dev_dv = o, dq.clone(), dk.clone(), dv.clone()

    # ---- end to end with host buffers: pinned host tensors in, pinned host tensors out, every step.  The
    # (batch x KV-head) groups are streamed in chunks so that copies and gqa_bwd calls overlap.
    from hopper_jeni_b200.hostpipe import HostBackward

    host_in = [t.cpu().pin_memory() for t in (q, k, v, o, do, lse)]
    host_out = [torch.empty_like(t, device="cpu").pin_memory() for t in (dq, dk, dv)]
    pipe = HostBackward(B, Hq, Hkv, S, D, causal=causal, scale=scale, chunks=8, device=dev)
    h2d, d2h = pipe.h2d_bytes, pipe.d2h_bytes

    def e2e_step():
        pipe(*host_in, *host_out)

    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    pipe.synchronize()
    barrier()
    e2e_ok = bool(torch.equal(host_out[1], dk.cpu()) and torch.equal(host_out[2], dv.cpu()))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    pipe.synchronize()
    e2e_ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_ms = float(e2e_ms.item())

    # the ceiling of that path: the bare copies, all ranks at once (they share the host's memory and PCIe roots)
    def copy_rate(pairs, nbytes):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(3):
            for dst, src in pairs:
                dst.copy_(src, non_blocking=True)
        b.record()
        b.synchronize()
        ms = torch.tensor([a.elapsed_time(b) / 3], dtype=torch.float64, device=dev)
        if dist is not None:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return nbytes / (float(ms.item()) * 1e-3) / 1e9

    h2d_gbs = copy_rate(list(zip((q, k, v, o, do, lse), host_in)), h2d)
    d2h_gbs = copy_rate(list(zip(host_out, (dq, dk, dv))), d2h)
    del pipe, host_in, host_out

    # ---- the same step back to back for >= 2 s: the power-capped regime (after every burst measurement).  No flush between steps: the inputs
    # and outputs of one step (270 MB + the 100 MB accumulator) exceed the 126 MB L2. ----
    n_sus = max(args.steps, int(math.ceil(args.sustain_seconds * 1e3 / (total_ms / args.steps))))
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_sus0 = time.time()
    s0.record()
    for _ in range(n_sus):
        step()
    s1.record()
    barrier()
    t_sus1 = time.time()
    sus_ms = torch.tensor([s0.elapsed_time(s1)], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(sus_ms, op=dist.ReduceOp.MAX)
    sus_ms = float(sus_ms.item()) / n_sus
    ops.check_status(ws)

    # ---- every rank's outputs are finite (NCCL, outside every timed region) ----
    sums = torch.stack([dq.float().abs().sum(), dk.float().abs().sum(), dv.float().abs().sum(),
                        torch.isfinite(dq.float()).all().float() * torch.isfinite(dk.float()).all().float()
                        * torch.isfinite(dv.float()).all().float()]).double()
    if dist is not None:
        gathered = [torch.empty_like(sums) for _ in range(world)]
        dist.all_gather(gathered, sums)
    else:
        gathered = [sums]
    all_finite = all(bool(g[3].item() == 1.0) and float(g[0].item()) > 0 for g in gathered)

    # ---- CPU baseline (rank 0): the reference's oracle path on the host cores; its gradients are the parity checker
    cpu = None
    if rank == 0 and not args.no_cpu_baseline:
        sec, threads, sample, ref = cpu_sdpa_backward_sample(3, 1, 2, HEADLINE, seed=42)
        cpu = {"sec": sec, "threads": threads, "sample": sample, "ref": ref}
    if dist is not None:
        dist.barrier()

    # ---- strong scaling: ONE problem cut over the ranks ----
    sharded = None
    if not args.no_sharded:
        sharded = {}
        # the headline problem of rank 0 (seed 42) on every rank
        if rank == 0:
            c2 = (q, k, v, do)
        else:
            c2 = tuple(t.to(dev) for t in host_inputs(B, Hq, Hkv, S, D, 42))
        r = sharded_problem("c2", HEADLINE, c2, gqa, ops, sharding, timer, dist, rank, world, peaks,
                            sdpa_sample=cpu["ref"] if cpu else None)
        if rank == 0:
            sharded["c2"] = r
        del c2
        L = LONG_CONTEXT
        c4 = device_inputs(L["B"], L["Hq"], L["Hkv"], L["S"], L["D"], dev, 4242)
        r = sharded_problem("c4", LONG_CONTEXT, c4, gqa, ops, sharding, timer, dist, rank, world, peaks,
                            sdpa_group_check=True)
        if rank == 0:
            sharded["c4"] = r
        del c4
        torch.cuda.empty_cache()

    if rank == 0:
        flops_rank = bwd_flops(B, Hq, S, D, causal)
        ms_per_step = total_ms / args.steps
        value = world * flops_rank / (ms_per_step * 1e-3) / 1e12
        executed = flops_rank * 10.0 / 16.0 / (main_ms * 1e-3) / 1e12
        clocks_head = sampler.window(t_head0, t_head1)
        clocks_sus = sampler.window(t_sus0, t_sus1)
        # the headline region is a few tens of milliseconds: report the clocks over it and the sustained region
        clocks_all = sampler.window(t_head0, t_sus1)
        sus_tf = flops_rank / (sus_ms * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {
                "workload": "GQA non-causal backward (whole gqa_bwd call: Delta preprocess + main + dQ finalise), "
                            "B8 Hq12 Hkv4 S4096 D64 bf16 per GPU, N(0,1) inputs",
                "parallelism": f"weak scaling: one headline-shaped batch per GPU on {world} GPU(s), no data-path "
                               "collective; the strong-scaling split of one problem is under `sharded`",
                "global_batch": B * world, "flop_convention": "backward = 4 x forward = 16*B*Hq*S^2*D",
                "l2": "256 MB memset before every timed step; inputs 270 MB > 126 MB L2",
                "frac_of_nominal_2250": value / world / NOMINAL_BF16_TFLOPS,
                "stage_ms": {"preprocess": pre_ms, "main": main_ms, "dq_finalise": fin_ms},
                "dq_path": "TMA reduce-add (fp32, L2) into an accumulator: not bit-reproducible; dK/dV single-writer, bit-reproducible",
                "outputs_finite_all_ranks": all_finite,
            },
            "roofline": {"bound": "tensor", "achieved": executed, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": executed / peaks["bf16_tflops"], "traffic": MAIN_KERNEL_DRAM_BYTES_PER_LAUNCH,
                         "kernel": "gqa_bwd_sm100_kernel<64>", "peak_source": peaks["source"] + " burst",
                         "flops_counted": "executed MMA work of the five GEMMs, 10*B*Hq*S^2*D per launch "
                                          "(10*128*128*D per 128x128 tile pair of a query head)",
                         "frac_of_sustained": executed / peaks["bf16_tflops_sustained"],
                         "achieved_reference_convention": executed * 16.0 / 10.0},
            "sustained": {"seconds": round(sus_ms * n_sus * 1e-3, 3), "steps": n_sus, "ms_per_step": sus_ms,
                          "tflops": world * sus_tf, "frac_of_nominal_2250": sus_tf / NOMINAL_BF16_TFLOPS,
                          "frac_executed_of_measured_sustained": sus_tf * 10 / 16 / peaks["bf16_tflops_sustained"],
                          "ms_times_median_sm_mhz": (sus_ms * clocks_sus["sm_mhz"]) if clocks_sus.get("sm_mhz") else None,
                          "clocks": clocks_sus, "l2": "no flush: one step touches 370 MB > 126 MB L2"},
            "clocks": {**clocks_all, "headline_region": clocks_head,
                       "note": "sampled every 20 ms over the headline and the sustained region"},
            "e2e": {"value": world * flops_rank / (e2e_ms / e2e_steps * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "path": "pinned host -> 8 chunks of (batch,KV-head) groups on 3 streams -> gqa_bwd -> pinned host",
                    "matches_device_resident_run": e2e_ok,
                    "bare_copy_gbs_per_rank": {"h2d": round(h2d_gbs, 1), "d2h": round(d2h_gbs, 1),
                                               "note": "all ranks copying at once, slowest rank"},
                    "copy_bound_tflops": world * flops_rank / max(h2d / (h2d_gbs * 1e9), d2h / (d2h_gbs * 1e9)) / 1e12},
            "gpu_launches": int(launches),
        }
        if fwd_ms is not None:
            f_tf = fwd_flops(B, Hq, S, D, causal) / (fwd_ms * 1e-3) / 1e12
            line["roofline_fwd"] = {"bound": "tensor", "achieved": f_tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                                    "frac": f_tf / peaks["bf16_tflops"], "traffic": FWD_KERNEL_DRAM_BYTES_PER_LAUNCH,
                                    "kernel": "gqa_fwd_sm100_kernel<64>", "ms": fwd_ms,
                                    "note": "4*B*Hq*S^2*D executed; at D = 64 the exp unit (16 384 exps per 128x128 "
                                            "tile = 1 024 cycles against 512 of tensor math) bounds this kernel"}
        if cpu is not None:
            line["cpu_baseline"] = {"value": bwd_flops(2, Hq, S, D, causal) / cpu["sec"] / 1e12, "unit": "TFLOP/s",
                                    "cores": cpu["threads"], "kind": "reference", "sample": cpu["sample"]}
            ro, rdq, rdk, rdv = cpu["ref"]
            pm = {"O": tensor_metrics(dev_o[:2].float().cpu(), ro), "dQ": tensor_metrics(dev_dq[:2].float().cpu(), rdq),
                  "dK": tensor_metrics(dev_dk[:2].float().cpu(), rdk), "dV": tensor_metrics(dev_dv[:2].float().cpu(), rdv)}
            line["parity"] = {
                **{n_: {"max_abs": m["max_abs"], "rel_rms": m["rel_rms"]} for n_, m in pm.items()},
                "gate_ok": all(m["gate_ok"] for m in pm.values()) and pm["O"]["rel_rms"] <= 1e-2
                           and all(pm[n_]["rel_rms"] <= 2e-2 for n_ in ("dQ", "dK", "dV")),
                "gate": "|d| <= 2e-2 + 2e-2|ref| element-wise, relative RMS <= 1e-2 (O) / 2e-2 (gradients)",
                "sample": "batches 0-1 of the timed problem (8 of 32 groups) against fp32 torch SDPA autograd on the host",
            }
        if sharded is not None:
            line["sharded"] = sharded
        if world == 1 and not args.no_other:
            line["config"]["other"] = other_configs(gqa, ops, dev, timer, peaks)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
