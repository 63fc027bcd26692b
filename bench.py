#!/usr/bin/env python
"""Headline benchmark: GQA backward TFLOP/s at B8 Hq12 Hkv4 S4096 D64 bf16 (non-causal).

    python bench.py --gpus N --steps K --warmup W            # N = 1
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...                      # the reference's CPU path (PyTorch SDPA autograd)

A step is one whole ``gqa_bwd`` call (Delta preprocess + tensor-core main kernel + dQ finalise) on one
batch of seeded synthetic inputs of the headline shape, through the C ABI.  With N ranks the (batch x
KV-head) groups are sharded with no data-path collective: every rank owns a full headline-shaped batch
(weak scaling, global batch 8*N); NCCL only gathers output checksums for verification after the timed
region.  FLOPs use the reference's convention, backward = 4 x forward = 16*B*Hq*S^2*D
(precision/baseline_gqa.py:532-533, src/attention/GQA_bwd.cu:16090).

Rank 0 prints ONE JSON line.  Keys beyond the base contract:
  roofline     tensor-core roofline of the dominant kernel (the backward main kernel), its duration
               measured live with CUDA events inside the library on the launching stream
  cpu_baseline the reference's oracle path (fp32 PyTorch SDPA autograd) on the host cores, bounded sample
  e2e          same metric with host (pinned) buffers: H2D of Q,K,V,O,dO,LSE + gqa_bwd + D2H of dQ,dK,dV
"""
from __future__ import annotations

import argparse
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
METRIC = "GQA bwd TFLOP/s (B8 Hq12 Hkv4 S4096 D64 bf16)"
NOMINAL_BF16_TFLOPS = 2250.0
# dram__bytes_read.sum + dram__bytes_write.sum of the backward main kernel from one ncu capture at B=4
# (B4 Hq12 Hkv4 S4096 D64: 123.8 MB read + 30.3 MB written = 154 MB), scaled by 2 to the headline batch: the
# (batch, KV-head) groups are independent, so traffic grows in proportion to B.
MAIN_KERNEL_DRAM_BYTES_PER_LAUNCH = 2 * 154.2e6


def bwd_flops(B, Hq, S, D, causal):
    f = 4.0 * B * Hq * S * S * D
    return 4.0 * (f * 0.5 if causal else f)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"bf16_tflops": float(p["bf16_tflops"]), "bf16_tflops_sustained": float(p["bf16_tflops_sustained"]),
                "hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # the busy samples are the ones that matter: keep the upper half (idle samples sit at low clocks)
        busy = sorted(sm)[len(sm) // 2:] if sm else []
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_sdpa_backward_sample(steps: int, warmup: int, sample_b: int, shape):
    """The reference's oracle path on the host: fp32 SDPA + autograd (precision/baseline_gqa.py:64-66,
    :429-435; harness/run_gqa_bwd_v44_bench.py:108-118) on `sample_b` of the B batches.  Returns the
    median backward seconds, the thread count and the sample description."""
    import torch.nn.functional as F

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    Hq, Hkv, S, D, causal = shape["Hq"], shape["Hkv"], shape["S"], shape["D"], shape["causal"]
    g = torch.Generator().manual_seed(42)
    mk = lambda h: torch.randn(sample_b, h, S, D, generator=g).bfloat16().float()
    q, k, v = mk(Hq).requires_grad_(True), mk(Hkv).requires_grad_(True), mk(Hkv).requires_grad_(True)
    do = torch.randn(sample_b, Hq, S, D, generator=torch.Generator().manual_seed(43)).bfloat16().float()
    times = []
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
    return statistics.median(times), threads, sample


def run_reference_arm(args, rank):
    if rank != 0:
        return
    shape = HEADLINE
    sample_b = 2
    sec, threads, sample = cpu_sdpa_backward_sample(max(1, args.steps), max(1, args.warmup), sample_b, shape)
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
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
    from hopper_jeni_b200 import ops

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)

    B, Hq, Hkv, S, D, causal = (HEADLINE[k] for k in ("B", "Hq", "Hkv", "S", "D", "causal"))
    scale = 1.0 / math.sqrt(D)
    gen = torch.Generator(device=dev).manual_seed(42 + rank)
    q = torch.randn(B, Hq, S, D, generator=gen, device=dev).bfloat16()
    k = torch.randn(B, Hkv, S, D, generator=gen, device=dev).bfloat16()
    v = torch.randn(B, Hkv, S, D, generator=gen, device=dev).bfloat16()
    do = torch.randn(B, Hq, S, D, generator=gen, device=dev).bfloat16()
    o, lse = gqa.gqa_forward(q, k, v, causal=causal, scale=scale)
    ws = torch.empty(gqa.bwd_workspace_bytes(B, Hq, Hkv, S, D, causal), dtype=torch.uint8, device=dev)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def step():
        gqa.gqa_backward(q, k, v, o, do, lse, causal=causal, scale=scale, workspace=ws, dq=dq, dk=dk, dv=dv)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # the clock sampler starts before the warm-up so that nvidia-smi is already reporting when the timed
    # region begins; idle samples are dropped when it is read out
    sampler = ClockSampler(local_rank) if rank == 0 else None
    for _ in range(args.warmup):
        step()
    barrier()
    ops.check_status(ws)

    # ---- timed region: K steps, device-timed per step, L2 flushed before each ----
    launches0 = gqa.launch_count()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier()
    for i in range(args.steps):
        flush.zero_()
        starts[i].record()
        step()
        stops[i].record()
    barrier()
    launches = gqa.launch_count() - launches0
    clocks = sampler.stop() if sampler else None
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
    barrier()
    e2e_ok = bool(torch.equal(host_out[1], dk.cpu()) and torch.equal(host_out[2], dv.cpu()))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_ms = float(e2e_ms.item())

    # ---- verification gather (NCCL, outside every timed region) ----
    sums = torch.stack([dq.float().abs().sum(), dk.float().abs().sum(), dv.float().abs().sum(),
                        torch.isfinite(dq.float()).all().float() * torch.isfinite(dk.float()).all().float()
                        * torch.isfinite(dv.float()).all().float()]).double()
    if dist is not None:
        gathered = [torch.empty_like(sums) for _ in range(world)]
        dist.all_gather(gathered, sums)
    else:
        gathered = [sums]
    all_finite = all(bool(g[3].item() == 1.0) and float(g[0].item()) > 0 for g in gathered)

    if rank == 0:
        flops_rank = bwd_flops(B, Hq, S, D, causal)
        ms_per_step = total_ms / args.steps
        value = world * flops_rank / (ms_per_step * 1e-3) / 1e12
        peaks = load_peaks()
        achieved = flops_rank / (main_ms * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {
                "workload": "GQA non-causal backward (whole gqa_bwd call: Delta preprocess + main + dQ finalise), "
                            "B8 Hq12 Hkv4 S4096 D64 bf16 per GPU, N(0,1) inputs",
                "parallelism": f"(batch x KV-head) groups sharded over {world} GPU(s), no data-path collective",
                "global_batch": B * world, "flop_convention": "backward = 4 x forward = 16*B*Hq*S^2*D",
                "l2": "256 MB memset before every timed step; inputs 270 MB > 126 MB L2",
                "frac_of_nominal_2250": value / world / NOMINAL_BF16_TFLOPS,
                "stage_ms": {"preprocess": pre_ms, "main": main_ms, "dq_finalise": fin_ms},
                "dq_path": "TMA reduce-add (fp32, L2) into an accumulator: not bit-reproducible; dK/dV single-writer, bit-reproducible",
                "outputs_finite_all_ranks": all_finite,
            },
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["bf16_tflops"], "traffic": MAIN_KERNEL_DRAM_BYTES_PER_LAUNCH,
                         "kernel": "gqa_bwd_sm100_kernel<64>", "peak_source": peaks["source"] + " burst",
                         "flop_convention": "achieved counts the reference's 16*B*Hq*S^2*D; the five GEMMs execute "
                                            "10*B*Hq*S^2*D, reported below",
                         "achieved_executed_mma": achieved * 10.0 / 16.0,
                         "frac_executed_mma": achieved * 10.0 / 16.0 / peaks["bf16_tflops"],
                         "frac_of_sustained": achieved / peaks["bf16_tflops_sustained"]},
            "clocks": clocks,
            "e2e": {"value": world * flops_rank / (e2e_ms / e2e_steps * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "path": "pinned host -> 8 chunks of (batch,KV-head) groups on 3 streams -> gqa_bwd -> pinned host",
                    "matches_device_resident_run": e2e_ok},
            "gpu_launches": int(launches),
        }
        if not args.no_cpu_baseline:
            sec, threads, sample = cpu_sdpa_backward_sample(3, 1, 2, HEADLINE)
            line["cpu_baseline"] = {"value": bwd_flops(2, Hq, S, D, causal) / sec / 1e12, "unit": "TFLOP/s",
                                    "cores": threads, "kind": "reference", "sample": sample}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
