#!/usr/bin/env python
"""Golden-file generator for the C++ harness (``hopper_jeni_b200/gqa_bench``).

TEST INFRASTRUCTURE.  Counterpart of ``save_reference`` in the reference
(precision/baseline_gqa.py:394-449): same file set and format (raw little-endian fp32 via
``numpy.tofile``; inputs are bf16-rounded values widened to fp32 so that the kernel and the reference
start from identical bits), same seeds (42 for q,k,v; 43 for dO), but

  * S, D and causal are arguments (the reference hard-codes S=4096, D=128, causal),
  * inputs are N(0,1) as the benchmark configs ask (``--uniform`` gives the reference's U[0,1)),
  * the targets are **fp32** SDPA + autograd on the bf16-rounded inputs
    (harness/bench_core.py:143-156, harness/run_gqa_bwd_v44_bench.py:108-118), computed on the CPU
    unless ``--device cuda`` is given.

    python oracle/make_ref.py B Hq Hkv [S=4096] [D=64] [causal=0] [--out data] [--do-mul 1.0]

writes gqa_{q,k,v,o,lse,do,dq,dk,dv}.bin.  LSE is computed head by head in fp32 as the reference's
``sdpa_lse`` does (precision/baseline_gqa.py:69-86).
"""
from __future__ import annotations

import argparse
import math
import os

import torch
import torch.nn.functional as F


def lse_by_head(q, k, scale, causal):
    B, Hq, S, _ = q.shape
    G = Hq // k.shape[1]
    lse = torch.empty(B, Hq, S, dtype=torch.float32, device=q.device)
    mask = torch.ones(S, S, dtype=torch.bool, device=q.device).tril() if causal else None
    for b in range(B):
        for hq in range(Hq):
            s = (q[b, hq] @ k[b, hq // G].t()) * scale
            if mask is not None:
                s = s.masked_fill(~mask, float("-inf"))
            lse[b, hq] = torch.logsumexp(s, dim=-1)
    return lse


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("dims", type=int, nargs="+", help="B Hq Hkv [S D causal]")
    ap.add_argument("--out", default="data")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--uniform", action="store_true")
    ap.add_argument("--do-mul", type=float, default=1.0)
    a = ap.parse_args()
    dims = a.dims + [4096, 64, 0][len(a.dims) - 3:] if len(a.dims) < 6 else a.dims
    B, Hq, Hkv, S, D, causal = dims[:6]
    causal = bool(causal)
    scale = 1.0 / math.sqrt(D)
    torch.set_num_threads(os.cpu_count() or 1)
    gen = torch.Generator().manual_seed(42)
    draw = torch.rand if a.uniform else torch.randn
    q = draw(B, Hq, S, D, generator=gen).bfloat16().float()
    k = draw(B, Hkv, S, D, generator=gen).bfloat16().float()
    v = draw(B, Hkv, S, D, generator=gen).bfloat16().float()
    do = (torch.randn(B, Hq, S, D, generator=torch.Generator().manual_seed(43)) * a.do_mul).bfloat16().float()
    dev = torch.device(a.device)
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    o = F.scaled_dot_product_attention(qd, kd, vd, scale=scale, is_causal=causal, enable_gqa=(Hq != Hkv))
    o.backward(do.to(dev))
    lse = lse_by_head(qd.detach(), kd.detach(), scale, causal)
    os.makedirs(a.out, exist_ok=True)
    for name, t in (("q", q), ("k", k), ("v", v), ("do", do), ("o", o.detach()), ("lse", lse),
                    ("dq", qd.grad), ("dk", kd.grad), ("dv", vd.grad)):
        t.detach().float().cpu().numpy().tofile(os.path.join(a.out, f"gqa_{name}.bin"))
    print(f"wrote 9 files to {a.out}/ for B={B} Hq={Hq} Hkv={Hkv} S={S} D={D} causal={int(causal)}")


if __name__ == "__main__":
    main()
