"""Generate the golden fixtures in this folder from the reference project's own Python code.

Run once in a container that has the reference checkout (read-only) and torch on CPU:

    python tests/golden/make_golden.py <path-to-reference-checkout>

It imports, unmodified, the reference's
  * ``fp64_reference`` / ``fp64_backward``   (precision/baseline_gqa.py:40-61, :169-197; causal only)
  * ``reference_output``                      (harness/bench_core.py:143-172; fp32 SDPA and fp64 loop)
  * ``reference_backward``                    (harness/run_gqa_bwd_v44_bench.py:108-118; fp32 SDPA autograd)
runs them on seeded CPU tensors and stores inputs (bf16 bit patterns, uint16) and outputs
(float32) as ``<case>.npz``.  The reference checkout is not available where the GPU tests
run, hence the committed files.  Seeds follow the reference (42 for q,k,v; 43 for dO,
precision/baseline_gqa.py:396, :422); the distributions are named per case.
"""
from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = {
    # name: (B, Hq, Hkv, S, D, causal, distribution of q/k/v, dO multiplier)
    "causal_uniform_b1_hq4_hkv2_s128_d64": (1, 4, 2, 128, 64, True, "uniform", 1.0),
    "noncausal_normal_b1_hq6_hkv2_s128_d64": (1, 6, 2, 128, 64, False, "normal", 1.0),
    "causal_normal_b1_hq2_hkv1_s256_d128": (1, 2, 1, 256, 128, True, "normal", 0.1),
}


def _load(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def _bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.int16).numpy().view(np.uint16).copy()


def main(ref_root: str) -> None:
    sys.argv = [sys.argv[0]]
    bg = _load("ref_baseline_gqa", os.path.join(ref_root, "precision", "baseline_gqa.py"))
    sys.path.insert(0, os.path.join(ref_root, "harness"))
    bc = _load("bench_core", os.path.join(ref_root, "harness", "bench_core.py"))
    bw = _load("ref_bwd_bench", os.path.join(ref_root, "harness", "run_gqa_bwd_v44_bench.py"))
    torch.set_num_threads(max(1, os.cpu_count() or 1))

    for name, (B, Hq, Hkv, S, D, causal, dist, do_mul) in CASES.items():
        gen = torch.Generator().manual_seed(42)
        draw = torch.rand if dist == "uniform" else torch.randn
        q = draw(B, Hq, S, D, generator=gen, dtype=torch.float32).bfloat16()
        k = draw(B, Hkv, S, D, generator=gen, dtype=torch.float32).bfloat16()
        v = draw(B, Hkv, S, D, generator=gen, dtype=torch.float32).bfloat16()
        gen = torch.Generator().manual_seed(43)
        do = (torch.randn(B, Hq, S, D, generator=gen, dtype=torch.float32) * do_mul).bfloat16()
        scale = 1.0 / (D ** 0.5)
        out = {"q": _bf16_bits(q), "k": _bf16_bits(k), "v": _bf16_bits(v), "do": _bf16_bits(do),
               "shape": np.array([B, Hq, Hkv, S, D, int(causal)], dtype=np.int32),
               "scale": np.array([scale], dtype=np.float64)}

        shape = bc.Shape(B, Hq, Hkv, S, D, causal=causal)
        out["o_fp32_sdpa"] = bc.reference_output(q, k, v, shape, mode="fp32").numpy()
        out["o_fp64"] = bc.reference_output(q, k, v, shape, mode="fp64").numpy()
        bshape = bw.Shape(B, Hq, Hkv, S, D, causal=causal)
        dq, dk, dv = bw.reference_backward(q, k, v, do, bshape)
        out["dq_fp32_sdpa"], out["dk_fp32_sdpa"], out["dv_fp32_sdpa"] = dq.numpy(), dk.numpy(), dv.numpy()

        if causal:
            # the reference's fp64 functions are causal-only and read the shape from module globals
            bg.B, bg.Hq, bg.Hkv, bg.S, bg.D, bg.G = B, Hq, Hkv, S, D, Hq // Hkv
            o64, lse64 = bg.fp64_reference(q, k, v, scale)
            dq64, dk64, dv64 = bg.fp64_backward(q, k, v, do, scale)
            out["o_fp64_baseline"] = o64.numpy()
            out["lse_fp64"] = lse64.numpy()
            out["dq_fp64"], out["dk_fp64"], out["dv_fp64"] = dq64.numpy(), dk64.numpy(), dv64.numpy()
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **out)
        print(name, {k_: v_.shape for k_, v_ in out.items()}, os.path.getsize(path))


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path-to-reference-checkout>")
    main(sys.argv[1])
