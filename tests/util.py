"""Shared helpers for the test-suite: seeded inputs, bf16 handling, error metrics and the tolerances."""
from __future__ import annotations

import math
import os

import numpy as np

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# bf16 tolerance of the parity gate, the one the reference's harness applies to its own kernels
# (src/attention/GQA_bwd_baseline.cu:677-679, harness/bench_core.py:175): |got - ref| <= ATOL + RTOL*|ref|,
# plus a relative-RMS bound ||got - ref|| / ||ref||.
ATOL = 2e-2
RTOL = 2e-2
REL_RMS_FWD = 1e-2
REL_RMS_BWD = 2e-2


def bf16_round(a: np.ndarray) -> np.ndarray:
    """Round float32 to the nearest bf16 (ties to even) and widen back to float32."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).reshape(a.shape)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def make_inputs(B, Hq, Hkv, S, D, seed=42, dist="normal", do_mul=1.0, bf16=True):
    """Seeded Q,K,V (seed) and dO (seed+1) as float32 holding bf16-representable values."""
    rng = np.random.default_rng(seed)
    draw = (lambda *s: rng.standard_normal(s, dtype=np.float32)) if dist == "normal" else \
           (lambda *s: rng.random(s, dtype=np.float32))
    q, k, v = draw(B, Hq, S, D), draw(B, Hkv, S, D), draw(B, Hkv, S, D)
    do = np.random.default_rng(seed + 1).standard_normal((B, Hq, S, D), dtype=np.float32) * np.float32(do_mul)
    if bf16:
        q, k, v, do = (bf16_round(x) for x in (q, k, v, do))
    return q, k, v, do


def metrics(got: np.ndarray, ref: np.ndarray) -> dict:
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    diff = np.abs(got - ref)
    denom = np.abs(ref)
    return {
        "max_abs": float(diff.max()),
        "mean_abs": float(diff.mean()),
        "max_rel": float(np.where(denom > 1e-5, diff / np.maximum(denom, 1e-30), diff).max()),
        "rel_rms": float(np.sqrt((diff ** 2).sum()) / max(np.sqrt((ref ** 2).sum()), 1e-30)),
        "gate_ok": bool((diff <= ATOL + RTOL * denom).all()),
    }


def assert_close_bf16(got, ref, name, rel_rms):
    m = metrics(got, ref)
    assert np.isfinite(np.asarray(got, dtype=np.float64)).all(), f"{name}: non-finite values"
    assert m["gate_ok"], f"{name}: |d| <= {ATOL} + {RTOL}|ref| violated: {m}"
    assert m["rel_rms"] <= rel_rms, f"{name}: relative RMS {m['rel_rms']:.3e} > {rel_rms}: {m}"
    return m


def default_scale(D):
    return 1.0 / math.sqrt(D)


def load_golden(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    B, Hq, Hkv, S, D, causal = (int(x) for x in z["shape"])
    out = {k: z[k] for k in z.files}
    for k in ("q", "k", "v", "do"):
        out[k] = bf16_bits_to_f32(z[k])
    out.update(B=B, Hq=Hq, Hkv=Hkv, S=S, D=D, causal=bool(causal), scale=float(z["scale"][0]))
    return out


GOLDEN_CASES = [
    "causal_uniform_b1_hq4_hkv2_s128_d64",
    "noncausal_normal_b1_hq6_hkv2_s128_d64",
    "causal_normal_b1_hq2_hkv1_s256_d128",
]


# ---- torch helpers (GPU tests) ----------------------------------------------------------------

def to_dev_bf16(a: np.ndarray):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a)).cuda().to(torch.bfloat16).contiguous()


def to_np(t):
    return t.detach().float().cpu().numpy()
