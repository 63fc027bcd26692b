"""Parity of gqa_fwd / gqa_bwd (through the C ABI) with PyTorch fp32 SDPA + autograd AT THE BENCHMARK CONFIG
SIZES, on the same seeded bf16-rounded inputs -- the gate the reference applies to its kernels at the full
benchmark shape before timing them (src/attention/GQA_bwd_baseline.cu:664-681, src/attention/GQA_fwd_v62.cu:95-110,
golden files from precision/baseline_gqa.py:394-449).  The kernels run once on the whole problem; the reference
is evaluated group by group (and, where a group's fp32 score block is too large, a few query heads at a time with
dK/dV accumulated over the group).

Tolerance (bf16): |got - ref| <= 2e-2 + 2e-2 |ref| element-wise, relative RMS <= 1e-2 (O) / 2e-2 (gradients),
LSE within 1e-3 relative + 2e-3 absolute.  Every case prints max-abs and relative-RMS per tensor.
"""
import math

import pytest
import torch

from oracle import sdpa_ref
import util
from hopper_jeni_b200 import ops

pytestmark = pytest.mark.gpu


def _inputs(B, Hq, Hkv, S, D, do_mul=1.0, seed=42):
    """Q, K, V ~ N(0,1) (seed), dO ~ N(0,1) * do_mul (seed + 1), rounded to bf16, on the device."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(B, Hq, S, D, generator=g, device="cuda").bfloat16()
    k = torch.randn(B, Hkv, S, D, generator=g, device="cuda").bfloat16()
    v = torch.randn(B, Hkv, S, D, generator=g, device="cuda").bfloat16()
    g2 = torch.Generator(device="cuda").manual_seed(seed + 1)
    do = (torch.randn(B, Hq, S, D, generator=g2, device="cuda") * do_mul).bfloat16()
    return q, k, v, do


def _check(name, got, ref, rel_rms, worst):
    m = sdpa_ref.metrics(got, ref)
    w = worst.setdefault(name, {"max_abs": 0.0, "rel_rms": 0.0})
    w["max_abs"], w["rel_rms"] = max(w["max_abs"], m["max_abs"]), max(w["rel_rms"], m["rel_rms"])
    assert m["finite"], f"{name}: non-finite values"
    assert m["gate_ok"], f"{name}: |d| <= 2e-2 + 2e-2|ref| violated: {m}"
    assert m["rel_rms"] <= rel_rms, f"{name}: relative RMS {m['rel_rms']:.3e} > {rel_rms}"


def _parity(B, Hq, Hkv, S, D, causal, do_mul=1.0, groups=None, backward=True, deterministic=False):
    """Runs forward (+ backward) on the whole problem, compares the listed (batch, KV-head) groups (all when None)."""
    G = Hq // Hkv
    sc = 1.0 / math.sqrt(D)
    q, k, v, do = _inputs(B, Hq, Hkv, S, D, do_mul)
    o, lse = ops.gqa_forward(q, k, v, causal=causal, scale=sc)
    ops.check_status()
    if backward:
        ws = torch.empty(ops.bwd_workspace_bytes(B, Hq, Hkv, S, D, causal), dtype=torch.uint8, device="cuda")
        dq, dk, dv = ops.gqa_backward(q, k, v, o, do, lse, causal=causal, scale=sc, workspace=ws,
                                      deterministic=deterministic)
        ops.check_status(ws)
    worst = {}
    for b, h in (groups if groups is not None else [(b, h) for b in range(B) for h in range(Hkv)]):
        hs = slice(h * G, (h + 1) * G)
        o_r, lse_r, dq_r, dk_r, dv_r = sdpa_ref.sdpa_group(q[b, hs], k[b, h], v[b, h], do[b, hs] if backward else None,
                                                           sc, causal)
        _check("O", o[b, hs], o_r, util.REL_RMS_FWD, worst)
        torch.testing.assert_close(lse[b, hs], lse_r, rtol=1e-3, atol=2e-3)
        if backward:
            _check("dQ", dq[b, hs], dq_r, util.REL_RMS_BWD, worst)
            _check("dK", dk[b, h], dk_r, util.REL_RMS_BWD, worst)
            _check("dV", dv[b, h], dv_r, util.REL_RMS_BWD, worst)
    print(f"\nparity B{B} Hq{Hq} Hkv{Hkv} S{S} D{D} causal={int(causal)}: "
          + ", ".join(f"{n} max_abs {w['max_abs']:.3e} rel_rms {w['rel_rms']:.3e}" for n, w in worst.items()))
    return worst


def test_headline_config_all_groups(gqa_lib):
    """B8 Hq12 Hkv4 S4096 D64 non-causal, forward + backward, every one of the 32 groups."""
    _parity(8, 12, 4, 4096, 64, causal=False)


def test_headline_config_deterministic_mode(gqa_lib):
    """Same shape through GQA_BWD_DETERMINISTIC (ordered dQ reductions), a quarter of the groups."""
    _parity(8, 12, 4, 4096, 64, causal=False, deterministic=True, groups=[(b, b % 4) for b in range(8)])


def test_causal_d128_config_all_groups(gqa_lib):
    """B4 Hq32 Hkv8 S8192 D128 causal, dO ~ 0.1 N(0,1), forward + backward, every one of the 32 groups."""
    _parity(4, 32, 8, 8192, 128, causal=True, do_mul=0.1)


def test_long_context_config_all_kv_heads(gqa_lib):
    """B1 Hq64 Hkv8 S32768 D128 causal, forward + backward, all eight KV-head groups (two query heads at a
    time on the reference side, dK/dV accumulated over the group)."""
    _parity(1, 64, 8, 32768, 128, causal=True)


@pytest.mark.parametrize("S,D,causal", [(4096, 64, False), (4096, 128, True), (16384, 64, True), (16384, 128, False),
                                        (1024, 128, False), (2048, 64, True)])
def test_forward_sweep_points(gqa_lib, S, D, causal):
    """Forward sweep B16 Hq16 Hkv2: the kernel runs the whole problem, O and LSE are compared on four groups."""
    _parity(16, 16, 2, S, D, causal=causal, backward=False, groups=[(0, 0), (5, 1), (10, 0), (15, 1)])


# The reference's own sweep: B in {2,4,8} x (Hq,Hkv) in {(12,4),(16,4),(24,8),(32,8)}, S = 4096, D = 128, causal
# (scripts/run_sweep.sh:17-18), inputs from its generator's distribution Q, K, V ~ U[0,1), dO ~ N(0,1)
# (precision/baseline_gqa.py:400-402, :422-423).
SWEEP = [(B, Hq, Hkv) for B in (2, 4, 8) for Hq, Hkv in ((12, 4), (16, 4), (24, 8), (32, 8))]


@pytest.mark.parametrize("B,Hq,Hkv", SWEEP)
def test_reference_sweep_uniform_inputs(gqa_lib, B, Hq, Hkv):
    """Two comparisons per tensor.  (1) Against fp32 SDPA autograd: the reference's own element-wise gate
    |d| <= 2e-2 + 2e-2|ref| (src/attention/GQA_bwd_baseline.cu:677-679) must hold; the relative RMS of dQ is
    reported, not bounded, because with these inputs it measures the INPUT contract, not the kernel: dP is
    Delta plus a fluctuation about half its size, the backward receives O rounded to bf16, and that rounding
    alone shifts Delta coherently along a row and moves dQ by about 10 % at S = 4096 in exact arithmetic
    (2.7 % at S = 128; tests/test_sdpa_ref.py pins the restatement used to show it).  (2) Against the same fp32
    backward handed the same bf16 O (the operator's contract): relative RMS <= 2e-2 for all three gradients."""
    S, D, G = 4096, 128, Hq // Hkv
    sc = 1.0 / math.sqrt(D)
    g = torch.Generator(device="cuda").manual_seed(42)
    q = torch.rand(B, Hq, S, D, generator=g, device="cuda").bfloat16()
    k = torch.rand(B, Hkv, S, D, generator=g, device="cuda").bfloat16()
    v = torch.rand(B, Hkv, S, D, generator=g, device="cuda").bfloat16()
    do = torch.randn(B, Hq, S, D, generator=torch.Generator(device="cuda").manual_seed(43), device="cuda").bfloat16()
    o, lse = ops.gqa_forward(q, k, v, causal=True, scale=sc)
    ops.check_status()
    ws = torch.empty(ops.bwd_workspace_bytes(B, Hq, Hkv, S, D, True), dtype=torch.uint8, device="cuda")
    dq, dk, dv = ops.gqa_backward(q, k, v, o, do, lse, causal=True, scale=sc, workspace=ws)
    ops.check_status(ws)
    vs_sdpa, vs_same_o = {}, {}
    for b in range(B):
        for h in range(Hkv):
            hs = slice(h * G, (h + 1) * G)
            o_r, _, dq_r, dk_r, dv_r = sdpa_ref.sdpa_group(q[b, hs], k[b, h], v[b, h], do[b, hs], sc, True, want_lse=False)
            _check("O", o[b, hs], o_r, util.REL_RMS_FWD, vs_sdpa)
            _check("dQ", dq[b, hs], dq_r, 1.0, vs_sdpa)          # element-wise gate only, see above
            _check("dK", dk[b, h], dk_r, util.REL_RMS_BWD, vs_sdpa)
            _check("dV", dv[b, h], dv_r, util.REL_RMS_BWD, vs_sdpa)
            dq_o, dk_o, dv_o = sdpa_ref.backward_given_o(q[b, hs], k[b, h], v[b, h], o[b, hs], do[b, hs], sc, True)
            _check("dQ", dq[b, hs], dq_o, util.REL_RMS_BWD, vs_same_o)
            _check("dK", dk[b, h], dk_o, util.REL_RMS_BWD, vs_same_o)
            _check("dV", dv[b, h], dv_o, util.REL_RMS_BWD, vs_same_o)
    fmt = lambda d: ", ".join(f"{n} max_abs {w['max_abs']:.3e} rel_rms {w['rel_rms']:.3e}" for n, w in d.items())
    print(f"\nuniform sweep B{B} Hq{Hq} Hkv{Hkv}: vs fp32 SDPA: {fmt(vs_sdpa)} | vs fp32 backward given the same bf16 O: "
          f"{fmt(vs_same_o)}")
