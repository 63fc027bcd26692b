"""GPU tests of the alternative dQ path (GQA_BWD_DQ_SEPARATE): dQ from a separate query-parallel pass, the layout of
the reference's first generations (a dQ kernel per query tile beside a dK/dV kernel per key tile,
src/attention/GQA_bwd.cu:29, :415, :1416), instead of fp32 reductions into an accumulator
(src/attention/GQA_bwd_baseline.cu:360-365).  All three gradients must match the oracle, dQ must be bit-identical
from run to run (its summation order is fixed), and dK / dV must be the bits the default path produces (the main
kernel computes them the same way with or without its dQ part)."""
import pytest
import torch

import util
from hopper_jeni_b200 import ops

pytestmark = pytest.mark.gpu

CASES = [
    # B, Hq, Hkv, S, D, causal
    (1, 2, 1, 128, 64, False),      # one tile
    (2, 6, 2, 512, 64, True),       # G = 3, diagonal blocks
    (1, 4, 4, 640, 64, False),      # MHA; five key blocks wrap the four-stage ring
    (1, 4, 2, 384, 128, True),      # D = 128 (two-stage ring)
    (1, 8, 1, 200, 96, True),       # padded head dimension, partial tile, MQA
    (1, 4, 2, 450, 64, False),      # ragged
]


@pytest.mark.parametrize("case", CASES)
def test_separate_dq_matches_oracle_and_is_bit_reproducible(gqa_lib, oracle, case):
    B, Hq, Hkv, S, D, causal = case
    q, k, v, do = util.make_inputs(B, Hq, Hkv, S, D, seed=23)
    sc = util.default_scale(D)
    tq, tk, tv, tdo = (util.to_dev_bf16(x) for x in (q, k, v, do))
    o_ref, lse_ref = oracle.forward(q, k, v, causal, sc)
    to = util.to_dev_bf16(util.bf16_round(o_ref))
    tlse = torch.from_numpy(lse_ref).cuda()
    ws = torch.empty(ops.bwd_workspace_bytes(B, Hq, Hkv, S, D, causal), dtype=torch.uint8, device="cuda")
    runs = []
    for _ in range(3):
        dq, dk, dv = (torch.full_like(t, float("nan")) for t in (tq, tk, tv))
        ops.gqa_backward(tq, tk, tv, to, tdo, tlse, causal=causal, scale=sc, workspace=ws, dq=dq, dk=dk, dv=dv,
                         dq_separate=True)
        ops.check_status(ws)
        runs.append((dq, dk, dv))
    dq_ref, dk_ref, dv_ref = oracle.backward(q, k, v, do, causal, sc)
    util.assert_close_bf16(util.to_np(runs[0][0]), dq_ref, "dQ", util.REL_RMS_BWD)
    util.assert_close_bf16(util.to_np(runs[0][1]), dk_ref, "dK", util.REL_RMS_BWD)
    util.assert_close_bf16(util.to_np(runs[0][2]), dv_ref, "dV", util.REL_RMS_BWD)
    for dq, dk, dv in runs[1:]:
        assert torch.equal(dq, runs[0][0]) and torch.equal(dk, runs[0][1]) and torch.equal(dv, runs[0][2])
    dq0, dk0, dv0 = ops.gqa_backward(tq, tk, tv, to, tdo, tlse, causal=causal, scale=sc, workspace=ws)
    assert torch.equal(dk0, runs[0][1]) and torch.equal(dv0, runs[0][2])
    assert util.metrics(util.to_np(runs[0][0]), util.to_np(dq0))["rel_rms"] < 5e-3


def test_separate_dq_at_the_headline_shape(gqa_lib):
    """B8 Hq12 Hkv4 S4096 D64: the two dQ paths agree (relative RMS; both are rounded to bf16 once)."""
    B, Hq, Hkv, S, D = 8, 12, 4, 4096, 64
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn(B, Hq, S, D, generator=g, device="cuda").bfloat16()
    k = torch.randn(B, Hkv, S, D, generator=g, device="cuda").bfloat16()
    v = torch.randn(B, Hkv, S, D, generator=g, device="cuda").bfloat16()
    do = torch.randn(B, Hq, S, D, generator=g, device="cuda").bfloat16()
    o, lse = ops.gqa_forward(q, k, v)
    ws = torch.empty(ops.bwd_workspace_bytes(B, Hq, Hkv, S, D), dtype=torch.uint8, device="cuda")
    dq_a, dk_a, dv_a = ops.gqa_backward(q, k, v, o, do, lse, workspace=ws)
    dq_b, dk_b, dv_b = ops.gqa_backward(q, k, v, o, do, lse, workspace=ws, dq_separate=True)
    ops.check_status(ws)
    assert torch.equal(dk_a, dk_b) and torch.equal(dv_a, dv_b)
    m = util.metrics(util.to_np(dq_b[:2]), util.to_np(dq_a[:2]))
    assert m["rel_rms"] < 3e-3 and m["gate_ok"], m
