"""GPU tests of GQA_BWD_SPLIT_HEADS: with few KV tiles in a call the backward may cut every tile's work over several
thread blocks by query head, keep fp32 partial dK / dV sums in the workspace and add them in a fixed order -- the
reference's per-head grid + gqa_dkdv_greduce (src/attention/GQA_bwd_baseline.cu:385-403, :594-599) on fp32 partials.
Results must match the oracle, stay bit-reproducible from run to run, and agree with the unsplit backward up to
the last bf16 bit."""
import pytest
import torch

import util
from hopper_jeni_b200 import capi, ops

pytestmark = pytest.mark.gpu

CASES = [
    # B, Hq, Hkv, S, D, causal        (all far below two KV tiles per SM)
    (1, 8, 1, 1024, 64, True),       # MQA, G = 8: the rule may split in 2, 4 or 8
    (1, 6, 2, 384, 64, False),       # G = 3: split in 3 or not at all
    (2, 8, 2, 512, 128, True),       # D = 128
    (1, 4, 2, 200, 96, True),        # padded head dimension, partial tile
]


@pytest.mark.parametrize("case", CASES)
def test_split_heads_matches_oracle_and_unsplit(gqa_lib, oracle, case):
    B, Hq, Hkv, S, D, causal = case
    q, k, v, do = util.make_inputs(B, Hq, Hkv, S, D, seed=17)
    sc = util.default_scale(D)
    tq, tk, tv, tdo = (util.to_dev_bf16(x) for x in (q, k, v, do))
    o_ref, lse_ref = oracle.forward(q, k, v, causal, sc)
    to = util.to_dev_bf16(util.bf16_round(o_ref))
    tlse = torch.from_numpy(lse_ref).cuda()
    need = ops.bwd_workspace_bytes(B, Hq, Hkv, S, D, causal, split_heads=True)
    assert need >= ops.bwd_workspace_bytes(B, Hq, Hkv, S, D, causal)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    runs = []
    for _ in range(3):
        dq, dk, dv = (torch.full_like(t, float("nan")) for t in (tq, tk, tv))
        ops.gqa_backward(tq, tk, tv, to, tdo, tlse, causal=causal, scale=sc, workspace=ws, dq=dq, dk=dk, dv=dv,
                         split_heads=True)
        ops.check_status(ws)
        runs.append((dq, dk, dv))
    dq_ref, dk_ref, dv_ref = oracle.backward(q, k, v, do, causal, sc)
    util.assert_close_bf16(util.to_np(runs[0][0]), dq_ref, "dQ", util.REL_RMS_BWD)
    util.assert_close_bf16(util.to_np(runs[0][1]), dk_ref, "dK", util.REL_RMS_BWD)
    util.assert_close_bf16(util.to_np(runs[0][2]), dv_ref, "dV", util.REL_RMS_BWD)
    for dq, dk, dv in runs[1:]:   # fixed-order sum: bit-reproducible
        assert torch.equal(dk, runs[0][1]) and torch.equal(dv, runs[0][2])
    # the unsplit backward gives the same dK / dV up to the last bf16 bit
    dq1, dk1, dv1 = ops.gqa_backward(tq, tk, tv, to, tdo, tlse, causal=causal, scale=sc)
    assert util.metrics(util.to_np(runs[0][1]), util.to_np(dk1))["rel_rms"] < 2e-3
    assert util.metrics(util.to_np(runs[0][2]), util.to_np(dv1))["rel_rms"] < 2e-3


def test_split_needs_the_matching_workspace(gqa_lib):
    B, Hq, Hkv, S, D = 1, 8, 1, 1024, 64
    small = ops.bwd_workspace_bytes(B, Hq, Hkv, S, D, True)
    big = ops.bwd_workspace_bytes(B, Hq, Hkv, S, D, True, split_heads=True)
    assert big > small          # this shape is split: the partial sums need room
    q = torch.zeros(B, Hq, S, D, dtype=torch.bfloat16, device="cuda")
    k = torch.zeros(B, Hkv, S, D, dtype=torch.bfloat16, device="cuda")
    lse = torch.zeros(B, Hq, S, dtype=torch.float32, device="cuda")
    ws = torch.empty(small, dtype=torch.uint8, device="cuda")
    with pytest.raises(capi.GqaError) as e:
        ops.gqa_backward(q, k, k, q, q, lse, causal=True, workspace=ws, split_heads=True)
    assert e.value.status == -3
