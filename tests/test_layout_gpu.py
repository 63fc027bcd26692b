"""GPU tests of the sequence-major layout (GQA_LAYOUT_BSHD): the same problem handed over as [B,S,H,D] tensors
must give the results of the canonical [B,H,S,D] call: O, LSE, dK, dV bit for bit (same arithmetic in the
same order), dQ up to the order of the fp32 reductions (bit for bit in the deterministic mode)."""
import pytest
import torch

import util
from hopper_jeni_b200 import ops

pytestmark = pytest.mark.gpu

SHAPES = [(2, 6, 2, 384, 64), (1, 8, 2, 512, 128), (2, 12, 4, 1024, 64)]


def _t(x):  # [B,H,S,D] -> contiguous [B,S,H,D]
    return x.transpose(1, 2).contiguous()


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_bshd_forward_and_backward_equal_bhsd(gqa_lib, shape, causal):
    B, Hq, Hkv, S, D = shape
    q, k, v, do = (util.to_dev_bf16(x) for x in util.make_inputs(B, Hq, Hkv, S, D, seed=81))
    o, lse = ops.gqa_forward(q, k, v, causal=causal)
    o2, lse2 = ops.gqa_forward(_t(q), _t(k), _t(v), causal=causal, layout="bshd")
    ops.check_status()
    assert o2.shape == (B, S, Hq, D)
    assert torch.equal(_t(o), o2) and torch.equal(lse, lse2)
    ws = torch.empty(ops.bwd_workspace_bytes(B, Hq, Hkv, S, D, causal), dtype=torch.uint8, device="cuda")
    dq, dk, dv = ops.gqa_backward(q, k, v, o, do, lse, causal=causal, workspace=ws, deterministic=True)
    ops.check_status(ws)
    dq2, dk2, dv2 = ops.gqa_backward(_t(q), _t(k), _t(v), o2, _t(do), lse2, causal=causal, workspace=ws,
                                     deterministic=True, layout="bshd")
    ops.check_status(ws)
    assert dq2.shape == (B, S, Hq, D) and dk2.shape == (B, S, Hkv, D)
    assert torch.equal(_t(dk), dk2) and torch.equal(_t(dv), dv2)
    assert torch.equal(_t(dq), dq2)
    # default mode: dK, dV again bit for bit between the layouts (against the ordered mode they may differ in the
    # order of the fp32 sums: without a mask the default mode starts its loops at other query tiles)
    _, dk0, dv0 = ops.gqa_backward(q, k, v, o, do, lse, causal=causal, workspace=ws)
    ops.check_status(ws)
    dq3, dk3, dv3 = ops.gqa_backward(_t(q), _t(k), _t(v), o2, _t(do), lse2, causal=causal, workspace=ws, layout="bshd")
    ops.check_status(ws)
    assert torch.equal(dk3, _t(dk0)) and torch.equal(dv3, _t(dv0))
    for got, want in ((dk3, dk2), (dv3, dv2)):
        m = util.metrics(util.to_np(got), util.to_np(want))
        assert m["rel_rms"] < 2e-3, m
    m = util.metrics(util.to_np(dq3), util.to_np(dq2))
    assert m["rel_rms"] < 2e-3, m


def test_bshd_backward_matches_oracle(gqa_lib, oracle):
    B, Hq, Hkv, S, D = 1, 4, 2, 256, 64
    qn, kn, vn, don = util.make_inputs(B, Hq, Hkv, S, D, seed=82)
    sc = util.default_scale(D)
    dq_ref, dk_ref, dv_ref = oracle.backward(qn, kn, vn, don, True, sc)
    q, k, v, do = (_t(util.to_dev_bf16(x)) for x in (qn, kn, vn, don))
    o, lse = ops.gqa_forward(q, k, v, causal=True, scale=sc, layout="bshd")
    dq, dk, dv = ops.gqa_backward(q, k, v, o, do, lse, causal=True, scale=sc, layout="bshd")
    util.assert_close_bf16(util.to_np(dq.transpose(1, 2).contiguous()), dq_ref, "dQ", util.REL_RMS_BWD)
    util.assert_close_bf16(util.to_np(dk.transpose(1, 2).contiguous()), dk_ref, "dK", util.REL_RMS_BWD)
    util.assert_close_bf16(util.to_np(dv.transpose(1, 2).contiguous()), dv_ref, "dV", util.REL_RMS_BWD)
