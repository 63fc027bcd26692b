"""GPU parity tests for head dimensions other than the two native ones.  The reference's tensor-core kernels
fix D = 128; its first two generations are generic in D % 16 == 0 (src/attention/GQA_bwd.cu:391-393).  Here any
multiple of 8 up to 128 runs on the kernel of the next native size (64 or 128): the tensor maps describe the real
columns, the boxes read zeros beyond them, and the epilogues store only the real columns.  Output buffers are
poisoned first so that a store beyond a row's real columns would show up in its neighbour."""
import numpy as np
import pytest
import torch

import util
from hopper_jeni_b200 import capi, ops

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("D", [8, 32, 48, 80, 96, 120])
def test_forward_backward_match_oracle(gqa_lib, oracle, D, causal):
    B, Hq, Hkv, S = 1, 4, 2, 200          # a partial last tile as well
    q, k, v, do = util.make_inputs(B, Hq, Hkv, S, D, seed=90 + D)
    sc = util.default_scale(D)
    tq, tk, tv, tdo = (util.to_dev_bf16(x) for x in (q, k, v, do))
    o = torch.full_like(tq, float("nan"))
    lse = torch.full((B, Hq, S), float("nan"), dtype=torch.float32, device="cuda")
    ops.gqa_forward(tq, tk, tv, causal=causal, scale=sc, out=o, lse=lse)
    ops.check_status()
    o_ref, lse_ref = oracle.forward(q, k, v, causal, sc)
    util.assert_close_bf16(util.to_np(o), o_ref, "O", util.REL_RMS_FWD)
    np.testing.assert_allclose(util.to_np(lse), lse_ref, rtol=1e-3, atol=2e-3)
    # backward from the oracle's forward, as the other backward tests do
    to = util.to_dev_bf16(util.bf16_round(o_ref))
    tlse = torch.from_numpy(lse_ref).cuda()
    dq, dk, dv = (torch.full_like(t, float("nan")) for t in (tq, tk, tv))
    ws = torch.empty(ops.bwd_workspace_bytes(B, Hq, Hkv, S, D, causal), dtype=torch.uint8, device="cuda")
    ops.gqa_backward(tq, tk, tv, to, tdo, tlse, causal=causal, scale=sc, workspace=ws, dq=dq, dk=dk, dv=dv)
    ops.check_status(ws)
    dq_ref, dk_ref, dv_ref = oracle.backward(q, k, v, do, causal, sc)
    util.assert_close_bf16(util.to_np(dq), dq_ref, "dQ", util.REL_RMS_BWD)
    util.assert_close_bf16(util.to_np(dk), dk_ref, "dK", util.REL_RMS_BWD)
    util.assert_close_bf16(util.to_np(dv), dv_ref, "dV", util.REL_RMS_BWD)
    # Delta on its own
    delta = ops.gqa_delta(to, tdo)
    np.testing.assert_allclose(util.to_np(delta), (util.bf16_round(o_ref) * do).sum(-1), rtol=1e-4, atol=1e-4)


def test_sequence_major_layout_needs_a_native_head_dimension(gqa_lib):
    q = torch.zeros(1, 128, 2, 96, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(capi.GqaError) as e:
        ops.gqa_forward(q, q, q, layout="bshd")
    assert e.value.status == -2
