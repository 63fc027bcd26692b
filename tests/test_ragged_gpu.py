"""GPU tests of sequence lengths that are not a multiple of the 128-row tile: the partial last tile reads zeros
beyond S (tensor maps with S as their own dimension), the forward masks the missing keys, and rows beyond S are
never stored.  Parity against the CPU oracle, forward and backward, both layouts."""
import pytest
import torch

import util
from hopper_jeni_b200 import ops

pytestmark = pytest.mark.gpu

CASES = [
    # B, Hq, Hkv, S, D
    (1, 2, 1, 72, 64),       # less than one tile
    (2, 6, 2, 200, 64),      # one full + one partial tile, second half-block partly masked
    (1, 4, 2, 333, 64),      # three tiles, odd length
    (1, 4, 2, 264, 128),     # D = 128, eight keys in the last tile
    (1, 8, 2, 450, 128),
]


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", CASES)
def test_ragged_forward_backward_match_oracle(gqa_lib, oracle, shape, causal):
    B, Hq, Hkv, S, D = shape
    qn, kn, vn, don = util.make_inputs(B, Hq, Hkv, S, D, seed=91)
    sc = util.default_scale(D)
    o_ref, lse_ref = oracle.forward(qn, kn, vn, causal, sc)
    dq_ref, dk_ref, dv_ref = oracle.backward(qn, kn, vn, don, causal, sc)
    q, k, v, do = (util.to_dev_bf16(x) for x in (qn, kn, vn, don))
    # poison the outputs: every element must be written, nothing outside them may be
    o = torch.full_like(q, float("nan"))
    lse = torch.full((B, Hq, S), float("nan"), dtype=torch.float32, device="cuda")
    ops.gqa_forward(q, k, v, causal=causal, scale=sc, out=o, lse=lse)
    ops.check_status()
    util.assert_close_bf16(util.to_np(o), o_ref, "O", util.REL_RMS_FWD)
    assert torch.allclose(lse.cpu(), torch.from_numpy(lse_ref), rtol=1e-3, atol=2e-3)
    ws = torch.empty(ops.bwd_workspace_bytes(B, Hq, Hkv, S, D, causal), dtype=torch.uint8, device="cuda")
    for det in (False, True):
        dq, dk, dv = (torch.full_like(t, float("nan")) for t in (q, k, v))
        ops.gqa_backward(q, k, v, o, do, lse, causal=causal, scale=sc, workspace=ws, dq=dq, dk=dk, dv=dv,
                         deterministic=det)
        ops.check_status(ws)
        util.assert_close_bf16(util.to_np(dq), dq_ref, "dQ", util.REL_RMS_BWD)
        util.assert_close_bf16(util.to_np(dk), dk_ref, "dK", util.REL_RMS_BWD)
        util.assert_close_bf16(util.to_np(dv), dv_ref, "dV", util.REL_RMS_BWD)


def test_ragged_bshd_equals_bhsd(gqa_lib):
    B, Hq, Hkv, S, D = 2, 6, 2, 300, 64
    q, k, v, do = (util.to_dev_bf16(x) for x in util.make_inputs(B, Hq, Hkv, S, D, seed=92))
    t = lambda x: x.transpose(1, 2).contiguous()
    o, lse = ops.gqa_forward(q, k, v, causal=True)
    o2, lse2 = ops.gqa_forward(t(q), t(k), t(v), causal=True, layout="bshd")
    assert torch.equal(t(o), o2) and torch.equal(lse, lse2)
    dq, dk, dv = ops.gqa_backward(q, k, v, o, do, lse, causal=True, deterministic=True)
    dq2, dk2, dv2 = ops.gqa_backward(t(q), t(k), t(v), o2, t(do), lse2, causal=True, deterministic=True, layout="bshd")
    assert torch.equal(t(dq), dq2) and torch.equal(t(dk), dk2) and torch.equal(t(dv), dv2)


def test_output_buffers_are_not_overrun(gqa_lib):
    """Outputs allocated inside a larger poisoned buffer: the bytes after them stay untouched."""
    B, Hq, Hkv, S, D = 1, 2, 1, 130, 64
    q, k, v, do = (util.to_dev_bf16(x) for x in util.make_inputs(B, Hq, Hkv, S, D, seed=93))
    nq, nkv = q.numel(), k.numel()
    pad = 128 * D
    big = torch.full((nq + pad + nq + pad + 2 * (nkv + pad),), 7.0, dtype=torch.bfloat16, device="cuda")
    o = big[:nq].view_as(q)
    dq = big[nq + pad:2 * nq + pad].view_as(q)
    dk = big[2 * nq + 2 * pad:2 * nq + 2 * pad + nkv].view_as(k)
    dv = big[2 * nq + 3 * pad + nkv:2 * nq + 3 * pad + 2 * nkv].view_as(k)
    lse_big = torch.full((B * Hq * S + 256,), 7.0, dtype=torch.float32, device="cuda")
    lse = lse_big[:B * Hq * S].view(B, Hq, S)
    ops.gqa_forward(q, k, v, out=o, lse=lse)
    ops.gqa_backward(q, k, v, o, do, lse, dq=dq, dk=dk, dv=dv)
    torch.cuda.synchronize()
    for a, b in ((nq, nq + pad), (2 * nq + pad, 2 * nq + 2 * pad), (2 * nq + 2 * pad + nkv, 2 * nq + 3 * pad + nkv)):
        assert (big[a:b] == 7.0).all()
    assert (big[2 * nq + 3 * pad + 2 * nkv:] == 7.0).all() and (lse_big[B * Hq * S:] == 7.0).all()
    assert torch.isfinite(big[:nq].float()).all() and torch.isfinite(lse).all()
