"""GPU parity tests of gqa_bwd (through the C ABI): CPU oracle and golden fixtures at small sizes,
the CUDA-core checker at medium sizes, and reference-free properties at the headline shape."""
import numpy as np
import pytest
import torch

import util
from hopper_jeni_b200 import capi, ops

pytestmark = pytest.mark.gpu

SMALL = [
    # B, Hq, Hkv, S, D
    (1, 2, 1, 128, 64),      # single tile, G = 2
    (2, 6, 2, 256, 64),      # G = 3
    (1, 4, 4, 384, 64),      # MHA
    (1, 8, 1, 256, 64),      # MQA, 16 iterations per CTA
    (1, 4, 2, 256, 128),     # D = 128 (dQ reuses the dP columns)
    (1, 2, 2, 512, 128),
]


def _run_bwd(q, k, v, do, causal, sc, fwd_from="oracle", oracle=None):
    tq, tk, tv, tdo = (util.to_dev_bf16(x) for x in (q, k, v, do))
    if fwd_from == "oracle":
        o_ref, lse_ref = oracle.forward(q, k, v, causal, sc)
        to = util.to_dev_bf16(util.bf16_round(o_ref))
        tlse = torch.from_numpy(lse_ref).cuda()
    else:
        to, tlse = ops.gqa_forward(tq, tk, tv, causal=causal, scale=sc)
    need = ops.bwd_workspace_bytes(*q.shape[:2], k.shape[1], q.shape[2], q.shape[3], causal)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    dq, dk, dv = ops.gqa_backward(tq, tk, tv, to, tdo, tlse, causal=causal, scale=sc, workspace=ws)
    ops.check_status(ws)
    return dq, dk, dv


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", SMALL)
def test_backward_matches_oracle(gqa_lib, oracle, shape, causal):
    B, Hq, Hkv, S, D = shape
    q, k, v, do = util.make_inputs(B, Hq, Hkv, S, D, seed=41)
    sc = util.default_scale(D)
    dq_ref, dk_ref, dv_ref = oracle.backward(q, k, v, do, causal, sc)
    dq, dk, dv = _run_bwd(q, k, v, do, causal, sc, oracle=oracle)
    util.assert_close_bf16(util.to_np(dq), dq_ref, "dQ", util.REL_RMS_BWD)
    util.assert_close_bf16(util.to_np(dk), dk_ref, "dK", util.REL_RMS_BWD)
    util.assert_close_bf16(util.to_np(dv), dv_ref, "dV", util.REL_RMS_BWD)


@pytest.mark.parametrize("name", util.GOLDEN_CASES)
def test_backward_matches_golden(gqa_lib, oracle, name):
    g = util.load_golden(name)
    dq, dk, dv = _run_bwd(g["q"], g["k"], g["v"], g["do"], g["causal"], g["scale"], oracle=oracle)
    # U[0,1) inputs (the reference generator's distribution): dP is Delta plus a fluctuation about half its size,
    # and the backward is handed O rounded to bf16, so Delta = rowsum(dO * O) carries a row-coherent error that
    # moves dQ by 2.7 % at this fixture in exact arithmetic (10 % at S = 4096; see test_config_parity_gpu.py).
    # Against fp32 SDPA the reference's element-wise gate holds and the relative-RMS bound is widened for that
    # fixture only; against the same fp32 backward given the same bf16 O the common bound holds (below).
    rel_rms = 6e-2 if "uniform" in name else util.REL_RMS_BWD
    for got, key in ((dq, "dq_fp32_sdpa"), (dk, "dk_fp32_sdpa"), (dv, "dv_fp32_sdpa")):
        util.assert_close_bf16(util.to_np(got), g[key], key, rel_rms)
    if g["causal"]:
        for got, key in ((dq, "dq_fp64"), (dk, "dk_fp64"), (dv, "dv_fp64")):
            util.assert_close_bf16(util.to_np(got), g[key], key, rel_rms)
    # same inputs, O as the operator received it (bf16): every gradient within the common relative-RMS bound
    from oracle import sdpa_ref

    G = g["Hq"] // g["Hkv"]
    o_ref, _ = oracle.forward(g["q"], g["k"], g["v"], g["causal"], g["scale"])
    o_in = torch.from_numpy(util.bf16_round(o_ref))
    tq, tk, tv, tdo = (torch.from_numpy(g[x]) for x in ("q", "k", "v", "do"))
    for b in range(g["B"]):
        for h in range(g["Hkv"]):
            hs = slice(h * G, (h + 1) * G)
            dq_o, dk_o, dv_o = sdpa_ref.backward_given_o(tq[b, hs], tk[b, h], tv[b, h], o_in[b, hs], tdo[b, hs],
                                                         g["scale"], g["causal"])
            util.assert_close_bf16(util.to_np(dq[b, hs]), dq_o.numpy(), "dQ given O", util.REL_RMS_BWD)
            util.assert_close_bf16(util.to_np(dk[b, h]), dk_o.numpy(), "dK given O", util.REL_RMS_BWD)
            util.assert_close_bf16(util.to_np(dv[b, h]), dv_o.numpy(), "dV given O", util.REL_RMS_BWD)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("D", [64, 128])
def test_backward_matches_checker_kernel_at_medium_size(gqa_lib, D, causal):
    B, Hq, Hkv, S = 1, 6, 2, 1024
    q, k, v, do = util.make_inputs(B, Hq, Hkv, S, D, seed=51)
    tq, tk, tv, tdo = (util.to_dev_bf16(x) for x in (q, k, v, do))
    o, lse = ops.checker_forward(tq, tk, tv, causal)
    ws = torch.empty(ops.bwd_workspace_bytes(B, Hq, Hkv, S, D, causal), dtype=torch.uint8, device="cuda")
    dq, dk, dv = ops.gqa_backward(tq, tk, tv, o, tdo, lse, causal=causal, workspace=ws)
    ops.check_status(ws)
    dq2, dk2, dv2 = ops.checker_backward(tq, tk, tv, o, tdo, lse, causal)
    util.assert_close_bf16(util.to_np(dq), util.to_np(dq2), "dQ", util.REL_RMS_BWD)
    util.assert_close_bf16(util.to_np(dk), util.to_np(dk2), "dK", util.REL_RMS_BWD)
    util.assert_close_bf16(util.to_np(dv), util.to_np(dv2), "dV", util.REL_RMS_BWD)


def test_backward_dkdv_bit_reproducible_dq_close(gqa_lib):
    """dK and dV have a single writer per element: bit-identical across runs.  dQ is reduced with
    fp32 atomics: equal up to the order of fp32 additions."""
    B, Hq, Hkv, S, D = 2, 6, 2, 1024, 64
    q, k, v, do = util.make_inputs(B, Hq, Hkv, S, D, seed=61)
    tq, tk, tv, tdo = (util.to_dev_bf16(x) for x in (q, k, v, do))
    o, lse = ops.gqa_forward(tq, tk, tv)
    ws = torch.empty(ops.bwd_workspace_bytes(B, Hq, Hkv, S, D), dtype=torch.uint8, device="cuda")
    runs = [ops.gqa_backward(tq, tk, tv, o, tdo, lse, workspace=ws) for _ in range(4)]
    torch.cuda.synchronize()
    for dq, dk, dv in runs[1:]:
        assert torch.equal(dk, runs[0][1]) and torch.equal(dv, runs[0][2])
        assert (dq.float() - runs[0][0].float()).abs().max().item() <= 2e-2


def test_backward_headline_shape_properties(gqa_lib):
    """Headline shape B8 Hq12 Hkv4 S4096 D64 non-causal, reference-free checks:
    (1) linearity in dO: bwd(2*dO) == 2*bwd(dO) up to bf16 rounding;
    (2) sum_s dV[b,hkv,s,:] == sum over the group's heads and rows of dO (columns of P sum over
        keys to one per query row);
    (3) dO = O-independent constant rows => Delta = dO.O and dS rows sum to zero => sum_j dS_ij = 0,
        checked through sum_s dK . 0 (skipped) -- instead check dQ, dK finite and non-trivial."""
    B, Hq, Hkv, S, D = 8, 12, 4, 4096, 64
    gen = torch.Generator(device="cuda").manual_seed(2)
    q = torch.randn(B, Hq, S, D, generator=gen, device="cuda").bfloat16()
    k = torch.randn(B, Hkv, S, D, generator=gen, device="cuda").bfloat16()
    v = torch.randn(B, Hkv, S, D, generator=gen, device="cuda").bfloat16()
    do = torch.randn(B, Hq, S, D, generator=gen, device="cuda").bfloat16()
    o, lse = ops.gqa_forward(q, k, v)
    ws = torch.empty(ops.bwd_workspace_bytes(B, Hq, Hkv, S, D), dtype=torch.uint8, device="cuda")
    dq, dk, dv = ops.gqa_backward(q, k, v, o, do, lse, workspace=ws)
    ops.check_status(ws)
    for t in (dq, dk, dv):
        assert torch.isfinite(t.float()).all() and t.float().abs().max().item() > 0
    dq2, dk2, dv2 = ops.gqa_backward(q, k, v, o, (do.float() * 2).bfloat16(), lse, workspace=ws)
    for a, b2 in ((dq, dq2), (dk, dk2), (dv, dv2)):
        m = util.metrics(util.to_np(b2), 2.0 * util.to_np(a))
        assert m["rel_rms"] < 1e-2, m
    col_sum = dv.float().sum(dim=2)                                   # [B, Hkv, D]
    want = do.float().view(B, Hkv, Hq // Hkv, S, D).sum(dim=(2, 3))    # [B, Hkv, D]
    assert (col_sum - want).abs().max().item() <= 2e-2 * want.abs().max().item() + 0.5


def test_backward_rejects_small_workspace(gqa_lib):
    q = torch.zeros(1, 2, 128, 64, dtype=torch.bfloat16, device="cuda")
    lse = torch.zeros(1, 2, 128, dtype=torch.float32, device="cuda")
    ws = torch.empty(1024, dtype=torch.uint8, device="cuda")
    with pytest.raises(capi.GqaError) as e:
        ops.gqa_backward(q, q, q, q, q, lse, workspace=ws)
    assert e.value.status == -3
