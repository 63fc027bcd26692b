"""GPU parity tests of gqa_fwd (through the C ABI) against the CPU oracle, the golden fixtures made
from the reference's own Python code, and -- at sizes the oracle cannot reach -- the CUDA-core checker
and size-independent properties."""
import numpy as np
import pytest
import torch

import util
from hopper_jeni_b200 import capi, ops

pytestmark = pytest.mark.gpu

SMALL = [
    # B, Hq, Hkv, S, D
    (1, 2, 1, 128, 64),      # one tile, second tile of the pair absent
    (1, 4, 2, 256, 64),      # one full tile pair
    (2, 6, 2, 512, 64),      # CPU plumbing config shape, G = 3
    (1, 4, 4, 384, 64),      # MHA (G = 1), odd tile count
    (1, 8, 1, 256, 128),     # MQA, D = 128
    (1, 4, 2, 640, 128),     # ring wrap-around with D = 128 (2 stages, 5 blocks)
]


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", SMALL)
def test_forward_matches_oracle(gqa_lib, oracle, shape, causal):
    B, Hq, Hkv, S, D = shape
    q, k, v, _ = util.make_inputs(B, Hq, Hkv, S, D, seed=21)
    sc = util.default_scale(D)
    o_ref, lse_ref = oracle.forward(q, k, v, causal, sc)
    o, lse = ops.gqa_forward(*(util.to_dev_bf16(x) for x in (q, k, v)), causal=causal, scale=sc)
    ops.check_status()
    util.assert_close_bf16(util.to_np(o), o_ref, "O", util.REL_RMS_FWD)
    np.testing.assert_allclose(util.to_np(lse), lse_ref, rtol=1e-3, atol=2e-3)


@pytest.mark.parametrize("name", util.GOLDEN_CASES)
def test_forward_matches_golden(gqa_lib, name):
    g = util.load_golden(name)
    o, lse = ops.gqa_forward(*(util.to_dev_bf16(g[x]) for x in "qkv"), causal=g["causal"], scale=g["scale"])
    ops.check_status()
    util.assert_close_bf16(util.to_np(o), g["o_fp32_sdpa"], "O vs fp32 SDPA", util.REL_RMS_FWD)
    util.assert_close_bf16(util.to_np(o), g["o_fp64"], "O vs fp64", util.REL_RMS_FWD)
    if g["causal"]:
        np.testing.assert_allclose(util.to_np(lse), g["lse_fp64"], rtol=1e-3, atol=2e-3)


def test_forward_large_logits_rescale_path(gqa_lib, oracle):
    """Logits that grow along the key axis force the running maximum to be refreshed (O rescale)."""
    B, Hq, Hkv, S, D = 1, 2, 1, 512, 64
    q, k, v, _ = util.make_inputs(B, Hq, Hkv, S, D, seed=5)
    ramp = np.linspace(0.2, 6.0, S, dtype=np.float32)[None, None, :, None]
    k = util.bf16_round(k * ramp)
    o_ref, lse_ref = oracle.forward(q, k, v, False, 0.5)
    o, lse = ops.gqa_forward(*(util.to_dev_bf16(x) for x in (q, k, v)), causal=False, scale=0.5)
    ops.check_status()
    util.assert_close_bf16(util.to_np(o), o_ref, "O", util.REL_RMS_FWD)
    np.testing.assert_allclose(util.to_np(lse), lse_ref, rtol=1e-3, atol=5e-3)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("D", [64, 128])
def test_forward_matches_checker_kernel_at_medium_size(gqa_lib, D, causal):
    B, Hq, Hkv, S = 2, 8, 2, 2048
    q, k, v, _ = util.make_inputs(B, Hq, Hkv, S, D, seed=31)
    tq, tk, tv = (util.to_dev_bf16(x) for x in (q, k, v))
    o, lse = ops.gqa_forward(tq, tk, tv, causal=causal)
    ops.check_status()
    o2, lse2 = ops.checker_forward(tq, tk, tv, causal)
    util.assert_close_bf16(util.to_np(o), util.to_np(o2), "O", util.REL_RMS_FWD)
    np.testing.assert_allclose(util.to_np(lse), util.to_np(lse2), rtol=1e-3, atol=2e-3)


def test_forward_headline_shape_properties(gqa_lib):
    """Full headline shape (B8 Hq12 Hkv4 S4096 D64): properties that need no reference.
    (1) with V = const per column, O equals that constant; (2) rows of P sum to one <=> with V = 1;
    (3) heads of one GQA group that are given identical Q produce identical O and LSE."""
    B, Hq, Hkv, S, D = 8, 12, 4, 4096, 64
    gen = torch.Generator(device="cuda").manual_seed(1)
    q = torch.randn(B, Hq, S, D, generator=gen, device="cuda").bfloat16()
    q[:, 1::3] = q[:, 0::3]                      # head 3g+1 duplicates head 3g (same KV head)
    k = torch.randn(B, Hkv, S, D, generator=gen, device="cuda").bfloat16()
    cols = torch.linspace(-2, 2, D, device="cuda").bfloat16()
    v = cols.expand(B, Hkv, S, D).contiguous()
    o, lse = ops.gqa_forward(q, k, v, causal=False)
    ops.check_status()
    assert torch.isfinite(o.float()).all() and torch.isfinite(lse).all()
    assert (o.float() - cols.float()).abs().max().item() <= 2e-2
    assert torch.equal(o[:, 1::3], o[:, 0::3]) and torch.equal(lse[:, 1::3], lse[:, 0::3])


def test_forward_rejects_unsupported_shapes(gqa_lib):
    q = torch.zeros(1, 2, 192, 100, dtype=torch.bfloat16, device="cuda")  # head dim not a multiple of 8
    with pytest.raises(capi.GqaError) as e:
        ops.gqa_forward(q, q, q)
    assert e.value.status == -2
    q = torch.zeros(1, 3, 128, 64, dtype=torch.bfloat16, device="cuda")   # Hq not a multiple of Hkv
    k = torch.zeros(1, 2, 128, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(capi.GqaError) as e:
        ops.gqa_forward(q, k, k)
    assert e.value.status == -2
