"""GPU test: the autograd wrapper against PyTorch fp32 SDPA autograd (the reference's oracle call,
precision/baseline_gqa.py:64-66, :429-435) on the same seeded inputs."""
import pytest
import torch
import torch.nn.functional as F

import util
from hopper_jeni_b200.autograd import gqa_attention

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("causal", [False, True])
def test_autograd_wrapper_matches_fp32_sdpa(gqa_lib, causal):
    B, Hq, Hkv, S, D = 2, 8, 2, 512, 64
    g = torch.Generator(device="cuda").manual_seed(5)
    q, k, v = (torch.randn(B, h, S, D, generator=g, device="cuda").bfloat16().requires_grad_(True) for h in (Hq, Hkv, Hkv))
    do = torch.randn(B, Hq, S, D, generator=g, device="cuda").bfloat16()
    gqa_attention(q, k, v, causal=causal).backward(do)
    q32, k32, v32 = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    F.scaled_dot_product_attention(q32, k32, v32, is_causal=causal, enable_gqa=True).backward(do.float())
    for got, ref, name in ((q.grad, q32.grad, "dQ"), (k.grad, k32.grad, "dK"), (v.grad, v32.grad, "dV")):
        util.assert_close_bf16(util.to_np(got), util.to_np(ref), name, util.REL_RMS_BWD)


def test_autograd_wrapper_sequence_major_ragged_deterministic(gqa_lib):
    """[B,S,H,D] tensors, a sequence length that is not a multiple of the tile, ordered dQ reductions: the
    gradients match fp32 SDPA autograd and two runs give the same bits."""
    B, Hq, Hkv, S, D = 1, 4, 2, 300, 128
    g = torch.Generator(device="cuda").manual_seed(6)
    q, k, v = (torch.randn(B, S, h, D, generator=g, device="cuda").bfloat16().requires_grad_(True) for h in (Hq, Hkv, Hkv))
    do = torch.randn(B, S, Hq, D, generator=g, device="cuda").bfloat16()
    grads = []
    for _ in range(2):
        for t in (q, k, v):
            t.grad = None
        gqa_attention(q, k, v, causal=True, layout="bshd", deterministic=True).backward(do)
        grads.append([t.grad.clone() for t in (q, k, v)])
    for a, b2 in zip(*grads):
        assert torch.equal(a, b2)
    q32, k32, v32 = (t.detach().float().transpose(1, 2).requires_grad_(True) for t in (q, k, v))
    F.scaled_dot_product_attention(q32, k32, v32, is_causal=True, enable_gqa=True).backward(do.float().transpose(1, 2))
    for got, ref, name in zip(grads[0], (q32.grad, k32.grad, v32.grad), ("dQ", "dK", "dV")):
        util.assert_close_bf16(util.to_np(got.transpose(1, 2).contiguous()), util.to_np(ref.contiguous()), name,
                               util.REL_RMS_BWD)


def test_autograd_wrapper_packed_varlen_matches_fp32_sdpa(gqa_lib):
    """Packed variable-length batch through the autograd wrapper: the gradients of every sequence match fp32 SDPA
    autograd run on that sequence alone."""
    from hopper_jeni_b200.autograd import gqa_attention_varlen

    lens, Hq, Hkv, D = [300, 128, 77, 515], 8, 2, 128
    T = sum(lens)
    g = torch.Generator(device="cuda").manual_seed(8)
    q, k, v = (torch.randn(T, h, D, generator=g, device="cuda").bfloat16().requires_grad_(True) for h in (Hq, Hkv, Hkv))
    do = torch.randn(T, Hq, D, generator=g, device="cuda").bfloat16()
    cu = torch.tensor([0, 300, 428, 505, 1020], dtype=torch.int32, device="cuda")
    gqa_attention_varlen(q, k, v, cu, max(lens), causal=True).backward(do)
    start = 0
    for n in lens:
        sl = slice(start, start + n)
        # [n,H,D] -> [1,H,n,D]
        q32, k32, v32 = (t.detach()[sl].float().transpose(0, 1).unsqueeze(0).requires_grad_(True) for t in (q, k, v))
        F.scaled_dot_product_attention(q32, k32, v32, is_causal=True, enable_gqa=True).backward(
            do[sl].float().transpose(0, 1).unsqueeze(0))
        for got, ref, name in ((q.grad, q32.grad, "dQ"), (k.grad, k32.grad, "dK"), (v.grad, v32.grad, "dV")):
            util.assert_close_bf16(util.to_np(got[sl].transpose(0, 1).unsqueeze(0)), util.to_np(ref), f"{name}@{start}",
                                   util.REL_RMS_BWD)
        start += n
