"""GPU test of the harness plug-ins: driven exactly as the reference harness drives a competitor
(available -> forward/backward on canonical [B,Hq,S,D] bf16 -> correctness gate against fp32 SDPA,
harness/bench_core.py:143-183, harness/run_gqa_bwd_v44_bench.py:108-131)."""
import math
from dataclasses import dataclass

import pytest
import torch
import torch.nn.functional as F

from hopper_jeni_b200.competitor import YourKernel, YourKernelBwd

pytestmark = pytest.mark.gpu


@dataclass
class Shape:  # same fields as harness/bench_core.py:21-36
    B: int
    Hq: int
    Hkv: int
    S: int
    D: int
    causal: bool = True
    dtype: str = "bf16"

    @property
    def G(self):
        return self.Hq // self.Hkv


def _gate(got, ref, atol=2e-2, rtol=2e-2):  # harness/bench_core.py:175-183
    return (got.float() - ref.float()).abs().max().item() <= atol + rtol * ref.float().abs().max().item()


@pytest.mark.parametrize("shape", [Shape(2, 12, 4, 1024, 128, True), Shape(2, 12, 4, 1024, 64, False)])
def test_plugins_pass_the_harness_gate(gqa_lib, shape):
    g = torch.Generator(device="cuda").manual_seed(42)
    mk = lambda h: torch.rand(shape.B, h, shape.S, shape.D, generator=g, device="cuda").bfloat16()
    q, k, v, do = mk(shape.Hq), mk(shape.Hkv), mk(shape.Hkv), mk(shape.Hq)   # U[0,1) like the harness
    fwd, bwd = YourKernel(), YourKernelBwd()
    assert fwd.available(shape) == (True, "") and bwd.available(shape) == (True, "")
    q32, k32, v32 = (t.float().requires_grad_(True) for t in (q, k, v))
    ref = F.scaled_dot_product_attention(q32, k32, v32, scale=1 / math.sqrt(shape.D), is_causal=shape.causal,
                                         enable_gqa=True)
    ref.backward(do.float())
    assert _gate(fwd.make(q, k, v, shape)(), ref)
    dq, dk, dv = bwd.make_bwd(q, k, v, do, shape)()
    assert _gate(dq, q32.grad) and _gate(dk, k32.grad) and _gate(dv, v32.grad)
    assert fwd.available(Shape(1, 4, 2, 100, 64))[0] is True      # any sequence length
    assert fwd.available(Shape(1, 4, 2, 128, 96))[0] is False     # head dims other than 64 and 128
