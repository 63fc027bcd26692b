"""CPU test: the sliced fp32-SDPA reference used by the config-size GPU parity tests (tests/sdpa_ref.py) agrees
with the C oracle (and so with the reference's fp64 loops) on forward, LSE and all three gradients."""
import numpy as np
import pytest
import torch

from oracle import sdpa_ref
import util


@pytest.mark.parametrize("causal", [False, True])
def test_sliced_sdpa_reference_matches_oracle(oracle, causal):
    B, Hq, Hkv, S, D = 1, 6, 2, 128, 64
    G = Hq // Hkv
    q, k, v, do = util.make_inputs(B, Hq, Hkv, S, D, seed=3)
    sc = util.default_scale(D)
    o_ref, lse_ref = oracle.forward(q, k, v, causal, sc)
    dq_ref, dk_ref, dv_ref = oracle.backward(q, k, v, do, causal, sc)
    tq, tk, tv, tdo = (torch.from_numpy(x) for x in (q, k, v, do))
    for h in range(Hkv):
        hs = slice(h * G, (h + 1) * G)
        o, lse, dq, dk, dv = sdpa_ref.sdpa_group(tq[0, hs], tk[0, h], tv[0, h], tdo[0, hs], sc, causal)
        np.testing.assert_allclose(o.numpy(), o_ref[0, hs], atol=5e-6)
        np.testing.assert_allclose(lse.numpy(), lse_ref[0, hs], atol=5e-6)
        np.testing.assert_allclose(dq.numpy(), dq_ref[0, hs], atol=2e-5)
        np.testing.assert_allclose(dk.numpy(), dk_ref[0, h], atol=2e-5)
        np.testing.assert_allclose(dv.numpy(), dv_ref[0, h], atol=2e-5)
        # the O-as-input restatement, given the exact O, is the same backward
        dq2, dk2, dv2 = sdpa_ref.backward_given_o(tq[0, hs], tk[0, h], tv[0, h], o, tdo[0, hs], sc, causal)
        np.testing.assert_allclose(dq2.numpy(), dq_ref[0, hs], atol=2e-5)
        np.testing.assert_allclose(dk2.numpy(), dk_ref[0, h], atol=2e-5)
        np.testing.assert_allclose(dv2.numpy(), dv_ref[0, h], atol=2e-5)


def test_heads_per_slice_divides_the_group():
    assert sdpa_ref.heads_per_slice(32768, 8) == 2
    assert sdpa_ref.heads_per_slice(8192, 4) == 4
    assert sdpa_ref.heads_per_slice(65536, 3) == 1
