"""GPU tests: the CUDA-core checker kernels and the Delta preprocess against the CPU oracle."""
import numpy as np
import pytest
import torch

import util
from hopper_jeni_b200 import ops

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(1, 4, 2, 96, 64), (2, 6, 2, 256, 64), (1, 2, 1, 128, 128)])
def test_checker_kernels_match_oracle(gqa_lib, oracle, shape, causal):
    B, Hq, Hkv, S, D = shape
    q, k, v, do = util.make_inputs(B, Hq, Hkv, S, D, seed=11)
    sc = util.default_scale(D)
    o_ref, lse_ref = oracle.forward(q, k, v, causal, sc)
    dq_ref, dk_ref, dv_ref = oracle.backward(q, k, v, do, causal, sc)
    tq, tk, tv, tdo = (util.to_dev_bf16(x) for x in (q, k, v, do))
    o, lse = ops.checker_forward(tq, tk, tv, causal, sc)
    util.assert_close_bf16(util.to_np(o), o_ref, "O", util.REL_RMS_FWD)
    np.testing.assert_allclose(util.to_np(lse), lse_ref, rtol=1e-4, atol=1e-4)
    dq, dk, dv = ops.checker_backward(tq, tk, tv, o, tdo, lse, causal, sc)
    torch.cuda.synchronize()
    util.assert_close_bf16(util.to_np(dq), dq_ref, "dQ", util.REL_RMS_BWD)
    util.assert_close_bf16(util.to_np(dk), dk_ref, "dK", util.REL_RMS_BWD)
    util.assert_close_bf16(util.to_np(dv), dv_ref, "dV", util.REL_RMS_BWD)


@pytest.mark.parametrize("D", [64, 128])
def test_delta_preprocess_matches_oracle(gqa_lib, oracle, D):
    rng = np.random.default_rng(5)
    o = util.bf16_round(rng.standard_normal((3, 5, 77, D), dtype=np.float32))
    do = util.bf16_round(rng.standard_normal((3, 5, 77, D), dtype=np.float32))
    got = ops.gqa_delta(util.to_dev_bf16(o), util.to_dev_bf16(do))
    np.testing.assert_allclose(util.to_np(got), oracle.delta(o, do), rtol=1e-5, atol=1e-4)
