"""CPU tests: the C oracle against the reference's own outputs (golden fixtures), against an
independent numpy restatement and against PyTorch fp32 SDPA autograd on the CPU plumbing config."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

import util


@pytest.mark.parametrize("name", util.GOLDEN_CASES)
def test_oracle_matches_reference_fp64_outputs(oracle, name):
    g = util.load_golden(name)
    o, lse = oracle.forward(g["q"], g["k"], g["v"], g["causal"], g["scale"])
    dq, dk, dv = oracle.backward(g["q"], g["k"], g["v"], g["do"], g["causal"], g["scale"])
    # bench_core.reference_output(mode="fp64") exists for causal and non-causal
    np.testing.assert_allclose(o, g["o_fp64"], rtol=1e-5, atol=2e-6)
    if g["causal"]:
        # precision/baseline_gqa.py fp64_reference / fp64_backward (causal only)
        np.testing.assert_allclose(o, g["o_fp64_baseline"], rtol=1e-5, atol=2e-6)
        np.testing.assert_allclose(lse, g["lse_fp64"], rtol=1e-6, atol=2e-6)
        for got, key in ((dq, "dq_fp64"), (dk, "dk_fp64"), (dv, "dv_fp64")):
            scale_ = max(1.0, float(np.abs(g[key]).max()))
            np.testing.assert_allclose(got, g[key], rtol=1e-5, atol=3e-6 * scale_)


@pytest.mark.parametrize("name", util.GOLDEN_CASES)
def test_oracle_matches_reference_fp32_sdpa_outputs(oracle, name):
    """The fp32 SDPA(+autograd) outputs are the parity target named for the GPU kernels; the oracle
    (double accumulation) must agree with them to fp32 round-off."""
    g = util.load_golden(name)
    o, _ = oracle.forward(g["q"], g["k"], g["v"], g["causal"], g["scale"])
    dq, dk, dv = oracle.backward(g["q"], g["k"], g["v"], g["do"], g["causal"], g["scale"])
    for got, key in ((o, "o_fp32_sdpa"), (dq, "dq_fp32_sdpa"), (dk, "dk_fp32_sdpa"), (dv, "dv_fp32_sdpa")):
        m = util.metrics(got, g[key])
        assert m["rel_rms"] < 2e-5 and m["max_abs"] < 2e-4 * max(1.0, float(np.abs(g[key]).max())), (key, m)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(1, 1, 1, 1, 16), (1, 3, 1, 7, 8), (2, 4, 4, 33, 16), (1, 8, 2, 65, 64)])
def test_oracle_vs_numpy_restatement_edge_shapes(oracle, shape, causal):
    """S = 1, ragged S, MQA (Hkv = 1), MHA (G = 1) and GQA."""
    B, Hq, Hkv, S, D = shape
    q, k, v, do = util.make_inputs(B, Hq, Hkv, S, D, seed=7, bf16=False)
    sc = util.default_scale(D)
    o, lse = oracle.forward(q, k, v, causal, sc)
    o2, lse2 = oracle.numpy_forward(q, k, v, causal, sc)
    np.testing.assert_allclose(o, o2, rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(lse, lse2, rtol=1e-6, atol=1e-6)
    got = oracle.backward(q, k, v, do, causal, sc)
    want = oracle.numpy_backward(q, k, v, do, causal, sc)
    for a, b in zip(got, want):
        np.testing.assert_allclose(a, b, rtol=1e-5, atol=1e-5)


def test_oracle_causal_first_row_sees_one_key(oracle):
    q, k, v, _ = util.make_inputs(1, 2, 1, 16, 8, seed=3, bf16=False)
    o, lse = oracle.forward(q, k, v, True, 0.3)
    np.testing.assert_allclose(o[0, :, 0], np.broadcast_to(v[0, 0, 0], (2, 8)), rtol=1e-6)
    np.testing.assert_allclose(lse[0, :, 0], 0.3 * (q[0, :, 0] @ k[0, 0, 0]), rtol=1e-5, atol=1e-6)


def test_oracle_rejects_bad_head_counts(oracle):
    q, k, v, _ = util.make_inputs(1, 3, 2, 8, 8, bf16=False)
    with pytest.raises(RuntimeError):
        oracle.forward(q, k, v, False, 1.0)


def test_oracle_matches_torch_sdpa_autograd_cpu_plumbing_config(oracle):
    """CPU plumbing config: fp32, B=2, Hq=6, Hkv=2 (G=3), S=512, D=64, non-causal, N(0,1)."""
    B, Hq, Hkv, S, D = 2, 6, 2, 512, 64
    q, k, v, do = util.make_inputs(B, Hq, Hkv, S, D, seed=42, bf16=False)
    sc = util.default_scale(D)
    tq, tk, tv = (torch.from_numpy(x).requires_grad_(True) for x in (q, k, v))
    out = F.scaled_dot_product_attention(tq, tk, tv, scale=sc, enable_gqa=True)
    out.backward(torch.from_numpy(do))
    o, _ = oracle.forward(q, k, v, False, sc)
    dq, dk, dv = oracle.backward(q, k, v, do, False, sc)
    for got, ref in ((o, out), (dq, tq.grad), (dk, tk.grad), (dv, tv.grad)):
        m = util.metrics(got, ref.detach().numpy())
        assert m["rel_rms"] < 5e-6, m


def test_oracle_delta(oracle):
    q, _, _, do = util.make_inputs(1, 2, 1, 32, 64, bf16=False)
    d = oracle.delta(q, do)
    np.testing.assert_allclose(d, (q.astype(np.float64) * do).sum(-1), rtol=1e-6, atol=1e-6)
