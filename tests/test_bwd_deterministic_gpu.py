"""GPU tests of the deterministic backward (gqa_bwd_ex with GQA_BWD_DETERMINISTIC): dQ is bit-identical from
run to run (what the reference's vj1d_determinism_probe.cu measures for its own kernel), agrees with the CPU
oracle, and equals the default mode up to the order of the fp32 additions."""
import ctypes

import pytest
import torch

import util
from hopper_jeni_b200 import capi, ops

pytestmark = pytest.mark.gpu


def _inputs(B, Hq, Hkv, S, D, causal, seed):
    q, k, v, do = util.make_inputs(B, Hq, Hkv, S, D, seed=seed)
    tq, tk, tv, tdo = (util.to_dev_bf16(x) for x in (q, k, v, do))
    o, lse = ops.gqa_forward(tq, tk, tv, causal=causal)
    return (q, k, v, do), (tq, tk, tv, tdo, o, lse)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(2, 6, 2, 256, 64), (1, 4, 2, 384, 128)])
def test_deterministic_backward_matches_oracle(gqa_lib, oracle, shape, causal):
    B, Hq, Hkv, S, D = shape
    (q, k, v, do), (tq, tk, tv, tdo, o, lse) = _inputs(B, Hq, Hkv, S, D, causal, seed=71)
    sc = util.default_scale(D)
    dq_ref, dk_ref, dv_ref = oracle.backward(q, k, v, do, causal, sc)
    ws = torch.empty(ops.bwd_workspace_bytes(B, Hq, Hkv, S, D, causal), dtype=torch.uint8, device="cuda")
    dq, dk, dv = ops.gqa_backward(tq, tk, tv, o, tdo, lse, causal=causal, scale=sc, workspace=ws, deterministic=True)
    ops.check_status(ws)
    util.assert_close_bf16(util.to_np(dq), dq_ref, "dQ", util.REL_RMS_BWD)
    util.assert_close_bf16(util.to_np(dk), dk_ref, "dK", util.REL_RMS_BWD)
    util.assert_close_bf16(util.to_np(dv), dv_ref, "dV", util.REL_RMS_BWD)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(2, 12, 4, 2048, 64), (2, 8, 2, 2048, 128), (8, 12, 4, 4096, 64)])
def test_deterministic_backward_is_bit_reproducible(gqa_lib, shape, causal):
    """More thread blocks than SMs, several per (batch, KV head) group: every dQ tile gets up to S/128 ordered
    reductions.  Four runs, all three gradients bit-identical; the default mode agrees up to the order of its fp32
    sums."""
    B, Hq, Hkv, S, D = shape
    gen = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn(B, Hq, S, D, generator=gen, device="cuda").bfloat16()
    k = torch.randn(B, Hkv, S, D, generator=gen, device="cuda").bfloat16()
    v = torch.randn(B, Hkv, S, D, generator=gen, device="cuda").bfloat16()
    do = torch.randn(B, Hq, S, D, generator=gen, device="cuda").bfloat16()
    o, lse = ops.gqa_forward(q, k, v, causal=causal)
    ws = torch.empty(ops.bwd_workspace_bytes(B, Hq, Hkv, S, D, causal), dtype=torch.uint8, device="cuda")
    runs = []
    for _ in range(4):
        runs.append(ops.gqa_backward(q, k, v, o, do, lse, causal=causal, workspace=ws, deterministic=True))
        ops.check_status(ws)
    for dq, dk, dv in runs[1:]:
        assert torch.equal(dq, runs[0][0]), "dQ differs between deterministic runs"
        assert torch.equal(dk, runs[0][1]) and torch.equal(dv, runs[0][2])
    dq0, dk0, dv0 = ops.gqa_backward(q, k, v, o, do, lse, causal=causal, workspace=ws)
    ops.check_status(ws)
    if causal:
        assert torch.equal(dk0, runs[0][1]) and torch.equal(dv0, runs[0][2])
    else:
        # without a mask the default mode starts each KV tile's loop over the query tiles at a different tile (the
        # ordered mode does not): the same fp32 sums in another order
        for got, want in ((dk0, runs[0][1]), (dv0, runs[0][2])):
            m = util.metrics(util.to_np(got), util.to_np(want))
            assert m["rel_rms"] < 2e-3, m
    m = util.metrics(util.to_np(dq0), util.to_np(runs[0][0]))
    assert m["rel_rms"] < 2e-3, m


def test_unknown_flag_bits_are_refused(gqa_lib):
    lib = capi.load_library()
    q = torch.zeros(1, 2, 128, 64, dtype=torch.bfloat16, device="cuda")
    lse = torch.zeros(1, 2, 128, dtype=torch.float32, device="cuda")
    ws = torch.empty(ops.bwd_workspace_bytes(1, 2, 2, 128, 64), dtype=torch.uint8, device="cuda")
    p = q.data_ptr()
    rc = lib.gqa_bwd_ex(p, p, p, p, p, lse.data_ptr(), p, p, p, 1, 2, 2, 128, 64, 0, 0.125, ws.data_ptr(), ws.numel(),
                        None, ctypes.c_uint(0x10))
    assert rc == -1
