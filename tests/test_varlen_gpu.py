"""GPU tests of packed variable-length batches (gqa_fwd_varlen / gqa_bwd_varlen): sequences of different lengths
back to back in [total_tokens, H, D] tensors, each attending only to itself.  Parity per sequence against the CPU
oracle (small lengths) and fp32 SDPA (long ones), lengths that are not multiples of the tile, a one-token and an
empty sequence, max_seqlen larger than needed, outputs poisoned beforehand and guarded behind."""
import numpy as np
import pytest
import torch

import util
from hopper_jeni_b200 import ops
from oracle import sdpa_ref

pytestmark = pytest.mark.gpu


def _cu(lens):
    return torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device="cuda")


def _packed_inputs(lens, Hq, Hkv, D, seed):
    """bf16-rounded fp32 numpy inputs in [B=1,H,T,D] order (the oracle's) for the whole packed batch."""
    T = int(sum(lens))
    return util.make_inputs(1, Hq, Hkv, T, D, seed=seed)


def _to_packed(x):  # numpy [1,H,T,D] -> device bf16 [T,H,D]
    return util.to_dev_bf16(x)[0].transpose(0, 1).contiguous()


def _from_packed(t):  # device [T,H,D] -> numpy [H,T,D]
    return util.to_np(t.transpose(0, 1).contiguous())


SMALL = [
    # lens, Hq, Hkv, D
    ([72, 200, 128, 333, 1, 256], 6, 2, 64),
    ([264, 450, 130, 50], 8, 2, 128),
    ([100, 0, 300, 0], 4, 4, 64),       # empty sequences, G = 1
    ([129], 4, 1, 128),                 # one sequence, one key in its second tile
]


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("case", SMALL)
def test_varlen_matches_oracle_per_sequence(gqa_lib, oracle, case, causal):
    lens, Hq, Hkv, D = case
    T = int(sum(lens))
    qn, kn, vn, don = _packed_inputs(lens, Hq, Hkv, D, seed=301)
    sc = util.default_scale(D)
    q, k, v, do = (_to_packed(x) for x in (qn, kn, vn, don))
    cu = _cu(lens)
    max_seqlen = max(lens) + 37  # larger than needed: only costs empty thread blocks
    max_seqlen = min(max_seqlen, T)
    # outputs poisoned and followed by a guard: every row must be written, nothing behind them may be
    guard = 4096

    def poisoned(like):
        buf = torch.full((like.numel() + guard,), float("nan"), dtype=like.dtype, device="cuda")
        return buf, buf[: like.numel()].view(like.shape)

    obuf, o = poisoned(q)
    lse = torch.full((Hq, T), float("nan"), dtype=torch.float32, device="cuda")
    ops.gqa_forward_varlen(q, k, v, cu, max_seqlen, causal=causal, scale=sc, out=o, lse=lse)
    ops.check_status()
    assert torch.isnan(obuf[q.numel():]).all(), "forward wrote behind O"
    ws = torch.empty(ops.bwd_varlen_workspace_bytes(T, Hq, Hkv, D), dtype=torch.uint8, device="cuda")
    dqbuf, dq = poisoned(q)
    dkbuf, dk = poisoned(k)
    dvbuf, dv = poisoned(v)
    ops.gqa_backward_varlen(q, k, v, o, do, lse, cu, max_seqlen, causal=causal, scale=sc, workspace=ws,
                            dq=dq, dk=dk, dv=dv)
    ops.check_status(ws)
    for buf, t, name in ((dqbuf, dq, "dQ"), (dkbuf, dk, "dK"), (dvbuf, dv, "dV")):
        assert torch.isnan(buf[t.numel():]).all(), f"backward wrote behind {name}"
    o_np, dq_np, dk_np, dv_np = (_from_packed(t) for t in (o, dq, dk, dv))
    lse_np = lse.cpu().numpy()
    start = 0
    for n in lens:
        if n == 0:
            continue
        sl = slice(start, start + n)
        qs, ks, vs, dos = (np.ascontiguousarray(x[:, :, sl]) for x in (qn, kn, vn, don))
        o_ref, lse_ref = oracle.forward(qs, ks, vs, causal, sc)
        dq_ref, dk_ref, dv_ref = oracle.backward(qs, ks, vs, dos, causal, sc)
        tag = f"seq@{start}+{n}"
        util.assert_close_bf16(o_np[None, :, sl], o_ref, f"O {tag}", util.REL_RMS_FWD)
        assert np.allclose(lse_np[None, :, sl], lse_ref, rtol=1e-3, atol=2e-3), tag
        # (a one-token sequence has dQ = dK = 0 exactly: only the absolute gate says anything there)
        rel = util.REL_RMS_BWD if n > 1 else float("inf")
        util.assert_close_bf16(dq_np[None, :, sl], dq_ref, f"dQ {tag}", rel)
        util.assert_close_bf16(dk_np[None, :, sl], dk_ref, f"dK {tag}", rel)
        util.assert_close_bf16(dv_np[None, :, sl], dv_ref, f"dV {tag}", util.REL_RMS_BWD)
        start += n


@pytest.mark.parametrize("D,causal", [(64, True), (64, False), (128, True)])
def test_varlen_long_sequences_match_fp32_sdpa(gqa_lib, D, causal):
    """More work items than SMs, sequences of 1 to 33 KV tiles: the persistent blocks skip the holes of the item
    list, and every sequence matches fp32 SDPA on the same inputs."""
    lens = [4096, 1000, 2500, 777, 3000, 128, 4200, 64]
    Hq, Hkv = (12, 4) if D == 64 else (8, 2)
    G = Hq // Hkv
    T = sum(lens)
    gen = torch.Generator(device="cuda").manual_seed(17)
    q = torch.randn(T, Hq, D, generator=gen, device="cuda").bfloat16()
    k = torch.randn(T, Hkv, D, generator=gen, device="cuda").bfloat16()
    v = torch.randn(T, Hkv, D, generator=gen, device="cuda").bfloat16()
    do = torch.randn(T, Hq, D, generator=gen, device="cuda").bfloat16()
    cu = _cu(lens)
    sc = util.default_scale(D)
    o, lse = ops.gqa_forward_varlen(q, k, v, cu, max(lens), causal=causal, scale=sc)
    ops.check_status()
    ws = torch.empty(ops.bwd_varlen_workspace_bytes(T, Hq, Hkv, D), dtype=torch.uint8, device="cuda")
    dq, dk, dv = ops.gqa_backward_varlen(q, k, v, o, do, lse, cu, max(lens), causal=causal, scale=sc, workspace=ws)
    ops.check_status(ws)
    dk2, dv2 = ops.gqa_backward_varlen(q, k, v, o, do, lse, cu, max(lens), causal=causal, scale=sc, workspace=ws)[1:]
    ops.check_status(ws)
    assert torch.equal(dk, dk2) and torch.equal(dv, dv2), "dK/dV differ between two runs"
    start = 0
    for n in lens:
        sl = slice(start, start + n)
        for hkv in range(Hkv):
            hs = slice(hkv * G, (hkv + 1) * G)
            o_ref, lse_ref, dq_ref, dk_ref, dv_ref = sdpa_ref.sdpa_group(
                q[sl, hs].transpose(0, 1), k[sl, hkv], v[sl, hkv], do[sl, hs].transpose(0, 1), sc, causal)
            for got, ref, name, tol in ((o[sl, hs].transpose(0, 1), o_ref, "O", 1e-2),
                                        (dq[sl, hs].transpose(0, 1), dq_ref, "dQ", 2e-2),
                                        (dk[sl, hkv], dk_ref, "dK", 2e-2), (dv[sl, hkv], dv_ref, "dV", 2e-2)):
                m = sdpa_ref.metrics(got.float(), ref)
                assert m["rel_rms"] <= tol, (name, start, n, hkv, m)
                assert m["gate_ok"], (name, start, n, hkv, m)
            assert torch.allclose(lse[hs, sl], lse_ref, rtol=1e-3, atol=2e-3)
        start += n


def test_varlen_equal_lengths_equal_the_batched_call(gqa_lib):
    """A packed batch of equal, tile-aligned lengths is the [B,S,H,D] problem: O, LSE, dK and dV bit for bit (same
    arithmetic in the same order), dQ up to the order of the fp32 reductions."""
    B, Hq, Hkv, S, D = 3, 8, 2, 512, 64
    gen = torch.Generator(device="cuda").manual_seed(23)
    q = torch.randn(B, S, Hq, D, generator=gen, device="cuda").bfloat16()
    k = torch.randn(B, S, Hkv, D, generator=gen, device="cuda").bfloat16()
    v = torch.randn(B, S, Hkv, D, generator=gen, device="cuda").bfloat16()
    do = torch.randn(B, S, Hq, D, generator=gen, device="cuda").bfloat16()
    cu = _cu([S] * B)
    for causal in (True, False):
        o, lse = ops.gqa_forward(q, k, v, causal=causal, layout="bshd")
        o2, lse2 = ops.gqa_forward_varlen(q.view(B * S, Hq, D), k.view(B * S, Hkv, D), v.view(B * S, Hkv, D), cu, S,
                                          causal=causal)
        ops.check_status()
        assert torch.equal(o.view(B * S, Hq, D), o2)
        assert torch.equal(lse.transpose(0, 1).reshape(Hq, B * S), lse2)
        ws = torch.empty(ops.bwd_workspace_bytes(B, Hq, Hkv, S, D, causal), dtype=torch.uint8, device="cuda")
        dq, dk, dv = ops.gqa_backward(q, k, v, o, do, lse, causal=causal, workspace=ws, layout="bshd")
        ops.check_status(ws)
        dq2, dk2, dv2 = ops.gqa_backward_varlen(q.view(B * S, Hq, D), k.view(B * S, Hkv, D), v.view(B * S, Hkv, D), o2,
                                                do.view(B * S, Hq, D), lse2, cu, S, causal=causal)
        assert torch.equal(dk.view(B * S, Hkv, D), dk2) and torch.equal(dv.view(B * S, Hkv, D), dv2), causal
        m = util.metrics(util.to_np(dq2), util.to_np(dq.view(B * S, Hq, D)))
        assert m["rel_rms"] < 2e-3, m


def test_varlen_rejects_bad_arguments(gqa_lib):
    from hopper_jeni_b200 import capi

    T, Hq, Hkv, D = 256, 4, 2, 64
    q = torch.zeros(T, Hq, D, dtype=torch.bfloat16, device="cuda")
    k = torch.zeros(T, Hkv, D, dtype=torch.bfloat16, device="cuda")
    cu = _cu([100, 156])
    with pytest.raises(capi.GqaError):
        ops.gqa_forward_varlen(q, k, k, cu, 0)          # max_seqlen must be positive
    with pytest.raises(capi.GqaError):
        ops.gqa_forward_varlen(q, k, k, cu, T + 1)      # ... and cannot exceed the token count
    q96 = torch.zeros(T, Hq, 96, dtype=torch.bfloat16, device="cuda")
    k96 = torch.zeros(T, Hkv, 96, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(capi.GqaError):
        ops.gqa_forward_varlen(q96, k96, k96, cu, 156)  # packed batches need D = 64 or 128
    with pytest.raises(ValueError):
        ops.gqa_forward_varlen(q, k, k, cu.cpu(), 156)  # cu_seqlens must be on the device
