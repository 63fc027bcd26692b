"""The reference side of the config-size parity tests: PyTorch fp32 scaled_dot_product_attention and its
autograd (the reference's own oracle call, precision/baseline_gqa.py:64-66, :429-435;
harness/run_gqa_bwd_v44_bench.py:108-118) on the same bf16-rounded inputs, evaluated on the GPU in slices
of (batch, KV-head) groups so that the fp32 score blocks of the long configs fit.

Test infrastructure: only tests/ and the checker legs of bench.py (outside every timed region) import it;
nothing in the package does.  tests/test_sdpa_ref.py pins it to the C oracle, which is pinned to the reference's
own fp64 loops by the golden fixtures.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch.nn.attention import SDPBackend, sdpa_kernel


def _no_tf32():
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False


def heads_per_slice(S: int, G: int, budget_bytes: float = 12e9) -> int:
    """Query heads of one group evaluated together: the fp32 score block [h, S, S] stays under the budget
    (the math backend keeps about five such blocks alive through the backward)."""
    h = max(1, int(budget_bytes // (4.0 * S * S)))
    while G % h:
        h -= 1
    return h


@torch.no_grad()
def lse_slice(q, k, scale, causal):
    """logsumexp of the scaled (masked) logits; q [h, S, D], k [S, D] fp32."""
    s = torch.matmul(q, k.t()) * scale
    if causal:
        S = s.shape[-1]
        s.masked_fill_(torch.ones(S, S, dtype=torch.bool, device=s.device).triu_(1), float("-inf"))
    return torch.logsumexp(s, dim=-1)


def sdpa_group(q, k, v, do, scale, causal, want_lse=True):
    """fp32 SDPA forward (+ backward when `do` is given) of ONE (batch, KV-head) group.
    q, do [G, S, D]; k, v [S, D] (bf16 or fp32, any device).  Returns fp32 o [G,S,D], lse [G,S] or None,
    dq [G,S,D], dk [S,D], dv [S,D] (None without `do`)."""
    _no_tf32()
    G, S, D = q.shape
    step = heads_per_slice(S, G)
    kf, vf = k.float(), v.float()
    o = torch.empty(G, S, D, dtype=torch.float32, device=q.device)
    lse = torch.empty(G, S, dtype=torch.float32, device=q.device) if want_lse else None
    dq = torch.empty_like(o) if do is not None else None
    dk = torch.zeros(S, D, dtype=torch.float32, device=q.device) if do is not None else None
    dv = torch.zeros_like(dk) if do is not None else None
    for h0 in range(0, G, step):
        qs = q[h0:h0 + step].float().unsqueeze(0).requires_grad_(do is not None)
        ks = kf.view(1, 1, S, D).clone().requires_grad_(do is not None)
        vs = vf.view(1, 1, S, D).clone().requires_grad_(do is not None)
        with sdpa_kernel(SDPBackend.MATH):
            os_ = F.scaled_dot_product_attention(qs, ks, vs, scale=scale, enable_gqa=True, is_causal=causal)
        o[h0:h0 + step] = os_.detach()[0]
        if do is not None:
            os_.backward(do[h0:h0 + step].float().unsqueeze(0))
            dq[h0:h0 + step] = qs.grad[0]
            dk += ks.grad[0, 0]
            dv += vs.grad[0, 0]
        del os_, qs, ks, vs
        if want_lse:
            lse[h0:h0 + step] = lse_slice(q[h0:h0 + step].float(), kf, scale, causal)
    return o, lse, dq, dk, dv


@torch.no_grad()
def backward_given_o(q, k, v, o, do, scale, causal):
    """fp32 backward of ONE (batch, KV-head) group that takes O as an INPUT, the way the operator does
    (Delta = rowsum(dO * O) from the O it is handed: src/attention/GQA_bwd_baseline.cu:273-298), with every
    other step exact: P = softmax(scale Q K^T), dP = dO V^T, dS = P (dP - Delta), dQ = scale dS K,
    dK = scale dS^T Q, dV = P^T dO (precision/baseline_gqa.py:169-197).  With O in fp32 this is SDPA autograd; with
    the bf16 O the operator really receives, it isolates the error that the input rounding of O alone puts
    into dQ/dK -- which dominates for inputs like U[0,1), where Delta is a large common offset of dP.
    q, o, do [G, S, D]; k, v [S, D].  Returns fp32 dq [G,S,D], dk [S,D], dv [S,D]."""
    _no_tf32()
    G, S, D = q.shape
    kf, vf = k.float(), v.float()
    dq = torch.empty(G, S, D, dtype=torch.float32, device=q.device)
    dk = torch.zeros(S, D, dtype=torch.float32, device=q.device)
    dv = torch.zeros_like(dk)
    mask = torch.ones(S, S, dtype=torch.bool, device=q.device).triu_(1) if causal else None
    for h in range(G):
        qf, dof = q[h].float(), do[h].float()
        s = torch.matmul(qf, kf.t()) * scale
        if causal:
            s.masked_fill_(mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        delta = (dof * o[h].float()).sum(-1, keepdim=True)
        ds = p * (torch.matmul(dof, vf.t()) - delta)
        dq[h] = torch.matmul(ds, kf) * scale
        dk += torch.matmul(ds.t(), qf) * scale
        dv += torch.matmul(p.t(), dof)
    return dq, dk, dv


def metrics(got: torch.Tensor, ref: torch.Tensor, atol=2e-2, rtol=2e-2):
    """max_abs, rel_rms and the element-wise gate |d| <= atol + rtol |ref| (on the device, fp64 sums)."""
    d = (got.double() - ref.double())
    return {
        "max_abs": float(d.abs().max()),
        "rel_rms": float(d.pow(2).sum().sqrt() / ref.double().pow(2).sum().sqrt().clamp_min(1e-30)),
        "gate_ok": bool((d.abs() <= atol + rtol * ref.double().abs()).all()),
        "finite": bool(torch.isfinite(got.float()).all()),
    }
