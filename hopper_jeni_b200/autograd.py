"""``torch.autograd.Function`` over the C ABI: forward keeps O and LSE for the backward, so the backward
does not recompute the forward (the hand-off the reference does through files, src/attention/GQA_bwd_baseline.cu:641-643)."""
from __future__ import annotations

import math

import torch

from . import ops


class _GqaAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale, layout, deterministic):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        o, lse = ops.gqa_forward(q, k, v, causal=causal, scale=scale, layout=layout)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.causal, ctx.scale, ctx.layout, ctx.deterministic = causal, scale, layout, deterministic
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = ops.gqa_backward(q, k, v, o, do.contiguous(), lse, causal=ctx.causal, scale=ctx.scale,
                                      layout=ctx.layout, deterministic=ctx.deterministic)
        return dq, dk, dv, None, None, None, None


def gqa_attention(q, k, v, causal: bool = False, scale: float | None = None, layout: str = "bhsd",
                  deterministic: bool = False):
    """Differentiable GQA attention on bf16 CUDA tensors ``[B,Hq,S,D]`` / ``[B,Hkv,S,D]``; same semantics as
    ``F.scaled_dot_product_attention(q, k, v, scale=scale, is_causal=causal, enable_gqa=True)``.
    ``layout="bshd"`` takes and returns ``[B,S,H,D]`` tensors; ``deterministic`` makes the gradient of q
    bit-reproducible (the other two always are)."""
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else float(scale)
    return _GqaAttention.apply(q, k, v, bool(causal), scale, layout, bool(deterministic))


class _GqaAttentionVarlen(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, max_seqlen, causal, scale):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        o, lse = ops.gqa_forward_varlen(q, k, v, cu_seqlens, max_seqlen, causal=causal, scale=scale)
        ctx.save_for_backward(q, k, v, o, lse, cu_seqlens)
        ctx.max_seqlen, ctx.causal, ctx.scale = max_seqlen, causal, scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, cu_seqlens = ctx.saved_tensors
        dq, dk, dv = ops.gqa_backward_varlen(q, k, v, o, do.contiguous(), lse, cu_seqlens, ctx.max_seqlen,
                                             causal=ctx.causal, scale=ctx.scale)
        return dq, dk, dv, None, None, None, None


def gqa_attention_varlen(q, k, v, cu_seqlens, max_seqlen: int, causal: bool = False, scale: float | None = None):
    """Differentiable GQA attention over a packed variable-length batch: q ``[T,Hq,D]``, k and v ``[T,Hkv,D]`` bf16,
    ``cu_seqlens`` int32 ``[n_seqs+1]`` on the same device; every sequence attends only to itself."""
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else float(scale)
    return _GqaAttentionVarlen.apply(q, k, v, cu_seqlens, int(max_seqlen), bool(causal), scale)
