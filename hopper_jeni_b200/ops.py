"""Tensor-level wrappers over the C ABI.

torch is used only for device memory and streams; all arithmetic happens inside the library.
Layouts follow the reference launchers (src/attention/GQA_bwd_baseline.cu:549-554,
src/attention/GQA_fwd_ref.cu:631-634): Q/O/dO/dQ ``[B,Hq,S,D]``, K/V/dK/dV ``[B,Hkv,S,D]`` bf16
contiguous, LSE ``[B,Hq,S]`` fp32 (natural log).
"""
from __future__ import annotations

import math

import torch

from . import capi


def _stream_ptr(stream=None) -> int:
    s = stream if stream is not None else torch.cuda.current_stream()
    return int(s.cuda_stream)


def _req(t: torch.Tensor, name: str, dtype) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (this library has no CPU path)")
    if t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _req_like(t: torch.Tensor, name: str, like: torch.Tensor, shape=None, dtype=None) -> None:
    """`t` must live on `like`'s device, be contiguous and have exactly the given shape and dtype: the C ABI
    receives raw pointers, so a wrong-sized or wrong-device tensor would become an out-of-bounds access."""
    _req(t, name, like.dtype if dtype is None else dtype)
    if t.device != like.device:
        raise ValueError(f"{name} is on {t.device}, expected {like.device}")
    want = tuple(like.shape if shape is None else shape)
    if tuple(t.shape) != want:
        raise ValueError(f"{name} has shape {tuple(t.shape)}, expected {want}")


def _dims(q, k, layout="bhsd"):
    if layout == "bshd":
        B, S, Hq, D = q.shape
        if k.shape[0] != B or k.shape[1] != S or k.shape[3] != D:
            raise ValueError(f"K/V shape {tuple(k.shape)} does not match Q {tuple(q.shape)}")
        return B, Hq, k.shape[2], S, D
    if layout != "bhsd":
        raise ValueError(f"layout must be 'bhsd' or 'bshd', got {layout!r}")
    B, Hq, S, D = q.shape
    if k.shape[0] != B or k.shape[2] != S or k.shape[3] != D:
        raise ValueError(f"K/V shape {tuple(k.shape)} does not match Q {tuple(q.shape)}")
    return B, Hq, k.shape[1], S, D


def launch_count() -> int:
    """Kernels launched by the library since it was loaded."""
    return int(capi.load_library().gqa_launch_count())


def gqa_forward(q, k, v, causal: bool = False, scale: float | None = None, out=None, lse=None, stream=None,
                layout: str = "bhsd"):
    """O, LSE = attention(Q, K, V).  Mirrors ``launch_gqa_v62`` with D and causal as arguments.
    ``layout="bshd"``: Q, K, V, O are [B,S,H,D] (``GQA_LAYOUT_BSHD``); LSE is [B,Hq,S] either way."""
    lib = capi.load_library()
    for t, n in ((q, "Q"), (k, "K"), (v, "V")):
        _req(t, n, torch.bfloat16)
    B, Hq, Hkv, S, D = _dims(q, k, layout)
    scale = 1.0 / math.sqrt(D) if scale is None else float(scale)
    out = torch.empty_like(q) if out is None else out
    lse = torch.empty((B, Hq, S), dtype=torch.float32, device=q.device) if lse is None else lse
    _req_like(v, "V", k)
    _req_like(out, "O", q)
    _req_like(lse, "LSE", q, shape=(B, Hq, S), dtype=torch.float32)
    with torch.cuda.device(q.device):
        rc = lib.gqa_fwd_ex(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                            B, Hq, Hkv, S, D, int(bool(causal)), scale, _stream_ptr(stream),
                            capi.GQA_LAYOUT_BSHD if layout == "bshd" else 0)
    capi.check("gqa_fwd_ex", rc)
    return out, lse


def bwd_workspace_bytes(B, Hq, Hkv, S, D, causal=False, split_heads: bool = False) -> int:
    """Bytes of scratch ``gqa_backward`` needs; with ``split_heads`` for calls that pass the same option."""
    lib = capi.load_library()
    if split_heads:
        return int(lib.gqa_bwd_workspace_bytes_ex(B, Hq, Hkv, S, D, int(bool(causal)), capi.GQA_BWD_SPLIT_HEADS))
    return int(lib.gqa_bwd_workspace_bytes(B, Hq, Hkv, S, D, int(bool(causal))))


def gqa_backward(q, k, v, o, do, lse, causal: bool = False, scale: float | None = None,
                 workspace=None, dq=None, dk=None, dv=None, stream=None, deterministic: bool = False,
                 layout: str = "bhsd", split_heads: bool = False, dq_separate: bool = False):
    """dQ, dK, dV.  Mirrors ``launch_gqa_backward_vj1d`` (G derived from the head counts).
    ``deterministic`` orders the dQ reductions (``GQA_BWD_DETERMINISTIC``): bit-reproducible dQ, slower.
    ``layout="bshd"``: all bf16 tensors are [B,S,H,D] (``GQA_LAYOUT_BSHD``); LSE is [B,Hq,S] either way.
    ``split_heads`` (``GQA_BWD_SPLIT_HEADS``): let a call with few KV tiles cut each tile's work over several thread
    blocks by query head (fp32 partial dK/dV, fixed-order sum); the workspace must be sized with the same option.
    ``dq_separate`` (``GQA_BWD_DQ_SEPARATE``): dQ from a separate query-parallel pass instead of the accumulator."""
    lib = capi.load_library()
    for t, n in ((q, "Q"), (k, "K"), (v, "V"), (o, "O"), (do, "dO")):
        _req(t, n, torch.bfloat16)
    _req(lse, "LSE", torch.float32)
    B, Hq, Hkv, S, D = _dims(q, k, layout)
    scale = 1.0 / math.sqrt(D) if scale is None else float(scale)
    need = bwd_workspace_bytes(B, Hq, Hkv, S, D, causal, split_heads)
    if need == 0:
        capi.check("gqa_bwd_workspace_bytes", -2)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
    dq = torch.empty_like(q) if dq is None else dq
    dk = torch.empty_like(k) if dk is None else dk
    dv = torch.empty_like(v) if dv is None else dv
    _req_like(v, "V", k)
    for t, n in ((o, "O"), (do, "dO"), (dq, "dQ")):
        _req_like(t, n, q)
    for t, n in ((dk, "dK"), (dv, "dV")):
        _req_like(t, n, k)
    _req_like(lse, "LSE", q, shape=(B, Hq, S), dtype=torch.float32)
    # its size is checked by the library (GQA_ERR_WORKSPACE, with the needed size in the error text)
    if not workspace.is_cuda or workspace.device != q.device or not workspace.is_contiguous():
        raise ValueError(f"workspace must be contiguous memory on {q.device}")
    with torch.cuda.device(q.device):
        args = (q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(),
                dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, Hq, Hkv, S, D, int(bool(causal)), scale,
                workspace.data_ptr(), workspace.numel() * workspace.element_size(), _stream_ptr(stream))
        flags = ((capi.GQA_BWD_DETERMINISTIC if deterministic else 0) | (capi.GQA_LAYOUT_BSHD if layout == "bshd" else 0)
                 | (capi.GQA_BWD_SPLIT_HEADS if split_heads else 0) | (capi.GQA_BWD_DQ_SEPARATE if dq_separate else 0))
        rc = lib.gqa_bwd_ex(*args, flags) if flags else lib.gqa_bwd(*args)
    capi.check("gqa_bwd_ex" if flags else "gqa_bwd", rc)
    return dq, dk, dv


def _packed_dims(q, k, cu_seqlens, max_seqlen):
    """Shapes of a packed variable-length batch: q [T,Hq,D], k [T,Hkv,D], cu_seqlens int32 [n_seqs+1] on the device."""
    if q.dim() != 3 or k.dim() != 3:
        raise ValueError("packed batches are [total_tokens, H, D]")
    T, Hq, D = q.shape
    if k.shape[0] != T or k.shape[2] != D:
        raise ValueError(f"K {tuple(k.shape)} does not match Q {tuple(q.shape)}")
    if (cu_seqlens.dtype != torch.int32 or cu_seqlens.dim() != 1 or cu_seqlens.numel() < 2 or not cu_seqlens.is_cuda
            or cu_seqlens.device != q.device or not cu_seqlens.is_contiguous()):
        raise ValueError(f"cu_seqlens must be a contiguous int32 vector of n_seqs + 1 entries on {q.device}")
    return T, Hq, k.shape[1], D, cu_seqlens.numel() - 1, int(max_seqlen)


def gqa_forward_varlen(q, k, v, cu_seqlens, max_seqlen: int, causal: bool = False, scale: float | None = None,
                       out=None, lse=None, stream=None):
    """O [T,Hq,D] and LSE [Hq,T] of a packed variable-length batch (``gqa_fwd_varlen``): sequence i is the rows
    cu_seqlens[i] .. cu_seqlens[i+1]-1 of q [T,Hq,D] and k, v [T,Hkv,D] and attends only to itself."""
    lib = capi.load_library()
    for t, n in ((q, "Q"), (k, "K"), (v, "V")):
        _req(t, n, torch.bfloat16)
    T, Hq, Hkv, D, n_seqs, max_seqlen = _packed_dims(q, k, cu_seqlens, max_seqlen)
    _req_like(v, "V", k)
    scale = 1.0 / math.sqrt(D) if scale is None else float(scale)
    out = torch.empty_like(q) if out is None else out
    lse = torch.empty(Hq, T, dtype=torch.float32, device=q.device) if lse is None else lse
    _req_like(out, "O", q)
    _req_like(lse, "LSE", q, shape=(Hq, T), dtype=torch.float32)
    with torch.cuda.device(q.device):
        rc = lib.gqa_fwd_varlen(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                cu_seqlens.data_ptr(), n_seqs, T, max_seqlen, Hq, Hkv, D, int(bool(causal)), scale,
                                _stream_ptr(stream))
    capi.check("gqa_fwd_varlen", rc)
    return out, lse


def bwd_varlen_workspace_bytes(total_tokens, Hq, Hkv, D) -> int:
    return int(capi.load_library().gqa_bwd_varlen_workspace_bytes(total_tokens, Hq, Hkv, D))


def gqa_backward_varlen(q, k, v, o, do, lse, cu_seqlens, max_seqlen: int, causal: bool = False,
                        scale: float | None = None, workspace=None, dq=None, dk=None, dv=None, stream=None):
    """dQ, dK, dV of a packed variable-length batch (``gqa_bwd_varlen``); tensors as in gqa_forward_varlen."""
    lib = capi.load_library()
    for t, n in ((q, "Q"), (k, "K"), (v, "V"), (o, "O"), (do, "dO")):
        _req(t, n, torch.bfloat16)
    _req(lse, "LSE", torch.float32)
    T, Hq, Hkv, D, n_seqs, max_seqlen = _packed_dims(q, k, cu_seqlens, max_seqlen)
    scale = 1.0 / math.sqrt(D) if scale is None else float(scale)
    need = bwd_varlen_workspace_bytes(T, Hq, Hkv, D)
    if need == 0:
        capi.check("gqa_bwd_varlen_workspace_bytes", -2)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
    dq = torch.empty_like(q) if dq is None else dq
    dk = torch.empty_like(k) if dk is None else dk
    dv = torch.empty_like(v) if dv is None else dv
    _req_like(v, "V", k)
    for t, n in ((o, "O"), (do, "dO"), (dq, "dQ")):
        _req_like(t, n, q)
    for t, n in ((dk, "dK"), (dv, "dV")):
        _req_like(t, n, k)
    _req_like(lse, "LSE", q, shape=(Hq, T), dtype=torch.float32)
    if not workspace.is_cuda or workspace.device != q.device or not workspace.is_contiguous():
        raise ValueError(f"workspace must be contiguous memory on {q.device}")
    with torch.cuda.device(q.device):
        rc = lib.gqa_bwd_varlen(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(),
                                dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), cu_seqlens.data_ptr(), n_seqs, T,
                                max_seqlen, Hq, Hkv, D, int(bool(causal)), scale, workspace.data_ptr(),
                                workspace.numel() * workspace.element_size(), _stream_ptr(stream))
    capi.check("gqa_bwd_varlen", rc)
    return dq, dk, dv


def bwd_stage_times(q, k, v, o, do, lse, causal, scale, workspace, dq, dk, dv, flush=None):
    """One backward with events around its stages; returns (preprocess_ms, main_ms, finalise_ms).
    `flush`, if given, is overwritten first so the working set starts outside L2."""
    import ctypes

    lib = capi.load_library()
    B, Hq, Hkv, S, D = _dims(q, k)
    if flush is not None:
        flush.zero_()
    ms = (ctypes.c_float * 3)()
    rc = lib.gqa_bwd_stage_times(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(),
                                 lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, Hq, Hkv, S, D,
                                 int(bool(causal)), float(scale), workspace.data_ptr(),
                                 workspace.numel() * workspace.element_size(), _stream_ptr(), ms)
    capi.check("gqa_bwd_stage_times", rc)
    return float(ms[0]), float(ms[1]), float(ms[2])


def gqa_delta(o, do, stream=None):
    """Delta = rowsum(dO * O) (stage 1 of the backward on its own)."""
    lib = capi.load_library()
    _req(o, "O", torch.bfloat16)
    _req(do, "dO", torch.bfloat16)
    D = o.shape[-1]
    rows = o.numel() // D
    out = torch.empty(o.shape[:-1], dtype=torch.float32, device=o.device)
    with torch.cuda.device(o.device):
        rc = lib.gqa_bwd_delta(o.data_ptr(), do.data_ptr(), out.data_ptr(), rows, D, _stream_ptr(stream))
    capi.check("gqa_bwd_delta", rc)
    return out


def check_status(workspace=None, stream=None) -> None:
    """Raise if a bounded device-side wait gave up in the last forward (``workspace=None``) or backward."""
    lib = capi.load_library()
    rc = lib.gqa_check_status(workspace.data_ptr() if workspace is not None else None, _stream_ptr(stream))
    capi.check("gqa_check_status", rc)


def checker_forward(q, k, v, causal=False, scale=None):
    """CUDA-core checker forward (diagnostics library; slow)."""
    lib = capi.load_selftest_library()
    B, Hq, Hkv, S, D = _dims(q, k)
    scale = 1.0 / math.sqrt(D) if scale is None else float(scale)
    out = torch.empty_like(q)
    lse = torch.empty((B, Hq, S), dtype=torch.float32, device=q.device)
    rc = lib.gqa_checker_fwd_simt(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                  B, Hq, Hkv, S, D, int(bool(causal)), scale, _stream_ptr())
    capi.check("gqa_checker_fwd_simt", rc)
    return out, lse


def checker_backward(q, k, v, o, do, lse, causal=False, scale=None):
    """CUDA-core checker backward (diagnostics library; slow)."""
    lib = capi.load_selftest_library()
    B, Hq, Hkv, S, D = _dims(q, k)
    scale = 1.0 / math.sqrt(D) if scale is None else float(scale)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    scratch = torch.empty((B, Hq, S), dtype=torch.float32, device=q.device)
    rc = lib.gqa_checker_bwd_simt(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(),
                                  lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), scratch.data_ptr(),
                                  B, Hq, Hkv, S, D, int(bool(causal)), scale, _stream_ptr())
    capi.check("gqa_checker_bwd_simt", rc)
    return dq, dk, dv


def selftest_umma(x, y, n: int, mode: int, use_tma: bool):
    """Run the UMMA building-block self test (diagnostics library); returns C [128, n] fp32."""
    lib = capi.load_selftest_library()
    c = torch.empty((128, n), dtype=torch.float32, device=x.device)
    rc = lib.gqa_selftest_umma(x.data_ptr(), y.data_ptr(), c.data_ptr(), n, mode, int(use_tma), _stream_ptr())
    capi.check("gqa_selftest_umma", rc)
    return c
