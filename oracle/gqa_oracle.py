"""ctypes front-end of the C oracle in ``gqa_ref.c``.

TEST INFRASTRUCTURE ONLY.  The oracle is the checker for the CUDA path (tests,
the smoke check, and the bench's CPU-baseline leg); the product package never
imports it.  Arrays are numpy float32, contiguous, in the reference layout
``[B, H, S, D]`` (precision/baseline_gqa.py:10-17).

``forward``/``backward`` follow ``fp64_reference`` / ``fp64_backward`` of the
reference (precision/baseline_gqa.py:40-61, :169-197); ``numpy_forward`` /
``numpy_backward`` are an independent dense restatement used to cross-check the C
code on small cases.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libgqa_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile ``gqa_ref.c`` into ``libgqa_oracle.so`` with gcc (idempotent)."""
    src = os.path.join(_HERE, "gqa_ref.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libgqa_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        build()
        lib = ctypes.CDLL(_LIB_PATH)
        fp = ctypes.POINTER(ctypes.c_float)
        i = ctypes.c_int
        lib.gqa_oracle_forward.argtypes = [fp, fp, fp, i, i, i, i, i, i, ctypes.c_float, fp, fp]
        lib.gqa_oracle_forward.restype = i
        lib.gqa_oracle_backward.argtypes = [fp, fp, fp, fp, i, i, i, i, i, i, ctypes.c_float, fp, fp, fp]
        lib.gqa_oracle_backward.restype = i
        lib.gqa_oracle_delta.argtypes = [fp, fp, ctypes.c_size_t, i, fp]
        lib.gqa_oracle_delta.restype = i
        lib.gqa_oracle_threads.restype = i
        _lib = lib
    return _lib


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def threads() -> int:
    return int(_load().gqa_oracle_threads())


def forward(q, k, v, causal: bool, scale: float):
    """Return (O [B,Hq,S,D], LSE [B,Hq,S]) as float32 from double accumulation."""
    lib = _load()
    q, qp = _f32(q); k, kp = _f32(k); v, vp = _f32(v)
    B, Hq, S, D = q.shape
    Hkv = k.shape[1]
    o = np.empty_like(q)
    lse = np.empty((B, Hq, S), dtype=np.float32)
    rc = lib.gqa_oracle_forward(qp, kp, vp, B, Hq, Hkv, S, D, int(causal), float(scale),
                                o.ctypes.data_as(ctypes.POINTER(ctypes.c_float)),
                                lse.ctypes.data_as(ctypes.POINTER(ctypes.c_float)))
    if rc != 0:
        raise RuntimeError(f"gqa_oracle_forward failed: {rc}")
    return o, lse


def backward(q, k, v, dout, causal: bool, scale: float):
    """Return (dQ, dK, dV) as float32 from double accumulation."""
    lib = _load()
    q, qp = _f32(q); k, kp = _f32(k); v, vp = _f32(v); dout, dp = _f32(dout)
    B, Hq, S, D = q.shape
    Hkv = k.shape[1]
    dq = np.empty_like(q); dk = np.empty_like(k); dv = np.empty_like(v)
    pf = ctypes.POINTER(ctypes.c_float)
    rc = lib.gqa_oracle_backward(qp, kp, vp, dp, B, Hq, Hkv, S, D, int(causal), float(scale),
                                 dq.ctypes.data_as(pf), dk.ctypes.data_as(pf), dv.ctypes.data_as(pf))
    if rc != 0:
        raise RuntimeError(f"gqa_oracle_backward failed: {rc}")
    return dq, dk, dv


def delta(o, dout):
    """Delta[b,h,s] = sum_d dO*O (precision/baseline_gqa.py:189)."""
    lib = _load()
    o, op = _f32(o); dout, dp = _f32(dout)
    rows = int(np.prod(o.shape[:-1]))
    out = np.empty(o.shape[:-1], dtype=np.float32)
    lib.gqa_oracle_delta(op, dp, rows, o.shape[-1], out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)))
    return out


# ---- independent dense numpy restatement (small cases only) -----------------

def _scores(q, k, causal, scale, G):
    kk = np.repeat(k.astype(np.float64), G, axis=1)
    s = np.einsum("bhid,bhjd->bhij", q.astype(np.float64), kk) * scale
    if causal:
        S = q.shape[2]
        s = np.where(np.tril(np.ones((S, S), dtype=bool)), s, -np.inf)
    return s


def numpy_forward(q, k, v, causal: bool, scale: float):
    G = q.shape[1] // k.shape[1]
    s = _scores(q, k, causal, scale, G)
    m = s.max(-1, keepdims=True)
    e = np.exp(s - m)
    l = e.sum(-1, keepdims=True)
    p = e / l
    o = np.einsum("bhij,bhjd->bhid", p, np.repeat(v.astype(np.float64), G, axis=1))
    return o.astype(np.float32), (m + np.log(l))[..., 0].astype(np.float32)


def numpy_backward(q, k, v, dout, causal: bool, scale: float):
    B, Hq, S, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    s = _scores(q, k, causal, scale, G)
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    vv = np.repeat(v.astype(np.float64), G, axis=1)
    kk = np.repeat(k.astype(np.float64), G, axis=1)
    do = dout.astype(np.float64)
    o = np.einsum("bhij,bhjd->bhid", p, vv)
    di = (do * o).sum(-1, keepdims=True)
    dp = np.einsum("bhid,bhjd->bhij", do, vv)
    ds = p * (dp - di)
    dq = np.einsum("bhij,bhjd->bhid", ds, kk) * scale
    dk = (np.einsum("bhij,bhid->bhjd", ds, q.astype(np.float64)) * scale).reshape(B, Hkv, G, S, D).sum(2)
    dv = np.einsum("bhij,bhid->bhjd", p, do).reshape(B, Hkv, G, S, D).sum(2)
    return dq.astype(np.float32), dk.astype(np.float32), dv.astype(np.float32)
