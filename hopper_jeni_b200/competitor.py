"""Plug-ins for the reference's Python benchmark harness.

The reference harness times attention implementations through two small duck-typed interfaces:

* forward  -- ``Competitor`` (harness/competitors.py:34-46): ``name``, ``role``, ``available(shape)``,
  ``forward(q, k, v, shape)``, ``make(q, k, v, shape)``; its slot for a user kernel is the stub
  ``YourKernel(so_path, entry="launch_gqa")`` (harness/competitors.py:396-415), which takes canonical
  ``[B,Hq,S,D]`` bf16 tensors and must return the same.
* backward -- ``BwdCompetitor`` (harness/run_gqa_bwd_v44_bench.py:181-194): ``available(shape)``,
  ``backward(q, k, v, do, shape) -> (dq, dk, dv)``, ``make_bwd(...)``; forward recomputation is part
  of what the harness times (run_gqa_bwd_v44_bench.py:12-13).

These classes implement both on top of the C ABI (``launch_gqa`` / ``gqa_fwd`` / ``gqa_bwd``).  They do
not import the harness: ``shape`` only needs ``B, Hq, Hkv, S, D, causal`` attributes, so the same object
works inside the reference harness (append an instance to its competitor list) and in this
repository's tests.
"""
from __future__ import annotations

import math
import os

import torch

from . import capi, ops


def _supported(shape):
    if shape.D not in (64, 128):
        return False, f"D={shape.D} not supported (64 or 128)"
    if shape.Hq % shape.Hkv:
        return False, "Hq is not a multiple of Hkv"
    if getattr(shape, "dtype", "bf16") != "bf16":
        return False, "bf16 only"
    if not torch.cuda.is_available() or torch.cuda.get_device_capability(0)[0] != 10:
        return False, "needs a compute-capability 10.x GPU"
    return True, ""


class YourKernel:
    """Forward plug-in: the filled-in version of the reference's ``YourKernel`` stub."""

    name = "yours"
    kind = "attention"
    role = "sm_100a tcgen05 GQA forward (this repository)"

    def __init__(self, so_path=None, entry="launch_gqa"):
        self.so_path = so_path or capi.lib_path()
        self.entry = entry
        self._fn = None

    def available(self, shape):
        if not os.path.exists(self.so_path):
            return False, f"{self.so_path} not found (build with `python -m hopper_jeni_b200.build`)"
        return _supported(shape)

    def _entry(self):
        if self._fn is None:
            import ctypes

            lib = ctypes.CDLL(self.so_path)
            fn = getattr(lib, self.entry)
            fn.restype, fn.argtypes = capi.EXPORTS["launch_gqa"]
            self._fn = fn
        return self._fn

    def forward(self, q, k, v, shape):
        o = torch.empty_like(q)
        lse = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device)
        rc = self._entry()(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                           shape.B, shape.Hq, shape.Hkv, shape.S, shape.D, int(bool(shape.causal)),
                           1.0 / math.sqrt(shape.D), int(torch.cuda.current_stream().cuda_stream))
        capi.check(self.entry, rc)
        return o

    def make(self, q, k, v, shape):
        return lambda: self.forward(q, k, v, shape)


class YourKernelBwd:
    """Backward plug-in.  ``backward`` recomputes the forward (as the harness's other entries do) and
    keeps its workspace between calls."""

    name = "yours_bwd"
    role = "sm_100a tcgen05 GQA backward (this repository)"

    def __init__(self):
        self._ws = None

    def available(self, shape):
        return _supported(shape)

    def backward(self, q, k, v, do, shape):
        scale = 1.0 / math.sqrt(shape.D)
        o, lse = ops.gqa_forward(q, k, v, causal=shape.causal, scale=scale)
        need = ops.bwd_workspace_bytes(shape.B, shape.Hq, shape.Hkv, shape.S, shape.D, shape.causal)
        if self._ws is None or self._ws.numel() < need or self._ws.device != q.device:
            self._ws = torch.empty(need, dtype=torch.uint8, device=q.device)
        return ops.gqa_backward(q, k, v, o, do, lse, causal=shape.causal, scale=scale, workspace=self._ws)

    def make_bwd(self, q, k, v, do, shape):
        return lambda: self.backward(q, k, v, do, shape)
