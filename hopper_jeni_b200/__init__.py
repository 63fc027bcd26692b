"""Blackwell (sm_100a) grouped-query attention: forward and three-stage backward behind a C ABI.

The compute lives in ``libgqa_b200.so`` (hand-written CUDA: tcgen05 MMA, TMEM accumulators, TMA-fed
swizzled shared memory).  This package is the thin host side: a ctypes binding of the C ABI
(:mod:`.capi`), tensor-level wrappers (:mod:`.ops`), the work sharding used on multi-GPU nodes
(:mod:`.sharding`) and the build helper (:mod:`.build`).  There is no CPU fallback: every operator
raises if the library or a CUDA device is missing.
"""
from .capi import GqaError, lib_path, load_library  # noqa: F401
from .ops import (  # noqa: F401
    bwd_varlen_workspace_bytes,
    bwd_workspace_bytes,
    gqa_backward,
    gqa_backward_varlen,
    gqa_delta,
    gqa_forward,
    gqa_forward_varlen,
    launch_count,
)

__all__ = ["GqaError", "lib_path", "load_library", "gqa_forward", "gqa_backward", "gqa_delta",
           "bwd_workspace_bytes", "launch_count", "gqa_forward_varlen", "gqa_backward_varlen",
           "bwd_varlen_workspace_bytes"]
