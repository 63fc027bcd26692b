"""GPU test of gqa_bwd_static_scratch, the backward for callers that are not allowed to allocate
device memory (a plugin that only receives its input/output buffers, code inside a memory-planned
region of a framework, a latency-critical loop).  It must give the same gradients as gqa_bwd, which
takes a caller-provided workspace, on two calls in a row -- the second call finds the built-in
scratch array dirty from the first -- and must refuse shapes whose scratch does not fit the array.

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test.  It passes alone in a fresh process as well (the first call does the one-time address
look-up of the array).
"""
import ctypes

import pytest
import torch

import util
from hopper_jeni_b200 import capi, ops

pytestmark = pytest.mark.gpu


def _call_static(lib, q, k, v, o, do, lse, dq, dk, dv, causal, scale):
    B, Hq, S, D = q.shape
    return lib.gqa_bwd_static_scratch(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(),
                                      lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                      B, Hq, k.shape[1], S, D, int(causal), float(scale),
                                      int(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("shape,causal", [((2, 6, 2, 512, 64), False), ((1, 4, 2, 384, 128), True)])
def test_static_scratch_backward_matches_gqa_bwd_twice(gqa_lib, shape, causal):
    B, Hq, Hkv, S, D = shape
    sc = util.default_scale(D)
    for call in range(2):  # second call: different inputs, scratch array still holds the first call's data
        q, k, v, do = util.make_inputs(B, Hq, Hkv, S, D, seed=71 + call)
        tq, tk, tv, tdo = (util.to_dev_bf16(x) for x in (q, k, v, do))
        o, lse = ops.gqa_forward(tq, tk, tv, causal=causal, scale=sc)
        ws = torch.empty(ops.bwd_workspace_bytes(B, Hq, Hkv, S, D, causal), dtype=torch.uint8, device="cuda")
        dq_ref, dk_ref, dv_ref = ops.gqa_backward(tq, tk, tv, o, tdo, lse, causal=causal, scale=sc, workspace=ws)
        ops.check_status(ws)
        dq = torch.full_like(tq, float("nan"))
        dk = torch.full_like(tk, float("nan"))
        dv = torch.full_like(tv, float("nan"))
        torch.cuda.synchronize()
        # Device-wide free memory as the driver reports it: unlike torch's allocator statistics it also sees
        # a cudaMalloc made inside the library.  Nothing else allocates between the two readings (the call
        # takes raw pointers; the first call's address look-up of the scratch array allocates nothing).
        free_before, _ = torch.cuda.mem_get_info()
        rc = _call_static(gqa_lib, tq, tk, tv, o, tdo, lse, dq, dk, dv, causal, sc)
        capi.check("gqa_bwd_static_scratch", rc)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        # Checked on the second call: the first one may make the driver load the library's device code and the
        # scratch array itself onto the GPU (lazy module loading), which is not an allocation made by the call.
        if call == 1:
            assert free_after >= free_before, f"device memory shrank by {free_before - free_after} bytes during the call"
        # dK and dV have one writer per element in both entry points: identical bits.  dQ is summed with
        # fp32 reductions at L2 in an order that changes from run to run: the bf16 parity tolerance applies.
        assert torch.equal(dk, dk_ref) and torch.equal(dv, dv_ref)
        util.assert_close_bf16(util.to_np(dq), util.to_np(dq_ref), "dQ", util.REL_RMS_BWD)


def test_static_scratch_backward_refuses_oversized_shapes(gqa_lib):
    cap = gqa_lib.gqa_bwd_static_scratch_bytes()
    assert cap == 32 << 20
    B, Hq, Hkv, S, D = 8, 12, 4, 4096, 64          # needs about 104 MB of scratch
    assert gqa_lib.gqa_bwd_workspace_bytes(B, Hq, Hkv, S, D, 0) > cap
    p = ctypes.c_void_p(4096)                       # never dereferenced: the size check comes first
    rc = gqa_lib.gqa_bwd_static_scratch(p, p, p, p, p, p, p, p, p, B, Hq, Hkv, S, D, 0, 0.125, None)
    assert rc == -3
    assert b"built-in array" in gqa_lib.gqa_last_cuda_error()
