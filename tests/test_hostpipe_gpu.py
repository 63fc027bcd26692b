"""GPU test: the chunked host-buffer backward equals the device-resident backward (dK/dV bit-identical)."""
import pytest
import torch

import util
from hopper_jeni_b200 import ops
from hopper_jeni_b200.hostpipe import HostBackward

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("causal,chunks", [(False, 3), (True, 8)])
def test_host_pipeline_matches_device_run(gqa_lib, causal, chunks):
    B, Hq, Hkv, S, D = 3, 8, 2, 512, 64
    q, k, v, do = util.make_inputs(B, Hq, Hkv, S, D, seed=81)
    tq, tk, tv, tdo = (util.to_dev_bf16(x) for x in (q, k, v, do))
    o, lse = ops.gqa_forward(tq, tk, tv, causal=causal)
    dq, dk, dv = ops.gqa_backward(tq, tk, tv, o, tdo, lse, causal=causal)
    host_in = [t.cpu().pin_memory() for t in (tq, tk, tv, o, tdo, lse)]
    host_out = [torch.empty_like(t, device="cpu").pin_memory() for t in (dq, dk, dv)]
    pipe = HostBackward(B, Hq, Hkv, S, D, causal=causal, chunks=chunks)
    for _ in range(2):  # second call reuses the staging slots
        pipe(*host_in, *host_out)
        pipe.synchronize()
    assert torch.equal(host_out[1], dk.cpu()) and torch.equal(host_out[2], dv.cpu())
    util.assert_close_bf16(host_out[0].float().numpy(), util.to_np(dq), "dQ", util.REL_RMS_BWD)
