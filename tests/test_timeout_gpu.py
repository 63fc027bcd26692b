"""GPU test of the give-up path of the bounded device-side waits.  The reference's waits spin without limit
(src/attention/GQA_bwd_baseline.cu:85-93): a protocol bug there hangs the GPU.  Here every wait has a limit, and
this test makes one run out on purpose -- safely: a self-test kernel waits, with a limit of about a millisecond,
on a barrier that nothing arrives at, then takes the same abort-flag / status-word / teardown path as the attention
kernels.  Nothing faults, traps or waits without a limit; the device must be fully usable afterwards."""
import time

import numpy as np
import pytest
import torch

import util
from hopper_jeni_b200 import capi, ops

pytestmark = pytest.mark.gpu


def test_bounded_wait_gives_up_reports_and_leaves_the_device_usable(gqa_lib, selftest_lib, oracle):
    stream = int(torch.cuda.current_stream().cuda_stream)
    word = torch.zeros(64, dtype=torch.int32, device="cuda")
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    blocks = min(1024, 3 * sms)              # three waves at one thread block per SM
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    rc = selftest_lib.gqa_selftest_timeout(word.data_ptr(), 2_000_000, blocks, stream)   # ~1 ms of SM cycles
    assert rc == 0, capi.STATUS_NAMES.get(rc, rc)
    rc = gqa_lib.gqa_check_status(word.data_ptr(), stream)
    elapsed = time.perf_counter() - t0
    assert rc == -5, f"expected GQA_ERR_DEVICE_TIMEOUT, got {capi.STATUS_NAMES.get(rc, rc)}"
    text = gqa_lib.gqa_last_cuda_error().decode()
    assert "wait site 7 gave up in block" in text, text
    with pytest.raises(capi.GqaError) as e:
        capi.check("gqa_check_status", rc)
    assert e.value.status == -5 and "timed out" in str(e.value)
    # the first wave waits out its limit; the later waves find the status word set and leave at once
    host = word.cpu().numpy().view(np.uint32)
    assert host[0] >> 31 == 1 and (host[0] >> 20) & 0x7FF == 7
    assert blocks - 2 * sms <= int(host[1]) <= blocks - 1, (int(host[1]), blocks, sms)
    assert elapsed < 1.0, f"the give-up path took {elapsed:.2f} s"

    # the context is intact: a forward + backward right after it still matches the oracle
    B, Hq, Hkv, S, D = 1, 4, 2, 256, 64
    q, k, v, do = util.make_inputs(B, Hq, Hkv, S, D, seed=9)
    sc = util.default_scale(D)
    tq, tk, tv, tdo = (util.to_dev_bf16(x) for x in (q, k, v, do))
    o, lse = ops.gqa_forward(tq, tk, tv, causal=True, scale=sc)
    ops.check_status()
    dq, dk, dv = ops.gqa_backward(tq, tk, tv, o, tdo, lse, causal=True, scale=sc)
    o_ref, _ = oracle.forward(q, k, v, True, sc)
    dq_ref, dk_ref, dv_ref = oracle.backward(q, k, v, do, True, sc)
    util.assert_close_bf16(util.to_np(o), o_ref, "O", util.REL_RMS_FWD)
    util.assert_close_bf16(util.to_np(dq), dq_ref, "dQ", util.REL_RMS_BWD)
    util.assert_close_bf16(util.to_np(dk), dk_ref, "dK", util.REL_RMS_BWD)
    util.assert_close_bf16(util.to_np(dv), dv_ref, "dV", util.REL_RMS_BWD)


def test_timeout_selftest_refuses_long_limits(selftest_lib):
    word = torch.zeros(64, dtype=torch.int32, device="cuda")
    assert selftest_lib.gqa_selftest_timeout(word.data_ptr(), 10 ** 9, 1, None) == -1      # > 0.1 s of cycles
    assert selftest_lib.gqa_selftest_timeout(word.data_ptr(), 1000, 5000, None) == -1      # too many blocks
