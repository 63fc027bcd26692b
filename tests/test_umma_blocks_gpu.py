"""GPU tests of the tensor-core building blocks (descriptor encodings, TMA panels, TMEM operands)."""
import numpy as np
import pytest
import torch

import util
from hopper_jeni_b200 import ops

pytestmark = pytest.mark.gpu


def _expected(x, y, n, mode):
    x = x.astype(np.float64)
    y = y.astype(np.float64)
    if mode in (0, 4):
        return x @ y[:n].T
    if mode == 6:
        return x @ y[:n].T + x[:, :16] @ y[:n, :16].T
    if mode in (1, 5):
        return x @ y[:, :n]
    if mode == 2:
        return x.T @ y[:n].T
    return x.T @ y[:, :n]


@pytest.mark.parametrize("use_tma", [False, True])
@pytest.mark.parametrize("n", [64, 128])
@pytest.mark.parametrize("mode", [0, 1, 2, 3, 4, 5, 6])
def test_umma_product(gqa_lib, mode, n, use_tma):
    rng = np.random.default_rng(100 + mode)
    x = util.bf16_round(rng.standard_normal((128, 128), dtype=np.float32))
    y = util.bf16_round(rng.standard_normal((128, 128), dtype=np.float32))
    c = ops.selftest_umma(util.to_dev_bf16(x), util.to_dev_bf16(y), n, mode, use_tma)
    torch.cuda.synchronize()
    want = _expected(x, y, n, mode)
    # exact products of bf16 values accumulated in fp32 over K = 128
    np.testing.assert_allclose(util.to_np(c), want, rtol=1e-4, atol=1e-3)


def test_issue_rate_probe(selftest_lib):
    """A lean warp-uniform issue loop keeps the tensor pipe busy: 128x128x16 products complete every
    ~64 cycles from one issuing warp, and two issuing warps share that rate (each sees ~128)."""
    import ctypes

    x = torch.randn(128, 128, device="cuda").bfloat16()
    y = torch.randn(128, 128, device="cuda").bfloat16()
    c = torch.empty(128, 128, device="cuda")
    out = {}
    for two in (0, 1):
        cy = ctypes.c_float()
        rc = selftest_lib.gqa_selftest_umma_cycles(x.data_ptr(), y.data_ptr(), c.data_ptr(), 128, 0, 64, two,
                                              ctypes.byref(cy), None)
        assert rc == 0
        out[two] = cy.value
    assert 60.0 < out[0] < 100.0, out
    assert out[1] < 2.3 * out[0], out
