"""CPU tests of the drop-in boundary: the library loads, exports every symbol include/gqa.h declares,
and rejects bad arguments with status codes before touching a device."""
import ctypes
import os
import re

import pytest

from hopper_jeni_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols(header="gqa.h"):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gqa_[a-z0-9_]+|launch_gqa)\s*\(", text)))


def test_header_and_binding_agree():
    assert _declared_symbols() == sorted(capi.EXPORTS)
    assert _declared_symbols("gqa_selftest.h") == sorted(capi.SELFTEST_EXPORTS)
    assert not set(capi.EXPORTS) & set(capi.SELFTEST_EXPORTS)


def test_library_exports_every_declared_symbol(gqa_lib, selftest_lib):
    for name in _declared_symbols():
        assert hasattr(gqa_lib, name), name
    for name in _declared_symbols("gqa_selftest.h"):
        assert hasattr(selftest_lib, name), name
        assert not hasattr(gqa_lib, name), f"{name}: diagnostics must not be exported by the product library"


def test_version_and_status_strings(gqa_lib):
    assert gqa_lib.gqa_version().decode().count(".") == 1
    for code in range(0, -7, -1):
        assert gqa_lib.gqa_status_string(code)
    assert gqa_lib.gqa_status_string(-99).decode() == "unknown status"


def test_workspace_bytes_formula(gqa_lib):
    B, Hq, Hkv, S, D = 8, 12, 4, 4096, 64
    rows = B * Hq * S
    need = gqa_lib.gqa_bwd_workspace_bytes(B, Hq, Hkv, S, D, 0)
    assert need >= rows * D * 4 + 2 * rows * 4 + 256
    assert need % 256 == 0
    # unsupported shapes report zero
    assert gqa_lib.gqa_bwd_workspace_bytes(B, Hq, Hkv, S, 100, 0) == 0        # rows must be multiples of 16 bytes
    assert gqa_lib.gqa_bwd_workspace_bytes(B, Hq, Hkv, S, 136, 0) == 0
    # other head dimensions run on the next native size up: the accumulator rows are padded to it
    assert gqa_lib.gqa_bwd_workspace_bytes(B, Hq, Hkv, S, 96, 0) == gqa_lib.gqa_bwd_workspace_bytes(B, Hq, Hkv, S, 128, 0)
    assert gqa_lib.gqa_bwd_workspace_bytes(B, Hq, Hkv, S, 40, 0) == need
    assert gqa_lib.gqa_bwd_workspace_bytes(B, Hq, Hkv, S + 60, D, 0) > need   # any S: partial tiles are masked
    assert gqa_lib.gqa_bwd_workspace_bytes(B, 10, 4, S, D, 0) == 0
    # with GQA_BWD_SPLIT_HEADS (4) the query covers the fp32 partial sums of shapes that are split: a shape with
    # plenty of KV tiles is not, one KV head of a long causal problem is
    assert gqa_lib.gqa_bwd_workspace_bytes_ex(B, Hq, Hkv, S, D, 0, 4) == need
    one_head = gqa_lib.gqa_bwd_workspace_bytes(1, 8, 1, 32768, 128, 1)
    assert gqa_lib.gqa_bwd_workspace_bytes_ex(1, 8, 1, 32768, 128, 1, 4) > one_head
    assert gqa_lib.gqa_bwd_workspace_bytes_ex(1, 8, 1, 32768, 128, 1, 64) == 0      # unknown flag


def test_argument_validation_needs_no_device(gqa_lib, selftest_lib):
    p = ctypes.c_void_p(4096)  # never dereferenced: validation fails first
    assert gqa_lib.gqa_fwd(None, p, p, p, None, 1, 4, 2, 128, 64, 0, 0.125, None) == -1
    assert gqa_lib.gqa_fwd(p, p, p, p, None, 1, 4, 2, 0, 64, 0, 0.125, None) == -1        # S <= 0
    assert gqa_lib.gqa_fwd(p, p, p, p, None, 1, 4, 2, 128, 100, 0, 0.125, None) == -2     # D % 8
    assert gqa_lib.gqa_fwd(p, p, p, p, None, 1, 4, 2, 128, 136, 0, 0.125, None) == -2     # D > 128
    assert gqa_lib.gqa_fwd_ex(p, p, p, p, None, 1, 4, 2, 128, 96, 0, 0.125, None, 2) == -2  # [B,S,H,D] needs D = 64 / 128
    assert gqa_lib.gqa_fwd(p, p, p, p, None, 1, 5, 2, 128, 64, 0, 0.125, None) == -2      # Hq % Hkv
    assert gqa_lib.gqa_fwd(p, p, p, p, None, 0, 4, 2, 128, 64, 0, 0.125, None) == -1      # B <= 0
    mis = ctypes.c_void_p(4096 + 2)
    assert gqa_lib.gqa_fwd(mis, p, p, p, None, 1, 4, 2, 128, 64, 0, 0.125, None) == -1    # misaligned
    assert gqa_lib.gqa_bwd(p, p, p, p, p, p, p, p, p, 1, 4, 2, 128, 64, 0, 0.125, None, 0, None) == -3
    assert gqa_lib.gqa_bwd(p, p, p, p, p, p, p, p, p, 1, 4, 2, 128, 64, 0, 0.125, p, 16, None) == -3
    assert gqa_lib.gqa_bwd(p, p, p, p, p, None, p, p, p, 1, 4, 2, 128, 64, 0, 0.125, p, 1 << 30, None) == -1
    assert gqa_lib.gqa_fwd(p, p, p, p, None, 1, 4, 2, 128, 64, 0, 0.0, None) == -1        # scale must be > 0
    assert gqa_lib.gqa_fwd(p, p, p, p, None, 1, 4, 2, 128, 64, 0, float("inf"), None) == -1
    assert gqa_lib.gqa_bwd(p, p, p, p, p, p, p, p, p, 1, 4, 2, 128, 64, 0, -0.125, p, 1 << 30, None) == -1
    assert selftest_lib.gqa_selftest_umma(p, p, p, 96, 0, 0, None) == -2
    assert selftest_lib.gqa_selftest_umma_cycles(p, p, p, 128, 0, 1 << 20, 0, None, None) == -1  # reps capped
    assert selftest_lib.gqa_selftest_timeout(p, 10 ** 10, 1, None) == -1                           # limit capped
    assert selftest_lib.gqa_selftest_timeout(None, 1000, 1, None) == -1
    assert gqa_lib.gqa_bwd_delta(p, p, p, 16, 36, None) == -2
    # packed variable-length batches: (..., cu_seqlens, n_seqs, total_tokens, max_seqlen, Hq, Hkv, D, causal, scale, ...)
    assert gqa_lib.gqa_fwd_varlen(p, p, p, p, None, None, 2, 256, 128, 4, 2, 64, 0, 0.125, None) == -1   # no cu_seqlens
    assert gqa_lib.gqa_fwd_varlen(p, p, p, p, None, p, 0, 256, 128, 4, 2, 64, 0, 0.125, None) == -1      # n_seqs <= 0
    assert gqa_lib.gqa_fwd_varlen(p, p, p, p, None, p, 2, 256, 0, 4, 2, 64, 0, 0.125, None) == -1        # max_seqlen <= 0
    assert gqa_lib.gqa_fwd_varlen(p, p, p, p, None, p, 2, 256, 300, 4, 2, 64, 0, 0.125, None) == -1      # ... > total
    assert gqa_lib.gqa_fwd_varlen(p, p, p, p, None, mis, 2, 256, 128, 4, 2, 64, 0, 0.125, None) == -1    # misaligned
    assert gqa_lib.gqa_fwd_varlen(p, p, p, p, None, p, 2, 256, 128, 4, 2, 96, 0, 0.125, None) == -2      # D = 64 / 128 only
    assert gqa_lib.gqa_fwd_varlen(p, p, p, p, None, p, 2, 256, 128, 5, 2, 64, 0, 0.125, None) == -2      # Hq % Hkv
    assert gqa_lib.gqa_bwd_varlen(p, p, p, p, p, p, p, p, p, p, 2, 256, 128, 4, 2, 64, 0, 0.125, p, 16, None) == -3
    assert gqa_lib.gqa_bwd_varlen(p, p, p, p, p, p, p, p, p, None, 2, 256, 128, 4, 2, 64, 0, 0.125, p, 1 << 30, None) == -1
    assert gqa_lib.gqa_bwd_varlen_workspace_bytes(256, 4, 2, 96) == 0
    assert gqa_lib.gqa_bwd_varlen_workspace_bytes(256, 4, 2, 64) == gqa_lib.gqa_bwd_workspace_bytes(1, 4, 2, 256, 64, 0)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setenv("GQA_B200_LIB", str(tmp_path / "nope.so"))
    monkeypatch.setattr(capi, "_LIB", None)
    with pytest.raises(FileNotFoundError):
        capi.load_library()


def test_ops_refuse_cpu_tensors():
    import torch

    import hopper_jeni_b200 as pkg

    q = torch.zeros(1, 2, 128, 64, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        pkg.gqa_forward(q, q, q)
