"""ctypes binding of the C ABI declared in ``include/gqa.h`` (``libgqa_b200.so``, the product) and in
``include/gqa_selftest.h`` (``libgqa_b200_selftest.so``, diagnostics used by the test-suite only).

Signatures here must stay in lock-step with those headers; ``EXPORTS`` / ``SELFTEST_EXPORTS`` list every
symbol each header declares and the test-suite checks that the built libraries export each of them.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_SELFTEST_LIB = None

GQA_OK = 0
GQA_BWD_DETERMINISTIC = 1
GQA_LAYOUT_BSHD = 2
GQA_BWD_SPLIT_HEADS = 4
GQA_BWD_DQ_SEPARATE = 8
STATUS_NAMES = {
    0: "GQA_OK", -1: "GQA_ERR_BAD_ARGUMENT", -2: "GQA_ERR_UNSUPPORTED", -3: "GQA_ERR_WORKSPACE",
    -4: "GQA_ERR_CUDA", -5: "GQA_ERR_DEVICE_TIMEOUT", -6: "GQA_ERR_ARCH",
}

_vp, _fp, _i, _f, _sz = ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t

#: symbol -> (restype, argtypes); one entry per declaration in include/gqa.h
EXPORTS = {
    "gqa_fwd": (_i, [_vp, _vp, _vp, _vp, _fp, _i, _i, _i, _i, _i, _i, _f, _vp]),
    "gqa_fwd_ex": (_i, [_vp, _vp, _vp, _vp, _fp, _i, _i, _i, _i, _i, _i, _f, _vp, ctypes.c_uint]),
    "launch_gqa": (_i, [_vp, _vp, _vp, _vp, _fp, _i, _i, _i, _i, _i, _i, _f, _vp]),
    "gqa_bwd_workspace_bytes": (_sz, [_i, _i, _i, _i, _i, _i]),
    "gqa_bwd_workspace_bytes_ex": (_sz, [_i, _i, _i, _i, _i, _i, ctypes.c_uint]),
    "gqa_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _fp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp, _sz, _vp]),
    "gqa_bwd_ex": (_i, [_vp, _vp, _vp, _vp, _vp, _fp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp, _sz, _vp,
                        ctypes.c_uint]),
    "gqa_fwd_varlen": (_i, [_vp, _vp, _vp, _vp, _fp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _vp]),
    "gqa_bwd_varlen_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "gqa_bwd_varlen": (_i, [_vp, _vp, _vp, _vp, _vp, _fp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _sz,
                            _vp]),
    "gqa_bwd_static_scratch_bytes": (_sz, []),
    "gqa_bwd_static_scratch": (_i, [_vp, _vp, _vp, _vp, _vp, _fp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp]),
    "gqa_bwd_stage_times": (_i, [_vp, _vp, _vp, _vp, _vp, _fp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp, _sz,
                                 _vp, ctypes.POINTER(ctypes.c_float)]),
    "gqa_bwd_delta": (_i, [_vp, _vp, _fp, _sz, _i, _vp]),
    "gqa_check_status": (_i, [_vp, _vp]),
    "gqa_status_string": (ctypes.c_char_p, [_i]),
    "gqa_last_cuda_error": (ctypes.c_char_p, []),
    "gqa_launch_count": (ctypes.c_ulonglong, []),
    "gqa_version": (ctypes.c_char_p, []),
}

#: symbol -> (restype, argtypes); one entry per declaration in include/gqa_selftest.h
SELFTEST_EXPORTS = {
    "gqa_selftest_umma": (_i, [_vp, _vp, _fp, _i, _i, _i, _vp]),
    "gqa_selftest_umma_cycles": (_i, [_vp, _vp, _fp, _i, _i, _i, _i, ctypes.POINTER(ctypes.c_float), _vp]),
    "gqa_checker_fwd_simt": (_i, [_vp, _vp, _vp, _vp, _fp, _i, _i, _i, _i, _i, _i, _f, _vp]),
    "gqa_checker_bwd_simt": (_i, [_vp, _vp, _vp, _vp, _vp, _fp, _vp, _vp, _vp, _fp,
                                  _i, _i, _i, _i, _i, _i, _f, _vp]),
    "gqa_selftest_timeout": (_i, [_vp, ctypes.c_longlong, _i, _vp]),
}


class GqaError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, fn: str, status: int, detail: str = ""):
        self.status = status
        name = STATUS_NAMES.get(status, str(status))
        super().__init__(f"{fn} failed with {name}" + (f": {detail}" if detail else ""))


def lib_path() -> str:
    return os.environ.get("GQA_B200_LIB", os.path.join(_HERE, "libgqa_b200.so"))


def load_library():
    """Load ``libgqa_b200.so``; raises if it has not been built (there is no fallback path)."""
    global _LIB
    if _LIB is None:
        path = lib_path()
        if not os.path.exists(path):
            raise FileNotFoundError(
                f"{path} not found: build it with `python -m hopper_jeni_b200.build` (needs nvcc); "
                "this package has no CPU or framework fallback")
        lib = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
        for name, (res, args) in EXPORTS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _LIB = lib
    return _LIB


def selftest_lib_path() -> str:
    return os.path.join(os.path.dirname(lib_path()), "libgqa_b200_selftest.so")


def load_selftest_library():
    """Load the diagnostics library (checker kernels, self tests); it links against the product library."""
    global _SELFTEST_LIB
    if _SELFTEST_LIB is None:
        load_library()  # resolves its dependency and fails first if the product is missing
        path = selftest_lib_path()
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path} not found: build it with `python -m hopper_jeni_b200.build`")
        lib = ctypes.CDLL(path)
        for name, (res, args) in SELFTEST_EXPORTS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _SELFTEST_LIB = lib
    return _SELFTEST_LIB


def check(fn: str, status: int) -> None:
    if status != GQA_OK:
        lib = load_library()
        detail = lib.gqa_status_string(status).decode()
        if status in (-3, -4, -5):
            detail += " | " + lib.gqa_last_cuda_error().decode()
        raise GqaError(fn, status, detail)
