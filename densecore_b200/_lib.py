"""ctypes loader for libdc_b200.so (the C ABI declared in include/dc_b200.h).

There is no fallback: if the shared library is missing the import of any op
fails with an error that says how to build it.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libdc_b200.so")

OK = 0
STATUS_NAMES = {
    0: "OK", -1: "INVALID_ARGUMENT", -2: "MODEL_LOAD_FAILED", -3: "OUT_OF_MEMORY",
    -5: "INTERNAL_ERROR", -6: "BACKEND_ERROR", -7: "UNSUPPORTED",
}


class DcError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"dc_b200 status {status} ({STATUS_NAMES.get(status, '?')}): {message}")
        self.status = status
        self.message = message


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m densecore_b200.build` "
                "(needs nvcc; there is no CPU fallback)")
        _lib = C.CDLL(LIB_PATH)
        _declare(_lib)
    return _lib


def _declare(l: C.CDLL) -> None:
    vp, i32, i64, sz = C.c_void_p, C.c_int, C.c_int64, C.c_size_t
    pp = C.POINTER(C.c_void_p)
    sigs = {
        "dc_b200_init": (i32, [i32, pp]),
        "dc_b200_destroy": (None, [vp]),
        "dc_b200_last_error": (C.c_char_p, [vp]),
        "dc_b200_stream": (vp, [vp]),
        "dc_b200_synchronize": (i32, [vp]),
        "dc_b200_set_option": (i32, [vp, C.c_char_p, i32]),
        "dc_b200_upload_weight": (i32, [vp, i32, C.POINTER(i64), vp, pp]),
        "dc_b200_free_weight": (i32, [vp, vp]),
        "dc_b200_weight_data": (vp, [vp, C.POINTER(sz)]),
        "dc_b200_quantize_q8k": (i32, [vp, vp, i32, i32, vp]),
        "dc_b200_quantize_q8k_dev": (i32, [vp, vp, i32, i32, vp]),
        "dc_b200_mul_mat": (i32, [vp, vp, vp, i32, vp]),
        "dc_b200_mul_mat_dev": (i32, [vp, vp, vp, i32, vp]),
        "dc_b200_mul_mat_block_sums": (i32, [vp, vp, vp, i32, vp, vp]),
    }
    sigs.update(_EXTRA_SIGS)
    for name, (res, args) in sigs.items():
        fn = getattr(l, name)
        fn.restype = res
        fn.argtypes = args


_EXTRA_SIGS: dict = {}


def exported_symbols() -> list[str]:
    """Names this binding expects the library to export (checked by the CPU tests)."""
    base = ["dc_b200_init", "dc_b200_destroy", "dc_b200_last_error", "dc_b200_stream", "dc_b200_synchronize",
            "dc_b200_set_option", "dc_b200_upload_weight", "dc_b200_free_weight", "dc_b200_weight_data",
            "dc_b200_quantize_q8k", "dc_b200_quantize_q8k_dev", "dc_b200_mul_mat", "dc_b200_mul_mat_dev",
            "dc_b200_mul_mat_block_sums"]
    return base + list(_EXTRA_SIGS)
