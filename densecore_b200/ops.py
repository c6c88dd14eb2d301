"""Host-side mirror of the reference's op interface over the C ABI.

Names follow the ggml ops the reference's custom-op callbacks implement:
mul_mat (cb_gemv_custom / cb_gemv_batched_custom), mul_mat_id (cb_moe_forward),
flash_attn_decode (cb_paged_attention_decode), verify_accept.  All arrays are
numpy host arrays; every call goes through libdc_b200.so.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from .blocks import BLOCK_BYTES, GGML_TYPE_Q4_K, GGML_TYPE_Q6_K, Q8K_BYTES, QK_K, row_bytes


def _vp(a: np.ndarray | None):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


class Weight:
    """Handle of a GGUF tensor resident in HBM in its native block bytes."""

    def __init__(self, ctx: "Context", handle: int, ggml_type: int, K: int, N: int, E: int):
        self.ctx, self.handle, self.type, self.K, self.N, self.E = ctx, handle, ggml_type, K, N, E

    @property
    def nbytes(self) -> int:
        return row_bytes(self.type, self.K) * self.N * self.E

    def free(self):
        if self.handle:
            self.ctx._check(_lib.lib().dc_b200_free_weight(self.ctx.handle, self.handle))
            self.handle = None


class Context:
    """One GPU, one stream (dc_b200_init)."""

    def __init__(self, device: int = 0):
        self.handle = None
        h = C.c_void_p()
        st = _lib.lib().dc_b200_init(int(device), C.byref(h))
        if st != 0:
            raise _lib.DcError(st, "dc_b200_init failed (no CPU fallback exists)")
        self.handle = h
        self.device = device

    def close(self):
        if self.handle:
            _lib.lib().dc_b200_destroy(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def last_error(self) -> str:
        return (_lib.lib().dc_b200_last_error(self.handle) or b"").decode()

    def _check(self, st: int):
        if st != 0:
            raise _lib.DcError(st, self.last_error())

    def synchronize(self):
        self._check(_lib.lib().dc_b200_synchronize(self.handle))

    def set_option(self, name: str, value: int):
        self._check(_lib.lib().dc_b200_set_option(self.handle, name.encode(), int(value)))

    # ---- weights
    def upload_weight(self, ggml_type: int, data: np.ndarray, K: int, N: int, E: int = 1) -> Weight:
        data = np.ascontiguousarray(data)
        want = row_bytes(ggml_type, K) * N * E
        if data.nbytes != want:
            raise ValueError(f"weight has {data.nbytes} bytes, expected {want}")
        ne = (C.c_int64 * 4)(K, N, E, 1)
        h = C.c_void_p()
        self._check(_lib.lib().dc_b200_upload_weight(self.handle, int(ggml_type), ne, _vp(data), C.byref(h)))
        return Weight(self, h, ggml_type, K, N, E)

    # ---- Q8_K
    def quantize_q8k(self, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(np.atleast_2d(x), dtype=np.float32)
        rows, K = x.shape
        out = np.zeros((rows, K // QK_K * Q8K_BYTES), dtype=np.uint8)
        self._check(_lib.lib().dc_b200_quantize_q8k(self.handle, _vp(x), rows, K, _vp(out)))
        return out

    # ---- MUL_MAT
    def mul_mat(self, w: Weight, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(np.atleast_2d(x), dtype=np.float32)
        M, K = x.shape
        if K != w.K:
            raise ValueError(f"x has K={K}, weight has K={w.K}")
        y = np.empty((M, w.N), dtype=np.float32)
        self._check(_lib.lib().dc_b200_mul_mat(self.handle, w.handle, _vp(x), M, _vp(y)))
        return y

    def mul_mat_block_sums(self, w: Weight, x: np.ndarray):
        x = np.ascontiguousarray(np.atleast_2d(x), dtype=np.float32)
        M, K = x.shape
        nb = K // QK_K
        I = np.zeros((M, w.N, nb), dtype=np.int32)
        Mn = np.zeros((M, w.N, nb), dtype=np.int32) if w.type == GGML_TYPE_Q4_K else None
        self._check(_lib.lib().dc_b200_mul_mat_block_sums(self.handle, w.handle, _vp(x), M, _vp(I), _vp(Mn)))
        return I, Mn
