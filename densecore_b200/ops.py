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

    def mul_mat_dev(self, w: Weight, x_dev: int, M: int, y_dev: int, noalloc: bool = False):
        """Device-pointer form: x_dev [M, K] f32 and y_dev [M, N] f32 are addresses from alloc().
        noalloc=True takes the entry point whose Q8_K scratch is built into the library
        (M <= 16, K <= 16384; performs no allocation)."""
        fn = _lib.lib().dc_b200_mul_mat_dev_noalloc if noalloc else _lib.lib().dc_b200_mul_mat_dev
        self._check(fn(self.handle, w.handle, C.c_void_p(x_dev), int(M), C.c_void_p(y_dev)))

    def mul_mat_block_sums(self, w: Weight, x: np.ndarray):
        x = np.ascontiguousarray(np.atleast_2d(x), dtype=np.float32)
        M, K = x.shape
        nb = K // QK_K
        I = np.zeros((M, w.N, nb), dtype=np.int32)
        Mn = np.zeros((M, w.N, nb), dtype=np.int32) if w.type == GGML_TYPE_Q4_K else None
        self._check(_lib.lib().dc_b200_mul_mat_block_sums(self.handle, w.handle, _vp(x), M, _vp(I), _vp(Mn)))
        return I, Mn

    # ---- device buffers
    def alloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        self._check(_lib.lib().dc_b200_alloc_device(self.handle, int(nbytes), C.byref(p)))
        return p.value

    def free(self, dev: int):
        self._check(_lib.lib().dc_b200_free_device(self.handle, C.c_void_p(dev)))

    def to_device(self, dev: int, a: np.ndarray):
        a = np.ascontiguousarray(a)
        self._check(_lib.lib().dc_b200_copy_to_device(self.handle, C.c_void_p(dev), _vp(a), a.nbytes))

    def from_device(self, dev: int, out: np.ndarray) -> np.ndarray:
        self._check(_lib.lib().dc_b200_copy_from_device(self.handle, _vp(out), C.c_void_p(dev), out.nbytes))
        return out

    def mul_mat_id_dev(self, router: Weight, gate: Weight, up: Weight, down: Weight, x_dev: int, T: int, top_k: int,
                       y_dev: int, ids_dev: int = 0, weights_dev: int = 0, routed_scale: float = 1.0):
        """Device-pointer form of mul_mat_id (enqueue only)."""
        self._check(_lib.lib().dc_b200_mul_mat_id_dev(self.handle, router.handle, gate.handle, up.handle, down.handle,
                                                      C.c_void_p(x_dev), int(T), int(top_k), routed_scale, C.c_void_p(y_dev),
                                                      C.c_void_p(ids_dev) if ids_dev else None,
                                                      C.c_void_p(weights_dev) if weights_dev else None))

    # ---- MUL_MAT_ID
    def mul_mat_id(self, router: Weight, gate: Weight, up: Weight, down: Weight, x: np.ndarray, top_k: int,
                   routed_scale: float = 1.0):
        """One MoE FFN layer.  Returns (y [T, hidden], ids [T, top_k], weights [T, top_k])."""
        x = np.ascontiguousarray(np.atleast_2d(x), dtype=np.float32)
        T, H = x.shape
        y = np.empty((T, H), dtype=np.float32)
        ids = np.zeros((T, top_k), dtype=np.int32)
        w = np.zeros((T, top_k), dtype=np.float32)
        self._check(_lib.lib().dc_b200_mul_mat_id(self.handle, router.handle, gate.handle, up.handle, down.handle,
                                                  _vp(x), T, top_k, routed_scale, _vp(y), _vp(ids), _vp(w)))
        return y, ids, w

    def moe_route(self, logits: np.ndarray, top_k: int, routed_scale: float = 1.0):
        logits = np.ascontiguousarray(np.atleast_2d(logits), dtype=np.float32)
        T, E = logits.shape
        ids = np.zeros((T, top_k), dtype=np.int32)
        w = np.zeros((T, top_k), dtype=np.float32)
        self._check(_lib.lib().dc_b200_moe_route(self.handle, _vp(logits), T, E, top_k, routed_scale, _vp(ids), _vp(w)))
        return ids, w

    # ---- sampling / verify
    def argmax(self, logits: np.ndarray) -> np.ndarray:
        logits = np.ascontiguousarray(np.atleast_2d(logits), dtype=np.float32)
        out = np.zeros(logits.shape[0], dtype=np.int32)
        self._check(_lib.lib().dc_b200_argmax(self.handle, _vp(logits), logits.shape[0], logits.shape[1], _vp(out)))
        return out

    def softmax(self, logits: np.ndarray, temperature: float) -> np.ndarray:
        logits = np.ascontiguousarray(np.atleast_2d(logits), dtype=np.float32)
        out = np.empty_like(logits)
        self._check(_lib.lib().dc_b200_softmax(self.handle, _vp(logits), logits.shape[0], logits.shape[1],
                                               temperature, _vp(out)))
        return out

    def verify_uniforms(self, seed: int, step: int, n: int) -> np.ndarray:
        out = np.zeros(n, dtype=np.float32)
        self._check(_lib.lib().dc_b200_verify_uniforms(self.handle, seed, step, n, _vp(out)))
        return out

    def verify_accept(self, target_logits: np.ndarray, draft_tokens, draft_probs=None, uniforms=None, seed: int = 0,
                      step: int = 0, mode: int = 0, temperature: float = 1.0):
        """Returns (n_accepted, next_token)."""
        tl = np.ascontiguousarray(target_logits, dtype=np.float32)
        gamma, vocab = tl.shape[0] - 1, tl.shape[1]
        dt = np.ascontiguousarray(draft_tokens, dtype=np.int32)
        dp = np.ascontiguousarray(draft_probs, dtype=np.float32) if draft_probs is not None else None
        u = np.ascontiguousarray(uniforms, dtype=np.float32) if uniforms is not None else None
        n, t = C.c_int(0), C.c_int(0)
        self._check(_lib.lib().dc_b200_verify_accept(self.handle, _vp(tl), _vp(dt), _vp(dp), _vp(u), seed, step,
                                                     gamma, vocab, mode, temperature, C.byref(n), C.byref(t)))
        return n.value, t.value

    # ---- paged KV
    def kv_cache(self, n_layer: int, n_kv_head: int, head_dim: int, max_blocks: int, max_seqs: int,
                 max_blocks_per_seq: int) -> "KVCache":
        return KVCache(self, n_layer, n_kv_head, head_dim, max_blocks, max_seqs, max_blocks_per_seq)


class KVCache:
    """Paged fp16 KV cache with 16-token blocks (dc_b200_kv_*)."""

    def __init__(self, ctx: Context, n_layer, n_kv_head, head_dim, max_blocks, max_seqs, max_blocks_per_seq):
        self.ctx, self.n_layer, self.n_kv, self.head_dim = ctx, n_layer, n_kv_head, head_dim
        h = C.c_void_p()
        ctx._check(_lib.lib().dc_b200_kv_create(ctx.handle, n_layer, n_kv_head, head_dim, max_blocks, max_seqs,
                                                max_blocks_per_seq, C.byref(h)))
        self.handle = h

    def close(self):
        if self.handle:
            _lib.lib().dc_b200_kv_destroy(self.handle)
            self.handle = None

    def seq_alloc(self) -> int:
        s = C.c_int(-1)
        self.ctx._check(_lib.lib().dc_b200_kv_seq_alloc(self.handle, C.byref(s)))
        return s.value

    def seq_free(self, seq: int):
        self.ctx._check(_lib.lib().dc_b200_kv_seq_free(self.handle, seq))

    def seq_reserve(self, seq: int, n_tokens: int):
        self.ctx._check(_lib.lib().dc_b200_kv_seq_reserve(self.handle, seq, n_tokens))

    def block_table(self, seq: int) -> np.ndarray:
        n = C.c_int(0)
        self.ctx._check(_lib.lib().dc_b200_kv_block_table(self.handle, seq, None, 0, C.byref(n)))
        out = np.zeros(max(n.value, 1), dtype=np.int32)
        self.ctx._check(_lib.lib().dc_b200_kv_block_table(self.handle, seq, _vp(out), out.size, C.byref(n)))
        return out[:n.value]

    def free_blocks(self) -> int:
        return _lib.lib().dc_b200_kv_free_blocks(self.handle)

    def read_block(self, layer: int, block: int):
        shape = (16, self.n_kv, self.head_dim)
        k = np.zeros(shape, dtype=np.float16)
        v = np.zeros(shape, dtype=np.float16)
        self.ctx._check(_lib.lib().dc_b200_kv_read_block(self.handle, layer, block, _vp(k), _vp(v)))
        return k, v

    def flash_attn_decode(self, layer: int, q, k, v, seq_ids, positions, scale: float) -> np.ndarray:
        """Writes the tokens' K/V at their positions, then attends.  q [T, n_head, hd]; k, v [T, n_kv, hd]."""
        q = np.ascontiguousarray(q, dtype=np.float32)
        k = np.ascontiguousarray(k, dtype=np.float32)
        v = np.ascontiguousarray(v, dtype=np.float32)
        T, n_head = q.shape[0], q.shape[1]
        seq_ids = np.ascontiguousarray(seq_ids, dtype=np.int32)
        positions = np.ascontiguousarray(positions, dtype=np.int32)
        out = np.empty((T, n_head, self.head_dim), dtype=np.float32)
        self.ctx._check(_lib.lib().dc_b200_flash_attn_decode(self.ctx.handle, self.handle, layer, _vp(q), _vp(k), _vp(v),
                                                             _vp(seq_ids), _vp(positions), T, n_head, scale, _vp(out)))
        return out

    def flash_attn_prefill(self, layer: int, q, k, v, seq: int, pos0: int, scale: float) -> np.ndarray:
        """Prompt chunk of one sequence: writes K/V at positions pos0.., then causal attention on the tensor cores."""
        q = np.ascontiguousarray(q, dtype=np.float32)
        k = np.ascontiguousarray(k, dtype=np.float32)
        v = np.ascontiguousarray(v, dtype=np.float32)
        n, n_head = q.shape[0], q.shape[1]
        out = np.empty((n, n_head, self.head_dim), dtype=np.float32)
        self.ctx._check(_lib.lib().dc_b200_flash_attn_prefill(self.ctx.handle, self.handle, layer, _vp(q), _vp(k), _vp(v), seq,
                                                              pos0, n, n_head, scale, _vp(out)))
        return out
