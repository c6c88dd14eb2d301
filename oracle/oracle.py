"""ctypes binding of the CPU oracle (oracle/dc_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by
the cpu_baseline / --impl reference legs of bench.py.  The product package
(densecore_b200) never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libdc_oracle.so")

TYPE_F32, TYPE_F16, TYPE_Q4_K, TYPE_Q6_K = 0, 1, 12, 14
BLOCK_BYTES = {TYPE_Q4_K: 144, TYPE_Q6_K: 210}
Q8K_BYTES = 292
KV_BLOCK = 16


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "dc_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libdc_oracle.so"], stdout=subprocess.DEVNULL)
    return _SO


# ---- the reference's own code where it compiles here (oracle/ref_shim.cpp -> oracle/_ref/libdc_ref.so) ----
_REF_SO = os.path.join(_HERE, "_ref", "libdc_ref.so")
_ref = None


def default_reference_root() -> str:
    """Where a DenseCore checkout is looked for: $DENSECORE_SRC, else a directory named
    `reference` beside this repository."""
    return os.environ.get("DENSECORE_SRC") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")


def build_ref(reference_root: str | None = None, force: bool = False) -> str | None:
    """Compiles the reference's sampler and Q6_K small-batch kernel from a DenseCore checkout.
    Returns the library path, or None when no checkout is present (a prebuilt library is then used as is)."""
    root = reference_root or default_reference_root()
    if not os.path.isdir(os.path.join(root, "core", "src", "sampler")):
        return _REF_SO if os.path.exists(_REF_SO) else None
    args = ["make", "-C", _HERE, "DENSECORE_SRC=" + root, "_ref/libdc_ref.so"]
    if force:
        args.insert(3, "-B")
    subprocess.check_call(args, stdout=subprocess.DEVNULL)
    return _REF_SO


def ref_lib():
    """ctypes handle of the compiled reference pieces, or None if they were never built."""
    global _ref
    if _ref is None and os.path.exists(_REF_SO):
        _ref = C.CDLL(_REF_SO)
    return _ref


def ref_argmax(v) -> int:
    v = _f32(v)
    return int(ref_lib().dcref_argmax(_p(v), v.size))


def ref_softmax_temperature(logits, temperature, seed: int = 42):
    """(probabilities, sampled token) of the reference's SampleTopP with top_p = 1."""
    logits = _f32(logits)
    p = np.zeros_like(logits)
    tok = ref_lib().dcref_softmax_temperature(_p(logits), logits.size, C.c_float(temperature), C.c_uint64(seed), _p(p))
    return p, int(tok)


def ref_q6k_q8k_m4(w_row: np.ndarray, q8_rows: np.ndarray, K: int) -> np.ndarray:
    """One Q6_K row against four Q8_K rows ([4, K/256*292] bytes) through the reference's AVX2 kernel."""
    q8 = np.ascontiguousarray(q8_rows, dtype=np.uint8)
    assert q8.shape[0] == 4
    # the kernel wants 4-byte aligned activation rows and a 2-byte aligned weight row
    wbuf = np.zeros(w_row.size + 8, dtype=np.uint8)
    off = (-wbuf.ctypes.data) % 8
    wbuf[off:off + w_row.size] = w_row
    out = np.zeros(4, dtype=np.float32)
    ok = ref_lib().dcref_q6k_q8k_m4(C.c_void_p(wbuf.ctypes.data + off), _p(q8), C.c_uint64(q8.shape[1]), int(K), _p(out))
    assert ok, "the reference kernel refused its arguments"
    return out


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        _lib.dco_fp16_to_fp32.restype = C.c_float
        _lib.dco_fp16_to_fp32.argtypes = [C.c_uint16]
        _lib.dco_fp32_to_fp16.restype = C.c_uint16
        _lib.dco_fp32_to_fp16.argtypes = [C.c_float]
        for n in ("dco_fast_exp", "dco_fast_exp_fma", "dco_det_exp"):
            getattr(_lib, n).restype = C.c_float
            getattr(_lib, n).argtypes = [C.c_float]
        _lib.dco_vec_dot_q4k_q8k.restype = C.c_float
        _lib.dco_vec_dot_q6k_q8k.restype = C.c_float
        _lib.dco_row_bytes.restype = C.c_int64
        _lib.dco_row_bytes.argtypes = [C.c_int, C.c_int64]
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def set_threads(n: int):
    lib().dco_set_threads(C.c_int(int(n)))


def max_threads() -> int:
    return int(lib().dco_max_threads())


def row_bytes(type_: int, K: int) -> int:
    return int(lib().dco_row_bytes(type_, C.c_int64(K)))


def fp16_to_fp32(h: int) -> float:
    return float(lib().dco_fp16_to_fp32(C.c_uint16(h)))


def fp32_to_fp16(f: float) -> int:
    return int(lib().dco_fp32_to_fp16(C.c_float(f)))


def fast_exp(x: float) -> float:
    return float(lib().dco_fast_exp(C.c_float(x)))


def fast_exp_fma(x: float) -> float:
    return float(lib().dco_fast_exp_fma(C.c_float(x)))


def det_exp(x: float) -> float:
    return float(lib().dco_det_exp(C.c_float(x)))


def quantize_q8k(x: np.ndarray) -> np.ndarray:
    """x: [rows, K] f32 -> uint8 [rows, K/256*292]."""
    x = _f32(np.atleast_2d(x))
    rows, K = x.shape
    out = np.zeros((rows, K // 256 * Q8K_BYTES), dtype=np.uint8)
    for r in range(rows):
        ok = lib().dco_quantize_row_q8k(_p(x[r]), _p(out[r]), C.c_int64(K))
        assert ok
    return out


def q8k_fields(q8: np.ndarray):
    """Split Q8_K bytes [rows, nb*292] into (d f32 [rows,nb], qs i8 [rows,nb,256], bsums i16 [rows,nb,16])."""
    rows = q8.shape[0]
    b = q8.reshape(rows, -1, Q8K_BYTES)
    d = b[:, :, 0:4].copy().view(np.float32)[..., 0]
    qs = b[:, :, 4:260].copy().view(np.int8)
    bs = b[:, :, 260:292].copy().view(np.int16)
    return d, qs, bs


def block_sums(type_: int, w_row: np.ndarray, q8_row: np.ndarray, K: int):
    nb = K // 256
    I = np.zeros(nb, dtype=np.int32)
    if type_ == TYPE_Q4_K:
        M = np.zeros(nb, dtype=np.int32)
        lib().dco_q4k_q8k_block_sums(_p(w_row), _p(q8_row), C.c_int64(K), _p(I), _p(M))
        return I, M
    lib().dco_q6k_q8k_block_sums(_p(w_row), _p(q8_row), C.c_int64(K), _p(I))
    return I, None


def vec_dot(type_: int, w_row: np.ndarray, q8_row: np.ndarray, K: int) -> float:
    fn = lib().dco_vec_dot_q4k_q8k if type_ == TYPE_Q4_K else lib().dco_vec_dot_q6k_q8k
    return float(fn(_p(w_row), _p(q8_row), C.c_int64(K)))


def dequantize(type_: int, w: np.ndarray, N: int, K: int) -> np.ndarray:
    rb = row_bytes(type_, K)
    w = np.ascontiguousarray(w, dtype=np.uint8).reshape(N, rb)
    out = np.zeros((N, K), dtype=np.float32)
    for n in range(N):
        lib().dco_dequantize_row(type_, _p(w[n]), _p(out[n]), C.c_int64(K))
    return out


def mul_mat(type_: int, w: np.ndarray, N: int, K: int, x: np.ndarray) -> np.ndarray:
    """y[M, N] = x[M, K] . W[N, K]^T through Q8_K activations (f32 weights: plain dot)."""
    x = _f32(np.atleast_2d(x))
    M = x.shape[0]
    w = np.ascontiguousarray(w)
    y = np.zeros((M, N), dtype=np.float32)
    ok = lib().dco_mul_mat(type_, _p(w), C.c_int64(N), C.c_int64(K), _p(x), C.c_int64(M), _p(y), None)
    assert ok
    return y


def route(logits: np.ndarray, top_k: int, mode: str = "stable", normalize: bool = True, scale: float = 1.0):
    logits = _f32(np.atleast_2d(logits))
    T, E = logits.shape
    ids = np.zeros((T, top_k), dtype=np.int32)
    w = np.zeros((T, top_k), dtype=np.float32)
    if mode == "stable":
        ok = lib().dco_route_stable_topk(_p(logits), T, E, top_k, C.c_float(scale), _p(ids), _p(w))
        assert ok
    else:
        lib().dco_route_softmax_topk(_p(logits), T, E, top_k, int(normalize), C.c_float(scale), _p(ids), _p(w))
    return ids, w


def build_reorder_map(ids: np.ndarray, n_experts: int):
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    T, k = ids.shape
    offsets = np.zeros(n_experts + 1, dtype=np.int32)
    tokens = np.zeros(T * k, dtype=np.int32)
    slot_of = np.zeros(T * k, dtype=np.int32)
    lib().dco_build_reorder_map(_p(ids), T, k, n_experts, _p(offsets), _p(tokens), _p(slot_of))
    return offsets, tokens, slot_of


def moe_forward(types, gate_w, up_w, down_w, n_experts, hidden, inter, x, ids, weights, fast_exp=True,
                f32ref=False, return_h=False):
    x = _f32(np.atleast_2d(x))
    T = x.shape[0]
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    weights = _f32(weights)
    top_k = ids.shape[1]
    out = np.zeros((T, hidden), dtype=np.float32)
    gt, ut, dt = types
    if f32ref:
        ok = lib().dco_moe_forward_f32ref(gt, ut, dt, _p(gate_w), _p(up_w), _p(down_w), n_experts, hidden, inter,
                                          _p(x), T, top_k, _p(ids), _p(weights), _p(out))
        assert ok
        return out
    h = np.zeros((T * top_k, inter), dtype=np.float32) if return_h else None
    ok = lib().dco_moe_forward(gt, ut, dt, _p(gate_w), _p(up_w), _p(down_w), n_experts, hidden, inter, _p(x), T,
                               top_k, _p(ids), _p(weights), int(fast_exp), _p(out), _p(h))
    assert ok
    return (out, h) if return_h else out


def kv_write(k_arena, v_arena, block_table, pos, n_kv, head_dim, k, v):
    lib().dco_kv_write(_p(k_arena), _p(v_arena), _p(block_table), int(pos), n_kv, head_dim, _p(_f32(k)), _p(_f32(v)))


def paged_attention(q, k_arena, v_arena, block_table, query_pos, n_head, n_kv, head_dim, scale, mode="blockwise"):
    q = _f32(q)
    out = np.zeros((n_head, head_dim), dtype=np.float32)
    fn = lib().dco_paged_attention_blockwise if mode == "blockwise" else lib().dco_paged_attention_scalar
    fn(_p(q), _p(k_arena), _p(v_arena), _p(block_table), int(query_pos), n_head, n_kv, head_dim, C.c_float(scale),
       _p(out))
    return out


def rms_norm(x, w, eps):
    x = _f32(x)
    out = np.zeros_like(x)
    wv = _f32(w) if w is not None else None
    lib().dco_rms_norm(_p(x), _p(wv), x.size, C.c_float(eps), _p(out))
    return out


def rope_table(max_pos, head_dim, theta):
    t = np.zeros((max_pos, head_dim), dtype=np.float32)
    lib().dco_rope_table(max_pos, head_dim, C.c_double(theta), _p(t))
    return t


def rope(x, cos_sin_row):
    x = _f32(x).copy()
    hd = cos_sin_row.shape[-1]
    row = _f32(cos_sin_row)
    for h in x.reshape(-1, hd):
        lib().dco_rope(_p(h), _p(row), hd)
    return x


def argmax(v) -> int:
    v = _f32(v)
    return int(lib().dco_argmax(_p(v), v.size))


def philox4x32_10(ctr, key):
    c = np.asarray(ctr, dtype=np.uint32)
    k = np.asarray(key, dtype=np.uint32)
    o = np.zeros(4, dtype=np.uint32)
    lib().dco_philox4x32_10(_p(c), _p(k), _p(o))
    return o


def verify_uniforms(seed: int, step: int, n: int) -> np.ndarray:
    u = np.zeros(n, dtype=np.float32)
    lib().dco_verify_uniforms(C.c_uint64(seed), C.c_uint32(step), n, _p(u))
    return u


def det_softmax(logits, temperature):
    logits = _f32(logits)
    p = np.zeros_like(logits)
    lib().dco_det_softmax(_p(logits), logits.size, C.c_float(temperature), _p(p))
    return p


def softmax_temperature(logits, temperature):
    """The sampler's temperature softmax with the C library's expf (sampler.cpp:235-262)."""
    logits = _f32(logits)
    p = np.zeros_like(logits)
    lib().dco_softmax_temperature(_p(logits), logits.size, C.c_float(temperature), _p(p))
    return p


def det_inverse_cdf(w, u) -> int:
    w = _f32(w)
    return int(lib().dco_det_inverse_cdf(_p(w), w.size, C.c_float(u)))


def verify_accept(target_logits, draft_tokens, draft_probs, u, mode, temperature=1.0):
    tl = _f32(target_logits)
    gamma = tl.shape[0] - 1
    vocab = tl.shape[1]
    dt = np.ascontiguousarray(draft_tokens, dtype=np.int32)
    dp = _f32(draft_probs) if draft_probs is not None else None
    uu = _f32(u) if u is not None else None
    n = C.c_int32(0)
    t = C.c_int32(0)
    ok = lib().dco_verify_accept(_p(tl), _p(dt), _p(dp), _p(uu), gamma, vocab, int(mode), C.c_float(temperature),
                                 C.byref(n), C.byref(t))
    assert ok
    return n.value, t.value


def synth_normal(seed, first_index, n, sigma):
    out = np.zeros(n, dtype=np.float32)
    lib().dco_synth_normal(C.c_uint64(seed), C.c_uint64(first_index), C.c_int64(n), C.c_float(sigma), _p(out))
    return out


def synth_quantized(type_, seed, N, K, sigma):
    out = np.zeros(N * (K // 256) * BLOCK_BYTES[type_], dtype=np.uint8)
    lib().dco_synth_quantized(type_, C.c_uint64(seed), C.c_int64(N), C.c_int64(K), C.c_float(sigma), _p(out))
    return out


def quantize_block(type_, x256):
    x = _f32(x256)
    out = np.zeros(BLOCK_BYTES[type_], dtype=np.uint8)
    (lib().dco_quantize_block_q4k if type_ == TYPE_Q4_K else lib().dco_quantize_block_q6k)(_p(x), _p(out))
    return out
