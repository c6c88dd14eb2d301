"""GGUF K-quant super-block byte layouts and seeded synthetic block generators.

Layouts (ggml block ABI as restated by DenseCore):
  Q4_K 144 B: fp16 d, fp16 dmin, u8 scales[12], u8 qs[128]   (core/src/kernels/hwy/hwy_moe_quant.cc:28-35)
  Q6_K 210 B: u8 ql[128], u8 qh[64], i8 scales[16], fp16 d    (core/src/llm/matmul/q6_small_batch.h:13-18)
  Q8_K 292 B: f32 d, i8 qs[256], i16 bsums[16]                (core/src/kernels/hwy/hwy_moe_quant.cc:47-51)

The generators produce raw random block bytes in the style of DenseCore's own
parity sweeps (core/tests/benchmarks/q6_small_batch.cpp:52-67): any byte
pattern is a legal input to the dot kernels.
"""
from __future__ import annotations

import numpy as np

GGML_TYPE_F32 = 0
GGML_TYPE_F16 = 1
GGML_TYPE_Q4_K = 12
GGML_TYPE_Q6_K = 14
QK_K = 256
BLOCK_BYTES = {GGML_TYPE_Q4_K: 144, GGML_TYPE_Q6_K: 210}
Q8K_BYTES = 292


def row_bytes(ggml_type: int, K: int) -> int:
    if ggml_type == GGML_TYPE_F32:
        return 4 * K
    if ggml_type == GGML_TYPE_F16:
        return 2 * K
    if ggml_type not in BLOCK_BYTES:
        raise ValueError(f"ggml type {ggml_type} is not supported (F32, F16, Q4_K, Q6_K)")
    if K % QK_K:
        raise ValueError(f"K={K} is not a multiple of {QK_K}")
    return K // QK_K * BLOCK_BYTES[ggml_type]


def pack_q4k_scales(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    """sc, mn: [..., 8] values 0..63 -> [..., 12] packed bytes.

    Inverse of the decode at core/src/kernels/hwy/hwy_moe_quant.cc:90-101.
    """
    sc = sc.astype(np.uint8)
    mn = mn.astype(np.uint8)
    out = np.zeros(sc.shape[:-1] + (12,), dtype=np.uint8)
    for j in range(4):
        out[..., j] = (sc[..., j] & 63) | ((sc[..., j + 4] >> 4) << 6)
        out[..., j + 4] = (mn[..., j] & 63) | ((mn[..., j + 4] >> 4) << 6)
        out[..., j + 8] = (sc[..., j + 4] & 0xF) | ((mn[..., j + 4] & 0xF) << 4)
    return out


def random_q4k(rng: np.random.Generator, N: int, K: int, d_sigma: float = 0.01) -> np.ndarray:
    """N rows of K/256 Q4_K blocks: nibbles uniform 0..15, scales and mins uniform 0..63,
    d and dmin = fp16(|N(0, d_sigma)|).  Returns uint8 [N, K/256*144]."""
    nb = K // QK_K
    blk = np.zeros((N, nb, 144), dtype=np.uint8)
    d = np.abs(rng.normal(0.0, d_sigma, size=(N, nb, 2))).astype(np.float16)
    blk[:, :, 0:4] = d.view(np.uint8).reshape(N, nb, 4)
    sc = rng.integers(0, 64, size=(N, nb, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, size=(N, nb, 8), dtype=np.uint8)
    blk[:, :, 4:16] = pack_q4k_scales(sc, mn)
    blk[:, :, 16:144] = rng.integers(0, 256, size=(N, nb, 128), dtype=np.uint8)
    return blk.reshape(N, nb * 144)


def random_q6k(rng: np.random.Generator, N: int, K: int, d_sigma: float = 0.01) -> np.ndarray:
    """N rows of K/256 Q6_K blocks: ql, qh random bytes, int8 scales uniform -32..31,
    d = fp16(|N(0, d_sigma)|).  Returns uint8 [N, K/256*210]."""
    nb = K // QK_K
    blk = np.zeros((N, nb, 210), dtype=np.uint8)
    blk[:, :, 0:192] = rng.integers(0, 256, size=(N, nb, 192), dtype=np.uint8)
    blk[:, :, 192:208] = rng.integers(-32, 32, size=(N, nb, 16), dtype=np.int8).view(np.uint8)
    d = np.abs(rng.normal(0.0, d_sigma, size=(N, nb, 1))).astype(np.float16)
    blk[:, :, 208:210] = d.view(np.uint8).reshape(N, nb, 2)
    return blk.reshape(N, nb * 210)


def random_weight(rng: np.random.Generator, ggml_type: int, N: int, K: int, d_sigma: float = 0.01) -> np.ndarray:
    if ggml_type == GGML_TYPE_Q4_K:
        return random_q4k(rng, N, K, d_sigma)
    if ggml_type == GGML_TYPE_Q6_K:
        return random_q6k(rng, N, K, d_sigma)
    raise ValueError(f"unsupported type {ggml_type}")
