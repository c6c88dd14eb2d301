"""Generates tests/golden/kquant_golden.npz: seeded inputs and the CPU oracle's
outputs for the K-quant ops.  DenseCore's own tests store no expected numbers
(every parity test there compares two implementations at run time), so these
vectors pin the oracle against itself across builds and, for the block decode,
against the independent `gguf` Python package (gguf.quants.dequantize), which
is only needed when this script runs.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from densecore_b200 import blocks as B  # noqa: E402
from oracle import oracle as o  # noqa: E402


def patterned(rows, cols, scale):
    """MakePatternedFloats of DenseCore's MoE tests (core/tests/moe/test_moe_ops.cpp:117-128)."""
    r = np.arange(rows)[:, None]
    c = np.arange(cols)[None, :]
    return (((r * 17 + c * 29 + 7) % 41 - 20) * scale).astype(np.float32)


def main():
    import gguf
    from gguf import quants
    rng = np.random.default_rng(20260913)  # seed style of core/tests/runtime/test_q8_small_batch.cpp
    out = {}
    K, N = 512, 6
    x = rng.normal(size=(3, K)).astype(np.float32)
    x[1, 256:] = 0.0                       # all-zero block
    x[2, 7] = -x[2].max() * 2              # largest magnitude negative
    out["x"] = x
    out["x_pat"] = patterned(2, K, 0.03125)
    out["q8_x"] = o.quantize_q8k(x)
    out["q8_x_pat"] = o.quantize_q8k(out["x_pat"])
    for name, t, gt in (("q4k", B.GGML_TYPE_Q4_K, gguf.GGMLQuantizationType.Q4_K),
                        ("q6k", B.GGML_TYPE_Q6_K, gguf.GGMLQuantizationType.Q6_K)):
        w = B.random_weight(rng, t, N, K)
        out[f"w_{name}"] = w
        deq = o.dequantize(t, w, N, K)
        ref = quants.dequantize(w, gt)
        assert np.array_equal(deq, ref), f"{name}: oracle dequant differs from gguf.quants"
        out[f"deq_{name}"] = deq
        out[f"y_{name}"] = o.mul_mat(t, w, N, K, x)
        rb = B.row_bytes(t, K)
        I = np.zeros((3, N, K // 256), np.int32)
        M = np.zeros((3, N, K // 256), np.int32)
        for m in range(3):
            for n in range(N):
                a, b = o.block_sums(t, w.reshape(N, rb)[n], out["q8_x"][m], K)
                I[m, n] = a
                if b is not None:
                    M[m, n] = b
        out[f"I_{name}"] = I
        out[f"M_{name}"] = M
    lg = rng.normal(size=(4, 16)).astype(np.float32)
    lg[1, 3] = lg[1, 9]
    out["route_logits"] = lg
    ids, w = o.route(lg, 4, mode="stable")
    out["route_ids"], out["route_w"] = ids, w
    ids2, w2 = o.route(lg, 4, mode="softmax")
    out["route_ids_softmax"], out["route_w_softmax"] = ids2, w2
    out["philox_kat"] = np.stack([o.philox4x32_10([0, 0, 0, 0], [0, 0]),
                                  o.philox4x32_10([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344],
                                                  [0xa4093822, 0x299f31d0])])
    out["uniforms_99_3"] = o.verify_uniforms(99, 3, 5)
    out["synth_q4k"] = o.synth_quantized(B.GGML_TYPE_Q4_K, 7, 2, 512, 0.02)
    out["synth_q6k"] = o.synth_quantized(B.GGML_TYPE_Q6_K, 7, 2, 512, 0.02)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kquant_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
