"""Golden vectors computed by DenseCore's own code (not by the oracle).

Needs a DenseCore checkout: oracle.build_ref() compiles core/src/sampler/sampler.cpp and
core/src/llm/matmul/q6_small_batch.h from it (recipe: oracle/Makefile, target _ref/libdc_ref.so).
The arrays written here travel with the repository, the checkout does not.

    python tests/golden/make_ref_golden.py

Contents of ref_golden.npz
  argmax_in [6, 1024] f32, argmax_out [6]         ArgmaxScalar (sampler.cpp:42-57): ties, all-equal, NaN, -inf rows
  sm_in [3, 2048] f32, sm_T [3], sm_out [3, 2048] SampleTopP's probabilities (sampler.cpp:235-262)
  q6_w [12, 8*210] u8, q6_x [4, 2048] f32, q6_q8 [4, 8*292] u8, q6_out [12, 4]
                                                   ComputeQ6KQ8KM4Native (q6_small_batch.h:36-103); weight bytes are
                                                   random blocks in the style of core/tests/benchmarks/q6_small_batch.cpp:52-67
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as o  # noqa: E402
from densecore_b200 import blocks as B  # noqa: E402


def main():
    assert o.build_ref(force=True), "no DenseCore checkout found (set DENSECORE_SRC)"
    rng = np.random.default_rng(20261125)
    a = rng.normal(size=(6, 1024)).astype(np.float32)
    a[1, 100] = a[1, 900] = 7.5            # equal maxima: the first wins
    a[2, :] = 1.25                          # all equal
    a[3, 17] = np.nan                       # NaN never compares greater
    a[4, :] = -np.inf
    a[4, 1023] = -1e30
    a[5, 0] = 50.0                          # maximum at index 0
    am = np.array([o.ref_argmax(r) for r in a], dtype=np.int32)
    sm_in = (rng.normal(size=(3, 2048)) * np.array([[1.0], [4.0], [0.25]])).astype(np.float32)
    sm_T = np.array([0.8, 1.0, 0.3], dtype=np.float32)
    sm_out = np.stack([o.ref_softmax_temperature(sm_in[i], float(sm_T[i]))[0] for i in range(3)])
    K = 2048
    q6_w = B.random_q6k(rng, 12, K).reshape(12, -1)
    q6_x = (rng.normal(size=(4, K)) * np.array([[1.0], [0.01], [30.0], [1.0]])).astype(np.float32)
    q6_x[3, :256] = 0.0                     # an all-zero activation block
    q6_q8 = o.quantize_q8k(q6_x)
    q6_out = np.stack([o.ref_q6k_q8k_m4(q6_w[r], q6_q8, K) for r in range(12)])
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_golden.npz"),
                        argmax_in=a, argmax_out=am, sm_in=sm_in, sm_T=sm_T, sm_out=sm_out, q6_w=q6_w, q6_x=q6_x,
                        q6_q8=q6_q8, q6_out=q6_out)
    print("wrote ref_golden.npz")


if __name__ == "__main__":
    main()
