"""The oracle against DenseCore's own code, for the functions of the path that compile from their
own sources without the ggml submodule: ArgmaxScalar and SampleTopP's softmax
(core/src/sampler/sampler.cpp:42-57, :235-262) and the Q6_K x Q8_K small-batch kernel
(core/src/llm/matmul/q6_small_batch.h:36-103, which DenseCore's own benchmark holds bitwise equal to
ggml's vec_dot, core/tests/benchmarks/q6_small_batch.cpp:38-87).

tests/golden/ref_golden.npz holds outputs of that code (made by tests/golden/make_ref_golden.py where a
DenseCore checkout exists); the oracle must reproduce them.  Where the compiled reference library is
present as well, it is called live on fresh random inputs.  No GPU needed.
"""
import os

import numpy as np
import pytest

from densecore_b200 import blocks as B

REF = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_golden.npz"))
Q6 = B.GGML_TYPE_Q6_K


def test_argmax_matches_reference_golden(oracle):
    got = [oracle.argmax(r) for r in REF["argmax_in"]]
    assert got == REF["argmax_out"].tolist()
    assert got[1] == 100 and got[2] == 0        # first of equal maxima


def test_temperature_softmax_matches_reference_golden(oracle):
    for x, T, want in zip(REF["sm_in"], REF["sm_T"], REF["sm_out"]):
        got = oracle.softmax_temperature(x, float(T))
        # the reference build may fuse v * (1/T) - max into one rounding; everything else is the same libm
        assert np.abs(got - want).max() <= 1e-6 * want.max()
        assert abs(float(got.sum()) - 1.0) < 1e-5
        # the verify step's fully specified exp agrees with it to float accuracy
        assert np.abs(oracle.det_softmax(x, float(T)) - want).max() <= 2e-6 * want.max()


def test_q6k_row_dot_is_bitwise_the_reference_kernel(oracle):
    """Float order of the Q6_K x Q8_K row dot: eight partial accumulators, fma per block, fixed
    final tree.  Bit-equal to the reference's AVX2 kernel, zero blocks and scaled rows included."""
    K = 2048
    assert np.array_equal(oracle.quantize_q8k(REF["q6_x"]), REF["q6_q8"])
    for r in range(REF["q6_w"].shape[0]):
        got = np.array([oracle.vec_dot(Q6, REF["q6_w"][r], REF["q6_q8"][m], K) for m in range(4)], dtype=np.float32)
        assert np.array_equal(got, REF["q6_out"][r]), r
    # the same through the oracle's MUL_MAT
    y = oracle.mul_mat(Q6, REF["q6_w"], 12, K, REF["q6_x"])
    assert np.array_equal(y.T, REF["q6_out"])


def test_live_reference_library_if_built(oracle):
    if oracle.ref_lib() is None:
        pytest.skip("oracle/_ref/libdc_ref.so was not built on this machine")
    rng = np.random.default_rng(77)
    for n in (1, 2, 33, 151936):
        v = rng.normal(size=n).astype(np.float32)
        if n > 2:
            v[n // 3] = v[2 * n // 3] = 11.0
        assert oracle.argmax(v) == oracle.ref_argmax(v)
    v = (rng.normal(size=151936) * 3).astype(np.float32)
    p_ref, _ = oracle.ref_softmax_temperature(v, 0.8)
    assert np.abs(oracle.softmax_temperature(v, 0.8) - p_ref).max() <= 1e-6 * p_ref.max()
    for K in (256, 768, 4096):
        w = B.random_q6k(rng, 5, K).reshape(5, -1)
        q8 = oracle.quantize_q8k(rng.normal(size=(4, K)).astype(np.float32))
        for r in range(5):
            got = np.array([oracle.vec_dot(Q6, w[r], q8[m], K) for m in range(4)], dtype=np.float32)
            assert np.array_equal(got, oracle.ref_q6k_q8k_m4(w[r], q8, K))
