"""The allocation-free MUL_MAT entry point against the ordinary one.

dc_b200_mul_mat_dev_noalloc exists for hosts that cannot call the CUDA
allocator on their compute path (an op callback under a graph executor with
fixed buffers, a serving loop after warm-up, code inside a stream capture): its
Q8_K scratch is an array inside the library instead of memory the context
allocates.  It must give the same numbers as dc_b200_mul_mat_dev, on repeated
calls, because the built-in array is shared and keeps the last call's contents.
This file sorts last so that a run stopping at the first failure has already
run every other test.
"""
import numpy as np
import pytest

import densecore_b200 as dc
from densecore_b200 import blocks as B

pytestmark = pytest.mark.gpu


def _run(ctx, W, x, noalloc):
    M, N = x.shape[0], W.N
    xd, yd = ctx.alloc(x.nbytes), ctx.alloc(M * N * 4)
    try:
        ctx.to_device(xd, x)
        ctx.to_device(yd, np.full((M, N), np.float32(-7.0)))
        ctx.mul_mat_dev(W, xd, M, yd, noalloc=noalloc)
        ctx.synchronize()
        return ctx.from_device(yd, np.empty((M, N), np.float32))
    finally:
        ctx.free(xd)
        ctx.free(yd)


def test_noalloc_matches_allocating_entry_point_twice_in_a_row(ctx):
    rng = np.random.default_rng(77)
    for t, N, K in ((B.GGML_TYPE_Q4_K, 512, 2048), (B.GGML_TYPE_Q6_K, 300, 768)):
        W = ctx.upload_weight(t, B.random_weight(rng, t, N, K), K, N)
        # second call: more rows of different values, so stale scratch contents would show
        for M in (3, 16):
            x = rng.normal(size=(M, K)).astype(np.float32)
            want = _run(ctx, W, x, noalloc=False)
            got = _run(ctx, W, x, noalloc=True)
            assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()
            assert np.array_equal(got, want)        # same kernels, same order: identical bits
        W.free()


def test_noalloc_at_the_full_extent_of_its_scratch(ctx):
    """16 rows of 16384 values fill the built-in array exactly (and make the kernel split the rows in two
    halves, which do not fit shared memory together)."""
    rng = np.random.default_rng(79)
    t, N, K = B.GGML_TYPE_Q4_K, 64, 16384
    W = ctx.upload_weight(t, B.random_weight(rng, t, N, K), K, N)
    x = rng.normal(size=(16, K)).astype(np.float32)
    assert np.array_equal(_run(ctx, W, x, noalloc=True), _run(ctx, W, x, noalloc=False))
    W.free()


def test_noalloc_refuses_shapes_beyond_its_scratch(ctx):
    rng = np.random.default_rng(78)
    W = ctx.upload_weight(B.GGML_TYPE_Q4_K, B.random_q4k(rng, 8, 256), 256, 8)
    xd, yd = ctx.alloc(17 * 256 * 4), ctx.alloc(17 * 8 * 4)
    with pytest.raises(dc.DcError) as e:
        ctx.mul_mat_dev(W, xd, 17, yd, noalloc=True)        # more than 16 rows
    assert e.value.status == -7 and "16 rows" in e.value.message
    ctx.free(xd)
    ctx.free(yd)
    W.free()
    K = 16640                                               # one super-block more than the array holds
    W = ctx.upload_weight(B.GGML_TYPE_Q4_K, B.random_q4k(rng, 2, K), K, 2)
    xd, yd = ctx.alloc(K * 4), ctx.alloc(2 * 4)
    with pytest.raises(dc.DcError) as e:
        ctx.mul_mat_dev(W, xd, 1, yd, noalloc=True)
    assert e.value.status == -7
    ctx.free(xd)
    ctx.free(yd)
    W.free()
