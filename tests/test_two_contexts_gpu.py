"""Two GPUs in one process: kernel attributes (dynamic shared memory opt-in) and occupancy answers are kept
per device, so a second context on another GPU launches the same kernels.  Skipped with fewer than two GPUs."""
import numpy as np
import pytest

import densecore_b200 as dc
from densecore_b200 import blocks as B

pytestmark = pytest.mark.gpu


def test_contexts_on_two_gpus_in_one_process(oracle):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    rng = np.random.default_rng(12)
    N, K = 2048, 2048
    w4, w6 = B.random_q4k(rng, N, K), B.random_q6k(rng, N, K)
    x = rng.normal(size=(5, K)).astype(np.float32)
    x64 = rng.normal(size=(64, K)).astype(np.float32)
    want4, want6 = oracle.mul_mat(B.GGML_TYPE_Q4_K, w4, N, K, x), oracle.mul_mat(B.GGML_TYPE_Q6_K, w6, N, K, x)
    want64 = oracle.mul_mat(B.GGML_TYPE_Q4_K, w4, N, K, x64)
    cfg = dc.Config(n_layer=2, hidden=512, n_head=4, n_kv_head=2, vocab=1000, n_expert=8, n_expert_used=2, expert_ffn=256,
                    max_seqs=2, max_ctx=128)
    prompt = rng.integers(0, 1000, size=45)
    tokens = []
    ctxs = [dc.Context(0), dc.Context(1)]
    # the second GPU first, so that nothing it needs was set up by an earlier call on the first
    for ctx in (ctxs[1], ctxs[0], ctxs[1]):
        W4 = ctx.upload_weight(B.GGML_TYPE_Q4_K, w4, K, N)
        W6 = ctx.upload_weight(B.GGML_TYPE_Q6_K, w6, K, N)
        assert np.array_equal(ctx.mul_mat(W4, x), want4) and np.array_equal(ctx.mul_mat(W6, x), want6)
        assert np.array_equal(ctx.mul_mat(W4, x64), want64)              # tensor-core kernel
        xd, yd = ctx.alloc(x.nbytes), ctx.alloc(5 * N * 4)
        ctx.to_device(xd, x)
        ctx.mul_mat_dev(W4, xd, 5, yd, noalloc=True)                      # the allocation-free entry point
        ctx.synchronize()
        assert np.array_equal(ctx.from_device(yd, np.zeros((5, N), np.float32)), want4)
        ctx.free(xd)
        ctx.free(yd)
        m = dc.Model(ctx, cfg)
        m.init_synthetic(5, 0.05)
        m.finalize()
        s = m.seq_alloc()
        first = m.prefill(s, prompt)                                      # chunked prefill on the tensor cores
        run, _ = m.decode_run([s], [first], 8)                            # persistent kernel
        m.set_option("persistent", 0)
        m.seq_truncate(s, prompt.size)
        run2, _ = m.decode_run([s], [first], 8)                           # per-op kernels
        assert np.array_equal(run, run2)
        tokens.append([first] + [int(t) for t in run[:, 0]])
        m.close()
        W4.free()
        W6.free()
    assert tokens[0] == tokens[1] == tokens[2]
    for c in ctxs:
        c.close()
