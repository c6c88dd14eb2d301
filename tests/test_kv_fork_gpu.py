"""Sequence fork with shared KV blocks and copy-on-write (BlockManager::Fork / CopyOnWrite of the
reference): a prompt is prefilled once, continuations share its blocks."""
import numpy as np
import pytest

import densecore_b200 as dc

pytestmark = pytest.mark.gpu


def test_fork_shares_blocks_and_copies_on_write(ctx):
    cfg = dc.Config(n_layer=2, hidden=512, n_head=4, n_kv_head=2, vocab=1000, n_expert=8, n_expert_used=2,
                    expert_ffn=256, max_seqs=4, max_ctx=128)
    m = dc.Model(ctx, cfg)
    m.init_synthetic(9, 0.05)
    m.finalize()
    rng = np.random.default_rng(2)
    prompt = rng.integers(0, cfg.vocab, size=40)     # 2 full blocks + 8 slots of a third
    free0 = m.free_blocks()
    a = m.seq_alloc()
    first = m.prefill(a, prompt)
    assert m.free_blocks() == free0 - 3
    b = m.seq_fork(a)
    c = m.seq_fork(a)
    assert m.free_blocks() == free0 - 3 and m.seq_len(b) == 40 == m.seq_len(c)   # nothing copied yet

    # three continuations from the same state, run together: identical tokens, and equal to a fresh sequence
    run, _ = m.decode_run([a, b, c], [first] * 3, 10)
    assert np.array_equal(run[:, 0], run[:, 1]) and np.array_equal(run[:, 0], run[:, 2])
    # the partly filled third block was copied for two of the three writers, the full blocks stay shared
    # (two copies), and each sequence took a fourth block for positions 48-49
    assert m.free_blocks() == free0 - 3 - 2 - 3
    d = m.seq_alloc()
    first_d = m.prefill(d, prompt)
    alone, _ = m.decode_run([d], [first_d], 10)
    assert first_d == first and np.array_equal(alone[:, 0], run[:, 0])
    m.seq_free(d)

    # different continuations diverge without disturbing each other
    m.seq_truncate(b, 40)
    m.seq_truncate(c, 40)
    other = (first + 7) % cfg.vocab
    rb, _ = m.decode_run([b], [other], 6)
    rc, _ = m.decode_run([c], [first], 6)
    assert np.array_equal(rc[:, 0], run[:6, 0]) and not np.array_equal(rb[:, 0], run[:6, 0])

    # the shared prefix outlives its first owner
    m.seq_free(a)
    m.seq_truncate(c, 40)
    rc2, _ = m.decode_run([c], [first], 6)
    assert np.array_equal(rc2[:, 0], run[:6, 0])
    m.seq_free(b)
    m.seq_free(c)
    assert m.free_blocks() == free0
    m.close()


def test_kv_fork_refcounts(ctx):
    kv = ctx.kv_cache(2, 2, 128, 16, 4, 8)
    lib = dc._lib.lib()
    import ctypes as C
    s0 = kv.seq_alloc()
    kv.seq_reserve(s0, 20)                      # two blocks
    blocks = kv.block_table(s0)
    s1 = C.c_int(-1)
    ctx._check(lib.dc_b200_kv_seq_fork(kv.handle, s0, C.byref(s1)))
    assert np.array_equal(kv.block_table(s1.value), blocks)
    assert [lib.dc_b200_kv_block_refcount(kv.handle, b) for b in blocks] == [2, 2]
    free = kv.free_blocks()
    kv.seq_free(s0)
    assert kv.free_blocks() == free            # still referenced by the fork
    assert [lib.dc_b200_kv_block_refcount(kv.handle, b) for b in blocks] == [1, 1]
    kv.seq_free(s1.value)
    assert kv.free_blocks() == free + 2
    kv.close()
