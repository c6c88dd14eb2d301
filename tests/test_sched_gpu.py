"""Step scheduler and hash-keyed prefix cache (core/src/runtime/scheduler.cpp:30-85,
core/src/runtime/memory/kv_cache_block_manager.cpp:364-416,515-522): requests that share a prompt prefix
prefill it once; at most four sequences decode together while one prompt is being prefilled in chunks."""
import ctypes as C

import numpy as np
import pytest

import densecore_b200 as dc

pytestmark = pytest.mark.gpu


def small_model(ctx, max_seqs=4, max_ctx=1280, blocks_per_seq=None):
    cfg = dc.Config(n_layer=2, hidden=512, n_head=4, n_kv_head=2, vocab=1000, n_expert=8, n_expert_used=2,
                    expert_ffn=256, max_seqs=max_seqs, max_ctx=max_ctx)
    m = dc.Model(ctx, cfg)
    m.init_synthetic(11, 0.05)
    m.finalize()
    return m, cfg


def fnv_prefix_hash(tokens):
    h = 14695981039346656037
    for t in tokens:
        h ^= int(t) & 0xFFFFFFFFFFFFFFFF
        h = (h * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


def test_two_requests_sharing_a_1024_token_prefix_prefill_it_once(ctx):
    m, cfg = small_model(ctx)
    # token-for-token comparison of a prompt run whole and run as cached prefix + tail: the sixteen-token prefill
    # path, whose results do not depend on where a prompt is cut
    m.set_option("tc_prefill", 0)
    rng = np.random.default_rng(5)
    prefix = rng.integers(0, cfg.vocab, size=1024)
    p1 = np.concatenate([prefix, rng.integers(0, cfg.vocab, size=37)])
    p2 = np.concatenate([prefix, rng.integers(0, cfg.vocab, size=21)])

    # without the cache: the tokens to expect
    want = []
    for p in (p1, p2):
        s = m.seq_alloc()
        first = m.prefill(s, p)
        run, _ = m.decode_run([s], [first], 8)
        want.append([first] + [int(t) for t in run[:, 0]])
        m.seq_free(s)
    base = m.prefix_stats()["prefill_tokens_run"]
    assert base == p1.size + p2.size

    m.set_option("prefix_cache", 1)
    free0 = m.free_blocks()
    got = []
    ran = []
    for p in (p1, p2):
        before = m.prefix_stats()["prefill_tokens_run"]
        s = m.seq_alloc()
        first = m.prefill(s, p)
        ran.append(m.prefix_stats()["prefill_tokens_run"] - before)
        run, _ = m.decode_run([s], [first], 8)
        got.append([first] + [int(t) for t in run[:, 0]])
        m.seq_free(s)
    assert ran == [p1.size, p2.size - 1024], ran           # the second request ran only its own 21 tokens
    assert got == want                                    # and decoded exactly the tokens of the uncached runs
    st = m.prefix_stats()
    assert st["hit_blocks"] == 64 and st["lookups"] == 2
    # both sequences are gone, the cached blocks stay resident but count as available
    assert st["resident_blocks"] == (p1.size // 16) + ((p2.size // 16) - 64) and m.free_blocks() == free0

    # a prompt that is exactly the cached prefix must leave one token to run: 63 blocks reused, 16 tokens run
    before = m.prefix_stats()["prefill_tokens_run"]
    s = m.seq_alloc()
    m.prefill(s, prefix)
    assert m.prefix_stats()["prefill_tokens_run"] - before == 16
    m.seq_free(s)
    # same block contents behind another left context do not match (the key is the whole prefix)
    other = np.concatenate([rng.integers(0, cfg.vocab, size=16), prefix[16:]])
    before = m.prefix_stats()
    s = m.seq_alloc()
    m.prefill(s, other)
    after = m.prefix_stats()
    assert after["hit_blocks"] == before["hit_blocks"] and after["prefill_tokens_run"] - before["prefill_tokens_run"] == other.size
    m.seq_free(s)
    m.close()


def test_prefix_cache_at_the_block_manager(ctx):
    """Attach / register on a bare cache: hashing, token verification, sharing and eviction order."""
    kv = ctx.kv_cache(1, 2, 128, 8, 4, 8)          # 8 blocks in all
    lib = dc._lib.lib()
    toks = np.arange(100, 100 + 48, dtype=np.int32)   # three whole blocks
    n = C.c_int(-1)

    def attach(seq, t):
        t = np.ascontiguousarray(t, dtype=np.int32)
        assert lib.dc_b200_kv_prefix_attach(kv.handle, seq, t.ctypes.data_as(C.c_void_p), t.size, C.byref(n)) == 0
        return n.value

    def register(seq, t):
        t = np.ascontiguousarray(t, dtype=np.int32)
        assert lib.dc_b200_kv_prefix_register(kv.handle, seq, t.ctypes.data_as(C.c_void_p), t.size) == 0

    def stats():
        out = (C.c_uint64 * 4)()
        assert lib.dc_b200_kv_prefix_stats(kv.handle, out) == 0
        return [int(v) for v in out]

    a = kv.seq_alloc()
    assert attach(a, toks) == 0                       # nothing cached yet
    kv.seq_reserve(a, 48)
    blocks_a = kv.block_table(a).tolist()
    register(a, toks)
    assert stats()[2] == 0                            # positions not written yet register nothing
    # the op-level cache learns a sequence's length from attention calls: write position 47
    q = np.zeros((1, 4, 128), np.float32)
    k = np.zeros((1, 2, 128), np.float32)
    kv.flash_attn_decode(0, q, k, k, [a], [47], 1.0)
    register(a, toks)
    assert stats()[2] == 3
    assert [lib.dc_b200_kv_block_refcount(kv.handle, b) for b in blocks_a] == [2, 2, 2]
    b = kv.seq_alloc()
    assert attach(b, np.concatenate([toks, [7]])) == 48          # all three blocks, one token left to run
    assert kv.block_table(b).tolist() == blocks_a
    c = kv.seq_alloc()
    assert attach(c, toks) == 32                                  # a prompt equal to the prefix keeps its last block to run
    d = kv.seq_alloc()
    wrong = toks.copy()
    wrong[20] += 1
    assert attach(d, np.concatenate([wrong, [7]])) == 16          # second block differs: only the first is reused
    for s in (a, b, c, d):
        lib.dc_b200_kv_seq_free(kv.handle, s)
    assert kv.free_blocks() == 8 and stats()[2] == 3              # resident, yet available
    # filling the cache evicts the least recently used resident blocks, and their prefixes stop matching
    e = kv.seq_alloc()
    kv.seq_reserve(e, 8 * 16)
    assert stats()[3] == 3 and stats()[2] == 0
    lib.dc_b200_kv_seq_free(kv.handle, e)
    f = kv.seq_alloc()
    assert attach(f, np.concatenate([toks, [7]])) == 0
    kv.close()


def test_scheduler_batches_four_sequences_with_one_prefill_at_a_time(ctx):
    m, cfg = small_model(ctx, max_seqs=4, max_ctx=512)
    # token-for-token comparison of differently chunked prompts: the sixteen-token prefill path, whose results do
    # not depend on where a prompt is cut (the tensor-core path's flash attention and Q6_K float order do, at 1e-4)
    m.set_option("tc_prefill", 0)
    rng = np.random.default_rng(8)
    prompts = [rng.integers(0, cfg.vocab, size=n) for n in (70, 33, 150, 20, 95, 64)]
    n_new = [12, 5, 9, 14, 7, 10]
    # every request decoded alone
    want = []
    for p, k in zip(prompts, n_new):
        s = m.seq_alloc()
        first = m.prefill(s, p)
        toks = [first]
        if k > 1:
            run, _ = m.decode_run([s], [first], k - 1)
            toks += [int(t) for t in run[:, 0]]
        want.append(toks)
        m.seq_free(s)

    free0 = m.free_blocks()
    sch = dc.Scheduler(m, max_num_seqs=4, max_prefill_chunk=48)
    ids = [sch.add(p, k) for p, k in zip(prompts, n_new)]
    assert ids == list(range(6)) and sch.pending() == 6
    out = {}
    finished = {}
    kinds = []
    while sch.pending() > 0:
        before = sch.stats()
        ev = sch.step()
        after = sch.stats()
        kinds.append("p" if after["prefill_chunks"] > before["prefill_chunks"] else "d")
        for rid, tok, fin in ev:
            assert rid not in finished
            out.setdefault(rid, []).append(tok)
            if fin:
                finished[rid] = fin
    st = sch.stats()
    assert sorted(finished) == ids and set(finished.values()) == {1}
    for rid in ids:
        assert out[rid] == want[rid], rid                       # batching changes no token
    assert st["max_batch"] == 4                                  # never more than four decode together
    assert st["decode_tokens"] == sum(n_new) - 6                 # the first token of each comes from its prefill
    # prompts ran in chunks of 48, one request at a time: ceil(n / 48) chunks each
    assert st["prefill_chunks"] == sum(-(-p.size // 48) for p in prompts)
    # while sequences were running, prompt chunks and decode steps alternated
    assert "pp" not in "".join(kinds)[kinds.index("d"):]
    assert sch.step() == []                                      # idle
    sch.close()
    assert m.free_blocks() == free0                              # every sequence slot and block came back
    m.close()


def test_scheduler_end_of_sequence_and_argument_checks(ctx):
    m, cfg = small_model(ctx, max_seqs=2, max_ctx=256)
    m.set_option("tc_prefill", 0)
    rng = np.random.default_rng(9)
    p = rng.integers(0, cfg.vocab, size=30)
    s = m.seq_alloc()
    first = m.prefill(s, p)
    run, _ = m.decode_run([s], [first], 6)
    m.seq_free(s)
    stream = [first] + [int(t) for t in run[:, 0]]
    eos = stream[3]
    cut = stream.index(eos)
    sch = dc.Scheduler(m, max_num_seqs=2, eos_token=eos)
    rid = sch.add(p, 20)
    out = sch.run()
    assert out[rid] == stream[:cut + 1]                          # stops with the end-of-sequence token
    with pytest.raises(dc.DcError):
        sch.add([], 4)
    with pytest.raises(dc.DcError):
        sch.add(p, 0)
    with pytest.raises(dc.DcError):
        sch.add([cfg.vocab], 4)
    with pytest.raises(dc.DcError):
        sch.add(p, 1000)                                          # beyond max_ctx
    sch.close()
    with pytest.raises(dc.DcError):
        dc.Scheduler(m, max_num_seqs=3)                           # the model holds two sequences
    m.close()
