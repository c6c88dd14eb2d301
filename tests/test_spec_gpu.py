"""Speculative decoding end to end: draft chain, one batched target forward, device-side greedy accept.
The emitted tokens must be the target's own greedy tokens whatever the draft proposes."""
import numpy as np
import pytest

import densecore_b200 as dc

pytestmark = pytest.mark.gpu


def models(ctx):
    tcfg = dc.Config(n_layer=2, hidden=512, n_head=4, n_kv_head=2, vocab=1000, n_expert=8, n_expert_used=2,
                     expert_ffn=256, max_seqs=2, max_ctx=256)
    dcfg = dc.Config(n_layer=1, hidden=512, n_head=4, n_kv_head=2, vocab=1000, ffn=512, tie_embeddings=True, max_seqs=2,
                     max_ctx=256)
    target, draft = dc.Model(ctx, tcfg), dc.Model(ctx, dcfg)
    target.init_synthetic(21, 0.05)
    draft.init_synthetic(22, 0.05)
    target.finalize()
    draft.finalize()
    return target, draft


def plain_greedy(m, prompt, n_out):
    s = m.seq_alloc()
    first = m.prefill(s, prompt)
    out = [first]
    last = first
    for _ in range(n_out - 1):     # one token per step through the batched entry point, as the verify forward does
        lg = m.forward_chunk(s, np.array([last], dtype=np.int32))
        last = int(np.argmax(lg[0]))
        out.append(last)
    m.seq_free(s)
    return np.array(out, dtype=np.int32)


def test_speculative_decode_emits_the_targets_greedy_tokens(ctx):
    target, draft = models(ctx)
    prompt = np.random.default_rng(1).integers(0, 1000, size=40)
    n_out = 48
    want = plain_greedy(target, prompt, n_out + 8)
    got, st = dc.speculative_decode(target, draft, prompt, n_out, gamma=4)
    assert st.steps > 0 and st.proposed == 4 * st.steps and 0 <= st.accepted <= st.proposed
    assert st.emitted == st.accepted + st.steps
    assert np.array_equal(got, want[:n_out]), (got, want[:n_out])

    # synthetic drafts at forced acceptance rates (drafts built from the target's own tokens)
    def forced(rate):
        def f(pos, gamma):
            true = want[pos:pos + gamma].copy()
            if rate == 0.0:
                true[0] = (true[0] + 1) % 1000
            elif rate == 0.5:
                true[gamma // 2] = (true[gamma // 2] + 1) % 1000
            return true
        return f
    for rate, per_step in ((1.0, 5.0), (0.5, 3.0), (0.0, 1.0)):
        got, st = dc.speculative_decode(target, draft, prompt, 40, gamma=4, forced_drafts=forced(rate))
        assert np.array_equal(got, want[:40]), rate
        assert abs(st.tokens_per_step - per_step) < 1e-9, (rate, st.tokens_per_step)
    target.close()
    draft.close()


def test_stochastic_speculative_decode_replays_on_the_cpu(ctx, oracle):
    """Config-5 style loop at temperature 0.8 with sampled drafts: every decision the device takes (the draft's
    sampled tokens, how many are accepted, the resampled or bonus token) is replayed by the CPU restatement of
    the rule from the very logits the device used and the same Philox uniforms, and must agree bit for bit."""
    from densecore_b200.spec import DRAFT_STREAM
    target, draft = models(ctx)
    prompt = np.random.default_rng(3).integers(0, 1000, size=24)
    gamma, T, seed = 4, 0.8, 777
    trace = []
    got, st = dc.speculative_decode(target, draft, prompt, 40, gamma=gamma, mode=1, temperature=T, seed=seed, trace=trace)
    assert st.steps == len(trace) and st.emitted == st.accepted + st.steps
    seen = set()
    pos = 1
    for rec in trace:
        u_d = oracle.verify_uniforms(seed ^ DRAFT_STREAM, rec["step"], gamma)
        q = np.stack([oracle.det_softmax(r, T) for r in rec["draft_logits"]])
        drafts = [oracle.det_inverse_cdf(q[i], float(u_d[i])) for i in range(gamma)]
        assert drafts == rec["drafts"].tolist(), rec["step"]
        u = oracle.verify_uniforms(seed, rec["step"], gamma + 1)
        n_acc, nxt = oracle.verify_accept(rec["target_logits"], drafts, q, u, 1, T)
        assert (n_acc, nxt) == (rec["n_accepted"], rec["next_token"]), rec["step"]
        emitted = drafts[:n_acc] + [nxt]
        assert got[pos:pos + len(emitted)].tolist() == emitted[:max(0, len(got) - pos)]
        pos += len(emitted)
        seen.add(n_acc)
    assert len(seen) > 1, "accepts and rejections should both occur"
    target.close()
    draft.close()
