"""Speculative decoding over two models that share a vocabulary: a draft model proposes a chain of gamma
tokens, the target model scores the chain in one batched forward of gamma + 1 tokens, and the accept step
runs on the device: greedy prefix match (mode 0), or the stochastic rule at a temperature (mode 1): the draft
samples its tokens from q = softmax(draft logits / T), token i is accepted iff u_i * q_i[t_i] < p_i[t_i], the
first rejected position is resampled from max(0, p - q), and a fully accepted chain earns a bonus token from
p.  All uniforms come from Philox4x32-10 keyed by (seed, step).  Host-side loop over the library's calls;
DenseCore loads a draft model but has no such loop (core/src/runtime/engine.cpp:593-645)."""
from __future__ import annotations

import ctypes as C
import time

import numpy as np

from . import _lib
from .model import Model
from .ops import _vp

DRAFT_STREAM = 0x9E3779B97F4A7C15      # the draft's uniforms come from (seed ^ this, step)


class SpecStats:
    def __init__(self):
        self.steps = self.proposed = self.accepted = self.emitted = 0
        self.seconds = 0.0

    @property
    def acceptance(self) -> float:
        return self.accepted / self.proposed if self.proposed else 0.0

    @property
    def tokens_per_step(self) -> float:
        return self.emitted / self.steps if self.steps else 0.0


def verify_accept_dev(target: Model, draft_tokens, gamma: int, mode: int = 0, draft_probs_dev: int = 0,
                      temperature: float = 1.0, seed: int = 0, step: int = 0) -> tuple[int, int]:
    """Accept step on the target's device-resident logits of the last forward_chunk."""
    lib = _lib.lib()
    logits_dev = lib.dc_b200_model_logits_dev(target.handle)
    dt = np.ascontiguousarray(draft_tokens, dtype=np.int32)
    n, t = C.c_int(0), C.c_int(0)
    target._check(lib.dc_b200_verify_accept_dev(target.ctx.handle, logits_dev, _vp(dt),
                                                C.c_void_p(draft_probs_dev) if mode == 1 else None, None, seed, step,
                                                gamma, target.cfg.vocab, mode, temperature, C.byref(n), C.byref(t)))
    return n.value, t.value


def sample_dev(model: Model, temperature: float, u: float, probs_dev: int) -> int:
    """One token drawn from the model's device-resident logits of its last single-token step; probs_dev receives
    the distribution it was drawn from."""
    lib = _lib.lib()
    tok = C.c_int(-1)
    model._check(lib.dc_b200_sample_dev(model.ctx.handle, lib.dc_b200_model_logits_dev(model.handle), model.cfg.vocab,
                                        temperature, u, C.c_void_p(probs_dev), C.byref(tok)))
    return tok.value


def speculative_decode(target: Model, draft: Model, prompt, n_out: int, gamma: int = 4, forced_drafts=None,
                       mode: int = 0, temperature: float = 0.8, seed: int = 1234, trace: list | None = None):
    """Speculative decoding.  Returns (tokens [n_out], SpecStats).

    mode 0: greedy drafts and greedy accept (the output is the target's greedy stream).  mode 1: sampled drafts
    and the stochastic accept rule at `temperature`.
    forced_drafts(position, gamma) -> ids, if given, replaces the draft model's proposals in mode 0 (used to
    sweep the acceptance rate with synthetic drafts).
    trace (mode 1, small vocabularies): every step appends the logits the device decided on, so that a checker
    can replay the step's decisions: dict(draft_logits [gamma, V], target_logits [gamma + 1, V], drafts,
    n_accepted, next_token, step)."""
    assert target.cfg.vocab == draft.cfg.vocab and 1 <= gamma <= 15
    prompt = np.ascontiguousarray(prompt, dtype=np.int32)
    ts, ds = target.seq_alloc(), draft.seq_alloc()
    stats = SpecStats()
    V = target.cfg.vocab
    ctx = target.ctx
    qbuf = ctx.alloc(gamma * V * 4) if mode == 1 else 0
    try:
        last = target.prefill(ts, prompt)           # first output token: the target's own pick
        draft.prefill(ds, prompt)
        out = [last]
        t0 = time.perf_counter()
        while len(out) < n_out:
            # the draft's cache may lack the newest committed tokens (all drafts accepted last time)
            committed = len(prompt) + len(out) - 1  # tokens whose K/V both caches must hold before `last`
            behind = committed - draft.seq_len(ds)
            if behind > 0:
                draft.forward_chunk(ds, np.array(out[-1 - behind:-1], dtype=np.int32), want_logits=False)
            step = stats.steps
            dl = []
            if mode == 1:
                u_d = ctx.verify_uniforms(seed ^ DRAFT_STREAM, step, gamma)
                drafts, tok = [], last
                for i in range(gamma):
                    if trace is not None:
                        _, lg = draft.decode_step([ds], [tok], want_logits=True)
                        dl.append(lg[0].copy())
                    else:
                        draft.decode_step([ds], [tok])
                    tok = sample_dev(draft, temperature, float(u_d[i]), qbuf + i * V * 4)
                    drafts.append(tok)
                drafts = np.array(drafts, dtype=np.int32)
            elif forced_drafts is None:
                run, _ = draft.decode_run([ds], [last], gamma)
                drafts = run[:, 0].astype(np.int32)
            else:
                drafts = np.asarray(forced_drafts(len(out), gamma), dtype=np.int32)
            tl = target.forward_chunk(ts, np.concatenate([[last], drafts]).astype(np.int32), want_logits=trace is not None)
            n_acc, nxt = verify_accept_dev(target, drafts, gamma, mode, qbuf, temperature, seed, step)
            if trace is not None:
                trace.append(dict(draft_logits=np.stack(dl) if dl else None, target_logits=tl.copy(), drafts=drafts.copy(),
                                  n_accepted=n_acc, next_token=nxt, step=step))
            # keep `last` and the accepted drafts in both caches; the bonus / correction token is next
            target.seq_truncate(ts, committed + 1 + n_acc)
            if draft.seq_len(ds) > committed + 1 + n_acc:
                draft.seq_truncate(ds, committed + 1 + n_acc)
            out.extend(int(x) for x in drafts[:n_acc])
            out.append(nxt)
            last = nxt
            stats.steps += 1
            stats.proposed += gamma
            stats.accepted += n_acc
        stats.seconds = time.perf_counter() - t0
        stats.emitted = len(out) - 1
        return np.array(out[:n_out], dtype=np.int32), stats
    finally:
        if qbuf:
            ctx.free(qbuf)
        target.seq_free(ts)
        draft.seq_free(ds)
