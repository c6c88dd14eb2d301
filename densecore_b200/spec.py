"""Speculative decoding over two models that share a vocabulary: a draft model proposes a chain of gamma
tokens, the target model scores the chain in one batched forward of gamma + 1 tokens, and the accept step
runs on the device (greedy prefix match).  Host-side loop over the library's calls; DenseCore loads a draft
model but has no such loop (core/src/runtime/engine.cpp:593-645)."""
from __future__ import annotations

import ctypes as C
import time

import numpy as np

from . import _lib
from .model import Model
from .ops import _vp


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


def verify_accept_dev(target: Model, draft_tokens, gamma: int) -> tuple[int, int]:
    """Greedy accept step on the target's device-resident logits of the last forward_chunk."""
    lib = _lib.lib()
    logits_dev = lib.dc_b200_model_logits_dev(target.handle)
    dt = np.ascontiguousarray(draft_tokens, dtype=np.int32)
    n, t = C.c_int(0), C.c_int(0)
    target._check(lib.dc_b200_verify_accept_dev(target.ctx.handle, logits_dev, _vp(dt), None, None, 0, 0, gamma,
                                                target.cfg.vocab, 0, 1.0, C.byref(n), C.byref(t)))
    return n.value, t.value


def speculative_decode(target: Model, draft: Model, prompt, n_out: int, gamma: int = 4, forced_drafts=None):
    """Greedy speculative decoding.  Returns (tokens [n_out], SpecStats).

    forced_drafts(position, gamma) -> ids, if given, replaces the draft model's proposals (used to sweep the
    acceptance rate with synthetic drafts)."""
    assert target.cfg.vocab == draft.cfg.vocab and 1 <= gamma <= 15
    prompt = np.ascontiguousarray(prompt, dtype=np.int32)
    ts, ds = target.seq_alloc(), draft.seq_alloc()
    stats = SpecStats()
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
            if forced_drafts is None:
                run, _ = draft.decode_run([ds], [last], gamma)
                drafts = run[:, 0].astype(np.int32)
            else:
                drafts = np.asarray(forced_drafts(len(out), gamma), dtype=np.int32)
            target.forward_chunk(ts, np.concatenate([[last], drafts]).astype(np.int32), want_logits=False)
            n_acc, nxt = verify_accept_dev(target, drafts, gamma)
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
        target.seq_free(ts)
        draft.seq_free(ds)
