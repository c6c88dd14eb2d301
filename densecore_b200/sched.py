"""Host mirror of the step scheduler (dc_b200_sched_*): continuous batching of at most four sequences with
one prefill in flight, DenseCore's engine policy for its CPU path (core/src/runtime/engine_internal.h:89,
core/src/runtime/scheduler.cpp:30-85)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from .model import Model
from .ops import _vp


class SchedEvent(C.Structure):
    _fields_ = [("request", C.c_int32), ("token", C.c_int32), ("finished", C.c_int32)]


class Scheduler:
    def __init__(self, model: Model, max_num_seqs: int = 0, max_prefill_chunk: int = 0, eos_token: int = -1):
        self.model = model
        h = C.c_void_p()
        model._check(_lib.lib().dc_b200_sched_create(model.handle, max_num_seqs, max_prefill_chunk, eos_token, C.byref(h)))
        self.handle = h
        self._ev = (SchedEvent * 16)()

    def close(self):
        if self.handle:
            _lib.lib().dc_b200_sched_destroy(self.handle)
            self.handle = None

    def add(self, prompt, max_new_tokens: int) -> int:
        p = np.ascontiguousarray(prompt, dtype=np.int32)
        rid = C.c_int(-1)
        self.model._check(_lib.lib().dc_b200_sched_add(self.handle, _vp(p), p.size, max_new_tokens, C.byref(rid)))
        return rid.value

    def step(self) -> list[tuple[int, int, int]]:
        """One unit of GPU work.  Returns [(request, token, finished)]."""
        n = C.c_int(0)
        self.model._check(_lib.lib().dc_b200_sched_step(self.handle, self._ev, 16, C.byref(n)))
        return [(self._ev[i].request, self._ev[i].token, self._ev[i].finished) for i in range(min(n.value, 16))]

    def pending(self) -> int:
        return _lib.lib().dc_b200_sched_pending(self.handle)

    def stats(self) -> dict:
        out = (C.c_uint64 * 6)()
        self.model._check(_lib.lib().dc_b200_sched_stats(self.handle, out))
        keys = ("steps", "prefill_chunks", "decode_steps", "decode_tokens", "max_batch", "prompt_tokens_cached")
        return dict(zip(keys, (int(v) for v in out)))

    def run(self) -> dict[int, list[int]]:
        """Steps until nothing is pending.  Returns request -> generated tokens."""
        out: dict[int, list[int]] = {}
        while self.pending() > 0:
            for rid, tok, _fin in self.step():
                out.setdefault(rid, []).append(tok)
        return out
