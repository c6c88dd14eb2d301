"""Decoder-level host mirror: model configs of the benchmark and the Model class
over dc_b200_model_* (the chained ops of one Qwen3-style decoder step)."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, asdict

import numpy as np

from . import _lib
from .blocks import GGML_TYPE_F32, GGML_TYPE_Q4_K, GGML_TYPE_Q6_K, row_bytes
from .ops import Context, _vp


@dataclass
class Config:
    n_layer: int
    hidden: int
    n_head: int
    n_kv_head: int
    vocab: int
    head_dim: int = 128
    ffn: int = 0
    n_expert: int = 0
    n_expert_used: int = 0
    expert_ffn: int = 0
    rms_eps: float = 1e-6
    rope_theta: float = 1e6
    routed_scale: float = 1.0
    tie_embeddings: bool = False
    qk_norm: bool = True
    max_seqs: int = 4
    max_ctx: int = 2560
    ep_rank: int = 0
    ep_size: int = 1

    def to_c(self) -> _lib.ModelConfig:
        d = asdict(self)
        c = _lib.ModelConfig()
        for k, v in d.items():
            setattr(c, k, int(v) if isinstance(v, bool) else v)
        return c


def dense_0p8b(**kw) -> Config:
    """Dense 0.8B-class Qwen3-style decoder: 28 layers, hidden 1024, FFN 3072, 16 Q / 8 KV heads, tied embeddings."""
    return Config(n_layer=28, hidden=1024, n_head=16, n_kv_head=8, vocab=151936, ffn=3072, tie_embeddings=True, **kw)


def moe_35b_a3b(**kw) -> Config:
    """35B-A3B-class MoE decoder: 48 layers, hidden 2048, 32 Q / 4 KV heads, 128 experts top-8 x 768, untied lm_head."""
    return Config(n_layer=48, hidden=2048, n_head=32, n_kv_head=4, vocab=151936, n_expert=128, n_expert_used=8,
                  expert_ffn=768, tie_embeddings=False, **kw)


def fnv1a64(name: str) -> int:
    h = 1469598103934665603
    for b in name.encode():
        h ^= b
        h = (h * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


def tensor_seed(seed: int, name: str) -> int:
    """Seed init_synthetic uses for one tensor: model seed + FNV-1a(name), mod 2^64."""
    return (seed + fnv1a64(name)) & 0xFFFFFFFFFFFFFFFF


class Model:
    def __init__(self, ctx: Context, cfg: Config):
        self.ctx, self.cfg = ctx, cfg
        self.handle = None
        h = C.c_void_p()
        cc = cfg.to_c()
        ctx._check(_lib.lib().dc_b200_model_create(ctx.handle, C.byref(cc), C.byref(h)))
        self.handle = h

    @classmethod
    def from_gguf(cls, ctx: Context, path: str, max_seqs: int = 4, max_ctx: int = 0, ep_rank: int = 0, ep_size: int = 1):
        """Model with configuration and tensors read from a GGUF file (not yet finalized)."""
        h = C.c_void_p()
        ctx._check(_lib.lib().dc_b200_model_from_gguf(ctx.handle, path.encode(), max_seqs, max_ctx, ep_rank, ep_size,
                                                      C.byref(h)))
        cc = _lib.ModelConfig()
        ctx._check(_lib.lib().dc_b200_model_get_config(h, C.byref(cc)))
        self = cls.__new__(cls)
        self.ctx, self.handle = ctx, h
        kw = {name: getattr(cc, name) for name, _ in _lib.ModelConfig._fields_}
        kw["tie_embeddings"], kw["qk_norm"] = bool(kw["tie_embeddings"]), bool(kw["qk_norm"])
        self.cfg = Config(**kw)
        return self

    def tensor_names(self):
        n = C.c_int(0)
        self._check(_lib.lib().dc_b200_model_tensor_names(self.handle, None, 0, C.byref(n)))
        arr = (C.c_char_p * n.value)()
        self._check(_lib.lib().dc_b200_model_tensor_names(self.handle, arr, n.value, C.byref(n)))
        return [a.decode() for a in arr]

    def close(self):
        if self.handle:
            _lib.lib().dc_b200_model_destroy(self.handle)
            self.handle = None

    def _check(self, st):
        self.ctx._check(st)

    def set_option(self, name: str, value: int):
        self._check(_lib.lib().dc_b200_model_set_option(self.handle, name.encode(), int(value)))

    def set_tensor(self, name: str, ggml_type: int, data: np.ndarray, K: int, N: int = 1, E: int = 1):
        data = np.ascontiguousarray(data)
        ne = (C.c_int64 * 4)(K, N, E, 1)
        self._check(_lib.lib().dc_b200_model_set_tensor(self.handle, name.encode(), ggml_type, ne, _vp(data)))

    def init_synthetic(self, seed: int, sigma: float = 0.02):
        self._check(_lib.lib().dc_b200_model_init_synthetic(self.handle, seed, sigma))

    def get_tensor_info(self, name: str):
        t = C.c_int(0)
        ne = (C.c_int64 * 4)()
        dev = C.c_void_p()
        nb = C.c_size_t(0)
        self._check(_lib.lib().dc_b200_model_get_tensor(self.handle, name.encode(), C.byref(t), ne, C.byref(dev),
                                                        C.byref(nb)))
        return t.value, tuple(ne), dev.value, nb.value

    def get_tensor(self, name: str):
        """Downloads a tensor's bytes: (ggml_type, (K, N, E), uint8 array or f32 array)."""
        t, ne, dev, nb = self.get_tensor_info(name)
        out = np.zeros(nb, dtype=np.uint8)
        self.ctx.from_device(dev, out)
        if t == GGML_TYPE_F32:
            out = out.view(np.float32)
        return t, ne[:3], out

    def ep_init(self, unique_id: bytes, nccl_path: str | None = None):
        buf = (C.c_char * 128).from_buffer_copy(unique_id)
        self._check(_lib.lib().dc_b200_model_ep_init(self.handle, nccl_path.encode() if nccl_path else None, buf))

    def ep_export(self) -> bytes:
        """64-byte handle of this rank's exchange buffer (hand it to every other rank)."""
        buf = (C.c_char * 64)()
        self._check(_lib.lib().dc_b200_model_ep_export(self.handle, buf))
        return bytes(buf.raw)

    def ep_import(self, rank: int, handle: bytes):
        buf = (C.c_char * 64).from_buffer_copy(handle)
        self._check(_lib.lib().dc_b200_model_ep_import(self.handle, rank, buf))

    def finalize(self):
        self._check(_lib.lib().dc_b200_model_finalize(self.handle))

    def weight_bytes(self) -> int:
        return int(_lib.lib().dc_b200_model_weight_bytes(self.handle))

    def seq_alloc(self) -> int:
        s = C.c_int(-1)
        self._check(_lib.lib().dc_b200_seq_alloc(self.handle, C.byref(s)))
        return s.value

    def seq_fork(self, seq: int) -> int:
        """New sequence sharing seq's KV blocks (copy-on-write)."""
        s = C.c_int(-1)
        self._check(_lib.lib().dc_b200_seq_fork(self.handle, seq, C.byref(s)))
        return s.value

    def free_blocks(self) -> int:
        return _lib.lib().dc_b200_model_free_blocks(self.handle)

    def seq_free(self, seq: int):
        self._check(_lib.lib().dc_b200_seq_free(self.handle, seq))

    def seq_len(self, seq: int) -> int:
        return _lib.lib().dc_b200_seq_len(self.handle, seq)

    def seq_truncate(self, seq: int, new_len: int):
        self._check(_lib.lib().dc_b200_seq_truncate(self.handle, seq, new_len))

    def prefill(self, seq: int, tokens, want_logits: bool = False):
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        logits = np.empty(self.cfg.vocab, dtype=np.float32) if want_logits else None
        nxt = C.c_int(0)
        self._check(_lib.lib().dc_b200_prefill(self.handle, seq, _vp(tokens), tokens.size, _vp(logits), C.byref(nxt)))
        return (nxt.value, logits) if want_logits else nxt.value

    def decode_step(self, seqs, tokens, want_logits: bool = False):
        seqs = np.ascontiguousarray(seqs, dtype=np.int32)
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        out = np.zeros(seqs.size, dtype=np.int32)
        logits = np.empty((seqs.size, self.cfg.vocab), dtype=np.float32) if want_logits else None
        self._check(_lib.lib().dc_b200_decode_step(self.handle, _vp(seqs), seqs.size, _vp(tokens), _vp(out), _vp(logits)))
        return (out, logits) if want_logits else out

    def decode_run(self, seqs, first_tokens, n_steps: int):
        """Device-resident greedy loop.  Returns (tokens [n_steps, n_seq], device milliseconds)."""
        seqs = np.ascontiguousarray(seqs, dtype=np.int32)
        first = np.ascontiguousarray(first_tokens, dtype=np.int32)
        out = np.zeros((n_steps, seqs.size), dtype=np.int32)
        ms = C.c_float(0.0)
        self._check(_lib.lib().dc_b200_decode_run(self.handle, _vp(seqs), seqs.size, _vp(first), n_steps, _vp(out),
                                                  C.byref(ms)))
        return out, ms.value

    def forward_chunk(self, seq: int, tokens, want_logits: bool = True):
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        logits = np.empty((tokens.size, self.cfg.vocab), dtype=np.float32) if want_logits else None
        self._check(_lib.lib().dc_b200_forward_chunk(self.handle, seq, _vp(tokens), tokens.size, _vp(logits)))
        return logits

    def prefix_stats(self) -> dict:
        """Prefix-cache counters: lookups, blocks hit, blocks resident, evictions, prompt tokens run."""
        out = (C.c_uint64 * 5)()
        self._check(_lib.lib().dc_b200_model_prefix_stats(self.handle, out))
        return dict(zip(("lookups", "hit_blocks", "resident_blocks", "evictions", "prefill_tokens_run"), (int(v) for v in out)))

    def read_layer_input(self, layer: int, n_tokens: int = 1) -> np.ndarray:
        """Hidden state that entered `layer` in the last step (layer == n_layer: what entered the output norm).
        Needs set_option("capture_layer_inputs", 1) before the step."""
        out = np.zeros((n_tokens, self.cfg.hidden), dtype=np.float32)
        self._check(_lib.lib().dc_b200_model_read_layer_input(self.handle, layer, n_tokens, _vp(out)))
        return out

    def read_kv(self, layer: int, seq: int, first: int, n_tokens: int):
        """fp16 K and V rows [n_tokens, n_kv_head, 128] (as uint16) of positions first.. of a sequence."""
        k = np.zeros((n_tokens, self.cfg.n_kv_head, 128), dtype=np.uint16)
        v = np.zeros_like(k)
        self._check(_lib.lib().dc_b200_model_read_kv(self.handle, layer, seq, first, n_tokens, _vp(k), _vp(v)))
        return k, v

    def step_stats(self):
        k = C.c_int(0)
        wb = C.c_double(0.0)
        kv = C.c_double(0.0)
        self._check(_lib.lib().dc_b200_model_step_stats(self.handle, C.byref(k), C.byref(wb), C.byref(kv)))
        return k.value, wb.value, kv.value

    def profile_step(self, seqs, tokens):
        """One eager decode step timed per kernel class.  Returns {class: (ms, launches, algorithmic bytes)}."""
        seqs = np.ascontiguousarray(seqs, dtype=np.int32)
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        n = 16
        ms = np.zeros(n, np.float32)
        launches = np.zeros(n, np.int32)
        nbytes = np.zeros(n, np.float64)
        self._check(_lib.lib().dc_b200_model_profile_step(self.handle, _vp(seqs), seqs.size, _vp(tokens), n, _vp(ms),
                                                          _vp(launches), _vp(nbytes)))
        out = {}
        for i in range(n):
            name = _lib.lib().dc_b200_kernel_class_name(i)
            if name and launches[i]:
                out[name.decode()] = (float(ms[i]), int(launches[i]), float(nbytes[i]))
        return out

    PHASES = ["(outside)", "x assemble", "attn_norm+q8", "qkv rows", "barrier", "scores", "barrier", "pv+merge", "barrier",
              "attn q8 fill", "o-proj rows", "barrier", "ffn_norm+q8", "router logits", "barrier", "top-k+buckets",
              "gate/up rows", "barrier", "h q8", "down rows", "barrier", "lm_head+barrier",
              "sub22", "sub23", "sub24", "sub25", "sub26", "sub27"]

    def phase_timing(self):
        """Nanoseconds per phase boundary accumulated by the persistent kernel (option phase_timing=1)."""
        out = np.zeros(len(self.PHASES), dtype=np.uint64)
        self._check(_lib.lib().dc_b200_model_phase_timing(self.handle, _vp(out), out.size))
        return dict(zip(range(len(self.PHASES)), zip(self.PHASES, out.tolist())))

    BARRIERS = ["after qkv rows", "after scores", "after pv+merge", "after o-proj", "after router logits",
                "after gate/up", "after down"]

    def barrier_trace(self, n_cta: int = 148):
        """(arrive, release) arrays [7, n_cta] of globaltimer nanoseconds: when each CTA reached and left the seven
        grid barriers of the second layer in the first step of the last launch.  All zero unless the library was
        built with -DDC_MEGA_SUBMARKS and phase_timing is on."""
        buf = np.zeros(32 + 14 * 160, dtype=np.uint64)
        self._check(_lib.lib().dc_b200_model_phase_timing(self.handle, _vp(buf), buf.size))
        tr = buf[32:].reshape(14, 160)[:, :n_cta].astype(np.int64)
        return tr[:7], tr[7:]

    WTRACE_POINTS = ["layer start", "norm+q8 done", "qkv rows done", "barrier", "scores done", "barrier", "pv+merge done",
                     "barrier", "o-proj rows done", "barrier", "norm+router done", "barrier", "top-k done",
                     "gate/up rows done", "barrier", "h q8 done", "down rows done", "barrier"]

    def warp_trace(self, n_cta: int = 148):
        """[18, n_cta, 16] globaltimer nanoseconds: when every warp of every CTA passed each point of the second
        layer in the first step of the last launch (instrumented build with phase_timing on; zeros otherwise)."""
        n = 32 + 14 * 160 + 18 * 2560
        buf = np.zeros(n, dtype=np.uint64)
        self._check(_lib.lib().dc_b200_model_phase_timing(self.handle, _vp(buf), buf.size))
        return buf[32 + 14 * 160:].reshape(18, 160, 16)[:, :n_cta].astype(np.int64)
