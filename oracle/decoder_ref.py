"""CPU reference of one decoder step, composed from the C oracle's ops.

TEST INFRASTRUCTURE ONLY (see oracle/dc_oracle.c).  Follows the graph DenseCore
builds for a Qwen3-style decoder (core/src/llm/graph/decoder.cpp: attn_norm :453,
QKV :1085-1100, per-head Q/K norm :1265-1343, RoPE :1422-1450, paged attention
:1846-1872, ffn_norm :2201, MoE :2217-2410 or SwiGLU FFN :2662-2730, lm_head :2997).
Tokens are processed one at a time; small models only.
"""
from __future__ import annotations

import numpy as np

from . import oracle as o

F32 = np.float32


def fast_exp_np(x: np.ndarray) -> np.ndarray:
    """Vectorised dco_fast_exp (core/src/backend/cpu_backend_internal.h:99-114): float32 steps, no FMA."""
    x = np.clip(x.astype(F32), F32(-50.0), F32(50.0))
    y = x * F32(1.4426950408889634)
    i = np.floor(y)
    f = (y - i).astype(F32)
    p = F32(1.0) + f * (F32(0.6960656421638072) + f * (F32(0.224494337302845) + f * F32(0.07944023841053369)))
    two_i = ((i.astype(np.int32) + 127) << 23).astype(np.int32).view(F32)
    return (two_i * p).astype(F32)


def silu_fast_np(g: np.ndarray) -> np.ndarray:
    g = g.astype(F32)
    return (g / (F32(1.0) + fast_exp_np(-g))).astype(F32)


class RefModel:
    def __init__(self, cfg, tensors: dict):
        """cfg: densecore_b200.model.Config-like.  tensors: name -> (ggml_type, (K, N, E), ndarray)."""
        self.cfg = cfg
        self.t = tensors
        self.bps = (cfg.max_ctx + 15) // 16
        shape = (cfg.max_seqs * self.bps * 16, cfg.n_kv_head, 128)
        self.k = [np.zeros(shape, dtype=np.uint16) for _ in range(cfg.n_layer)]
        self.v = [np.zeros(shape, dtype=np.uint16) for _ in range(cfg.n_layer)]
        self.rope = o.rope_table(cfg.max_ctx, 128, cfg.rope_theta)
        self.lens = {}
        self.last_route = None

    def table(self, seq: int) -> np.ndarray:
        return np.arange(seq * self.bps, (seq + 1) * self.bps, dtype=np.int32)

    def mm(self, name: str, x: np.ndarray) -> np.ndarray:
        ty, (K, N, E), data = self.t[name]
        return o.mul_mat(ty, data, N, K, x.reshape(1, K))[0]

    def vec(self, name: str) -> np.ndarray:
        return self.t[name][2]

    def embed(self, tok: int) -> np.ndarray:
        ty, (K, N, E), data = self.t["token_embd.weight"]
        rb = o.row_bytes(ty, K)
        row = np.ascontiguousarray(data.reshape(N, rb)[tok])
        return o.dequantize(ty, row, 1, K)[0]

    def layer(self, il: int, x: np.ndarray, pos: int, k_arena: np.ndarray, v_arena: np.ndarray, table: np.ndarray,
              route_mode: str = "stable"):
        """One decoder layer for one token at position `pos`: x [hidden] -> x_out [hidden].  The token's K/V
        row is written into (k_arena, v_arena) at `pos` through `table`; earlier rows are whatever the arenas
        hold.  Also records the router logits and the routing of the layer in self.last_route."""
        c = self.cfg
        p = f"blk.{il}."
        scale = F32(1.0 / np.sqrt(np.float32(c.head_dim)))
        xn = o.rms_norm(x, self.vec(p + "attn_norm.weight"), c.rms_eps)
        q = self.mm(p + "attn_q.weight", xn).reshape(c.n_head, 128)
        k = self.mm(p + "attn_k.weight", xn).reshape(c.n_kv_head, 128)
        v = self.mm(p + "attn_v.weight", xn).reshape(c.n_kv_head, 128)
        if c.qk_norm:
            qw, kw = self.vec(p + "attn_q_norm.weight"), self.vec(p + "attn_k_norm.weight")
            q = np.stack([o.rms_norm(h, qw, c.rms_eps) for h in q])
            k = np.stack([o.rms_norm(h, kw, c.rms_eps) for h in k])
        q = o.rope(q, self.rope[pos])
        k = o.rope(k, self.rope[pos])
        o.kv_write(k_arena, v_arena, table, pos, c.n_kv_head, 128, k, v)
        att = o.paged_attention(q, k_arena, v_arena, table, pos, c.n_head, c.n_kv_head, 128, float(scale),
                                mode="blockwise")
        x = (x + self.mm(p + "attn_output.weight", att.reshape(-1))).astype(F32)
        xn = o.rms_norm(x, self.vec(p + "ffn_norm.weight"), c.rms_eps)
        if c.n_expert > 0:
            rl = self.mm(p + "ffn_gate_inp.weight", xn)
            ids, w = o.route(rl, c.n_expert_used, mode=route_mode, scale=c.routed_scale)
            self.last_route = (rl, ids, w)
            gt, _, gd = self.t[p + "ffn_gate_exps.weight"]
            ut, _, ud = self.t[p + "ffn_up_exps.weight"]
            dt, _, dd = self.t[p + "ffn_down_exps.weight"]
            y = o.moe_forward((gt, ut, dt), gd, ud, dd, c.n_expert, c.hidden, c.expert_ffn, xn.reshape(1, -1), ids,
                              w, fast_exp=True)[0]
            return (x + y).astype(F32)
        gate = self.mm(p + "ffn_gate.weight", xn)
        up = self.mm(p + "ffn_up.weight", xn)
        h = (silu_fast_np(gate) * up).astype(F32)
        return (x + self.mm(p + "ffn_down.weight", h)).astype(F32)

    def head(self, x: np.ndarray) -> np.ndarray:
        """Output norm and lm_head: x [hidden] -> logits [vocab]."""
        c = self.cfg
        xn = o.rms_norm(x, self.vec("output_norm.weight"), c.rms_eps)
        return self.mm("token_embd.weight" if c.tie_embeddings else "output.weight", xn)

    def step(self, seq: int, tok: int, want_logits: bool = True, route_mode: str = "stable"):
        c = self.cfg
        pos = self.lens.get(seq, 0)
        table = self.table(seq)
        x = self.embed(tok)
        for il in range(c.n_layer):
            x = self.layer(il, x, pos, self.k[il], self.v[il], table, route_mode)
        self.lens[seq] = pos + 1
        return self.head(x) if want_logits else None
