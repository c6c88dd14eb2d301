#!/usr/bin/env python
"""Benchmark of the quantized decode hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): the 35B-A3B-class Q4_K_M MoE decoder (48 layers, hidden 2048,
32 Q / 4 KV heads x 128, 128 experts top-8 x 768, vocab 151936, untied lm_head),
seeded synthetic weights generated and quantised on the device, a 2048-token
random-id prompt per stream prefilled into the paged fp16 KV cache (untimed
set-up), then greedy decode.  A "step" is one decode step (one new token per
stream).  `value` = output tokens per second at 1 stream with inputs resident in
HBM (device-side token feedback, CUDA-graph replays, device time from CUDA
events on the launching stream).  `e2e` = the same metric through
dc_b200_decode_step with host buffers: every step copies the token ids host ->
device and the picked ids device -> host.  4-stream numbers ride along in
`streams4`.

N > 1: expert parallel (experts sharded in contiguous ranges, everything else
replicated, one NCCL all-reduce per MoE layer); every rank decodes the same
streams, so the whole job's tokens/s is streams x steps / max-over-ranks time
and scaling is "strong".

--impl reference: the CPU restatement of DenseCore's ggml path (oracle/) timed on
the host cores with all threads, on a bounded sample of the same step.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode tok/s (1 & 4 streams), 35B-A3B-class Q4_K_M; % HBM roofline"
UNIT = "tok/s"
PROMPT = 2048
WORKLOAD = ("moe35b_a3b_q4km decode: 48 layers, hidden 2048, 128 experts top-8, vocab 151936; "
            "2048-token random prompt per stream, greedy, paged fp16 KV")
CPU_CTX = PROMPT + 128     # context length of the CPU sample: the middle of a 256-token generation
SAMPLE_LAYERS = 4          # layers of the model the CPU baseline times per sample
SAMPLE_REPS = 12           # repeats of the sample (median taken)
# DRAM bytes (read + write) of one launch of the persistent kernel divided by its algorithmic bytes,
# measured with one ncu capture of the model cut to 4 layers (traffic is the weights, which scale with the layers)
DRAM_TRAFFIC_RATIO = 1.03


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ----------------------------------------------------------------- clocks
class ClockSampler:
    """Samples nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.proc, self.lines, self.first = gpu_index, None, [], 0

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def wait_ready(self, timeout: float = 3.0):
        """nvidia-smi takes a few hundred milliseconds to start: wait until it is sampling."""
        t0 = time.perf_counter()
        while self.proc and not self.lines and time.perf_counter() - t0 < timeout:
            time.sleep(0.01)

    def mark(self):
        """Samples from here on belong to the timed region."""
        self.first = len(self.lines)

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines[self.first:]:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------ CPU baseline
def cpu_sample_setup(layers: int, ctx_len: int, seed: int = 1):
    """Random-byte weights with the model's shapes for `layers` layers plus the lm_head, and a
    random fp16 KV cache of ctx_len tokens: values do not matter for timing."""
    from densecore_b200 import blocks as B
    rng = np.random.default_rng(seed)
    H, QD, KD, E, F, V = 2048, 4096, 512, 128, 768, 151936

    def rnd(t, n, k):
        out = rng.integers(0, 256, size=n * B.row_bytes(t, k), dtype=np.uint8)
        bb = B.BLOCK_BYTES[t]
        blk = out.reshape(-1, bb)
        if t == B.GGML_TYPE_Q4_K:
            blk[:, 0:4] = np.array([0x00, 0x1E, 0x00, 0x1E], np.uint8)   # d, dmin = fp16 ~0.006
        else:
            blk[:, 208:210] = np.array([0x00, 0x1E], np.uint8)
        return out
    L = []
    for il in range(layers):
        L.append(dict(q=rnd(12, QD, H), k=rnd(12, KD, H), v=rnd(14, KD, H), o=rnd(12, H, QD),
                      router=(rng.normal(size=(E, H)) * 0.02).astype(np.float32),
                      gate=rnd(12, E * F, H), up=rnd(12, E * F, H), down=rnd(14 if il % 2 == 0 else 12, E * H, F),
                      down_t=14 if il % 2 == 0 else 12))
    blocks = (ctx_len + 15) // 16
    kv = (rng.integers(0, 0x3C00, size=(blocks * 16, 4, 128), dtype=np.uint16),
          rng.integers(0, 0x3C00, size=(blocks * 16, 4, 128), dtype=np.uint16))
    return dict(layers=L, lm_head=rnd(14, V, H), kv=kv, table=np.arange(blocks, dtype=np.int32), ctx=ctx_len)


def cpu_sample_run(o, S, n_streams: int, rng) -> float:
    """One decode step of `len(S['layers'])` layers + lm_head through the CPU path's matmul, attention, router
    and MoE calls (norms, RoPE and residual adds are left out: they are negligible).  Returns seconds."""
    H, QD, KD, E, F, V = 2048, 4096, 512, 128, 768, 151936
    x = rng.normal(size=(n_streams, H)).astype(np.float32)
    scale = float(1 / np.sqrt(128.0))
    t0 = time.perf_counter()
    for Ly in S["layers"]:
        q = o.mul_mat(12, Ly["q"], QD, H, x)
        o.mul_mat(12, Ly["k"], KD, H, x)
        o.mul_mat(14, Ly["v"], KD, H, x)
        att = np.stack([o.paged_attention(q[s].reshape(32, 128), S["kv"][0], S["kv"][1], S["table"], S["ctx"] - 1, 32, 4,
                                          128, scale, "blockwise").reshape(-1) for s in range(n_streams)])
        o.mul_mat(12, Ly["o"], H, QD, att)
        lg = o.mul_mat(0, Ly["router"], E, H, x)
        ids, w = o.route(lg, 8, mode="stable")
        x = o.moe_forward((12, 12, Ly["down_t"]), Ly["gate"], Ly["up"], Ly["down"], E, H, F, x, ids, w, fast_exp=True)
    t_layers = time.perf_counter() - t0
    t0 = time.perf_counter()
    o.mul_mat(14, S["lm_head"], V, H, x)
    t_head = time.perf_counter() - t0
    return t_layers, t_head


def cpu_reference(o, reps: int, warm: int = 2):
    """The CPU restatement of DenseCore's ggml path, all host threads, on the bounded sample both CPU legs
    use: SAMPLE_LAYERS of 48 layers (QKV/O matmuls, paged attention at ctx CPU_CTX, router, MoE FFN) plus
    the lm_head per batch-1 decode step, scaled to 48 layers (norms, RoPE and residual adds are left out:
    they are below 1 % of the step).  Returns (tok/s, seconds per step, threads, sample text)."""
    threads = o.max_threads()
    o.set_threads(threads)
    rng = np.random.default_rng(0)
    S = cpu_sample_setup(SAMPLE_LAYERS, CPU_CTX)
    for _ in range(warm):
        cpu_sample_run(o, S, 1, rng)
    per = []
    for _ in range(reps):
        tl, th = cpu_sample_run(o, S, 1, rng)
        per.append(tl / SAMPLE_LAYERS * 48 + th)
    step_s = float(np.median(per))
    sample = (f"{SAMPLE_LAYERS} of 48 layers (QKV/O matmuls, paged attention at ctx {CPU_CTX}, router, MoE FFN) + lm_head "
              f"of one batch-1 decode step, median of {reps} repeats after {warm} warm-ups, scaled to 48 layers; norms, RoPE "
              f"and residual adds left out; CPU restatement of DenseCore's ggml path")
    return 1.0 / step_s, step_s, threads, sample


def bench_config(streams: int = 1, layers: int = 48, prompt: int = PROMPT, world: int = 1) -> dict:
    return {"workload": WORKLOAD, "streams": streams, "layers": layers, "prompt_tokens": prompt, "parallelism": f"ep{world}"}


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from oracle import oracle as o
    o.build()
    t_all = time.perf_counter()
    value, step_s, threads, sample = cpu_reference(o, args.steps, max(1, min(args.warmup, 2)))
    cfg = bench_config(1, 48, PROMPT, max(1, args.gpus))
    cfg["parallelism"] = "cpu threads"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8 x int4/int6 block dots, f32 accumulate", "data": "synthetic",
        "config": cfg,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t_all,
    }
    print(json.dumps(line))
    return 0


# ------------------------------------------------------- single-op timing
def _stream_of(ctx):
    import torch
    import densecore_b200 as dc
    return torch.cuda.ExternalStream(dc._lib.lib().dc_b200_stream(ctx.handle))


def _time_graph(ctx, enqueue, reps: int, warm: int = 3):
    """Device time of `enqueue()` (library calls on the context's stream), captured once as a CUDA graph and
    replayed `reps` times back to back: microseconds per replay from CUDA events on that stream."""
    import torch
    st = _stream_of(ctx)
    enqueue()                                   # eager: kernel attributes, scratch growth
    ctx.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=st):
        enqueue()
    for _ in range(warm):
        g.replay()
    ctx.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(st):
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps


def op_gemv(ctx, ggml_type: int, N: int, K: int, M: int, ring: int, reps: int, peak_gbs: float) -> dict:
    """MUL_MAT of one [N x K] K-quant matrix with M activation rows, over a ring of distinct weight copies
    (larger than L2 together) so that every launch reads its weights from HBM.  One op = Q8_K quantiser +
    GEMV kernel, as dc_b200_mul_mat_dev enqueues them."""
    from densecore_b200 import blocks as B
    rng = np.random.default_rng(1234)
    ws = [ctx.upload_weight(ggml_type, B.random_weight(rng, ggml_type, N, K), K, N) for _ in range(ring)]
    x = rng.normal(size=(M, K)).astype(np.float32)
    xd, yd = ctx.alloc(x.nbytes), ctx.alloc(M * N * 4)
    ctx.to_device(xd, x)

    def enqueue():
        for w in ws:
            ctx.mul_mat_dev(w, xd, M, yd)
    us = _time_graph(ctx, enqueue, reps) / ring
    nbytes = B.row_bytes(ggml_type, K) * N + M * K * 4 + M * N * 4
    for w in ws:
        w.free()
    ctx.free(xd)
    ctx.free(yd)
    return {"us": us, "bytes": nbytes, "gbs": nbytes / us / 1e3, "frac": nbytes / us / 1e3 / peak_gbs,
            "floor_us": nbytes / peak_gbs / 1e3, "ring_copies": ring, "M": M}


def op_moe_layer(ctx, T: int, reps: int, peak_gbs: float, weights=None) -> dict:
    """One MoE FFN layer (hidden 2048, 128 experts top-8, FFN 768, gate/up Q4_K, down Q6_K, F32 router) on T
    tokens, over a ring of different inputs so that successive calls route to different experts and read them
    from HBM.  Bytes: router + 3 059 712 per distinct expert hit (counted from the returned ids) + 16 384 T."""
    from densecore_b200 import blocks as B
    H, F, E, k = 2048, 768, 128, 8
    rng = np.random.default_rng(4242)
    own = weights is None
    if own:
        router = (rng.normal(size=(E, H)) * 0.02).astype(np.float32)
        weights = (ctx.upload_weight(B.GGML_TYPE_F32, router, H, E),
                   ctx.upload_weight(B.GGML_TYPE_Q4_K, B.random_weight(rng, B.GGML_TYPE_Q4_K, E * F, H), H, F, E),
                   ctx.upload_weight(B.GGML_TYPE_Q4_K, B.random_weight(rng, B.GGML_TYPE_Q4_K, E * F, H), H, F, E),
                   ctx.upload_weight(B.GGML_TYPE_Q6_K, B.random_weight(rng, B.GGML_TYPE_Q6_K, E * H, F), F, H, E))
    Wr, Wg, Wu, Wd = weights
    ring = max(2, 48 // T)
    xs = rng.normal(size=(ring, T, H)).astype(np.float32)
    xd, yd, idd = ctx.alloc(xs.nbytes), ctx.alloc(T * H * 4), ctx.alloc(ring * T * k * 4)
    ctx.to_device(xd, xs)

    def enqueue():
        for r in range(ring):
            ctx.mul_mat_id_dev(Wr, Wg, Wu, Wd, xd + r * T * H * 4, T, k, yd, ids_dev=idd + r * T * k * 4)
    us = _time_graph(ctx, enqueue, reps) / ring
    ids = ctx.from_device(idd, np.zeros((ring, T * k), np.int32))
    U = float(np.mean([len(set(r.tolist())) for r in ids]))
    nbytes = E * H * 4 + U * 3059712 + T * 16384
    for d in (xd, yd, idd):
        ctx.free(d)
    if own:
        for w in weights:
            w.free()
    return {"T": T, "us": us, "distinct_experts": U, "bytes": nbytes, "gbs": nbytes / us / 1e3,
            "frac": nbytes / us / 1e3 / peak_gbs, "floor_us": nbytes / peak_gbs / 1e3, "ring_inputs": ring}


def moe_layer_sweep(ctx, reps, peak):
    from densecore_b200 import blocks as B
    H, F, E = 2048, 768, 128
    rng = np.random.default_rng(4242)
    router = (rng.normal(size=(E, H)) * 0.02).astype(np.float32)
    weights = (ctx.upload_weight(B.GGML_TYPE_F32, router, H, E),
               ctx.upload_weight(B.GGML_TYPE_Q4_K, B.random_weight(rng, B.GGML_TYPE_Q4_K, E * F, H), H, F, E),
               ctx.upload_weight(B.GGML_TYPE_Q4_K, B.random_weight(rng, B.GGML_TYPE_Q4_K, E * F, H), H, F, E),
               ctx.upload_weight(B.GGML_TYPE_Q6_K, B.random_weight(rng, B.GGML_TYPE_Q6_K, E * H, F), F, H, E))
    out = [op_moe_layer(ctx, T, reps, peak, weights) for T in (1, 4, 8, 16)]
    for w in weights:
        w.free()
    return out


def bench_dense_0p8b(ctx, peak_gbs: float, n_decode: int = 256) -> dict:
    """Config 2: dense 0.8B-class decoder, 512-token random prompt, greedy decode of 256 tokens at batch 1."""
    import densecore_b200 as dc
    cfg = dc.dense_0p8b(max_seqs=1, max_ctx=512 + n_decode + 64)
    m = dc.Model(ctx, cfg)
    m.init_synthetic(2, 0.02)
    m.finalize()
    rng = np.random.default_rng(2)
    seq = m.seq_alloc()
    t0 = time.perf_counter()
    first = m.prefill(seq, rng.integers(0, cfg.vocab, size=512))
    prefill_s = time.perf_counter() - t0
    toks, _ = m.decode_run([seq], [first], 16)
    toks, ms = m.decode_run([seq], toks[-1], n_decode - 16)
    _, wbytes, kvb = m.step_stats()
    ctx_mid = 512 + 16 + (n_decode - 16) // 2
    step_bytes = wbytes + kvb * ctx_mid
    tok_s = (n_decode - 16) / (ms * 1e-3)
    m.close()
    return {"tok_s": tok_s, "ms_per_step": ms / (n_decode - 16), "step_bytes": step_bytes,
            "floor_tok_s": peak_gbs * 1e9 / step_bytes, "frac": tok_s * step_bytes / 1e9 / peak_gbs,
            "prefill_512_ms": prefill_s * 1e3}


def spec_sweep(ctx, model, cfg, rng, seqs_to_free) -> dict:
    """Config 5: target = the benchmark model, draft = the dense 0.8B-class model, gamma 4, 1024-token prompt,
    128 output tokens; greedy accept with synthetic drafts at forced 0 / 50 / 100 % acceptance, and the
    stochastic rule at temperature 0.8 with the draft model's own sampled proposals."""
    import densecore_b200 as dc
    dcfg = dc.dense_0p8b(max_seqs=2, max_ctx=1024 + 512)
    draft = dc.Model(ctx, dcfg)
    draft.init_synthetic(4321, 0.02)
    draft.finalize()
    prompt = rng.integers(0, cfg.vocab, size=1024)
    n_out, gamma = 128, 4
    for s in seqs_to_free:
        model.seq_free(s)   # the decode runs hold all four sequence slots
    want, st0 = dc.speculative_decode(model, draft, prompt, n_out + gamma + 1, gamma=gamma)
    out = {"gamma": gamma, "prompt_tokens": 1024, "output_tokens": n_out,
           "draft_model_greedy": {"acceptance": st0.acceptance, "tokens_per_step": st0.tokens_per_step,
                                  "tok_s": st0.emitted / st0.seconds, "ms_per_verify_step": st0.seconds / st0.steps * 1e3}}

    def forced(rate):
        def f(pos, g):
            true = want[pos:pos + g].copy()
            if rate == 0.0:
                true[0] = (true[0] + 1) % cfg.vocab
            elif rate == 0.5:
                true[g // 2] = (true[g // 2] + 1) % cfg.vocab
            return true
        return f
    for rate in (0.0, 0.5, 1.0):
        got, st = dc.speculative_decode(model, draft, prompt, n_out, gamma=gamma, forced_drafts=forced(rate))
        out[f"forced_{int(rate * 100)}"] = {"acceptance": st.acceptance, "tokens_per_step": st.tokens_per_step,
                                            "tok_s": st.emitted / st.seconds, "ms_per_verify_step": st.seconds / st.steps * 1e3,
                                            "equals_greedy_stream": bool(np.array_equal(got, want[:n_out]))}
    got, st = dc.speculative_decode(model, draft, prompt, 64, gamma=gamma, mode=1, temperature=0.8, seed=99)
    out["stochastic_T0.8"] = {"acceptance": st.acceptance, "tokens_per_step": st.tokens_per_step,
                              "tok_s": st.emitted / st.seconds, "ms_per_verify_step": st.seconds / st.steps * 1e3}
    draft.close()
    return out


def op_gemm(ctx, ggml_type: int, N: int, K: int, M: int, reps: int) -> dict:
    """Prompt-sized MUL_MAT (M token rows) through the tensor-core kernel: activation tiling + GEMM, as
    dc_b200_mul_mat_dev enqueues them.  Reported in int8 multiply-accumulate operations (2 N K M per call)."""
    from densecore_b200 import blocks as B
    rng = np.random.default_rng(7)
    w = ctx.upload_weight(ggml_type, B.random_weight(rng, ggml_type, N, K), K, N)
    x = rng.normal(size=(M, K)).astype(np.float32)
    xd, yd = ctx.alloc(x.nbytes), ctx.alloc(M * N * 4)
    ctx.to_device(xd, x)
    us = _time_graph(ctx, lambda: ctx.mul_mat_dev(w, xd, M, yd), reps)
    ctx.free(xd)
    ctx.free(yd)
    w.free()
    return {"N": N, "K": K, "M": M, "type": ggml_type, "us": us, "tops": 2.0 * N * K * M / us / 1e6}


def run_single_op(args) -> int:
    """--op: one operator alone (for profiling runs and for the per-config figures of the main line)."""
    import densecore_b200 as dc
    from densecore_b200 import blocks as B
    ctx = dc.Context(0)
    peak, _ = measured_peaks()
    if args.op == "gemv-config1":
        out = op_gemv(ctx, B.GGML_TYPE_Q4_K, 6144, 2048, 1, 64, args.steps, peak)
    elif args.op == "gemv-q4-big":
        out = op_gemv(ctx, B.GGML_TYPE_Q4_K, 65536, 2048, 1, 4, args.steps, peak)
    elif args.op == "gemv-lm-head":
        out = op_gemv(ctx, B.GGML_TYPE_Q6_K, 151936, 2048, 1, 2, args.steps, peak)
    elif args.op == "gemm-q4":
        out = op_gemm(ctx, B.GGML_TYPE_Q4_K, 4096, 2048, 2048, args.steps)
    elif args.op == "gemm-q6":
        out = op_gemm(ctx, B.GGML_TYPE_Q6_K, 2048, 768, 4096, args.steps)
    elif args.op == "moe-layer":
        out = {"T": moe_layer_sweep(ctx, args.steps, peak)}
    elif args.op == "dense-0p8b":
        out = bench_dense_0p8b(ctx, peak)
    else:
        raise SystemExit(f"unknown --op {args.op}")
    print(json.dumps({"op": args.op, **out}))
    ctx.close()
    return 0


# -------------------------------------------------------------- our arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=48, help="debug: fewer layers (the result is then not the benchmark)")
    ap.add_argument("--prompt", type=int, default=PROMPT)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile-classes", action="store_true", help="print the per-kernel-class table to stderr")
    ap.add_argument("--path", default="persistent", choices=["persistent", "per-op"],
                    help="persistent: one cooperative kernel per decode run where the model fits its plan (default); "
                         "per-op: one kernel per op, replayed as a CUDA graph")
    ap.add_argument("--phase-timing", action="store_true",
                    help="print the persistent kernel's per-phase device time (CTA 0's view) to stderr")
    ap.add_argument("--ep-exchange", default="peer", choices=["peer", "nccl"],
                    help="N > 1: peer = the persistent kernel stores expert outputs into all GPUs' buffers over NVLink "
                         "(default); nccl = per-op kernels with one all-reduce per layer")
    ap.add_argument("--streams", default="1,4", help="stream counts to time (the JSON line needs 1)")
    ap.add_argument("--profiler-range", action="store_true",
                    help="bracket the timed 1-stream decode run with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    ap.add_argument("--no-extras", action="store_true", help="skip the other workloads (single ops, dense model, speculative sweep)")
    ap.add_argument("--op", default=None, choices=["gemv-config1", "gemv-lm-head", "gemv-q4-big", "gemm-q4", "gemm-q6", "moe-layer", "dense-0p8b"],
                    help="time one operator alone and print its own JSON line (not the benchmark line)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.op:
        return run_single_op(args)
    if args.impl == "reference":
        return reference_arm(args)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    import torch
    import densecore_b200 as dc
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("gloo", rank=rank, world_size=world)   # control plane only; data plane is NCCL in the library
    torch.cuda.set_device(local_rank)
    ctx = dc.Context(local_rank)
    cfg = dc.moe_35b_a3b(max_seqs=4, max_ctx=args.prompt + 512, ep_rank=rank, ep_size=world)
    cfg.n_layer = args.layers
    model = dc.Model(ctx, cfg)
    model.init_synthetic(1234, 0.02)
    if world > 1:
        import ctypes as C
        import nvidia.nccl
        nccl_path = os.path.join(list(nvidia.nccl.__path__)[0], "lib", "libnccl.so.2")
        buf = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            raw = (C.c_char * 128)()
            ctx._check(dc._lib.lib().dc_b200_ep_unique_id(ctx.handle, nccl_path.encode(), raw))
            buf = torch.frombuffer(bytearray(raw.raw), dtype=torch.uint8).clone()
        dist.broadcast(buf, 0)
        model.ep_init(bytes(buf.numpy().tobytes()), nccl_path)
        peer_ok = args.ep_exchange == "peer"
        if peer_ok:
            # exchange buffers of the persistent kernel: every rank's handle to every rank
            try:
                mine = torch.frombuffer(bytearray(model.ep_export()), dtype=torch.uint8).clone()
            except dc.DcError as e:
                print(f"rank {rank}: ep_export failed: {e}", file=sys.stderr)
                mine, peer_ok = torch.zeros(64, dtype=torch.uint8), False
            allh = [torch.zeros(64, dtype=torch.uint8) for _ in range(world)]
            dist.all_gather(allh, mine)
            for r in range(world):
                if r != rank and peer_ok:
                    try:
                        model.ep_import(r, bytes(allh[r].numpy().tobytes()))
                    except dc.DcError as e:
                        print(f"rank {rank}: ep_import({r}) failed: {e}", file=sys.stderr)
                        peer_ok = False
            # all ranks must take the same path: one failure sends everyone to the per-op kernels and NCCL
            flag = torch.tensor([1 if peer_ok else 0], dtype=torch.int32)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            peer_ok = bool(flag.item())
        ep_force_per_op = not peer_ok
    model.finalize()
    if args.path == "per-op" or (world > 1 and ep_force_per_op):
        model.set_option("persistent", 0)

    rng = np.random.default_rng(0)
    seqs = [model.seq_alloc() for _ in range(4)]
    prompts = [rng.integers(0, cfg.vocab, size=args.prompt) for _ in seqs]
    first, ttfts = [], []
    for s, p in zip(seqs, prompts):                       # host prompt in, first token out: time to first token
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        first.append(model.prefill(s, p))
        ttfts.append((time.perf_counter() - t0) * 1e3)
    ttft_first_ms, ttft_ms = ttfts[0], float(np.median(ttfts[1:]))   # the first call also allocates the chunk buffers

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if dist is None:
            return v
        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    results = {}
    clocks = None
    stream_counts = sorted({int(x) for x in args.streams.split(",")} | {1})
    for n_streams in stream_counts:
        sq = seqs[:n_streams]
        sampler = ClockSampler(local_rank) if (n_streams == 1 and rank == 0) else None
        if sampler:
            sampler.start()
            sampler.wait_ready()
        toks, _ = model.decode_run(sq, first[:n_streams], args.warmup)        # warm-up: eager pass, capture, replays
        barrier()
        if sampler:
            sampler.mark()
        if args.profiler_range and n_streams == 1:
            dc._lib.lib().dc_b200_profiler_range(1)
        t0 = time.perf_counter()
        toks, ms = model.decode_run(sq, toks[-1], args.steps)                 # K steps, device time from CUDA events
        barrier()
        wall = time.perf_counter() - t0
        if args.profiler_range and n_streams == 1:
            dc._lib.lib().dc_b200_profiler_range(0)
        run_launches = model.step_stats()[0]
        ms = max_over_ranks(ms)
        # end to end: host buffers every step
        last = toks[-1]
        for _ in range(args.warmup):
            last = model.decode_step(sq, last)
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            last = model.decode_step(sq, last)
        barrier()
        e2e_s = max_over_ranks(time.perf_counter() - t0)
        if sampler:
            clocks = sampler.stop()           # samples cover the device-timed run and the end-to-end run
        results[n_streams] = dict(ms=ms, wall=wall, e2e_s=e2e_s, ctx=model.seq_len(sq[0]), last=last, run_launches=run_launches)

    _, weight_bytes, kv_bytes_per_tok = model.step_stats()
    peak_gbs, peak_kind = measured_peaks()
    r1 = results[1]
    ms_per_step = r1["ms"] / args.steps
    value = 1 * args.steps / (r1["ms"] * 1e-3)
    # algorithmic bytes of one step: every weight byte the step must read (attention and router weights, the
    # selected experts, lm_head) + the K and V rows of the context, at the context length mid-way through the run
    step_bytes = weight_bytes + kv_bytes_per_tok * (r1["ctx"] - args.steps // 2)
    persistent = r1["run_launches"] == 1
    if persistent:
        # one launch of the persistent kernel runs all K steps: bytes per launch = K x step bytes, duration =
        # the run's device time (CUDA events on the launching stream around that launch)
        achieved = step_bytes * args.steps / (r1["ms"] * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": "k_decode_mega", "achieved": achieved, "peak": peak_gbs, "unit": "GB/s",
                    "frac": achieved / peak_gbs, "peak_kind": f"of {peak_kind}",
                    "traffic": DRAM_TRAFFIC_RATIO * step_bytes * args.steps,
                    "traffic_note": "dram__bytes_read+write of one launch from an ncu capture of the model cut to 4 layers, "
                                    "scaled by algorithmic bytes",
                    "launches": 1, "bytes_per_launch": step_bytes * args.steps, "us_per_launch": r1["ms"] * 1e3}
        gpu_launches = 1
    else:
        # per-op path: device time of one eager step per kernel class (CUDA events around every launch)
        prof = model.profile_step(seqs[:1], r1["last"][:1])
        prof = model.profile_step(seqs[:1], r1["last"][:1])
        dom_name, (dom_ms, dom_n, dom_bytes) = max(prof.items(), key=lambda kv: kv[1][0])
        achieved = dom_bytes / (dom_ms * 1e-3) / 1e9 if dom_ms > 0 else 0.0
        roofline = {"bound": "hbm", "kernel": dom_name, "achieved": achieved, "peak": peak_gbs, "unit": "GB/s",
                    "frac": achieved / peak_gbs, "peak_kind": f"of {peak_kind}", "traffic": None,
                    "launches_per_step": dom_n, "bytes_per_launch": dom_bytes / dom_n,
                    "us_per_launch": dom_ms * 1e3 / dom_n}
        gpu_launches = r1["run_launches"] * args.steps
    if args.phase_timing and persistent and rank == 0:
        for n_streams in stream_counts:
            model.set_option("phase_timing", 1)
            _, ms_pt = model.decode_run(seqs[:n_streams], results[n_streams]["last"], 32)
            pt = model.phase_timing()
            arrive, release = model.barrier_trace()
            model.set_option("phase_timing", 0)
            if model.step_stats()[0] != 1:
                print(f"streams {n_streams}: per-op path ({ms_pt / 32 * 1e3:.1f} us/step), no phases", file=sys.stderr)
                continue
            print(f"streams {n_streams}: {ms_pt / 32 * 1e3:.1f} us/step, {args.layers} layers; us per layer (CTA 0):", file=sys.stderr)
            for i, (name, ns) in pt.items():
                if ns:
                    print(f"  {i:2d} {name:18s} {ns / 32 / args.layers / 1e3:8.2f}", file=sys.stderr)
            if arrive.any():   # instrumented build only
                print("  barriers of layer 1, first step: spread of CTA arrivals and release latency (us)", file=sys.stderr)
                for b, name in enumerate(model.BARRIERS):
                    a, r = arrive[b], release[b]
                    print(f"    {name:20s} median-first {(np.median(a) - a.min()) / 1e3:6.2f}  last-median "
                          f"{(a.max() - np.median(a)) / 1e3:6.2f}  release-last {(np.median(r) - a.max()) / 1e3:6.2f}",
                          file=sys.stderr)
    if args.profile_classes and rank == 0:
        for n_streams in stream_counts:
            last = results[n_streams]["last"][:n_streams]
            prof = model.profile_step(seqs[:n_streams], last)
            prof = model.profile_step(seqs[:n_streams], last)
            tot = sum(v[0] for v in prof.values())
            print(f"per-op kernels, one eager step, {n_streams} stream(s): {tot * 1e3:.1f} us in kernels", file=sys.stderr)
            for k, (ms_, n_, b_) in sorted(prof.items(), key=lambda kv: -kv[1][0]):
                print(f"  {k:22s} launches {n_:4d}  {ms_ * 1e3:9.1f} us  {ms_ / tot * 100:5.1f} %  "
                      f"{b_ / n_ / 1e6:8.2f} MB/launch  {b_ / (ms_ * 1e-3) / 1e9 if ms_ else 0:8.1f} GB/s", file=sys.stderr)

    extras = {}
    if world == 1 and not args.no_extras:
        # the other workloads of the benchmark family, each on its own configuration (not the headline number)
        extras["gemv_6144x2048_q4k"] = op_gemv(ctx, 12, 6144, 2048, 1, 32, 20, peak_gbs)
        extras["lm_head_151936x2048_q6k"] = op_gemv(ctx, 14, 151936, 2048, 1, 2, 20, peak_gbs)
        extras["moe_layer"] = moe_layer_sweep(ctx, 20, peak_gbs)
        extras["dense_0p8b_decode"] = bench_dense_0p8b(ctx, peak_gbs)
        extras["speculative"] = spec_sweep(ctx, model, cfg, rng, seqs[3:])
        seqs = seqs[:3]

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8 x int4/int6 block dots (dp4a), f32 accumulate", "data": "synthetic",
        "config": dict(bench_config(1, args.layers, args.prompt, world), ctx_at_timing=r1["ctx"],
                       path="persistent kernel" if persistent else "per-op CUDA graph",
                       l2="each step reads ~1.9 GB of weights, far more than the 126 MB L2, so no flush is needed"),
        "ttft_ms": ttft_ms, "ttft_first_call_ms": ttft_first_ms,
        "prefill_tok_s": args.prompt / (ttft_ms * 1e-3),
        "hbm_fraction_of_step": step_bytes / (ms_per_step * 1e-3) / 1e9 / (peak_gbs * world),
        "e2e": {"value": args.steps / r1["e2e_s"], "unit": UNIT, "h2d_bytes_per_step": 12, "d2h_bytes_per_step": 4,
                "api": "dc_b200_decode_step"},
        "gpu_launches": gpu_launches,
        "clocks": clocks,
        "roofline": roofline,
    }
    if 4 in results:
        r4 = results[4]
        # bytes of a 4-stream step: shared weights once, the distinct experts four tokens route to (expected
        # 128 (1 - (1 - 8/128)^4) = 29.1 of 128 per layer under uniform routing), four K/V histories
        n_moe = args.layers
        expert_bytes = 3059712
        shared = weight_bytes - n_moe * 8 * expert_bytes
        b4 = shared + n_moe * 29.1 * expert_bytes + 4 * kv_bytes_per_tok * (r4["ctx"] - args.steps // 2)
        line["streams4"] = {"value": 4 * args.steps / (r4["ms"] * 1e-3), "ms_per_step": r4["ms"] / args.steps,
                            "e2e": 4 * args.steps / r4["e2e_s"], "ctx_at_timing": r4["ctx"],
                            "step_bytes_expected": b4,
                            "hbm_fraction_of_step": b4 / (r4["ms"] / args.steps * 1e-3) / 1e9 / (peak_gbs * world)}
    if world > 1:
        # byte model of expert parallelism: replicated bytes (attention, router, dense matrices, lm_head, KV) are read
        # by every GPU, expert bytes are split; the ceiling is what that would buy if the step were bandwidth-bound
        expert_bytes_step = args.layers * 8 * 3059712
        repl = step_bytes - expert_bytes_step
        line["ep_model"] = {"replicated_bytes_per_step": repl, "expert_bytes_per_step": expert_bytes_step,
                            "speedup_ceiling": step_bytes / (repl + expert_bytes_step / world),
                            "note": "one stream is latency-bound: every layer adds one NVLink store-signal round trip"}
    if extras:
        line["other_workloads"] = extras
    if rank == 0 and not args.no_cpu_baseline:
        from oracle import oracle as o
        o.build()
        v, step_s, threads, sample = cpu_reference(o, SAMPLE_REPS)
        line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample}
    if rank == 0:
        print(json.dumps(line))
    model.close()
    ctx.close()
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
