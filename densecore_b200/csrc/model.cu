// Decoder: the per-op kernels chained into one Qwen3-style model step (dense FFN
// or MoE), captured as a CUDA graph per batch shape.  Follows the graph that
// BuildTransformerGraph lays out (core/src/llm/graph/decoder.cpp: :453 attn_norm,
// :1085-1100 QKV, :1265-1343 Q/K norm, :1422-1450 RoPE, :1846-1872 paged attention,
// :2201 ffn_norm, :2217-2410 MoE, :2662-2730 dense FFN, :2997 lm_head) and the
// decode loop of core/src/runtime/worker.cpp (:2534 build, :4242 compute, :5895
// sample).  Host code only; every arithmetic step is a kernel from the other files.
#include <math.h>
#include <stdio.h>
#include <string.h>

#include <map>
#include <string>
#include <vector>

#include "dc_common.cuh"
#include "dc_internal.h"
#include "dc_kv.h"
#include "dc_mega.h"
#include "dc_model.h"

#define DC_TRY(expr)                       \
    do {                                   \
        int _st = (expr);                  \
        if (_st != DC_B200_OK) return _st; \
    } while (0)

static uint64_t fnv1a64(const char* s) {
    uint64_t h = 1469598103934665603ull;
    for (; *s; ++s) {
        h ^= (uint8_t)*s;
        h *= 1099511628211ull;
    }
    return h;
}

static size_t row_bytes_of(int type, int64_t K) {
    switch (type) {
    case DC_TYPE_F32: return (size_t)K * 4;
    case DC_TYPE_F16: return (size_t)K * 2;
    case DC_TYPE_Q4_K: return (size_t)(K / DC_QK_K) * DC_Q4K_BYTES;
    case DC_TYPE_Q6_K: return (size_t)(K / DC_QK_K) * DC_Q6K_BYTES;
    }
    return 0;
}

static dc_weight* new_weight(dc_model* m, int type, int64_t K, int64_t N, int64_t E) {
    dc_weight* w = new dc_weight();
    w->type = type;
    w->K = K;
    w->N = N;
    w->E = E;
    w->row_bytes = row_bytes_of(type, K);
    w->bytes = w->row_bytes * (size_t)N * (size_t)E;
    if (cudaMalloc(&w->dev, w->bytes + 64) != cudaSuccess) {
        delete w;
        return nullptr;
    }
    cudaMemsetAsync(w->dev + w->bytes, 0, 64, m->ctx->stream);
    return w;
}

// name -> slot, expected shape
struct TensorSlot {
    dc_weight** slot;
    int64_t K, N, E;
    int synth_type;   // type used by init_synthetic
    int kind;         // 0 matrix, 1 norm vector (synthetic value 1 + noise), 2 router
};

static bool find_slot(dc_model* m, const std::string& name, TensorSlot* out) {
    const dc_model_config& c = m->cfg;
    const int64_t H = c.hidden, QD = (int64_t)c.n_head * c.head_dim, KD = (int64_t)c.n_kv_head * c.head_dim;
    auto set = [&](dc_weight** s, int64_t K, int64_t N, int64_t E, int type, int kind) {
        *out = TensorSlot{s, K, N, E, type, kind};
        return true;
    };
    if (name == "token_embd.weight") return set(&m->tok_embd, H, c.vocab, 1, c.tie_embeddings ? DC_TYPE_Q6_K : DC_TYPE_Q4_K, 0);
    if (name == "output_norm.weight") return set(&m->out_norm, H, 1, 1, DC_TYPE_F32, 1);
    if (name == "output.weight") {
        if (c.tie_embeddings) return false;
        return set(&m->output, H, c.vocab, 1, DC_TYPE_Q6_K, 0);
    }
    int il = -1;
    char rest[96];
    if (sscanf(name.c_str(), "blk.%d.%95s", &il, rest) != 2 || il < 0 || il >= c.n_layer) return false;
    dc_layer& L = m->layers[il];
    const std::string r = rest;
    const int down_type = (il % 2 == 0) ? DC_TYPE_Q6_K : DC_TYPE_Q4_K;
    if (r == "attn_norm.weight") return set(&L.attn_norm, H, 1, 1, DC_TYPE_F32, 1);
    if (r == "attn_q.weight") return set(&L.wq, H, QD, 1, DC_TYPE_Q4_K, 0);
    if (r == "attn_k.weight") return set(&L.wk, H, KD, 1, DC_TYPE_Q4_K, 0);
    if (r == "attn_v.weight") return set(&L.wv, H, KD, 1, DC_TYPE_Q6_K, 0);
    if (r == "attn_output.weight") return set(&L.wo, QD, H, 1, DC_TYPE_Q4_K, 0);
    if (r == "attn_q_norm.weight" && c.qk_norm) return set(&L.q_norm, c.head_dim, 1, 1, DC_TYPE_F32, 1);
    if (r == "attn_k_norm.weight" && c.qk_norm) return set(&L.k_norm, c.head_dim, 1, 1, DC_TYPE_F32, 1);
    if (r == "ffn_norm.weight") return set(&L.ffn_norm, H, 1, 1, DC_TYPE_F32, 1);
    if (c.n_expert > 0) {
        if (r == "ffn_gate_inp.weight") return set(&L.router, H, c.n_expert, 1, DC_TYPE_F32, 2);
        if (r == "ffn_gate_exps.weight") return set(&L.gate_exps, H, c.expert_ffn, c.n_expert, DC_TYPE_Q4_K, 0);
        if (r == "ffn_up_exps.weight") return set(&L.up_exps, H, c.expert_ffn, c.n_expert, DC_TYPE_Q4_K, 0);
        if (r == "ffn_down_exps.weight") return set(&L.down_exps, c.expert_ffn, H, c.n_expert, down_type, 0);
    } else {
        if (r == "ffn_gate.weight") return set(&L.ffn_gate, H, c.ffn, 1, DC_TYPE_Q4_K, 0);
        if (r == "ffn_up.weight") return set(&L.ffn_up, H, c.ffn, 1, DC_TYPE_Q4_K, 0);
        if (r == "ffn_down.weight") return set(&L.ffn_down, c.ffn, H, 1, down_type, 0);
    }
    return false;
}

static std::vector<std::string> tensor_names(const dc_model* m) {
    const dc_model_config& c = m->cfg;
    std::vector<std::string> v = {"token_embd.weight", "output_norm.weight"};
    if (!c.tie_embeddings) v.push_back("output.weight");
    for (int il = 0; il < c.n_layer; ++il) {
        const std::string p = "blk." + std::to_string(il) + ".";
        for (const char* n : {"attn_norm.weight", "attn_q.weight", "attn_k.weight", "attn_v.weight", "attn_output.weight",
                              "ffn_norm.weight"})
            v.push_back(p + n);
        if (c.qk_norm) {
            v.push_back(p + "attn_q_norm.weight");
            v.push_back(p + "attn_k_norm.weight");
        }
        if (c.n_expert > 0)
            for (const char* n : {"ffn_gate_inp.weight", "ffn_gate_exps.weight", "ffn_up_exps.weight", "ffn_down_exps.weight"})
                v.push_back(p + n);
        else
            for (const char* n : {"ffn_gate.weight", "ffn_up.weight", "ffn_down.weight"}) v.push_back(p + n);
    }
    return v;
}

template <typename T>
static int dev_alloc(dc_ctx* ctx, T** p, size_t n) {
    return dc_check_cuda(ctx, cudaMalloc((void**)p, n * sizeof(T) + 256), "cudaMalloc(step buffer)");
}

static int alloc_step_buffers(dc_model* m) {
    const dc_model_config& c = m->cfg;
    dc_ctx* ctx = m->ctx;
    const size_t T = DC_MAX_T, H = c.hidden, QD = (size_t)c.n_head * 128, KD = (size_t)c.n_kv_head * 128;
    const size_t F = c.n_expert > 0 ? c.expert_ffn : c.ffn;
    const size_t A = c.n_expert > 0 ? T * c.n_expert_used : T;
    dc_step_buffers& b = m->buf;
    DC_TRY(dev_alloc(ctx, &b.tokens, T));
    DC_TRY(dev_alloc(ctx, &b.seq_ids, T));
    DC_TRY(dev_alloc(ctx, &b.positions, T));
    DC_TRY(dev_alloc(ctx, &b.out_tokens, T));
    DC_TRY(dev_alloc(ctx, &b.argmax_keys, T));
    DC_TRY(dev_alloc(ctx, &b.x, T * H));
    DC_TRY(dev_alloc(ctx, &b.xn, T * H));
    DC_TRY(dev_alloc(ctx, &b.qkv, T * (QD + 2 * KD)));
    DC_TRY(dev_alloc(ctx, &b.q, T * QD));
    DC_TRY(dev_alloc(ctx, &b.h, A * F));
    DC_TRY(dev_alloc(ctx, &b.dn, A * H));
    DC_TRY(dev_alloc(ctx, &b.moe_out, T * H));
    DC_TRY(dev_alloc(ctx, &b.logits, T * (size_t)c.vocab));
    const size_t att_bytes = dc_attention_scratch_bytes((int)T, c.n_head, c.n_kv_head, m->kv.max_blocks_per_seq, m->nsplit);
    DC_TRY(dev_alloc(ctx, &b.attn_mem, att_bytes));
    dc_attn_scratch_bind(&b.attn, b.attn_mem, (int)T, c.n_head, c.n_kv_head, m->kv.max_blocks_per_seq, m->nsplit);
    DC_TRY(dc_check_cuda(ctx, cudaMemsetAsync(b.attn.tickets, 0, T * c.n_head * 4, ctx->stream), "memset"));
    DC_TRY(dev_alloc(ctx, &b.q8_x, T * (H / 256) * 292));
    DC_TRY(dev_alloc(ctx, &b.q8_attn, T * (QD / 256) * 292));
    DC_TRY(dev_alloc(ctx, &b.q8_h, A * (F / 256) * 292));
    DC_TRY(dev_alloc(ctx, &b.history, (size_t)DC_HISTORY_CAP * T));
    DC_TRY(dev_alloc(ctx, &b.history_len, 1));
    if (c.n_expert > 0) {
        DC_TRY(dev_alloc(ctx, &b.route_mem, (size_t)(1 << 20)));
        dc_moe_route_bind(&b.route, b.route_mem, (int)T, c.n_expert, c.n_expert_used);
        DC_TRY(dc_check_cuda(ctx, cudaMemsetAsync(b.route.ticket, 0, sizeof(int), ctx->stream), "memset"));
    }
    DC_TRY(dc_check_cuda(ctx, cudaMemsetAsync(b.argmax_keys, 0, T * sizeof(unsigned long long), ctx->stream), "memset"));
    DC_TRY(dc_check_cuda(ctx, cudaMemsetAsync(b.history_len, 0, sizeof(int), ctx->stream), "memset"));
    // RoPE table computed in double: [pos][2i]=cos, [2i+1]=sin of pos*theta^(-2i/d)
    std::vector<float> cs((size_t)c.max_ctx * 128);
    for (int p = 0; p < c.max_ctx; ++p)
        for (int i = 0; i < 64; ++i) {
            const double a = (double)p * pow((double)c.rope_theta, -2.0 * i / 128.0);
            cs[(size_t)p * 128 + 2 * i] = (float)cos(a);
            cs[(size_t)p * 128 + 2 * i + 1] = (float)sin(a);
        }
    DC_TRY(dev_alloc(ctx, &b.cos_sin, cs.size()));
    DC_TRY(dc_check_cuda(ctx, cudaMemcpy(b.cos_sin, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice), "rope table"));
    DC_TRY(dc_check_cuda(ctx, cudaMallocHost((void**)&m->h_stage, 4096), "cudaMallocHost"));
    return DC_B200_OK;
}

// ------------------------------------------------------------- one step
// lm_mode: 0 no logits, 1 last row only, 2 every row.
static int enqueue_forward(dc_model* m, int T, int lm_mode, bool feedback) {
    const dc_model_config& c = m->cfg;
    dc_ctx* ctx = m->ctx;
    dc_step_buffers& b = m->buf;
    const int H = c.hidden, QD = c.n_head * 128, KD = c.n_kv_head * 128, QKV = QD + 2 * KD;
    const float scale = 1.0f / sqrtf((float)c.head_dim);
    const int E = c.n_expert, top_k = c.n_expert_used;
    const int ep_lo = m->ep_lo, ep_hi = m->ep_hi;
    int launches = 0;
    // cls: kernel class for the per-class timing; bytes: algorithmic bytes of the launch
#define L(cls, bytes, n, expr)                                          \
    do {                                                                \
        dc_model::ProfRec _r = {cls, nullptr, nullptr, (double)(bytes)}; \
        if (m->prof) {                                                  \
            cudaEventCreate(&_r.e0);                                    \
            cudaEventCreate(&_r.e1);                                    \
            cudaEventRecord(_r.e0, ctx->stream);                        \
        }                                                               \
        DC_TRY(expr);                                                   \
        if (m->prof) {                                                  \
            cudaEventRecord(_r.e1, ctx->stream);                        \
            m->prof_recs.push_back(_r);                                 \
        }                                                               \
        launches += (n);                                                \
    } while (0)
    const double q8x = (double)T * (H / 256) * 292, xb = (double)T * H * 4;
    L(DC_K_EMBED, m->tok_embd->row_bytes * T + xb, 1, dc_launch_embed(ctx, m->tok_embd, b.tokens, T, b.x));
    const float* pending = nullptr;  // MoE output of the previous layer, added in the next norm
    for (int il = 0; il < c.n_layer; ++il) {
        dc_layer& Ly = m->layers[il];
        L(DC_K_RMSNORM, xb + q8x + H * 4, 1,
          dc_launch_rmsnorm_q8k(ctx, b.x, pending, (const float*)Ly.attn_norm->dev, T, H, c.rms_eps, nullptr, b.q8_x));
        pending = nullptr;
        if (m->dbg_x)
            DC_TRY(dc_check_cuda(ctx, cudaMemcpyAsync(m->dbg_x + (size_t)il * DC_MAX_T * H, b.x, (size_t)T * H * 4, cudaMemcpyDeviceToDevice, ctx->stream), "capture"));
        dc_gemv_seg qkv[3] = {
            {Ly.wq->dev, Ly.wq->type, QD, (int)Ly.wq->row_bytes, b.qkv, QKV},
            {Ly.wk->dev, Ly.wk->type, KD, (int)Ly.wk->row_bytes, b.qkv + QD, QKV},
            {Ly.wv->dev, Ly.wv->type, KD, (int)Ly.wv->row_bytes, b.qkv + QD + KD, QKV},
        };
        L(DC_K_GEMV_QKV, (double)Ly.wq->bytes + Ly.wk->bytes + Ly.wv->bytes + q8x + (double)T * QKV * 4, 1,
          dc_launch_gemv(ctx, qkv, 3, DC_EPI_STORE, b.q8_x, T, H, nullptr));
        __half* ka = m->kv.k_arena + m->kv.layer_elems * il;
        __half* va = m->kv.v_arena + m->kv.layer_elems * il;
        L(DC_K_QKROPE, (double)T * QKV * 4 * 2, 1,
          dc_launch_qknorm_rope_kv(ctx, b.qkv, Ly.q_norm ? (const float*)Ly.q_norm->dev : nullptr,
                                   Ly.k_norm ? (const float*)Ly.k_norm->dev : nullptr, b.cos_sin, c.max_ctx, b.positions,
                                   b.seq_ids, m->kv.d_tables, m->kv.max_blocks_per_seq, ka, va, c.n_head, c.n_kv_head,
                                   c.rms_eps, T, b.q));
        // KV bytes depend on the context length; filled in by the caller of the profile
        L(DC_K_ATTENTION, 0.0, 2,
          dc_launch_attention(ctx, b.q, ka, va, m->kv.d_tables, m->kv.max_blocks_per_seq, b.seq_ids, b.positions, T,
                              c.n_head, c.n_kv_head, scale, m->nsplit, &b.attn, nullptr, b.q8_attn));
        dc_gemv_seg wo = {Ly.wo->dev, Ly.wo->type, H, (int)Ly.wo->row_bytes, b.x, H};
        L(DC_K_GEMV_O, (double)Ly.wo->bytes + (double)T * (QD / 256) * 292 + 2 * xb, 1,
          dc_launch_gemv(ctx, &wo, 1, DC_EPI_ACC, b.q8_attn, T, QD, nullptr));
        L(DC_K_RMSNORM, xb * (E > 0 ? 2 : 1) + q8x + H * 4, 1,
          dc_launch_rmsnorm_q8k(ctx, b.x, nullptr, (const float*)Ly.ffn_norm->dev, T, H, c.rms_eps,
                                E > 0 ? b.xn : nullptr, b.q8_x));
        if (E > 0) {
            const int A = T * top_k, F = c.expert_ffn;
            // distinct experts hit: top_k for one token; for T > 1 the host only knows the bound
            const double U = T == 1 ? top_k : (A < E ? A : E);
            const double local = (double)(ep_hi - ep_lo) / E;
            L(DC_K_ROUTER, (double)Ly.router->bytes + xb, 1,
              dc_launch_router(ctx, Ly.router, b.xn, E, T, top_k, c.routed_scale, ep_lo, ep_hi, &b.route, m->route_mode));
            L(DC_K_MOE_GATEUP, U * local * 2.0 * F * Ly.gate_exps->row_bytes + q8x + (double)A * F * 4, 1,
              dc_launch_moe_mm(ctx, true, Ly.gate_exps, Ly.up_exps, b.q8_x, T, T, top_k, ep_lo, &b.route, b.h));
            L(DC_K_QUANT_H, (double)A * F * 4 + (double)A * (F / 256) * 292, 1,
              dc_launch_quantize_q8k(ctx, b.h, A, F, b.q8_h));
            L(DC_K_MOE_DOWN, U * local * H * Ly.down_exps->row_bytes + (double)A * (F / 256) * 292 + (double)A * H * 4, 1,
              dc_launch_moe_mm(ctx, false, Ly.down_exps, nullptr, b.q8_h, A, T, top_k, ep_lo, &b.route, b.dn));
            L(DC_K_COMBINE, (double)A * H * 4 + xb, 1,
              dc_launch_moe_combine(ctx, b.dn, b.route.ids, b.route.weights, T, top_k, H, ep_lo, ep_hi, b.moe_out));
            if (c.ep_size > 1) L(DC_K_ALLREDUCE, xb, 1, dc_ep_allreduce(m, b.moe_out, (size_t)T * H));
            pending = b.moe_out;
        } else {
            dc_gemv_seg gu[2] = {
                {Ly.ffn_gate->dev, Ly.ffn_gate->type, c.ffn, (int)Ly.ffn_gate->row_bytes, b.h, c.ffn},
                {Ly.ffn_up->dev, Ly.ffn_up->type, c.ffn, (int)Ly.ffn_up->row_bytes, b.h, c.ffn},
            };
            L(DC_K_FFN_GATEUP, (double)Ly.ffn_gate->bytes + Ly.ffn_up->bytes + q8x + (double)T * c.ffn * 4, 1,
              dc_launch_gemv(ctx, gu, 2, DC_EPI_SWIGLU, b.q8_x, T, H, nullptr));
            L(DC_K_QUANT_H, (double)T * c.ffn * 4 + (double)T * (c.ffn / 256) * 292, 1,
              dc_launch_quantize_q8k(ctx, b.h, T, c.ffn, b.q8_h));
            dc_gemv_seg dw = {Ly.ffn_down->dev, Ly.ffn_down->type, H, (int)Ly.ffn_down->row_bytes, b.x, H};
            L(DC_K_FFN_DOWN, (double)Ly.ffn_down->bytes + (double)T * (c.ffn / 256) * 292 + 2 * xb, 1,
              dc_launch_gemv(ctx, &dw, 1, DC_EPI_ACC, b.q8_h, T, c.ffn, nullptr));
        }
    }
    if (lm_mode != 0) {
        const int rows = lm_mode == 1 ? 1 : T, first = lm_mode == 1 ? T - 1 : 0;
        L(DC_K_RMSNORM, (double)rows * H * 4 * 2 + (double)rows * (H / 256) * 292, 1,
          dc_launch_rmsnorm_q8k(ctx, b.x + (size_t)first * H, pending ? pending + (size_t)first * H : nullptr,
                                (const float*)m->out_norm->dev, rows, H, c.rms_eps, nullptr, b.q8_x));
        if (m->dbg_x)
            DC_TRY(dc_check_cuda(ctx, cudaMemcpyAsync(m->dbg_x + ((size_t)c.n_layer * DC_MAX_T + first) * H, b.x + (size_t)first * H, (size_t)rows * H * 4, cudaMemcpyDeviceToDevice, ctx->stream), "capture"));
        const dc_weight* out_w = c.tie_embeddings ? m->tok_embd : m->output;
        dc_gemv_seg lm = {out_w->dev, out_w->type, c.vocab, (int)out_w->row_bytes, b.logits, c.vocab};
        L(DC_K_LM_HEAD, (double)out_w->bytes + (double)rows * (H / 256) * 292 + (double)rows * c.vocab * 4, 1,
          dc_launch_gemv(ctx, &lm, 1, DC_EPI_STORE, b.q8_x, rows, H, b.argmax_keys));
        L(DC_K_ARGMAX, 64.0, 1,
          dc_launch_argmax_finish(ctx, b.argmax_keys, rows, b.out_tokens, feedback ? b.tokens : nullptr,
                                  feedback ? b.positions : nullptr, feedback ? b.history : nullptr,
                                  feedback ? b.history_len : nullptr, DC_HISTORY_CAP));
    }
#undef L
    m->last_launches = launches;
    return DC_B200_OK;
}

// Captured once per (T, lm_mode, feedback); replayed afterwards.
static int run_forward(dc_model* m, int T, int lm_mode, bool feedback) {
    dc_ctx* ctx = m->ctx;
    if (!m->use_graphs || m->dbg_x) return enqueue_forward(m, T, lm_mode, feedback);
    const int key = T * 8 + lm_mode * 2 + (feedback ? 1 : 0);
    auto it = m->graphs.find(key);
    if (it == m->graphs.end()) {
        // one eager pass first: it sets kernel attributes, which is not allowed while capturing
        if (!m->warmed[key]) {
            m->warmed[key] = true;
            return enqueue_forward(m, T, lm_mode, feedback);
        }
        cudaGraph_t g = nullptr;
        cudaGraphExec_t ge = nullptr;
        DC_TRY(dc_check_cuda(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal), "begin capture"));
        int st = enqueue_forward(m, T, lm_mode, feedback);
        cudaError_t e = cudaStreamEndCapture(ctx->stream, &g);
        if (st != DC_B200_OK) {
            if (g) cudaGraphDestroy(g);
            return st;
        }
        DC_TRY(dc_check_cuda(ctx, e, "end capture"));
        e = cudaGraphInstantiate(&ge, g, 0);
        cudaGraphDestroy(g);
        DC_TRY(dc_check_cuda(ctx, e, "graph instantiate"));
        dc_graph gr;
        gr.exec = ge;
        gr.launches = m->last_launches;
        it = m->graphs.emplace(key, gr).first;
    }
    m->last_launches = it->second.launches;
    return dc_check_cuda(ctx, cudaGraphLaunch(it->second.exec, ctx->stream), "graph launch");
}

static int upload_step_inputs(dc_model* m, const int32_t* tokens, const int32_t* seqs, const int32_t* positions, int T) {
    // one pinned staging area, three small copies ordered on the stream
    int32_t* st = m->h_stage + m->stage_slot * 64;
    m->stage_slot = (m->stage_slot + 1) % 16;
    if (m->stage_slot == 0) cudaStreamSynchronize(m->ctx->stream);
    memcpy(st, tokens, (size_t)T * 4);
    memcpy(st + 16, seqs, (size_t)T * 4);
    memcpy(st + 32, positions, (size_t)T * 4);
    dc_ctx* ctx = m->ctx;
    DC_TRY(dc_check_cuda(ctx, cudaMemcpyAsync(m->buf.tokens, st, (size_t)T * 4, cudaMemcpyHostToDevice, ctx->stream), "H2D tokens"));
    DC_TRY(dc_check_cuda(ctx, cudaMemcpyAsync(m->buf.seq_ids, st + 16, (size_t)T * 4, cudaMemcpyHostToDevice, ctx->stream), "H2D seqs"));
    DC_TRY(dc_check_cuda(ctx, cudaMemcpyAsync(m->buf.positions, st + 32, (size_t)T * 4, cudaMemcpyHostToDevice, ctx->stream), "H2D positions"));
    return DC_B200_OK;
}

// The persistent kernel serves decode steps of MoE models.  With two or more streams every phase is bound
// by instruction issue and the per-op kernels (more resident warps per SM) are faster (measured: 1116 vs
// 1284 us per step at 2 streams, 1546 vs 2059 at 4, 8-layer cut), so the default sends one stream to it.
static bool mega_ok(dc_model* m, int T) {
    if (!m->use_mega || (m->use_mega == 1 && T > 1)) return false;
    MegaParams p;
    const char* why = "";
    return dc_mega_plan(m, T, &p, &why);
}

static bool model_complete(dc_model* m, std::string* missing) {
    for (const std::string& n : tensor_names(m)) {
        TensorSlot s;
        if (!find_slot(m, n, &s) || !*s.slot) {
            *missing = n;
            return false;
        }
    }
    return true;
}

static int check_seq(dc_model* m, int seq) {
    if (seq < 0 || seq >= m->kv.max_seqs || !m->kv.seqs[seq].used)
        return dc_fail(m->ctx, DC_B200_INVALID_ARGUMENT, "sequence %d is not allocated", seq);
    return DC_B200_OK;
}

static int forward_chunk(dc_model* m, int seq, const int32_t* tokens, int n, int lm_mode) {
    dc_kv_seq& s = m->kv.seqs[seq];
    if (s.len + n > m->cfg.max_ctx) return dc_fail(m->ctx, DC_B200_OUT_OF_MEMORY, "sequence %d would exceed max_ctx %d", seq, m->cfg.max_ctx);
    for (int i = 0; i < n; ++i)
        if (tokens[i] < 0 || tokens[i] >= m->cfg.vocab) return dc_fail(m->ctx, DC_B200_INVALID_ARGUMENT, "token id %d out of range", tokens[i]);
    DC_TRY(dc_kv_seq_reserve(&m->kv, seq, s.len + n));
    int32_t seqs[DC_MAX_T], pos[DC_MAX_T];
    for (int i = 0; i < n; ++i) {
        seqs[i] = seq;
        pos[i] = s.len + i;
    }
    DC_TRY(upload_step_inputs(m, tokens, seqs, pos, n));
    DC_TRY(run_forward(m, n, lm_mode, false));
    s.len += n;
    return DC_B200_OK;
}

extern "C" {

int dc_b200_model_create(dc_ctx* ctx, const dc_model_config* cfg, dc_model** out) {
    if (!ctx || !cfg || !out) return DC_B200_INVALID_ARGUMENT;
    *out = nullptr;
    const dc_model_config& c = *cfg;
    if (c.head_dim != 128 || c.n_layer < 1 || c.hidden % 256 || c.n_head < 2 || c.n_kv_head < 1 || c.n_head % c.n_kv_head ||
        c.n_head / c.n_kv_head > 8 || (c.n_head & 1) || c.vocab < 2 || c.max_seqs < 1 || c.max_seqs > DC_MAX_T || c.max_ctx < 16)
        return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "model_create: unsupported shape (head_dim must be 128, hidden %% 256 == 0)");
    if (c.n_expert > 0 && (c.n_expert_used < 1 || c.n_expert_used > 16 || c.n_expert > 256 || c.expert_ffn % 256 || c.expert_ffn < 256))
        return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "model_create: unsupported MoE shape");
    if (c.n_expert == 0 && (c.ffn % 256 || c.ffn < 256)) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "model_create: ffn must be a multiple of 256");
    if (c.ep_size > 1 && (c.n_expert == 0 || c.n_expert % c.ep_size || c.ep_rank < 0 || c.ep_rank >= c.ep_size))
        return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "model_create: bad expert-parallel shard %d/%d", c.ep_rank, c.ep_size);
    cudaSetDevice(ctx->device);
    dc_model* m = new dc_model();
    m->ctx = ctx;
    m->cfg = c;
    if (m->cfg.ep_size < 1) m->cfg.ep_size = 1;
    if (m->cfg.routed_scale == 0.0f) m->cfg.routed_scale = 1.0f;
    m->layers.resize(c.n_layer);
    m->ep_lo = 0;
    m->ep_hi = c.n_expert;
    if (c.n_expert > 0 && m->cfg.ep_size > 1) {
        const int per = c.n_expert / m->cfg.ep_size;
        m->ep_lo = m->cfg.ep_rank * per;
        m->ep_hi = m->ep_lo + per;
    }
    const int blocks_per_seq = (c.max_ctx + DC_KV_BLOCK - 1) / DC_KV_BLOCK;
    int st = dc_kv_init(ctx, &m->kv, c.n_layer, c.n_kv_head, c.head_dim, blocks_per_seq * c.max_seqs, c.max_seqs, blocks_per_seq);
    // split count: about two CTAs per SM for a single-token step, at least 4 KV blocks per split at full context
    if (st == DC_B200_OK) {
        int ns = (2 * ctx->num_sms) / c.n_kv_head;
        const int max_useful = (blocks_per_seq + 3) / 4;
        if (ns > max_useful) ns = max_useful;
        if (ns > 64) ns = 64;
        if (ns < 1) ns = 1;
        m->nsplit = ns;
        st = alloc_step_buffers(m);
    }
    if (st != DC_B200_OK) {
        dc_b200_model_destroy(m);
        return st;
    }
    *out = m;
    return DC_B200_OK;
}

void dc_b200_model_destroy(dc_model* m) {
    if (!m) return;
    cudaSetDevice(m->ctx->device);
    cudaStreamSynchronize(m->ctx->stream);
    for (auto& kvp : m->graphs) cudaGraphExecDestroy(kvp.second.exec);
    dc_ep_destroy(m);
    for (dc_weight* w : m->owned) {
        if (w) {
            cudaFree(w->dev);
            delete w;
        }
    }
    dc_step_buffers& b = m->buf;
    void* ptrs[] = {b.tokens, b.seq_ids, b.positions, b.out_tokens, b.argmax_keys, b.x, b.xn, b.qkv, b.q, b.h, b.dn,
                    b.moe_out, b.logits, b.attn_mem, b.q8_x, b.q8_attn, b.q8_h, b.history, b.history_len,
                    b.route_mem, b.cos_sin, b.verify_mem};
    for (void* p : ptrs)
        if (p) cudaFree(p);
    if (m->dbg_x) cudaFree(m->dbg_x);
    dc_prefill_release(m);
    if (m->mega_layers) cudaFree(m->mega_layers);
    if (m->mega_counter) cudaFree(m->mega_counter);
    dc_mega_release_xch(m);
    if (m->h_stage) cudaFreeHost(m->h_stage);
    dc_kv_release(&m->kv);
    delete m;
}

int dc_b200_model_get_config(dc_model* m, dc_model_config* out) {
    if (!m || !out) return DC_B200_INVALID_ARGUMENT;
    *out = m->cfg;
    return DC_B200_OK;
}

int dc_b200_model_tensor_names(dc_model* m, const char** names_out, int capacity, int* n_out) {
    if (!m || !n_out) return DC_B200_INVALID_ARGUMENT;
    if (m->all_names.empty()) m->all_names = tensor_names(m);
    *n_out = (int)m->all_names.size();
    if (names_out)
        for (int i = 0; i < capacity && i < *n_out; ++i) names_out[i] = m->all_names[i].c_str();
    return DC_B200_OK;
}

int dc_b200_model_set_tensor(dc_model* m, const char* name, int ggml_type, const int64_t ne[4], const void* data_host) {
    if (!m || !name || !ne || !data_host) return DC_B200_INVALID_ARGUMENT;
    cudaSetDevice(m->ctx->device);
    TensorSlot s;
    if (!find_slot(m, name, &s)) return dc_fail(m->ctx, DC_B200_MODEL_LOAD_FAILED, "set_tensor: '%s' is not a tensor of this model", name);
    const int64_t E = ne[2] > 0 ? ne[2] : 1, N = ne[1] > 0 ? ne[1] : 1;
    if (ne[0] != s.K || N != s.N || E != s.E)
        return dc_fail(m->ctx, DC_B200_MODEL_LOAD_FAILED, "set_tensor: '%s' has shape [%lld,%lld,%lld], expected [%lld,%lld,%lld]",
                       name, (long long)ne[0], (long long)N, (long long)E, (long long)s.K, (long long)s.N, (long long)s.E);
    const bool is_vec = s.kind == 1 || s.kind == 2;
    if (is_vec && ggml_type != DC_TYPE_F32) return dc_fail(m->ctx, DC_B200_UNSUPPORTED, "set_tensor: '%s' must be F32", name);
    if (!is_vec && ggml_type != DC_TYPE_Q4_K && ggml_type != DC_TYPE_Q6_K)
        return dc_fail(m->ctx, DC_B200_UNSUPPORTED, "set_tensor: '%s' has ggml type %d; only Q4_K and Q6_K matrices are supported", name, ggml_type);
    if (*s.slot) return dc_fail(m->ctx, DC_B200_MODEL_LOAD_FAILED, "set_tensor: '%s' was already set", name);
    // expert tensors keep only this GPU's contiguous range of experts
    const int64_t e_first = s.E > 1 ? m->ep_lo : 0, e_count = s.E > 1 ? m->ep_hi - m->ep_lo : 1;
    dc_weight* w = new_weight(m, ggml_type, s.K, s.N, e_count);
    if (!w) return dc_fail(m->ctx, DC_B200_OUT_OF_MEMORY, "set_tensor: out of device memory for '%s'", name);
    const uint8_t* src = (const uint8_t*)data_host + (size_t)e_first * s.N * w->row_bytes;
    cudaError_t e = cudaMemcpyAsync(w->dev, src, w->bytes, cudaMemcpyHostToDevice, m->ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(m->ctx->stream);
    if (e != cudaSuccess) {
        cudaFree(w->dev);
        delete w;
        return dc_check_cuda(m->ctx, e, "set_tensor");
    }
    *s.slot = w;
    m->owned.push_back(w);
    m->names[name] = w;
    return DC_B200_OK;
}

int dc_b200_model_init_synthetic(dc_model* m, uint64_t seed, float sigma) {
    if (!m) return DC_B200_INVALID_ARGUMENT;
    cudaSetDevice(m->ctx->device);
    for (const std::string& n : tensor_names(m)) {
        TensorSlot s;
        if (!find_slot(m, n, &s)) return dc_fail(m->ctx, DC_B200_INTERNAL_ERROR, "init_synthetic: no slot for %s", n.c_str());
        if (*s.slot) continue;
        const int64_t e_first = s.E > 1 ? m->ep_lo : 0, e_count = s.E > 1 ? m->ep_hi - m->ep_lo : 1;
        dc_weight* w = new_weight(m, s.synth_type, s.K, s.N, e_count);
        if (!w) return dc_fail(m->ctx, DC_B200_OUT_OF_MEMORY, "init_synthetic: out of device memory for '%s'", n.c_str());
        const uint64_t ts = seed + fnv1a64(n.c_str());
        int st;
        if (s.kind == 0) st = dc_launch_synth_quantized(m->ctx, s.synth_type, ts, e_first * s.N, s.N * e_count, s.K, sigma, w->dev);
        else st = dc_launch_synth_f32(m->ctx, ts, s.K * s.N * s.E, sigma, s.kind == 1 ? 1.0f : 0.0f, (float*)w->dev);
        if (st != DC_B200_OK) {
            cudaFree(w->dev);
            delete w;
            return st;
        }
        *s.slot = w;
        m->owned.push_back(w);
        m->names[n] = w;
    }
    return dc_b200_synchronize(m->ctx);
}

int dc_b200_model_get_tensor(dc_model* m, const char* name, int* ggml_type, int64_t ne[4], void** dev, size_t* bytes) {
    if (!m || !name) return DC_B200_INVALID_ARGUMENT;
    auto it = m->names.find(name);
    if (it == m->names.end()) return dc_fail(m->ctx, DC_B200_INVALID_ARGUMENT, "get_tensor: '%s' is not set", name);
    const dc_weight* w = it->second;
    if (ggml_type) *ggml_type = w->type;
    if (ne) {
        ne[0] = w->K;
        ne[1] = w->N;
        ne[2] = w->E;
        ne[3] = 1;
    }
    if (dev) *dev = w->dev;
    if (bytes) *bytes = w->bytes;
    return DC_B200_OK;
}

int dc_b200_model_finalize(dc_model* m) {
    if (!m) return DC_B200_INVALID_ARGUMENT;
    std::string missing;
    if (!model_complete(m, &missing)) return dc_fail(m->ctx, DC_B200_MODEL_LOAD_FAILED, "finalize: tensor '%s' is missing", missing.c_str());
    if (m->cfg.ep_size > 1 && !m->ep_ready) return dc_fail(m->ctx, DC_B200_MODEL_LOAD_FAILED, "finalize: expert-parallel communicator not initialised");
    if (!m->mega_layers) DC_TRY(dc_mega_prepare(m));
    m->finalized = true;
    return DC_B200_OK;
}

size_t dc_b200_model_weight_bytes(dc_model* m) {
    size_t n = 0;
    if (m)
        for (dc_weight* w : m->owned) n += w->bytes;
    return n;
}

int dc_b200_seq_alloc(dc_model* m, int* out_seq) { return (m && out_seq) ? dc_kv_seq_alloc(&m->kv, out_seq) : DC_B200_INVALID_ARGUMENT; }
int dc_b200_seq_free(dc_model* m, int seq) { return m ? dc_kv_seq_free(&m->kv, seq) : DC_B200_INVALID_ARGUMENT; }
int dc_b200_seq_fork(dc_model* m, int src_seq, int* out_seq) {
    if (!m || !out_seq) return DC_B200_INVALID_ARGUMENT;
    cudaSetDevice(m->ctx->device);
    return dc_kv_seq_fork(&m->kv, src_seq, out_seq);
}
int dc_b200_model_free_blocks(dc_model* m) { return m ? dc_kv_available_blocks(&m->kv) : DC_B200_INVALID_ARGUMENT; }
int dc_b200_seq_len(dc_model* m, int seq) {
    if (!m || seq < 0 || seq >= m->kv.max_seqs || !m->kv.seqs[seq].used) return DC_B200_INVALID_ARGUMENT;
    return m->kv.seqs[seq].len;
}
int dc_b200_seq_truncate(dc_model* m, int seq, int new_len) {
    if (!m) return DC_B200_INVALID_ARGUMENT;
    DC_TRY(check_seq(m, seq));
    if (new_len < 0 || new_len > m->kv.seqs[seq].len) return dc_fail(m->ctx, DC_B200_INVALID_ARGUMENT, "seq_truncate: bad length %d", new_len);
    m->kv.seqs[seq].len = new_len;  // blocks stay reserved; later positions are simply overwritten
    return DC_B200_OK;
}

}  // extern "C"

int dc_model_prefill_range(dc_model* m, int seq, const int32_t* tokens_host, int n, bool final, int32_t* next_token) {
    for (int i0 = 0; i0 < n;) {
        const int left = n - i0;
        if (dc_prefill_tc_ok(m, left)) {
            // enough tokens for the tensor-core matmuls: one chunk of up to prefill_chunk tokens
            const int c = left < m->prefill_chunk ? left : m->prefill_chunk;
            DC_TRY(dc_prefill_chunk_tc(m, seq, tokens_host + i0, c, final && i0 + c >= n));
            i0 += c;
        } else {
            const int c = left < DC_MAX_T ? left : DC_MAX_T;
            DC_TRY(forward_chunk(m, seq, tokens_host + i0, c, (final && i0 + c >= n) ? 1 : 0));
            i0 += c;
        }
    }
    m->prefill_tokens_run += (uint64_t)n;
    if (!final) return DC_B200_OK;
    dc_ctx* ctx = m->ctx;
    int32_t* pin = m->h_stage + 1000;
    DC_TRY(dc_check_cuda(ctx, cudaMemcpyAsync(pin, m->buf.out_tokens, 4, cudaMemcpyDeviceToHost, ctx->stream), "D2H token"));
    DC_TRY(dc_b200_synchronize(ctx));
    if (next_token) *next_token = pin[0];
    return DC_B200_OK;
}

extern "C" {

int dc_b200_prefill(dc_model* m, int seq, const int32_t* tokens_host, int n, float* logits_host, int32_t* next_token) {
    if (!m || !tokens_host || n < 1) return m ? dc_fail(m->ctx, DC_B200_INVALID_ARGUMENT, "prefill: bad argument") : DC_B200_INVALID_ARGUMENT;
    if (!m->finalized) return dc_fail(m->ctx, DC_B200_MODEL_LOAD_FAILED, "prefill: model is not finalized");
    cudaSetDevice(m->ctx->device);
    DC_TRY(check_seq(m, seq));
    // with the prefix cache on, a sequence that holds nothing yet first takes over the cached blocks of the
    // longest whole-block prefix of its prompt (at least one token is always left to run)
    const bool fresh = m->kv.seqs[seq].len == 0 && m->kv.seqs[seq].blocks.empty();
    int skip = 0;
    if (m->prefix_cache && fresh) DC_TRY(dc_kv_prefix_attach(&m->kv, seq, tokens_host, n, &skip));
    DC_TRY(dc_model_prefill_range(m, seq, tokens_host + skip, n - skip, true, next_token));
    if (logits_host) {
        DC_TRY(dc_check_cuda(m->ctx, cudaMemcpyAsync(logits_host, m->buf.logits, (size_t)m->cfg.vocab * 4, cudaMemcpyDeviceToHost, m->ctx->stream), "D2H logits"));
        DC_TRY(dc_b200_synchronize(m->ctx));
    }
    if (m->prefix_cache && fresh) DC_TRY(dc_kv_prefix_register(&m->kv, seq, tokens_host, n));
    return DC_B200_OK;
}

int dc_b200_model_prefix_stats(dc_model* m, uint64_t out[5]) {
    if (!m || !out) return DC_B200_INVALID_ARGUMENT;
    out[0] = m->kv.prefix_lookups;
    out[1] = m->kv.prefix_hit_blocks;
    out[2] = (uint64_t)m->kv.prefix.size();
    out[3] = m->kv.prefix_evictions;
    out[4] = m->prefill_tokens_run;
    return DC_B200_OK;
}

int dc_b200_forward_chunk(dc_model* m, int seq, const int32_t* tokens_host, int n, float* logits_host) {
    if (!m || !tokens_host || n < 1 || n > DC_MAX_T) return m ? dc_fail(m->ctx, DC_B200_INVALID_ARGUMENT, "forward_chunk: bad argument") : DC_B200_INVALID_ARGUMENT;
    if (!m->finalized) return dc_fail(m->ctx, DC_B200_MODEL_LOAD_FAILED, "forward_chunk: model is not finalized");
    cudaSetDevice(m->ctx->device);
    DC_TRY(check_seq(m, seq));
    DC_TRY(forward_chunk(m, seq, tokens_host, n, 2));
    if (logits_host) {
        DC_TRY(dc_check_cuda(m->ctx, cudaMemcpyAsync(logits_host, m->buf.logits, (size_t)n * m->cfg.vocab * 4, cudaMemcpyDeviceToHost, m->ctx->stream), "D2H logits"));
        return dc_b200_synchronize(m->ctx);
    }
    return DC_B200_OK;
}

void* dc_b200_model_logits_dev(dc_model* m) { return m ? m->buf.logits : nullptr; }

int dc_b200_model_phase_timing(dc_model* m, uint64_t* ns_out, int n) {
    if (!m || !ns_out || n < 1 || n > DC_MEGA_TIMING_SLOTS || !m->mega_counter) return DC_B200_INVALID_ARGUMENT;
    cudaSetDevice(m->ctx->device);
    cudaStreamSynchronize(m->ctx->stream);
    return dc_check_cuda(m->ctx, cudaMemcpy(ns_out, (uint8_t*)m->mega_counter + 64, (size_t)n * 8, cudaMemcpyDeviceToHost), "phase timing");
}

int dc_b200_decode_step(dc_model* m, const int32_t* seqs, int n_seq, const int32_t* tokens_host, int32_t* next_tokens_host, float* logits_host) {
    if (!m || !seqs || !tokens_host || !next_tokens_host || n_seq < 1 || n_seq > DC_MAX_T)
        return m ? dc_fail(m->ctx, DC_B200_INVALID_ARGUMENT, "decode_step: bad argument") : DC_B200_INVALID_ARGUMENT;
    if (!m->finalized) return dc_fail(m->ctx, DC_B200_MODEL_LOAD_FAILED, "decode_step: model is not finalized");
    cudaSetDevice(m->ctx->device);
    dc_ctx* ctx = m->ctx;
    int32_t pos[DC_MAX_T];
    for (int i = 0; i < n_seq; ++i) {
        DC_TRY(check_seq(m, seqs[i]));
        for (int j = 0; j < i; ++j)
            if (seqs[j] == seqs[i]) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "decode_step: sequence %d appears twice", seqs[i]);
        if (tokens_host[i] < 0 || tokens_host[i] >= m->cfg.vocab) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "decode_step: token id out of range");
        dc_kv_seq& s = m->kv.seqs[seqs[i]];
        if (s.len + 1 > m->cfg.max_ctx) return dc_fail(ctx, DC_B200_OUT_OF_MEMORY, "decode_step: sequence %d is at max_ctx", seqs[i]);
        DC_TRY(dc_kv_seq_reserve(&m->kv, seqs[i], s.len + 1));
        pos[i] = s.len;
    }
    DC_TRY(upload_step_inputs(m, tokens_host, seqs, pos, n_seq));
    if (!m->prof && mega_ok(m, n_seq)) DC_TRY(dc_mega_run(m, n_seq, 1, false));
    else DC_TRY(run_forward(m, n_seq, 2, false));
    int32_t* pin = m->h_stage + 1000;
    DC_TRY(dc_check_cuda(ctx, cudaMemcpyAsync(pin, m->buf.out_tokens, (size_t)n_seq * 4, cudaMemcpyDeviceToHost, ctx->stream), "D2H tokens"));
    if (logits_host) DC_TRY(dc_check_cuda(ctx, cudaMemcpyAsync(logits_host, m->buf.logits, (size_t)n_seq * m->cfg.vocab * 4, cudaMemcpyDeviceToHost, ctx->stream), "D2H logits"));
    DC_TRY(dc_check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "sync"));
    for (int i = 0; i < n_seq; ++i) {
        next_tokens_host[i] = pin[i];
        m->kv.seqs[seqs[i]].len += 1;
    }
    return DC_B200_OK;
}

int dc_b200_decode_run(dc_model* m, const int32_t* seqs, int n_seq, const int32_t* first_tokens_host, int n_steps,
                       int32_t* out_tokens_host, float* ms_out) {
    if (!m || !seqs || !first_tokens_host || n_seq < 1 || n_seq > DC_MAX_T || n_steps < 1 || n_steps > DC_HISTORY_CAP)
        return m ? dc_fail(m->ctx, DC_B200_INVALID_ARGUMENT, "decode_run: bad argument (n_steps <= %d)", DC_HISTORY_CAP) : DC_B200_INVALID_ARGUMENT;
    if (!m->finalized) return dc_fail(m->ctx, DC_B200_MODEL_LOAD_FAILED, "decode_run: model is not finalized");
    cudaSetDevice(m->ctx->device);
    dc_ctx* ctx = m->ctx;
    int32_t pos[DC_MAX_T];
    for (int i = 0; i < n_seq; ++i) {
        DC_TRY(check_seq(m, seqs[i]));
        for (int j = 0; j < i; ++j)
            if (seqs[j] == seqs[i]) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "decode_run: sequence %d appears twice", seqs[i]);
        if (first_tokens_host[i] < 0 || first_tokens_host[i] >= m->cfg.vocab) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "decode_run: token id out of range");
        dc_kv_seq& s = m->kv.seqs[seqs[i]];
        if (s.len + n_steps > m->cfg.max_ctx) return dc_fail(ctx, DC_B200_OUT_OF_MEMORY, "decode_run: sequence %d would exceed max_ctx", seqs[i]);
        DC_TRY(dc_kv_seq_reserve(&m->kv, seqs[i], s.len + n_steps));
        pos[i] = s.len;
    }
    DC_TRY(upload_step_inputs(m, first_tokens_host, seqs, pos, n_seq));
    DC_TRY(dc_check_cuda(ctx, cudaMemsetAsync(m->buf.history_len, 0, sizeof(int), ctx->stream), "memset"));
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (ms_out) {
        cudaEventCreate(&e0);
        cudaEventCreate(&e1);
        cudaEventRecord(e0, ctx->stream);
    }
    int st = DC_B200_OK;
    if (mega_ok(m, n_seq)) st = dc_mega_run(m, n_seq, n_steps, true);   // all steps in one cooperative launch
    else
        for (int i = 0; i < n_steps && st == DC_B200_OK; ++i) st = run_forward(m, n_seq, 2, true);
    if (ms_out) {
        cudaEventRecord(e1, ctx->stream);
        cudaEventSynchronize(e1);
        cudaEventElapsedTime(ms_out, e0, e1);
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
    }
    DC_TRY(st);
    if (out_tokens_host)
        DC_TRY(dc_check_cuda(ctx, cudaMemcpyAsync(out_tokens_host, m->buf.history, (size_t)n_steps * n_seq * 4, cudaMemcpyDeviceToHost, ctx->stream), "D2H history"));
    DC_TRY(dc_b200_synchronize(ctx));
    for (int i = 0; i < n_seq; ++i) m->kv.seqs[seqs[i]].len += n_steps;
    return DC_B200_OK;
}

static const char* kClassNames[DC_K_COUNT] = {"embed", "rmsnorm_q8k", "gemv_qkv", "qknorm_rope_kv", "attention",
                                               "gemv_attn_out", "router_topk", "moe_gate_up_swiglu", "quantize_h",
                                               "moe_down", "moe_combine", "ep_allreduce", "ffn_gate_up_swiglu",
                                               "ffn_down", "lm_head_argmax", "argmax_finish"};

const char* dc_b200_kernel_class_name(int cls) { return (cls >= 0 && cls < DC_K_COUNT) ? kClassNames[cls] : nullptr; }

int dc_b200_model_profile_step(dc_model* m, const int32_t* seqs, int n_seq, const int32_t* tokens_host, int n_classes,
                               float* ms_out, int* launches_out, double* bytes_out) {
    if (!m || !seqs || !tokens_host || !ms_out || !launches_out || !bytes_out || n_classes < DC_K_COUNT)
        return m ? dc_fail(m->ctx, DC_B200_INVALID_ARGUMENT, "profile_step: need room for %d classes", DC_K_COUNT) : DC_B200_INVALID_ARGUMENT;
    const bool graphs = m->use_graphs;
    const int pdl = m->ctx->use_pdl;
    m->use_graphs = false;   // events between launches need eager, serialised launches
    m->ctx->use_pdl = 0;
    m->prof = true;
    m->prof_recs.clear();
    int32_t next[DC_MAX_T];
    int st = dc_b200_decode_step(m, seqs, n_seq, tokens_host, next, nullptr);
    m->prof = false;
    m->use_graphs = graphs;
    m->ctx->use_pdl = pdl;
    for (int i = 0; i < n_classes; ++i) {
        ms_out[i] = 0.0f;
        launches_out[i] = 0;
        bytes_out[i] = 0.0;
    }
    const double kv_bytes = 2.0 * m->cfg.n_kv_head * m->cfg.head_dim * 2.0;  // K and V, fp16, per token of context
    for (auto& r : m->prof_recs) {
        float ms = 0.0f;
        if (st == DC_B200_OK) cudaEventElapsedTime(&ms, r.e0, r.e1);
        cudaEventDestroy(r.e0);
        cudaEventDestroy(r.e1);
        ms_out[r.cls] += ms;
        launches_out[r.cls] += 1;
        double bytes = r.bytes;
        if (r.cls == DC_K_ATTENTION)
            for (int i = 0; i < n_seq; ++i) bytes += kv_bytes * m->kv.seqs[seqs[i]].len;
        bytes_out[r.cls] += bytes;
    }
    m->prof_recs.clear();
    return st;
}

int dc_b200_model_set_option(dc_model* m, const char* name, int value) {
    if (!m || !name) return DC_B200_INVALID_ARGUMENT;
    if (!strcmp(name, "graphs")) {
        m->use_graphs = value != 0;
        return DC_B200_OK;
    }
    if (!strcmp(name, "persistent")) {
        m->use_mega = value < 0 ? 0 : value > 2 ? 2 : value;
        return DC_B200_OK;
    }
    if (!strcmp(name, "route_mode")) {
        if (value != DC_ROUTE_STABLE && value != DC_ROUTE_SOFTMAX) return dc_fail(m->ctx, DC_B200_INVALID_ARGUMENT, "route_mode must be 0 or 1");
        if (value != m->route_mode) {   // captured step graphs hold the old launch parameters
            cudaStreamSynchronize(m->ctx->stream);
            for (auto& kvp : m->graphs) cudaGraphExecDestroy(kvp.second.exec);
            m->graphs.clear();
        }
        m->route_mode = value;
        return DC_B200_OK;
    }
    if (!strcmp(name, "capture_layer_inputs")) {
        cudaSetDevice(m->ctx->device);
        cudaStreamSynchronize(m->ctx->stream);
        if (value && !m->dbg_x) {
            const size_t n = (size_t)(m->cfg.n_layer + 1) * DC_MAX_T * m->cfg.hidden;
            cudaError_t e = cudaMalloc((void**)&m->dbg_x, n * sizeof(float));
            if (e == cudaSuccess) e = cudaMemset(m->dbg_x, 0, n * sizeof(float));
            if (e != cudaSuccess) {
                m->dbg_x = nullptr;
                return dc_check_cuda(m->ctx, e, "capture buffer");
            }
        } else if (!value && m->dbg_x) {
            cudaFree(m->dbg_x);
            m->dbg_x = nullptr;
        }
        return DC_B200_OK;
    }
    // Test hooks for the bounded waits of the persistent kernel: a limit small enough to run out, so that
    // the error path (status code, usable context afterwards) can be exercised without any real failure.
    if (!strcmp(name, "tc_prefill")) {
        m->use_tc_prefill = value != 0;
        return DC_B200_OK;
    }
    if (!strcmp(name, "prefill_attention")) {
        m->prefill_flash = value != 0;
        return DC_B200_OK;
    }
    if (!strcmp(name, "prefill_chunk")) {
        if (value < 32 || value > 4096) return dc_fail(m->ctx, DC_B200_INVALID_ARGUMENT, "prefill_chunk must be 32..4096");
        if (m->prefill) return dc_fail(m->ctx, DC_B200_INVALID_ARGUMENT, "prefill_chunk is fixed once a chunk has run");
        m->prefill_chunk = value;
        return DC_B200_OK;
    }
    if (!strcmp(name, "prefix_cache")) {
        m->prefix_cache = value != 0;
        return DC_B200_OK;
    }
    if (!strcmp(name, "test_ep_loopback")) return value ? dc_mega_test_loopback(m) : DC_B200_OK;
    if (!strcmp(name, "test_barrier_polls")) {
        m->test_barrier_polls = value < 0 ? 0u : (unsigned)value;
        return DC_B200_OK;
    }
    if (!strcmp(name, "test_ep_wait_us")) {
        m->test_ep_wait_ns = value < 0 ? 0ull : (unsigned long long)value * 1000ull;
        return DC_B200_OK;
    }
    if (!strcmp(name, "phase_timing")) {
        m->mega_timing = value != 0;
        if (m->mega_counter) cudaMemsetAsync((uint8_t*)m->mega_counter + 64, 0, DC_MEGA_TIMING_SLOTS * 8, m->ctx->stream);
        return DC_B200_OK;
    }
    return dc_fail(m->ctx, DC_B200_INVALID_ARGUMENT, "unknown model option '%s'", name);
}

int dc_b200_model_read_layer_input(dc_model* m, int layer, int n_tokens, float* x_host) {
    if (!m || !x_host) return DC_B200_INVALID_ARGUMENT;
    if (!m->dbg_x) return dc_fail(m->ctx, DC_B200_INVALID_ARGUMENT, "read_layer_input: set option capture_layer_inputs first");
    if (layer < 0 || layer > m->cfg.n_layer || n_tokens < 1 || n_tokens > DC_MAX_T)
        return dc_fail(m->ctx, DC_B200_INVALID_ARGUMENT, "read_layer_input: layer %d / %d tokens out of range", layer, n_tokens);
    cudaSetDevice(m->ctx->device);
    DC_TRY(dc_check_cuda(m->ctx, cudaMemcpyAsync(x_host, m->dbg_x + (size_t)layer * DC_MAX_T * m->cfg.hidden, (size_t)n_tokens * m->cfg.hidden * 4,
                                                 cudaMemcpyDeviceToHost, m->ctx->stream), "D2H layer input"));
    return dc_b200_synchronize(m->ctx);
}

int dc_b200_model_read_kv(dc_model* m, int layer, int seq, int first, int n_tokens, void* k_host, void* v_host) {
    if (!m || !k_host || !v_host) return DC_B200_INVALID_ARGUMENT;
    DC_TRY(check_seq(m, seq));
    const dc_kv_seq& s = m->kv.seqs[seq];
    if (layer < 0 || layer >= m->cfg.n_layer || first < 0 || n_tokens < 1 || first + n_tokens > (int)s.blocks.size() * DC_KV_BLOCK)
        return dc_fail(m->ctx, DC_B200_INVALID_ARGUMENT, "read_kv: layer %d, tokens [%d, %d) out of range", layer, first, first + n_tokens);
    cudaSetDevice(m->ctx->device);
    const size_t row = (size_t)m->cfg.n_kv_head * 128;   // fp16 elements per token
    const __half* ka = m->kv.k_arena + m->kv.layer_elems * layer;
    const __half* va = m->kv.v_arena + m->kv.layer_elems * layer;
    for (int t = first; t < first + n_tokens;) {
        const int blk = s.blocks[t / DC_KV_BLOCK], slot = t % DC_KV_BLOCK;
        int n = DC_KV_BLOCK - slot;
        if (n > first + n_tokens - t) n = first + n_tokens - t;
        const size_t src = ((size_t)blk * DC_KV_BLOCK + slot) * row, dst = (size_t)(t - first) * row * 2;
        DC_TRY(dc_check_cuda(m->ctx, cudaMemcpyAsync((uint8_t*)k_host + dst, ka + src, (size_t)n * row * 2, cudaMemcpyDeviceToHost, m->ctx->stream), "D2H K"));
        DC_TRY(dc_check_cuda(m->ctx, cudaMemcpyAsync((uint8_t*)v_host + dst, va + src, (size_t)n * row * 2, cudaMemcpyDeviceToHost, m->ctx->stream), "D2H V"));
        t += n;
    }
    return dc_b200_synchronize(m->ctx);
}

int dc_b200_model_step_stats(dc_model* m, int* kernels_per_step, double* weight_bytes_per_step, double* kv_bytes_per_token_ctx) {
    if (!m) return DC_B200_INVALID_ARGUMENT;
    const dc_model_config& c = m->cfg;
    if (kernels_per_step) *kernels_per_step = m->last_launches;
    // bytes one single-token step must read: every dense tensor once, top-k experts per layer, the output matrix
    double wb = 0.0;
    for (int il = 0; il < c.n_layer; ++il) {
        const dc_layer& L = m->layers[il];
        for (const dc_weight* w : {L.attn_norm, L.wq, L.wk, L.wv, L.wo, L.q_norm, L.k_norm, L.ffn_norm, L.router, L.ffn_gate, L.ffn_up, L.ffn_down})
            if (w) wb += (double)w->bytes;
        for (const dc_weight* w : {L.gate_exps, L.up_exps, L.down_exps})
            if (w) wb += (double)w->bytes / (double)w->E * c.n_expert_used;  // whole job: all ranks together read top-k experts
    }
    const dc_weight* out_w = c.tie_embeddings ? m->tok_embd : m->output;
    if (out_w) wb += (double)out_w->bytes;
    if (m->out_norm) wb += (double)m->out_norm->bytes;
    if (m->tok_embd) wb += (double)m->tok_embd->row_bytes;
    if (weight_bytes_per_step) *weight_bytes_per_step = wb;
    if (kv_bytes_per_token_ctx) *kv_bytes_per_token_ctx = 2.0 * c.n_layer * c.n_kv_head * c.head_dim * 2.0;
    return DC_B200_OK;
}

}  // extern "C"
