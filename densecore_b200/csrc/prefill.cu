// Prompt processing in chunks of up to 2048 tokens: every matmul of the decoder runs as one tensor-core
// MUL_MAT over the whole chunk (gemm_tc.cu) instead of sixteen tokens at a time through the row-streaming
// kernels, which re-read every weight for each sixteen tokens.  The CPU side of this is DenseCore's batched
// matmul path for prefill chunks (core/src/llm/matmul/batched_exec.cpp:1040-1240, chunks up to M = 4096,
// core/src/llm/matmul/dispatch.cpp:622,985-989) and ggml_flash_attn_ext (core/src/llm/attention/exec.cpp:255-275).
//
// Per layer: RMSNorm (the decode kernel, one CTA per token) -> tiled Q8_K -> Q, K, V GEMMs -> per-head norm,
// RoPE and cache write (the decode kernel) -> causal attention of every chunk token over the paged cache
// (attn_prefill.cu on the tensor cores; or the decode kernels' exact chain, one grid for the chunk) -> output projection accumulated into the residual ->
// RMSNorm -> router (logits, then one warp per token) -> assignments grouped by expert into 64-slot tiles ->
// gate and up GEMMs with an expert per tile -> SwiGLU + tiled Q8_K -> down GEMM scattered back to
// assignment order -> weighted combine (the decode kernel).  The last chunk ends with the decode path's
// output norm, lm_head row-streaming kernel and greedy pick for its last token.
#include <algorithm>

#include "dc_common.cuh"
#include "dc_gemm_tc.h"
#include "dc_model.h"

#define DC_TRY(expr)                       \
    do {                                   \
        int st_ = (expr);                  \
        if (st_ != DC_B200_OK) return st_; \
    } while (0)

using namespace dc;

struct dc_prefill_buffers {
    int cap = 0;               // tokens per chunk
    int max_tiles = 0;         // 64-slot tiles of the grouped expert matmuls
    int32_t *tokens = nullptr, *seq_ids = nullptr, *positions = nullptr;
    float *x = nullptr, *xn = nullptr, *qkv = nullptr, *q = nullptr, *att = nullptr, *g = nullptr,
          *dn = nullptr, *moe_out = nullptr, *logits = nullptr, *weights = nullptr;
    int32_t* ids = nullptr;
    int32_t *slot_assign = nullptr, *slot_token = nullptr, *tile_expert = nullptr, *pair_tile0 = nullptr, *pair_nset = nullptr;
    uint8_t *act_x = nullptr, *act_att = nullptr, *act_moe = nullptr, *act_h = nullptr, *attn_mem = nullptr;
    dc_attn_scratch attn = {};
    int32_t* h_stage = nullptr;   // pinned: ring of (tokens, seq ids, positions) triples
    int stage_slot = 0;
    std::vector<void*> owned;
};

static constexpr int PF_STAGE_SLOTS = 4;

void dc_prefill_release(dc_model* m) {
    dc_prefill_buffers* P = m->prefill;
    if (!P) return;
    for (void* p : P->owned) cudaFree(p);
    if (P->h_stage) cudaFreeHost(P->h_stage);
    delete P;
    m->prefill = nullptr;
}

template <typename T>
static int pf_alloc(dc_model* m, T** p, size_t n) {
    DC_TRY(dc_check_cuda(m->ctx, cudaMalloc((void**)p, n * sizeof(T) + 256), "cudaMalloc(prefill buffer)"));
    m->prefill->owned.push_back((void*)*p);
    return DC_B200_OK;
}

static int prefill_prepare(dc_model* m) {
    if (m->prefill) return DC_B200_OK;
    const dc_model_config& c = m->cfg;
    dc_prefill_buffers* P = m->prefill = new dc_prefill_buffers();
    const size_t C = (size_t)m->prefill_chunk, H = c.hidden, QD = (size_t)c.n_head * 128, KD = (size_t)c.n_kv_head * 128;
    const bool moe = c.n_expert > 0;
    const size_t F = moe ? c.expert_ffn : c.ffn;
    const size_t A = moe ? C * c.n_expert_used : C;
    // every expert's assignments are padded to whole tiles: at most one partly filled tile per expert
    P->max_tiles = moe ? (int)(A / 64 + c.n_expert) : (int)((C + 63) / 64);
    const size_t slots = (size_t)P->max_tiles * 64;
    P->cap = (int)C;
    int st = DC_B200_OK;
    auto A_ = [&](int s) { if (st == DC_B200_OK) st = s; };
    A_(pf_alloc(m, &P->tokens, C));
    A_(pf_alloc(m, &P->seq_ids, C));
    A_(pf_alloc(m, &P->positions, C));
    A_(pf_alloc(m, &P->x, C * H));
    A_(pf_alloc(m, &P->xn, C * H));
    A_(pf_alloc(m, &P->qkv, C * (QD + 2 * KD)));
    A_(pf_alloc(m, &P->q, C * QD));
    A_(pf_alloc(m, &P->att, C * QD));
    A_(pf_alloc(m, &P->g, slots * 2 * F));      // gate | up, 2 F columns per slot
    A_(pf_alloc(m, &P->act_x, dc_gemm_tc_act_bytes((int)C, (int)H)));
    A_(pf_alloc(m, &P->act_att, dc_gemm_tc_act_bytes((int)C, (int)QD)));
    A_(pf_alloc(m, &P->act_h, dc_gemm_tc_act_bytes((int)slots, (int)F)));
    if (moe) {
        A_(pf_alloc(m, &P->dn, A * H));
        A_(pf_alloc(m, &P->moe_out, C * H));
        A_(pf_alloc(m, &P->logits, C * c.n_expert));
        A_(pf_alloc(m, &P->weights, A));
        A_(pf_alloc(m, &P->ids, A));
        A_(pf_alloc(m, &P->slot_assign, slots));
        A_(pf_alloc(m, &P->slot_token, slots));
        A_(pf_alloc(m, &P->tile_expert, (size_t)P->max_tiles));
        A_(pf_alloc(m, &P->pair_tile0, (size_t)P->max_tiles));
        A_(pf_alloc(m, &P->pair_nset, (size_t)P->max_tiles));
        A_(pf_alloc(m, &P->act_moe, dc_gemm_tc_act_bytes((int)slots, (int)H)));
    }
    if (st == DC_B200_OK) st = dc_check_cuda(m->ctx, cudaMallocHost((void**)&P->h_stage, PF_STAGE_SLOTS * 3 * C * 4), "cudaMallocHost");
    if (st != DC_B200_OK) dc_prefill_release(m);
    return st;
}

// ---- grouping of the chunk's expert assignments ----------------------------------------------------------
// ids [C][top_k] -> the assignments of every expert (ascending experts) in runs padded to whole 64-slot tiles:
// slot_assign[slot] = t * top_k + k or -1, slot_token[slot] = t or -1, tile_expert[tile] = expert or -1.
// tile_expert holds the expert's slab index on this GPU.  Slots of one expert are filled in arrival order (the rows of a tile are independent, and results return to
// assignment order through slot_assign).  One CTA.
__global__ void __launch_bounds__(1024) k_moe_group(const int32_t* __restrict__ ids, int A, int top_k, int E, int max_tiles,
                                                    int ep_lo, int ep_hi, int32_t* __restrict__ slot_assign,
                                                    int32_t* __restrict__ slot_token, int32_t* __restrict__ tile_expert,
                                                    int32_t* __restrict__ pair_tile0, int32_t* __restrict__ pair_nset) {
    __shared__ int s_cnt[256], s_off[256], s_fill[256], s_total, s_pairs;
    const int tid = threadIdx.x;
    if (tid < 256) s_cnt[tid] = s_fill[tid] = 0;
    __syncthreads();
    for (int i = tid; i < A; i += blockDim.x) atomicAdd(&s_cnt[ids[i]], 1);
    __syncthreads();
    if (tid < 256) {
        int off = 0;
        for (int i = 0; i < tid; ++i) off += (s_cnt[i] + 63) / 64;
        s_off[tid] = off;
        const int tiles = tid < E ? (s_cnt[tid] + 63) / 64 : 0;
        // expert parallel: this GPU stores experts [ep_lo, ep_hi) only, as slabs 0 .. ep_hi - ep_lo - 1; tiles of the
        // others are skipped here and their share of the layer arrives by all-reduce
        const int local = (tid >= ep_lo && tid < ep_hi) ? tid - ep_lo : -1;
        for (int t = 0; t < tiles; ++t) tile_expert[off + t] = local;
        if (tid == 255) s_total = off + tiles;
        // pairs of neighbouring tiles of one expert (the work items of the matmul kernel's second form)
        int poff = 0;
        for (int i = 0; i < tid; ++i) poff += ((s_cnt[i] + 63) / 64 + 1) / 2;
        const int pairs = (tiles + 1) / 2;
        for (int j = 0; j < pairs; ++j) {
            pair_tile0[poff + j] = local >= 0 ? off + 2 * j : -1;
            pair_nset[poff + j] = min(2, tiles - 2 * j);
        }
        if (tid == 255) s_pairs = poff + pairs;
    }
    for (int sl = tid; sl < max_tiles * 64; sl += blockDim.x) {
        slot_assign[sl] = -1;
        slot_token[sl] = -1;
    }
    __syncthreads();
    for (int t = s_total + tid; t < max_tiles; t += blockDim.x) tile_expert[t] = -1;
    for (int t = s_pairs + tid; t < max_tiles; t += blockDim.x) pair_tile0[t] = -1;
    for (int i = tid; i < A; i += blockDim.x) {
        const int e = ids[i];
        const int slot = s_off[e] * 64 + atomicAdd(&s_fill[e], 1);
        slot_assign[slot] = i;
        slot_token[slot] = i / top_k;
    }
}

// h = silu(g) * u per slot (the production SwiGLU of the CPU kernels, see silu_fast), quantised to the
// tiled Q8_K layout of the down projection's activations.  One warp per (slot, 256-value block);
// slot_valid (optional): slots whose entry is negative hold zeros.
__global__ void __launch_bounds__(256) k_swiglu_q8k_tiled(const float* __restrict__ g, const float* __restrict__ u, int ld, int F,
                                                          int n_slots_data, uint8_t* __restrict__ act, int n_tt,
                                                          const int32_t* __restrict__ slot_valid) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = F / DC_QK_K;
    const long long total = (long long)n_tt * 64 * nb;
    for (long long item = (long long)blockIdx.x * 8 + warp; item < total; item += (long long)gridDim.x * 8) {
        const int b = (int)(item % nb), slot = (int)(item / nb);
        const bool live = slot < n_slots_data && (!slot_valid || slot_valid[slot] >= 0);
        uint8_t* tile = act + ((size_t)b * n_tt + slot / TC_NTOK) * TC_ACT_TILE;
        uint32_t w0 = 0, w1 = 0, bw = 0;
        float d = 0.0f;
        if (live) {
            const size_t base = (size_t)slot * ld + (size_t)b * DC_QK_K + 8 * lane;
            const float4 g0 = *reinterpret_cast<const float4*>(g + base), g1 = *reinterpret_cast<const float4*>(g + base + 4);
            const float4 u0 = *reinterpret_cast<const float4*>(u + base), u1 = *reinterpret_cast<const float4*>(u + base + 4);
            const float v[8] = {__fmul_rn(silu_fast(g0.x), u0.x), __fmul_rn(silu_fast(g0.y), u0.y),
                                __fmul_rn(silu_fast(g0.z), u0.z), __fmul_rn(silu_fast(g0.w), u0.w),
                                __fmul_rn(silu_fast(g1.x), u1.x), __fmul_rn(silu_fast(g1.y), u1.y),
                                __fmul_rn(silu_fast(g1.z), u1.z), __fmul_rn(silu_fast(g1.w), u1.w)};
            q8k_block_core(v, lane, w0, w1, bw, d);
        }
        tc_act_store(tile, slot % TC_NTOK, lane, w0, w1, bw, d);
    }
}

// g, u: rows of ld floats per slot
static int launch_swiglu(dc_ctx* ctx, const float* g, const float* u, int ld, int F, int n_slots_data, uint8_t* act, int n_tt,
                         const int32_t* slot_valid) {
    const long long items = (long long)n_tt * 64 * (F / DC_QK_K);
    long long blocks = (items + 7) / 8;
    if (blocks > 148 * 16) blocks = 148 * 16;
    k_swiglu_q8k_tiled<<<(unsigned)blocks, 256, 0, ctx->stream>>>(g, u, ld, F, n_slots_data, act, n_tt, slot_valid);
    return dc_check_cuda(ctx, cudaGetLastError(), "k_swiglu_q8k_tiled");
}

// Scratch of the decode kernels' exact attention chain for a whole chunk (scores of every token over the whole
// context): only allocated when that attention is asked for.
static int prefill_exact_attention_scratch(dc_model* m) {
    dc_prefill_buffers* P = m->prefill;
    if (P->attn_mem) return DC_B200_OK;
    const dc_model_config& c = m->cfg;
    const size_t att_bytes = dc_attention_scratch_bytes(P->cap, c.n_head, c.n_kv_head, m->kv.max_blocks_per_seq, m->nsplit);
    DC_TRY(pf_alloc(m, &P->attn_mem, att_bytes));
    dc_attn_scratch_bind(&P->attn, P->attn_mem, P->cap, c.n_head, c.n_kv_head, m->kv.max_blocks_per_seq, m->nsplit);
    return dc_check_cuda(m->ctx, cudaMemsetAsync(P->attn.tickets, 0, (size_t)P->cap * c.n_head * 4, m->ctx->stream), "memset");
}

// ---- one chunk ---------------------------------------------------------------------------------------------
bool dc_prefill_tc_ok(dc_model* m, int n) {
    const dc_model_config& c = m->cfg;
    if (!m->use_tc_prefill || n < m->ctx->gemm_tc_min_rows || (c.ep_size > 1 && !m->ep_ready) || m->dbg_x || m->prof) return false;
    for (const dc_layer& L : m->layers) {
        const dc_weight* ws[] = {L.wq, L.wk, L.wv, L.wo, L.gate_exps, L.up_exps, L.down_exps, L.ffn_gate, L.ffn_up, L.ffn_down};
        for (const dc_weight* w : ws)
            if (w && !dc_gemm_tc_supports(w)) return false;
    }
    return true;
}

// Appends n <= prefill_chunk tokens to the sequence; lm: also the logits and greedy pick of the last token
// (left in the step buffers of the decode path).
int dc_prefill_chunk_tc(dc_model* m, int seq, const int32_t* tokens, int n, bool lm) {
    DC_TRY(prefill_prepare(m));
    if (!m->prefill_flash) DC_TRY(prefill_exact_attention_scratch(m));
    dc_prefill_buffers& P = *m->prefill;
    const dc_model_config& c = m->cfg;
    dc_ctx* ctx = m->ctx;
    dc_kv_seq& s = m->kv.seqs[seq];
    if (n > P.cap) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "prefill chunk of %d tokens exceeds %d", n, P.cap);
    if (s.len + n > c.max_ctx) return dc_fail(ctx, DC_B200_OUT_OF_MEMORY, "sequence %d would exceed max_ctx %d", seq, c.max_ctx);
    for (int i = 0; i < n; ++i)
        if (tokens[i] < 0 || tokens[i] >= c.vocab) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "token id %d out of range", tokens[i]);
    DC_TRY(dc_kv_seq_reserve(&m->kv, seq, s.len + n));
    // inputs through a pinned ring
    if (P.stage_slot == 0) cudaStreamSynchronize(ctx->stream);
    int32_t* st = P.h_stage + (size_t)P.stage_slot * 3 * P.cap;
    P.stage_slot = (P.stage_slot + 1) % PF_STAGE_SLOTS;
    for (int i = 0; i < n; ++i) {
        st[i] = tokens[i];
        st[P.cap + i] = seq;
        st[2 * P.cap + i] = s.len + i;
    }
    DC_TRY(dc_check_cuda(ctx, cudaMemcpyAsync(P.tokens, st, (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream), "H2D tokens"));
    DC_TRY(dc_check_cuda(ctx, cudaMemcpyAsync(P.seq_ids, st + P.cap, (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream), "H2D seqs"));
    DC_TRY(dc_check_cuda(ctx, cudaMemcpyAsync(P.positions, st + 2 * P.cap, (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream), "H2D positions"));

    const int H = c.hidden, QD = c.n_head * 128, KD = c.n_kv_head * 128, QKV = QD + 2 * KD;
    const float scale = 1.0f / sqrtf((float)c.head_dim);
    const int E = c.n_expert, top_k = c.n_expert_used;
    const int n_tt = dc_gemm_tc_tiles(n);
    DC_TRY(dc_launch_embed(ctx, m->tok_embd, P.tokens, n, P.x));
    const float* pending = nullptr;   // MoE output of the previous layer, added in the next norm
    for (int il = 0; il < c.n_layer; ++il) {
        dc_layer& Ly = m->layers[il];
        DC_TRY(dc_launch_rmsnorm_q8k(ctx, P.x, pending, (const float*)Ly.attn_norm->dev, n, H, c.rms_eps, P.xn, nullptr));
        pending = nullptr;
        DC_TRY(dc_launch_quantize_q8k_tiled(ctx, P.xn, H, n, H, P.act_x, n_tt, nullptr));
        {
            // Q | K | V in as few launches as their types allow (V is often Q6_K beside Q4_K Q and K)
            const dc_weight* ws[3] = {Ly.wq, Ly.wk, Ly.wv};
            const int offs[3] = {0, QD, QD + KD};
            for (int i = 0; i < 3;) {
                int j = i + 1;
                while (j < 3 && ws[j]->type == ws[i]->type && ws[j]->row_bytes == ws[i]->row_bytes) ++j;
                DC_TRY(dc_launch_gemm_tc_multi(ctx, ws + i, offs + i, j - i, P.act_x, n, P.qkv, QKV));
                i = j;
            }
        }
        __half* ka = m->kv.k_arena + m->kv.layer_elems * il;
        __half* va = m->kv.v_arena + m->kv.layer_elems * il;
        DC_TRY(dc_launch_qknorm_rope_kv(ctx, P.qkv, Ly.q_norm ? (const float*)Ly.q_norm->dev : nullptr,
                                        Ly.k_norm ? (const float*)Ly.k_norm->dev : nullptr, m->buf.cos_sin, c.max_ctx, P.positions,
                                        P.seq_ids, m->kv.d_tables, m->kv.max_blocks_per_seq, ka, va, c.n_head, c.n_kv_head,
                                        c.rms_eps, n, P.q));
        if (m->prefill_flash)
            DC_TRY(dc_launch_attention_prefill(ctx, P.q, ka, va, m->kv.d_tables + (size_t)seq * m->kv.max_blocks_per_seq, s.len, n,
                                               c.n_head, c.n_kv_head, scale, P.att));
        else
            DC_TRY(dc_launch_attention(ctx, P.q, ka, va, m->kv.d_tables, m->kv.max_blocks_per_seq, P.seq_ids, P.positions, n,
                                       c.n_head, c.n_kv_head, scale, m->nsplit, &P.attn, P.att, nullptr));
        DC_TRY(dc_launch_quantize_q8k_tiled(ctx, P.att, QD, n, QD, P.act_att, n_tt, nullptr));
        DC_TRY(dc_launch_gemm_tc(ctx, Ly.wo, P.act_att, n, P.x, H, nullptr, nullptr, true));
        DC_TRY(dc_launch_rmsnorm_q8k(ctx, P.x, nullptr, (const float*)Ly.ffn_norm->dev, n, H, c.rms_eps, P.xn, nullptr));
        if (E > 0) {
            const int A = n * top_k, F = c.expert_ffn;
            DC_TRY(dc_launch_router_batched(ctx, Ly.router, P.xn, n, top_k, c.routed_scale, P.logits, P.ids, P.weights, m->route_mode));
            k_moe_group<<<1, 1024, 0, ctx->stream>>>(P.ids, A, top_k, E, P.max_tiles, m->ep_lo, m->ep_hi, P.slot_assign, P.slot_token,
                                                     P.tile_expert, P.pair_tile0, P.pair_nset);
            DC_TRY(dc_check_cuda(ctx, cudaGetLastError(), "k_moe_group"));
            const int slots = P.max_tiles * 64;
            DC_TRY(dc_launch_quantize_q8k_tiled(ctx, P.xn, H, n, H, P.act_moe, P.max_tiles, P.slot_token));
            if (Ly.gate_exps->type == Ly.up_exps->type) {
                // gate | up in one launch: g and u are one buffer of 2 F columns per slot (gate first)
                const dc_weight* ws[2] = {Ly.gate_exps, Ly.up_exps};
                const int offs[2] = {0, F};
                DC_TRY(dc_launch_gemm_tc_multi(ctx, ws, offs, 2, P.act_moe, slots, P.g, 2 * F, P.tile_expert, nullptr, false, P.pair_tile0,
                                               P.pair_nset, P.max_tiles));
            } else {
                DC_TRY(dc_launch_gemm_tc(ctx, Ly.gate_exps, P.act_moe, slots, P.g, 2 * F, P.tile_expert, nullptr, false, P.pair_tile0,
                                         P.pair_nset, P.max_tiles));
                DC_TRY(dc_launch_gemm_tc(ctx, Ly.up_exps, P.act_moe, slots, P.g + F, 2 * F, P.tile_expert, nullptr, false, P.pair_tile0,
                                         P.pair_nset, P.max_tiles));
            }
            DC_TRY(launch_swiglu(ctx, P.g, P.g + F, 2 * F, F, slots, P.act_h, P.max_tiles, P.slot_assign));
            DC_TRY(dc_launch_gemm_tc(ctx, Ly.down_exps, P.act_h, slots, P.dn, H, P.tile_expert, P.slot_assign, false, P.pair_tile0,
                                     P.pair_nset, P.max_tiles));
            DC_TRY(dc_launch_moe_combine(ctx, P.dn, P.ids, P.weights, n, top_k, H, m->ep_lo, m->ep_hi, P.moe_out));
            if (c.ep_size > 1) DC_TRY(dc_ep_allreduce(m, P.moe_out, (size_t)n * H));
            pending = P.moe_out;
        } else {
            const int F = c.ffn;
            DC_TRY(dc_launch_quantize_q8k_tiled(ctx, P.xn, H, n, H, P.act_x, n_tt, nullptr));
            if (Ly.ffn_gate->type == Ly.ffn_up->type) {
                const dc_weight* ws[2] = {Ly.ffn_gate, Ly.ffn_up};
                const int offs[2] = {0, F};
                DC_TRY(dc_launch_gemm_tc_multi(ctx, ws, offs, 2, P.act_x, n, P.g, 2 * F));
            } else {
                DC_TRY(dc_launch_gemm_tc(ctx, Ly.ffn_gate, P.act_x, n, P.g, 2 * F));
                DC_TRY(dc_launch_gemm_tc(ctx, Ly.ffn_up, P.act_x, n, P.g + F, 2 * F));
            }
            DC_TRY(launch_swiglu(ctx, P.g, P.g + F, 2 * F, F, n, P.act_h, n_tt, nullptr));
            DC_TRY(dc_launch_gemm_tc(ctx, Ly.ffn_down, P.act_h, n, P.x, H, nullptr, nullptr, true));
        }
    }
    if (lm) {
        // the last token through the decode path's output norm, lm_head and greedy pick
        dc_step_buffers& b = m->buf;
        const size_t off = (size_t)(n - 1) * H;
        DC_TRY(dc_launch_rmsnorm_q8k(ctx, P.x + off, pending ? pending + off : nullptr, (const float*)m->out_norm->dev, 1, H,
                                     c.rms_eps, nullptr, b.q8_x));
        const dc_weight* out_w = c.tie_embeddings ? m->tok_embd : m->output;
        dc_gemv_seg lmh = {out_w->dev, out_w->type, c.vocab, (int)out_w->row_bytes, b.logits, c.vocab};
        DC_TRY(dc_launch_gemv(ctx, &lmh, 1, DC_EPI_STORE, b.q8_x, 1, H, b.argmax_keys));
        DC_TRY(dc_launch_argmax_finish(ctx, b.argmax_keys, 1, b.out_tokens, nullptr, nullptr, nullptr, nullptr, DC_HISTORY_CAP));
    }
    s.len += n;
    return DC_B200_OK;
}
