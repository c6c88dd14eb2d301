// C-ABI entry points for single ops with host buffers: MUL_MAT_ID, paged
// flash-decode attention, sampling and the speculative verify step.  Each call
// stages its inputs in the context's scratch area, runs the same kernels the
// decoder uses, and copies the result back.
#include <string.h>

#include <vector>

#include "dc_common.cuh"
#include "dc_internal.h"
#include "dc_kv.h"

#define DC_TRY(expr)                       \
    do {                                   \
        int _st = (expr);                  \
        if (_st != DC_B200_OK) return _st; \
    } while (0)

namespace {
struct Bump {
    uint8_t* base;
    size_t off = 0;
    template <typename T>
    T* take(size_t n) {
        T* p = reinterpret_cast<T*>(base + off);
        off += (n * sizeof(T) + 255) & ~(size_t)255;
        return p;
    }
};
int h2d(dc_ctx* ctx, void* d, const void* h, size_t n) {
    return dc_check_cuda(ctx, cudaMemcpyAsync(d, h, n, cudaMemcpyHostToDevice, ctx->stream), "H2D");
}
int d2h(dc_ctx* ctx, void* h, const void* d, size_t n) {
    return dc_check_cuda(ctx, cudaMemcpyAsync(h, d, n, cudaMemcpyDeviceToHost, ctx->stream), "D2H");
}
}  // namespace

size_t dc_moe_route_bind(dc_moe_route* rt, uint8_t* base, int T, int E, int top_k) {
    Bump b{base};
    rt->logits = b.take<float>((size_t)T * E);
    rt->ids = b.take<int32_t>((size_t)T * top_k);
    rt->weights = b.take<float>((size_t)T * top_k);
    rt->ticket = b.take<int>(1);
    rt->n_active = b.take<int>(1);
    rt->uexp = b.take<int32_t>(E);
    rt->uoff = b.take<int32_t>(E + 1);
    rt->uassign = b.take<int32_t>((size_t)T * top_k);
    return b.off;
}

extern "C" {

int dc_b200_alloc_device(dc_ctx* ctx, size_t bytes, void** out_dev) {
    if (!ctx || !out_dev) return DC_B200_INVALID_ARGUMENT;
    cudaSetDevice(ctx->device);
    return dc_check_cuda(ctx, cudaMalloc(out_dev, bytes), "alloc_device");
}
int dc_b200_free_device(dc_ctx* ctx, void* dev) {
    if (!ctx) return DC_B200_INVALID_ARGUMENT;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    return dc_check_cuda(ctx, cudaFree(dev), "free_device");
}
int dc_b200_copy_to_device(dc_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes) {
    if (!ctx || !dst_dev || !src_host) return DC_B200_INVALID_ARGUMENT;
    cudaSetDevice(ctx->device);
    DC_TRY(h2d(ctx, dst_dev, src_host, bytes));
    return dc_check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "copy_to_device");
}
int dc_b200_copy_from_device(dc_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes) {
    if (!ctx || !dst_host || !src_dev) return DC_B200_INVALID_ARGUMENT;
    cudaSetDevice(ctx->device);
    DC_TRY(d2h(ctx, dst_host, src_dev, bytes));
    return dc_check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "copy_from_device");
}

int dc_b200_moe_route(dc_ctx* ctx, const float* logits_host, int T, int n_expert, int top_k, float routed_scale,
                      int32_t* ids_out, float* weights_out) {
    if (!ctx) return DC_B200_INVALID_ARGUMENT;
    if (!logits_host || !ids_out || !weights_out || T < 1 || T > DC_MAX_T)
        return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "moe_route: bad argument");
    // checked before anything is carved, cleared or copied: the scratch is sized from these
    if (n_expert < 1 || n_expert > 256 || top_k < 1 || top_k > 16 || top_k > n_expert)
        return dc_fail(ctx, DC_B200_UNSUPPORTED, "moe_route: n_expert=%d top_k=%d out of range (1..256 experts, top_k <= min(16, n_expert))",
                       n_expert, top_k);
    cudaSetDevice(ctx->device);
    dc_moe_route rt;
    const size_t need = dc_moe_route_bind(&rt, nullptr, T, n_expert, top_k);
    uint8_t* s = dc_scratch(ctx, need + 256);
    if (!s) return DC_B200_OUT_OF_MEMORY;
    dc_moe_route_bind(&rt, s, T, n_expert, top_k);
    DC_TRY(dc_check_cuda(ctx, cudaMemsetAsync(rt.ticket, 0, sizeof(int), ctx->stream), "memset"));
    DC_TRY(h2d(ctx, rt.logits, logits_host, (size_t)T * n_expert * 4));
    DC_TRY(dc_launch_router(ctx, nullptr, nullptr, n_expert, T, top_k, routed_scale, 0, n_expert, &rt, ctx->route_mode));
    DC_TRY(d2h(ctx, ids_out, rt.ids, (size_t)T * top_k * 4));
    DC_TRY(d2h(ctx, weights_out, rt.weights, (size_t)T * top_k * 4));
    return dc_b200_synchronize(ctx);
}

// router == nullptr: the caller supplies the router logits (cb_moe_forward's src1)
static int mul_mat_id_check(dc_ctx* ctx, const dc_weight* router, const dc_weight* gate, const dc_weight* up,
                            const dc_weight* down, int T, int top_k, bool need_router = true) {
    if ((need_router && !router) || !gate || !up || !down || T < 1 || T > DC_MAX_T)
        return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "mul_mat_id: bad argument (T=%d)", T);
    const int H = (int)gate->K, F = (int)gate->N, E = (int)gate->E;
    if ((router && (router->K != H || router->N != E)) || up->K != H || up->N != F || up->E != E || down->K != F ||
        down->N != H || down->E != E)
        return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "mul_mat_id: tensor shapes do not agree");
    if (E < 1 || E > 256 || top_k < 1 || top_k > 16 || top_k > E)
        return dc_fail(ctx, DC_B200_UNSUPPORTED, "mul_mat_id: n_expert=%d top_k=%d out of range (1..256 experts, top_k <= min(16, n_expert))", E, top_k);
    if (H % 256 || F % 256) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "mul_mat_id: hidden and ffn sizes must be multiples of 256");
    return DC_B200_OK;
}

// Enqueues one MoE layer on device buffers: x_dev [T, H] -> y_dev [T, H]; ids_dev / w_dev (optional) receive the
// routing.  Scratch comes from the context (grown on first use).
static int moe_layer_dev(dc_ctx* ctx, const dc_weight* router, const float* logits_dev, const dc_weight* gate,
                         const dc_weight* up, const dc_weight* down, const float* x_dev, int T, int top_k,
                         float routed_scale, float* y_dev, int32_t* ids_dev, float* weights_dev) {
    if (!ctx) return DC_B200_INVALID_ARGUMENT;
    if (!x_dev || !y_dev || (!router && !logits_dev)) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "mul_mat_id_dev: null buffer");
    DC_TRY(mul_mat_id_check(ctx, router, gate, up, down, T, top_k, router != nullptr));
    const int H = (int)gate->K, F = (int)gate->N, E = (int)gate->E;
    cudaSetDevice(ctx->device);
    const int A = T * top_k;
    dc_moe_route rt_size;
    const size_t need = (size_t)T * (H / 256) * 292 + (size_t)A * F * 4 + (size_t)A * (F / 256) * 292 + (size_t)A * H * 4 +
                        dc_moe_route_bind(&rt_size, nullptr, T, E, top_k) + 4096;
    uint8_t* s = dc_scratch(ctx, need);
    if (!s) return DC_B200_OUT_OF_MEMORY;
    Bump b{s};
    uint8_t* xq = b.take<uint8_t>((size_t)T * (H / 256) * 292);
    float* h = b.take<float>((size_t)A * F);
    uint8_t* hq = b.take<uint8_t>((size_t)A * (F / 256) * 292);
    float* dn = b.take<float>((size_t)A * H);
    dc_moe_route rt;
    dc_moe_route_bind(&rt, s + b.off, T, E, top_k);
    DC_TRY(dc_check_cuda(ctx, cudaMemsetAsync(rt.ticket, 0, sizeof(int), ctx->stream), "memset"));
    if (!router)
        DC_TRY(dc_check_cuda(ctx, cudaMemcpyAsync(rt.logits, logits_dev, (size_t)T * E * 4, cudaMemcpyDeviceToDevice, ctx->stream), "logits"));
    DC_TRY(dc_launch_router(ctx, router, x_dev, E, T, top_k, routed_scale, 0, E, &rt, ctx->route_mode));
    DC_TRY(dc_launch_quantize_q8k(ctx, x_dev, T, H, xq));
    DC_TRY(dc_launch_moe_mm(ctx, true, gate, up, xq, T, T, top_k, 0, &rt, h));
    DC_TRY(dc_launch_quantize_q8k(ctx, h, A, F, hq));
    DC_TRY(dc_launch_moe_mm(ctx, false, down, nullptr, hq, A, T, top_k, 0, &rt, dn));
    DC_TRY(dc_launch_moe_combine(ctx, dn, rt.ids, rt.weights, T, top_k, H, 0, E, y_dev));
    if (ids_dev) DC_TRY(dc_check_cuda(ctx, cudaMemcpyAsync(ids_dev, rt.ids, (size_t)A * 4, cudaMemcpyDeviceToDevice, ctx->stream), "ids"));
    if (weights_dev) DC_TRY(dc_check_cuda(ctx, cudaMemcpyAsync(weights_dev, rt.weights, (size_t)A * 4, cudaMemcpyDeviceToDevice, ctx->stream), "weights"));
    return DC_B200_OK;
}

int dc_b200_mul_mat_id_dev(dc_ctx* ctx, const dc_weight* router, const dc_weight* gate, const dc_weight* up,
                           const dc_weight* down, const float* x_dev, int T, int top_k, float routed_scale,
                           float* y_dev, int32_t* ids_dev, float* weights_dev) {
    if (ctx && !router) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "mul_mat_id_dev: null router");
    return moe_layer_dev(ctx, router, nullptr, gate, up, down, x_dev, T, top_k, routed_scale, y_dev, ids_dev, weights_dev);
}

static int moe_layer_host(dc_ctx* ctx, const dc_weight* router, const float* logits_host, const dc_weight* gate,
                          const dc_weight* up, const dc_weight* down, const float* x_host, int T, int top_k,
                          float routed_scale, float* y_host, int32_t* ids_out, float* weights_out);

int dc_b200_mul_mat_id(dc_ctx* ctx, const dc_weight* router, const dc_weight* gate, const dc_weight* up,
                       const dc_weight* down, const float* x_host, int T, int top_k, float routed_scale,
                       float* y_host, int32_t* ids_out, float* weights_out) {
    if (ctx && !router) {
        if (y_host && gate && T > 0 && T <= DC_MAX_T) memset(y_host, 0, (size_t)T * gate->K * sizeof(float));
        return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "mul_mat_id: null router");
    }
    return moe_layer_host(ctx, router, nullptr, gate, up, down, x_host, T, top_k, routed_scale, y_host, ids_out, weights_out);
}

int dc_b200_moe_forward(dc_ctx* ctx, const dc_weight* gate, const dc_weight* up, const dc_weight* down,
                        const float* x_host, const float* gate_logits_host, int T, int top_k, float routed_scale,
                        float* y_host, int32_t* ids_out, float* weights_out) {
    if (ctx && !gate_logits_host) {
        if (y_host && gate && T > 0 && T <= DC_MAX_T) memset(y_host, 0, (size_t)T * gate->K * sizeof(float));
        return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "moe_forward: null gate logits");
    }
    return moe_layer_host(ctx, nullptr, gate_logits_host, gate, up, down, x_host, T, top_k, routed_scale, y_host, ids_out,
                          weights_out);
}

static int moe_layer_host(dc_ctx* ctx, const dc_weight* router, const float* logits_host, const dc_weight* gate,
                          const dc_weight* up, const dc_weight* down, const float* x_host, int T, int top_k,
                          float routed_scale, float* y_host, int32_t* ids_out, float* weights_out) {
    if (!ctx) return DC_B200_INVALID_ARGUMENT;
    if (!gate || !x_host || !y_host || T < 1 || T > DC_MAX_T)
        return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "mul_mat_id: bad argument (T=%d)", T);
    const int H = (int)gate->K;
    auto fail_closed = [&](int st) {
        memset(y_host, 0, (size_t)T * H * sizeof(float));  // zero-fill on failure (moe/exec.cpp:397-414)
        return st;
    };
    int st = mul_mat_id_check(ctx, router, gate, up, down, T, top_k, router != nullptr);
    if (st != DC_B200_OK) return fail_closed(st);
    cudaSetDevice(ctx->device);
    const int A = T * top_k;
    const size_t lb = router ? 0 : (size_t)T * gate->E * 4;
    // staging buffers of this call live in pinned-size device allocations of their own (the context's scratch
    // belongs to the device-level call)
    float *x = nullptr, *y = nullptr, *w = nullptr;
    int32_t* ids = nullptr;
    const size_t xb = (size_t)T * H * 4;
    cudaError_t e = cudaMalloc((void**)&x, 2 * xb + (size_t)A * 8 + lb + 1024);
    if (e != cudaSuccess) return fail_closed(dc_check_cuda(ctx, e, "mul_mat_id staging"));
    y = (float*)((uint8_t*)x + xb);
    ids = (int32_t*)((uint8_t*)y + xb);
    w = (float*)(ids + A);
    float* lg = router ? nullptr : w + A;
    st = h2d(ctx, x, x_host, xb);
    if (st == DC_B200_OK && lg) st = h2d(ctx, lg, logits_host, lb);
    if (st == DC_B200_OK) st = moe_layer_dev(ctx, router, lg, gate, up, down, x, T, top_k, routed_scale, y, ids, w);
    if (st == DC_B200_OK) st = d2h(ctx, y_host, y, xb);
    if (st == DC_B200_OK && ids_out) st = d2h(ctx, ids_out, ids, (size_t)A * 4);
    if (st == DC_B200_OK && weights_out) st = d2h(ctx, weights_out, w, (size_t)A * 4);
    if (st == DC_B200_OK) st = dc_b200_synchronize(ctx);
    else cudaStreamSynchronize(ctx->stream);
    cudaFree(x);
    return st == DC_B200_OK ? st : fail_closed(st);
}

int dc_b200_flash_attn_decode(dc_ctx* ctx, dc_kv_cache* kv, int layer, const float* q_host, const float* k_host,
                              const float* v_host, const int32_t* seq_ids, const int32_t* positions, int T, int n_head,
                              float scale, float* out_host) {
    if (!ctx) return DC_B200_INVALID_ARGUMENT;
    if (!out_host || T < 1 || n_head < 1) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "flash_attn_decode: bad argument");
    const size_t out_n = (size_t)T * n_head * 128;
    auto fail_closed = [&](int st) {
        memset(out_host, 0, out_n * sizeof(float));  // zero-fill on failure (paged_exec.cpp:358-412)
        return st;
    };
    if (!kv || !q_host || !k_host || !v_host || !seq_ids || !positions || T > DC_MAX_T || layer < 0 ||
        layer >= kv->n_layer)
        return fail_closed(dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "flash_attn_decode: bad argument (T=%d layer=%d)", T, layer));
    for (int t = 0; t < T; ++t) {
        const int s = seq_ids[t];
        if (s < 0 || s >= kv->max_seqs || !kv->seqs[s].used || positions[t] < 0)
            return fail_closed(dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "flash_attn_decode: token %d has a bad sequence or position", t));
    }
    cudaSetDevice(ctx->device);
    for (int t = 0; t < T; ++t) {
        int st = dc_kv_seq_reserve(kv, seq_ids[t], positions[t] + 1);
        if (st != DC_B200_OK) return fail_closed(st);
        if (kv->seqs[seq_ids[t]].len < positions[t] + 1) kv->seqs[seq_ids[t]].len = positions[t] + 1;
    }
    const int n_kv = kv->n_kv, heads = n_head + 2 * n_kv, nsplit = 16;
    const size_t att_bytes = dc_attention_scratch_bytes(T, n_head, n_kv, kv->max_blocks_per_seq, nsplit);
    uint8_t* s = dc_scratch(ctx, (size_t)T * heads * 128 * 4 * 3 + att_bytes + (1 << 16));
    if (!s) return fail_closed(DC_B200_OUT_OF_MEMORY);
    Bump b{s};
    float* qkv = b.take<float>((size_t)T * heads * 128);
    float* q = b.take<float>((size_t)T * n_head * 128);
    float* out = b.take<float>(out_n);
    uint8_t* att_mem = b.take<uint8_t>(att_bytes);
    dc_attn_scratch asc;
    dc_attn_scratch_bind(&asc, att_mem, T, n_head, n_kv, kv->max_blocks_per_seq, nsplit);
    int32_t* d_seq = b.take<int32_t>(T);
    int32_t* d_pos = b.take<int32_t>(T);
    std::vector<float> packed((size_t)T * heads * 128);
    for (int t = 0; t < T; ++t) {
        float* row = packed.data() + (size_t)t * heads * 128;
        memcpy(row, q_host + (size_t)t * n_head * 128, (size_t)n_head * 128 * 4);
        memcpy(row + (size_t)n_head * 128, k_host + (size_t)t * n_kv * 128, (size_t)n_kv * 128 * 4);
        memcpy(row + (size_t)(n_head + n_kv) * 128, v_host + (size_t)t * n_kv * 128, (size_t)n_kv * 128 * 4);
    }
    int st = dc_check_cuda(ctx, cudaMemsetAsync(asc.tickets, 0, (size_t)T * n_kv * 4, ctx->stream), "memset");
    if (st == DC_B200_OK) st = dc_check_cuda(ctx, cudaMemcpyAsync(qkv, packed.data(), packed.size() * 4, cudaMemcpyHostToDevice, ctx->stream), "H2D qkv");
    if (st == DC_B200_OK) st = h2d(ctx, d_seq, seq_ids, (size_t)T * 4);
    if (st == DC_B200_OK) st = h2d(ctx, d_pos, positions, (size_t)T * 4);
    // pageable sources: make sure the copies are done before `packed` goes away
    if (st == DC_B200_OK) st = dc_check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "sync");
    __half* ka = kv->k_arena + kv->layer_elems * layer;
    __half* va = kv->v_arena + kv->layer_elems * layer;
    if (st == DC_B200_OK)
        st = dc_launch_qknorm_rope_kv(ctx, qkv, nullptr, nullptr, nullptr, 0, d_pos, d_seq, kv->d_tables,
                                      kv->max_blocks_per_seq, ka, va, n_head, n_kv, 0.0f, T, q);
    if (st == DC_B200_OK)
        st = dc_launch_attention(ctx, q, ka, va, kv->d_tables, kv->max_blocks_per_seq, d_seq, d_pos, T, n_head, n_kv,
                                 scale, nsplit, &asc, out, nullptr);
    if (st == DC_B200_OK) st = d2h(ctx, out_host, out, out_n * 4);
    if (st == DC_B200_OK) st = dc_b200_synchronize(ctx);
    return st == DC_B200_OK ? st : fail_closed(st);
}

// Prompt-chunk form of the attention op: n tokens of ONE sequence at positions pos0 .. pos0 + n - 1 (their K/V
// rows are written first), causal attention on the tensor cores (ggml_flash_attn_ext on the CPU,
// core/src/llm/attention/exec.cpp:255-275).
int dc_b200_flash_attn_prefill(dc_ctx* ctx, dc_kv_cache* kv, int layer, const float* q_host, const float* k_host,
                               const float* v_host, int seq, int pos0, int n, int n_head, float scale, float* out_host) {
    if (!ctx) return DC_B200_INVALID_ARGUMENT;
    if (!out_host || n < 1 || n_head < 1) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "flash_attn_prefill: bad argument");
    const size_t out_n = (size_t)n * n_head * 128;
    auto fail_closed = [&](int st) {
        memset(out_host, 0, out_n * sizeof(float));
        return st;
    };
    if (!kv || !q_host || !k_host || !v_host || n > 4096 || layer < 0 || layer >= kv->n_layer || seq < 0 ||
        seq >= kv->max_seqs || !kv->seqs[seq].used || pos0 < 0 || n_head % kv->n_kv)
        return fail_closed(dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "flash_attn_prefill: bad argument (n=%d layer=%d seq=%d)", n, layer, seq));
    cudaSetDevice(ctx->device);
    int st = dc_kv_seq_reserve(kv, seq, pos0 + n);
    if (st != DC_B200_OK) return fail_closed(st);
    if (kv->seqs[seq].len < pos0 + n) kv->seqs[seq].len = pos0 + n;
    const int n_kv = kv->n_kv, heads = n_head + 2 * n_kv;
    uint8_t* s = dc_scratch(ctx, (size_t)n * heads * 128 * 4 * 3 + (size_t)n * 8 + (1 << 16));
    if (!s) return fail_closed(DC_B200_OUT_OF_MEMORY);
    Bump b{s};
    float* qkv = b.take<float>((size_t)n * heads * 128);
    float* q = b.take<float>((size_t)n * n_head * 128);
    float* out = b.take<float>(out_n);
    int32_t* d_seq = b.take<int32_t>(n);
    int32_t* d_pos = b.take<int32_t>(n);
    std::vector<float> packed((size_t)n * heads * 128);
    std::vector<int32_t> meta(2 * (size_t)n);
    for (int t = 0; t < n; ++t) {
        float* row = packed.data() + (size_t)t * heads * 128;
        memcpy(row, q_host + (size_t)t * n_head * 128, (size_t)n_head * 128 * 4);
        memcpy(row + (size_t)n_head * 128, k_host + (size_t)t * n_kv * 128, (size_t)n_kv * 128 * 4);
        memcpy(row + (size_t)(n_head + n_kv) * 128, v_host + (size_t)t * n_kv * 128, (size_t)n_kv * 128 * 4);
        meta[t] = seq;
        meta[n + t] = pos0 + t;
    }
    st = dc_check_cuda(ctx, cudaMemcpyAsync(qkv, packed.data(), packed.size() * 4, cudaMemcpyHostToDevice, ctx->stream), "H2D qkv");
    if (st == DC_B200_OK) st = h2d(ctx, d_seq, meta.data(), (size_t)n * 4);
    if (st == DC_B200_OK) st = h2d(ctx, d_pos, meta.data() + n, (size_t)n * 4);
    if (st == DC_B200_OK) st = dc_check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "sync");
    __half* ka = kv->k_arena + kv->layer_elems * layer;
    __half* va = kv->v_arena + kv->layer_elems * layer;
    if (st == DC_B200_OK)
        st = dc_launch_qknorm_rope_kv(ctx, qkv, nullptr, nullptr, nullptr, 0, d_pos, d_seq, kv->d_tables,
                                      kv->max_blocks_per_seq, ka, va, n_head, n_kv, 0.0f, n, q);
    if (st == DC_B200_OK)
        st = dc_launch_attention_prefill(ctx, q, ka, va, kv->d_tables + (size_t)seq * kv->max_blocks_per_seq, pos0, n, n_head,
                                         n_kv, scale, out);
    if (st == DC_B200_OK) st = d2h(ctx, out_host, out, out_n * 4);
    if (st == DC_B200_OK) st = dc_b200_synchronize(ctx);
    return st == DC_B200_OK ? st : fail_closed(st);
}

int dc_b200_argmax(dc_ctx* ctx, const float* logits_host, int rows, int n, int32_t* out_ids) {
    if (!ctx || !logits_host || !out_ids || rows < 1 || n < 1) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "argmax: bad argument");
    cudaSetDevice(ctx->device);
    uint8_t* s = dc_scratch(ctx, (size_t)rows * n * 4 + rows * 4 + 512);
    if (!s) return DC_B200_OUT_OF_MEMORY;
    Bump b{s};
    float* l = b.take<float>((size_t)rows * n);
    int32_t* o = b.take<int32_t>(rows);
    DC_TRY(h2d(ctx, l, logits_host, (size_t)rows * n * 4));
    DC_TRY(dc_launch_argmax_rows(ctx, l, rows, n, o));
    DC_TRY(d2h(ctx, out_ids, o, (size_t)rows * 4));
    return dc_b200_synchronize(ctx);
}

int dc_b200_verify_uniforms(dc_ctx* ctx, uint64_t seed, uint32_t step, int n, float* out_host) {
    if (!ctx || !out_host || n < 1 || n > 32) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "verify_uniforms: bad argument");
    cudaSetDevice(ctx->device);
    uint8_t* s = dc_scratch(ctx, 1024);
    if (!s) return DC_B200_OUT_OF_MEMORY;
    DC_TRY(dc_launch_verify_uniforms(ctx, seed, step, n, (float*)s));
    DC_TRY(d2h(ctx, out_host, s, (size_t)n * 4));
    return dc_b200_synchronize(ctx);
}

int dc_b200_softmax(dc_ctx* ctx, const float* logits_host, int rows, int n, float temperature, float* probs_host) {
    if (!ctx || !logits_host || !probs_host || rows < 1 || n < 1 || !(temperature > 0.0f))
        return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "softmax: bad argument");
    cudaSetDevice(ctx->device);
    uint8_t* s = dc_scratch(ctx, (size_t)rows * n * 8 + 512);
    if (!s) return DC_B200_OUT_OF_MEMORY;
    Bump b{s};
    float* l = b.take<float>((size_t)rows * n);
    float* p = b.take<float>((size_t)rows * n);
    DC_TRY(h2d(ctx, l, logits_host, (size_t)rows * n * 4));
    DC_TRY(dc_launch_det_softmax(ctx, l, rows, n, temperature, p));
    DC_TRY(d2h(ctx, probs_host, p, (size_t)rows * n * 4));
    return dc_b200_synchronize(ctx);
}

// Temperature sampling on device-resident logits: probs_dev [vocab] receives softmax(logits / temperature)
// (the draft distribution q of a speculative step), *token_out one draw from it by inverse CDF with uniform u.
int dc_b200_sample_dev(dc_ctx* ctx, const float* logits_dev, int vocab, float temperature, float u, float* probs_dev,
                       int32_t* token_out) {
    if (!ctx) return DC_B200_INVALID_ARGUMENT;
    if (!logits_dev || !probs_dev || !token_out || vocab < 2 || !(temperature > 0.0f) || !(u >= 0.0f && u < 1.0f))
        return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "sample_dev: bad argument");
    cudaSetDevice(ctx->device);
    uint8_t* s = dc_scratch(ctx, 1024);
    if (!s) return DC_B200_OUT_OF_MEMORY;
    float* ud = (float*)s;
    int32_t* res = (int32_t*)(s + 256);
    DC_TRY(h2d(ctx, ud, &u, 4));
    DC_TRY(dc_check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "sync"));   // `u` is a stack value
    DC_TRY(dc_launch_sample(ctx, logits_dev, vocab, temperature, ud, probs_dev, res));
    int32_t out = -1;
    DC_TRY(d2h(ctx, &out, res, 4));
    DC_TRY(dc_b200_synchronize(ctx));
    *token_out = out;
    return DC_B200_OK;
}

int dc_b200_verify_accept(dc_ctx* ctx, const float* target_logits_host, const int32_t* draft_tokens,
                          const float* draft_probs_host, const float* uniforms, uint64_t seed, uint32_t step,
                          int gamma, int vocab, int mode, float temperature, int32_t* n_accepted,
                          int32_t* next_token) {
    if (!ctx) return DC_B200_INVALID_ARGUMENT;
    if (!target_logits_host || !draft_tokens || !n_accepted || !next_token || gamma < 1 || gamma > 16 || vocab < 2 ||
        (mode != 0 && mode != 1) || (mode == 1 && !draft_probs_host))
        return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "verify_accept: bad argument");
    for (int i = 0; i < gamma; ++i)
        if (draft_tokens[i] < 0 || draft_tokens[i] >= vocab)
            return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "verify_accept: draft token %d out of range", i);
    cudaSetDevice(ctx->device);
    const size_t row = (size_t)vocab * 4;
    uint8_t* s = dc_scratch(ctx, row * (gamma + 1) * 2 + row * gamma + 4096);
    if (!s) return DC_B200_OUT_OF_MEMORY;
    Bump b{s};
    float* tl = b.take<float>((size_t)(gamma + 1) * vocab);
    float* probs = b.take<float>((size_t)(gamma + 1) * vocab);
    float* dp = b.take<float>((size_t)gamma * vocab);
    int32_t* dt = b.take<int32_t>(gamma);
    float* u = b.take<float>(gamma + 1);
    int32_t* am = b.take<int32_t>(gamma + 1);
    int32_t* res = b.take<int32_t>(2);
    DC_TRY(h2d(ctx, tl, target_logits_host, row * (gamma + 1)));
    DC_TRY(h2d(ctx, dt, draft_tokens, (size_t)gamma * 4));
    if (mode == 1) {
        DC_TRY(h2d(ctx, dp, draft_probs_host, row * gamma));
        if (uniforms) DC_TRY(h2d(ctx, u, uniforms, (size_t)(gamma + 1) * 4));
        else DC_TRY(dc_launch_verify_uniforms(ctx, seed, step, gamma + 1, u));
    }
    DC_TRY(dc_launch_verify(ctx, mode, gamma, vocab, tl, dt, dp, u, temperature, am, probs, res));
    int32_t out[2] = {0, 0};
    DC_TRY(d2h(ctx, out, res, 8));
    DC_TRY(dc_b200_synchronize(ctx));
    *n_accepted = out[0];
    *next_token = out[1];
    return DC_B200_OK;
}

// Device-resident variant: target logits [gamma+1, vocab] (for example dc_b200_model_logits_dev after a
// forward_chunk) and, in mode 1, draft probabilities [gamma, vocab] are already on this GPU; only the draft
// token ids go in and the two result ints come out.
int dc_b200_verify_accept_dev(dc_ctx* ctx, const float* target_logits_dev, const int32_t* draft_tokens,
                              const float* draft_probs_dev, const float* uniforms, uint64_t seed, uint32_t step,
                              int gamma, int vocab, int mode, float temperature, int32_t* n_accepted,
                              int32_t* next_token) {
    if (!ctx) return DC_B200_INVALID_ARGUMENT;
    if (!target_logits_dev || !draft_tokens || !n_accepted || !next_token || gamma < 1 || gamma > 16 || vocab < 2 ||
        (mode != 0 && mode != 1) || (mode == 1 && !draft_probs_dev))
        return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "verify_accept_dev: bad argument");
    for (int i = 0; i < gamma; ++i)
        if (draft_tokens[i] < 0 || draft_tokens[i] >= vocab)
            return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "verify_accept_dev: draft token %d out of range", i);
    cudaSetDevice(ctx->device);
    const size_t row = (size_t)vocab * 4;
    uint8_t* s = dc_scratch(ctx, row * (gamma + 1) + 4096);
    if (!s) return DC_B200_OUT_OF_MEMORY;
    Bump b{s};
    float* probs = b.take<float>((size_t)(gamma + 1) * vocab);
    int32_t* dt = b.take<int32_t>(gamma);
    float* u = b.take<float>(gamma + 1);
    int32_t* am = b.take<int32_t>(gamma + 1);
    int32_t* res = b.take<int32_t>(2);
    DC_TRY(h2d(ctx, dt, draft_tokens, (size_t)gamma * 4));
    if (mode == 1) {
        if (uniforms) DC_TRY(h2d(ctx, u, uniforms, (size_t)(gamma + 1) * 4));
        else DC_TRY(dc_launch_verify_uniforms(ctx, seed, step, gamma + 1, u));
    }
    DC_TRY(dc_launch_verify(ctx, mode, gamma, vocab, target_logits_dev, dt, draft_probs_dev, u, temperature, am, probs, res));
    int32_t out[2] = {0, 0};
    DC_TRY(d2h(ctx, out, res, 8));
    DC_TRY(dc_b200_synchronize(ctx));
    *n_accepted = out[0];
    *next_token = out[1];
    return DC_B200_OK;
}

}  // extern "C"
