// ggml-shaped custom-op callbacks over the C ABI (include/dc_ggml_compat.h).
//
// Host code only: every callback validates its node the way DenseCore's own callback does, then makes one
// call into the library.  Thread 0 of the executor's nth threads does the work; the others return.
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "dc_ggml_compat.h"

namespace {

std::atomic<uint64_t> g_fail_closed{0};

size_t dense_f32_bytes(const ggml_tensor* t) {
    return (size_t)t->ne[0] * (size_t)t->ne[1] * (size_t)t->ne[2] * (size_t)t->ne[3] * sizeof(float);
}

void zero_fill(ggml_tensor* dst) {
    if (dst && dst->data && dst->type == GGML_TYPE_F32 && dst->ne[0] > 0 && dst->ne[1] > 0 && dst->ne[2] > 0 && dst->ne[3] > 0)
        memset(dst->data, 0, dense_f32_bytes(dst));
}

// A node this callback cannot run: zero result, one line, one count.
void reject(ggml_tensor* dst, const char* fmt, ...) {
    char buf[384];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    zero_fill(dst);
    g_fail_closed.fetch_add(1, std::memory_order_relaxed);
    fprintf(stderr, "[dc_b200] CRITICAL: %s\n", buf);
}

// The library call itself failed: it has zero-filled the result and written its own line.
void library_failed(ggml_tensor* dst) {
    zero_fill(dst);
    g_fail_closed.fetch_add(1, std::memory_order_relaxed);
}

bool dense_rows(const ggml_tensor* t) {   // rows of ne[0] floats, packed back to back in every outer dimension
    if (t->nb[0] != sizeof(float)) return false;
    size_t want = (size_t)t->ne[0] * sizeof(float);
    for (int d = 1; d < 4; ++d) {
        if (t->ne[d] > 1 && t->nb[d] != want) return false;
        want *= (size_t)t->ne[d];
    }
    return true;
}

}  // namespace

extern "C" {

uint64_t dc_b200_shim_fail_closed_count(void) { return g_fail_closed.load(std::memory_order_relaxed); }

void cb_gemv_b200(struct ggml_tensor* dst, int ith, int nth, void* userdata) {
    (void)nth;
    if (ith != 0) return;
    auto* ud = static_cast<dc_b200_gemv_userdata*>(userdata);
    if (!dst || !dst->data) return;   // nothing to fill (gemv_exec.cpp:102,128 return likewise)
    if (!ud || !ud->ctx) return reject(dst, "GEMV callback without userdata or context");
    const ggml_tensor* x = dst->src[0];
    const ggml_tensor* w = dst->src[1];
    if (!x || !x->data) return reject(dst, "GEMV input tensor is null or has no data");
    if (!w || (!w->data && !ud->weight)) return reject(dst, "GEMV weight tensor is null or has no data");
    if (w->type != GGML_TYPE_Q4_K && w->type != GGML_TYPE_Q6_K)
        return reject(dst, "GEMV weight type %d is not Q4_K or Q6_K", (int)w->type);
    if (x->type != GGML_TYPE_F32 || dst->type != GGML_TYPE_F32) return reject(dst, "GEMV input and output must be F32");
    const int64_t n_in = w->ne[0], k_out = w->ne[1], m = x->ne[1];
    if (dst->ne[0] != k_out)
        return reject(dst, "GEMV buffer mismatch! dst->ne[0](%ld) != weight->ne[1](%ld). Output tensor was sized incorrectly.",
                      (long)dst->ne[0], (long)k_out);
    if (x->ne[0] != n_in || dst->ne[1] != m || m < 1 || x->ne[2] != 1 || x->ne[3] != 1 || w->ne[2] != 1 || w->ne[3] != 1)
        return reject(dst, "GEMV shapes do not agree: input [%ld, %ld], weight [%ld, %ld], output [%ld, %ld]", (long)x->ne[0],
                      (long)x->ne[1], (long)n_in, (long)k_out, (long)dst->ne[0], (long)dst->ne[1]);
    if (!dense_rows(x) || !dense_rows(dst)) return reject(dst, "GEMV input and output rows must be contiguous");
    if (!ud->weight) {
        const int64_t ne[4] = {n_in, k_out, 1, 1};
        if (dc_b200_upload_weight(ud->ctx, (int)w->type, ne, w->data, &ud->weight) != DC_B200_OK) return library_failed(dst);
    }
    if (dc_b200_mul_mat(ud->ctx, ud->weight, (const float*)x->data, (int)m, (float*)dst->data) != DC_B200_OK)
        library_failed(dst);
}

void cb_moe_forward_b200(struct ggml_tensor* dst, const struct ggml_tensor* src0, const struct ggml_tensor* src1, int ith,
                         int nth, void* userdata) {
    (void)nth;
    if (ith != 0) return;
    auto* ud = static_cast<dc_b200_moe_userdata*>(userdata);
    if (!dst || !dst->data) return;
    if (!ud || !ud->ctx) return reject(dst, "MoE callback missing userdata/context");
    if (!ud->gate_exps || !ud->up_exps || !ud->down_exps) return reject(dst, "MoE callback missing registered experts");
    if (!src0 || !src0->data || !src1 || !src1->data) return reject(dst, "MoE callback input or router logits missing");
    if (src0->type != GGML_TYPE_F32 || src1->type != GGML_TYPE_F32 || dst->type != GGML_TYPE_F32)
        return reject(dst, "MoE callback tensors must be F32");
    const int64_t hidden = src0->ne[0], tokens = src0->ne[1], n_expert = src1->ne[0];
    if (tokens < 1 || src1->ne[1] != tokens || dst->ne[0] != hidden || dst->ne[1] != tokens)
        return reject(dst, "MoE shapes do not agree: input [%ld, %ld], logits [%ld, %ld], output [%ld, %ld]", (long)hidden,
                      (long)tokens, (long)n_expert, (long)src1->ne[1], (long)dst->ne[0], (long)dst->ne[1]);
    if (!dense_rows(src0) || !dense_rows(src1) || !dense_rows(dst)) return reject(dst, "MoE tensors must be contiguous");
    const float scale = (ud->routed_scaling_factor != 0.0f) ? ud->routed_scaling_factor : 1.0f;
    // tokens are independent: chunks of at most 16 (the library's limit per call)
    for (int64_t t0 = 0; t0 < tokens; t0 += 16) {
        const int n = (int)(tokens - t0 < 16 ? tokens - t0 : 16);
        const int st = dc_b200_moe_forward(ud->ctx, ud->gate_exps, ud->up_exps, ud->down_exps,
                                           (const float*)src0->data + t0 * hidden, (const float*)src1->data + t0 * n_expert, n,
                                           ud->k, scale, (float*)dst->data + t0 * hidden, nullptr, nullptr);
        if (st != DC_B200_OK) return library_failed(dst);
    }
}

void cb_paged_attention_decode_b200(struct ggml_tensor* dst, int ith, int nth, void* userdata) {
    if (ith != 0 || nth <= 0) return;
    auto* ud = static_cast<dc_b200_attn_userdata*>(userdata);
    if (!ud || !ud->cache || !ud->ctx || !dst || !dst->data) return;   // paged_exec.cpp:345
    const ggml_tensor *q = dst->src[0], *k = dst->src[1], *v = dst->src[2];
    if (!q || !k || !v) return;                                       // paged_exec.cpp:351
    if (!q->data || !k->data || !v->data) return reject(dst, "paged attention: q, k or v has no data");
    const int64_t tokens = q->ne[2];
    if (tokens <= 0 || ud->head_dim <= 0 || ud->n_head <= 0 || ud->n_head_kv <= 0 || ud->n_head % ud->n_head_kv)
        return reject(dst, "paged attention: bad head layout (%d heads, %d kv heads, dim %d, %ld tokens)", ud->n_head,
                      ud->n_head_kv, ud->head_dim, (long)tokens);
    if (q->type != GGML_TYPE_F32 || k->type != GGML_TYPE_F32 || v->type != GGML_TYPE_F32 || dst->type != GGML_TYPE_F32)
        return reject(dst, "paged attention: tensors must be F32");
    if (q->ne[0] != ud->head_dim || q->ne[1] != ud->n_head || k->ne[0] != ud->head_dim || k->ne[1] != ud->n_head_kv ||
        v->ne[0] != ud->head_dim || v->ne[1] != ud->n_head_kv || k->ne[2] != tokens || v->ne[2] != tokens ||
        dst->ne[0] != ud->head_dim || dst->ne[1] != ud->n_head || dst->ne[2] != tokens)
        return reject(dst, "paged attention: shapes do not agree with %d heads / %d kv heads of dim %d over %ld tokens", ud->n_head,
                      ud->n_head_kv, ud->head_dim, (long)tokens);
    if (!dense_rows(q) || !dense_rows(k) || !dense_rows(v) || !dense_rows(dst))
        return reject(dst, "paged attention: tensors must be contiguous");
    if (!ud->seq_id || !ud->pos) return reject(dst, "paged attention: batch has no sequence ids or positions");
    const float scale = ud->scale != 0.0f ? ud->scale : 1.0f / sqrtf((float)ud->head_dim);
    const int64_t qrow = (int64_t)ud->n_head * ud->head_dim, kvrow = (int64_t)ud->n_head_kv * ud->head_dim;
    for (int64_t t0 = 0; t0 < tokens; t0 += 16) {
        const int n = (int)(tokens - t0 < 16 ? tokens - t0 : 16);
        const int st = dc_b200_flash_attn_decode(ud->ctx, ud->cache, ud->layer, (const float*)q->data + t0 * qrow,
                                                 (const float*)k->data + t0 * kvrow, (const float*)v->data + t0 * kvrow,
                                                 ud->seq_id + t0, ud->pos + t0, n, ud->n_head, scale,
                                                 (float*)dst->data + t0 * qrow);
        if (st != DC_B200_OK) return library_failed(dst);
    }
}

}  // extern "C"
