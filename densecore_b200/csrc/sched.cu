// Step scheduler over one decoder: continuous batching of at most max_num_seqs sequences with one prefill
// in flight at a time, the policy of DenseCore's engine for its CPU path (max_num_seqs = 4 by default,
// core/src/runtime/engine_internal.h:89; admission and prefix reuse, core/src/runtime/scheduler.cpp:30-85).
//
// Host code only.  One call of step() does one unit of GPU work:
//   * a chunk of the prompt of the request that is being prefilled (admitting the oldest waiting request first
//     if no prefill is in flight and a sequence slot is free), or
//   * one decode step for all running sequences together (their tokens form one batch of the decoder),
// alternating between the two when both are possible, so that a long prompt does not stall running streams.
// A newly admitted request first takes over the cached blocks of its longest cached prompt prefix (model
// option "prefix_cache"); only the rest of the prompt runs.
#include <deque>
#include <vector>

#include "dc_common.cuh"
#include "dc_model.h"

#define DC_TRY(expr)                       \
    do {                                   \
        int st_ = (expr);                  \
        if (st_ != DC_B200_OK) return st_; \
    } while (0)

struct dc_sched_request {
    int id = 0;
    std::vector<int32_t> prompt;
    int max_new = 0;
    int seq = -1;
    int done = 0;        // prompt tokens in the cache so far (prefill), cached prefix included
    int cached = 0;      // prompt tokens taken from the prefix cache
    int generated = 0;
    int32_t last = 0;    // last emitted token: the next decode input
};

struct dc_sched {
    dc_model* m = nullptr;
    int max_num_seqs = 4, chunk = 512, eos = -1;
    int next_id = 0;
    bool last_was_prefill = false;
    std::deque<dc_sched_request> waiting;
    std::vector<dc_sched_request> prefilling;   // at most one
    std::vector<dc_sched_request> running;
    uint64_t steps = 0, prefill_chunks = 0, decode_steps = 0, decode_tokens = 0, max_batch = 0, prompt_tokens_cached = 0;
};

namespace {

int emit(dc_sched_event* ev, int cap, int* n, int request, int32_t token, int finished) {
    if (*n < cap) ev[*n] = {request, token, finished};
    ++*n;
    return finished;
}

// 0: keeps running, 1: reached its token budget, 2: produced the end-of-sequence token
int finish_reason(const dc_sched* s, const dc_sched_request& r) {
    if (s->eos >= 0 && r.last == s->eos) return 2;
    return r.generated >= r.max_new ? 1 : 0;
}

int prefill_step(dc_sched* s, dc_sched_event* ev, int cap, int* n) {
    dc_model* m = s->m;
    if (s->prefilling.empty()) {
        dc_sched_request r = std::move(s->waiting.front());
        s->waiting.pop_front();
        DC_TRY(dc_b200_seq_alloc(m, &r.seq));
        if (m->prefix_cache) {
            int st = dc_kv_prefix_attach(&m->kv, r.seq, r.prompt.data(), (int)r.prompt.size(), &r.cached);
            if (st != DC_B200_OK) {
                dc_b200_seq_free(m, r.seq);
                return st;
            }
            s->prompt_tokens_cached += (uint64_t)r.cached;
        }
        r.done = r.cached;
        s->prefilling.push_back(std::move(r));
    }
    dc_sched_request& r = s->prefilling[0];
    const int left = (int)r.prompt.size() - r.done;
    const int c = left < s->chunk ? left : s->chunk;
    const bool final = c == left;
    int32_t next = -1;
    int st = dc_model_prefill_range(m, r.seq, r.prompt.data() + r.done, c, final, &next);
    if (st != DC_B200_OK) {   // the request fails as a whole; its slot returns
        dc_b200_seq_free(m, r.seq);
        emit(ev, cap, n, r.id, -1, 3);
        s->prefilling.clear();
        return st;
    }
    r.done += c;
    ++s->prefill_chunks;
    if (!final) return DC_B200_OK;
    if (m->prefix_cache) dc_kv_prefix_register(&m->kv, r.seq, r.prompt.data(), (int)r.prompt.size());
    r.last = next;
    r.generated = 1;
    const int fin = finish_reason(s, r);
    emit(ev, cap, n, r.id, next, fin);
    if (fin) dc_b200_seq_free(m, r.seq);
    else s->running.push_back(std::move(r));
    s->prefilling.clear();
    return DC_B200_OK;
}

int decode_step(dc_sched* s, dc_sched_event* ev, int cap, int* n) {
    const int B = (int)s->running.size();
    int32_t seqs[DC_MAX_T], toks[DC_MAX_T], next[DC_MAX_T];
    for (int i = 0; i < B; ++i) {
        seqs[i] = s->running[i].seq;
        toks[i] = s->running[i].last;
    }
    DC_TRY(dc_b200_decode_step(s->m, seqs, B, toks, next, nullptr));
    ++s->decode_steps;
    s->decode_tokens += (uint64_t)B;
    if ((uint64_t)B > s->max_batch) s->max_batch = (uint64_t)B;
    std::vector<dc_sched_request> keep;
    for (int i = 0; i < B; ++i) {
        dc_sched_request& r = s->running[i];
        r.last = next[i];
        ++r.generated;
        const int fin = finish_reason(s, r);
        emit(ev, cap, n, r.id, next[i], fin);
        if (fin) dc_b200_seq_free(s->m, r.seq);
        else keep.push_back(std::move(r));
    }
    s->running.swap(keep);
    return DC_B200_OK;
}

}  // namespace

extern "C" {

int dc_b200_sched_create(dc_model* m, int max_num_seqs, int max_prefill_chunk, int eos_token, dc_sched** out) {
    if (!m || !out) return DC_B200_INVALID_ARGUMENT;
    *out = nullptr;
    if (!m->finalized) return dc_fail(m->ctx, DC_B200_MODEL_LOAD_FAILED, "sched_create: model is not finalized");
    if (max_num_seqs <= 0) max_num_seqs = 4;   // KVCacheConfig::max_num_seqs, engine_internal.h:89
    if (max_num_seqs > m->cfg.max_seqs || max_num_seqs > DC_MAX_T)
        return dc_fail(m->ctx, DC_B200_INVALID_ARGUMENT, "sched_create: %d sequences asked, the model holds %d", max_num_seqs, m->cfg.max_seqs);
    if (max_prefill_chunk <= 0) max_prefill_chunk = 512;
    dc_sched* s = new dc_sched();
    s->m = m;
    s->max_num_seqs = max_num_seqs;
    s->chunk = (max_prefill_chunk + DC_KV_BLOCK - 1) / DC_KV_BLOCK * DC_KV_BLOCK;   // whole cache blocks per chunk
    s->eos = eos_token;
    *out = s;
    return DC_B200_OK;
}

void dc_b200_sched_destroy(dc_sched* s) {
    if (!s) return;
    for (auto& r : s->prefilling) dc_b200_seq_free(s->m, r.seq);
    for (auto& r : s->running) dc_b200_seq_free(s->m, r.seq);
    delete s;
}

int dc_b200_sched_add(dc_sched* s, const int32_t* prompt, int n_prompt, int max_new_tokens, int* request_id) {
    if (!s || !request_id) return DC_B200_INVALID_ARGUMENT;
    if (!prompt || n_prompt < 1 || max_new_tokens < 1)
        return dc_fail(s->m->ctx, DC_B200_INVALID_ARGUMENT, "sched_add: empty prompt or no tokens to generate");
    if (n_prompt + max_new_tokens > s->m->cfg.max_ctx)
        return dc_fail(s->m->ctx, DC_B200_INVALID_ARGUMENT, "sched_add: %d prompt + %d new tokens exceed max_ctx %d", n_prompt,
                       max_new_tokens, s->m->cfg.max_ctx);
    for (int i = 0; i < n_prompt; ++i)
        if (prompt[i] < 0 || prompt[i] >= s->m->cfg.vocab) return dc_fail(s->m->ctx, DC_B200_INVALID_ARGUMENT, "sched_add: token id out of range");
    dc_sched_request r;
    r.id = s->next_id++;
    r.prompt.assign(prompt, prompt + n_prompt);
    r.max_new = max_new_tokens;
    *request_id = r.id;
    s->waiting.push_back(std::move(r));
    return DC_B200_OK;
}

int dc_b200_sched_pending(dc_sched* s) {
    return s ? (int)(s->waiting.size() + s->prefilling.size() + s->running.size()) : DC_B200_INVALID_ARGUMENT;
}

int dc_b200_sched_step(dc_sched* s, dc_sched_event* events, int capacity, int* n_events) {
    if (!s || !n_events || (capacity > 0 && !events)) return DC_B200_INVALID_ARGUMENT;
    *n_events = 0;
    const bool slot_free = (int)(s->running.size() + s->prefilling.size()) < s->max_num_seqs;
    const bool can_prefill = !s->prefilling.empty() || (!s->waiting.empty() && slot_free);
    const bool can_decode = !s->running.empty();
    if (!can_prefill && !can_decode) return DC_B200_OK;
    cudaSetDevice(s->m->ctx->device);
    ++s->steps;
    const bool do_prefill = can_prefill && (!can_decode || !s->last_was_prefill);
    s->last_was_prefill = do_prefill;
    return do_prefill ? prefill_step(s, events, capacity, n_events) : decode_step(s, events, capacity, n_events);
}

int dc_b200_sched_stats(dc_sched* s, uint64_t out[6]) {
    if (!s || !out) return DC_B200_INVALID_ARGUMENT;
    out[0] = s->steps;
    out[1] = s->prefill_chunks;
    out[2] = s->decode_steps;
    out[3] = s->decode_tokens;
    out[4] = s->max_batch;
    out[5] = s->prompt_tokens_cached;
    return DC_B200_OK;
}

}  // extern "C"
