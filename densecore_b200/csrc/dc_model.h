// Decoder state shared by model.cu, ep.cu and spec.cu.
#pragma once
#include <map>
#include <string>
#include <vector>

#include "dc_internal.h"
#include "dc_kv.h"

#define DC_HISTORY_CAP 4096

enum {
    DC_K_EMBED = 0, DC_K_RMSNORM, DC_K_GEMV_QKV, DC_K_QKROPE, DC_K_ATTENTION, DC_K_GEMV_O, DC_K_ROUTER, DC_K_MOE_GATEUP,
    DC_K_QUANT_H, DC_K_MOE_DOWN, DC_K_COMBINE, DC_K_ALLREDUCE, DC_K_FFN_GATEUP, DC_K_FFN_DOWN, DC_K_LM_HEAD, DC_K_ARGMAX,
    DC_K_COUNT
};

struct dc_layer {
    dc_weight *attn_norm = nullptr, *wq = nullptr, *wk = nullptr, *wv = nullptr, *wo = nullptr;
    dc_weight *q_norm = nullptr, *k_norm = nullptr, *ffn_norm = nullptr;
    dc_weight *router = nullptr, *gate_exps = nullptr, *up_exps = nullptr, *down_exps = nullptr;
    dc_weight *ffn_gate = nullptr, *ffn_up = nullptr, *ffn_down = nullptr;
};

struct dc_step_buffers {
    int32_t *tokens = nullptr, *seq_ids = nullptr, *positions = nullptr, *out_tokens = nullptr;
    unsigned long long* argmax_keys = nullptr;
    float *x = nullptr, *xn = nullptr, *qkv = nullptr, *q = nullptr, *h = nullptr, *dn = nullptr, *moe_out = nullptr;
    float *logits = nullptr, *cos_sin = nullptr;
    uint8_t *q8_x = nullptr, *q8_attn = nullptr, *q8_h = nullptr, *route_mem = nullptr, *verify_mem = nullptr;
    uint8_t* attn_mem = nullptr;
    dc_attn_scratch attn = {};
    int32_t* history = nullptr;
    int* history_len = nullptr;
    dc_moe_route route = {};
};

struct dc_graph {
    cudaGraphExec_t exec = nullptr;
    int launches = 0;
};

struct dc_prefill_buffers;

struct dc_model {
    dc_ctx* ctx = nullptr;
    dc_model_config cfg = {};
    std::vector<dc_layer> layers;
    dc_weight *tok_embd = nullptr, *out_norm = nullptr, *output = nullptr;
    std::vector<dc_weight*> owned;
    std::map<std::string, dc_weight*> names;
    std::vector<std::string> all_names;   // every tensor the decoder needs, in load order
    dc_kv_cache kv;
    dc_step_buffers buf;
    int nsplit = 16;
    bool finalized = false;
    bool use_graphs = true;
    std::map<int, dc_graph> graphs;
    std::map<int, bool> warmed;
    int last_launches = 0;
    // per-kernel-class device timing of one eager step (dc_b200_model_profile_step)
    bool prof = false;
    struct ProfRec { int cls; cudaEvent_t e0, e1; double bytes; };
    std::vector<ProfRec> prof_recs;
    int ep_lo = 0, ep_hi = 0;    // experts stored on this GPU
    int32_t* h_stage = nullptr;  // pinned, 1024 ints
    int stage_slot = 0;
    // persistent decode kernel (mega.cu)
    void* mega_layers = nullptr;     // device array of MegaLayer
    unsigned* mega_counter = nullptr;
    int use_mega = 1;            // 0 never, 1 for one stream (where it is the faster path), 2 wherever it fits
    bool mega_timing = false;
    int route_mode = 0;          // DC_ROUTE_STABLE / DC_ROUTE_SOFTMAX
    // parity aid: the hidden state entering every layer (slot il) and the output norm (slot n_layer) of the
    // last step, [n_layer + 1][DC_MAX_T][hidden] floats; allocated by option "capture_layer_inputs"
    float* dbg_x = nullptr;
    // bounded-wait test hooks: poll limits of the persistent kernel's waits (0 = the defaults)
    unsigned test_barrier_polls = 0;
    unsigned long long test_ep_wait_ns = 0;
    // prompt chunks through the tensor-core matmuls (prefill.cu): option "tc_prefill" (default on), chunk
    // length option "prefill_chunk" (default 2048, fixed once the first chunk has run)
    bool use_tc_prefill = true;
    int prefill_chunk = 2048;
    bool prefill_flash = true;            // option "prefill_attention": 1 tensor-core flash attention, 0 the decode kernels' exact chain
    dc_prefill_buffers* prefill = nullptr;
    bool prefix_cache = false;            // option "prefix_cache": prefill looks up and registers block prefixes
    uint64_t prefill_tokens_run = 0;      // prompt tokens that went through the decoder (cached ones do not)
    // expert parallel
    bool ep_ready = false;
    void* ep_comm = nullptr;     // ncclComm_t
    void* ep_lib = nullptr;      // dlopen handle of libnccl
    // exchange buffer of the persistent kernel's expert-parallel path: flags, then two halves of rows;
    // xch_peer[r] is rank r's buffer mapped into this process (own rank: xch itself)
    uint8_t* xch = nullptr;
    uint8_t* xch_peer[8] = {};
    int xch_connected = 0;       // peers mapped so far
    bool xch_loopback = false;   // test hook: the peer buffer is a local allocation (dc_mega_test_loopback)
    unsigned xepoch = 0;         // exchanges completed by earlier launches
};

// ---- synth.cu ----
int dc_launch_synth_quantized(dc_ctx* ctx, int type, uint64_t seed, int64_t first_row, int64_t rows, int64_t K, float sigma,
                              uint8_t* out);
int dc_launch_synth_f32(dc_ctx* ctx, uint64_t seed, int64_t n, float sigma, float offset, float* out);
// ---- mega.cu ----
void dc_mega_release_xch(dc_model* m);
int dc_mega_test_loopback(dc_model* m);
struct MegaParams;
bool dc_mega_plan(dc_model* m, int T, MegaParams* out, const char** why);
int dc_mega_run(dc_model* m, int T, int n_steps, bool feedback);
// Appends tokens[0..n) to a sequence in chunks; if `final`, the last chunk also picks the next token (and leaves
// its logits in the step buffer) and *next_token receives it after a synchronize.
int dc_model_prefill_range(dc_model* m, int seq, const int32_t* tokens_host, int n, bool final, int32_t* next_token);
int dc_mega_prepare(dc_model* m);
// ---- prefill.cu ----
bool dc_prefill_tc_ok(dc_model* m, int n);
int dc_prefill_chunk_tc(dc_model* m, int seq, const int32_t* tokens, int n, bool lm);
void dc_prefill_release(dc_model* m);
// ---- ep.cu ----
int dc_ep_allreduce(dc_model* m, float* buf, size_t n);
void dc_ep_destroy(dc_model* m);
