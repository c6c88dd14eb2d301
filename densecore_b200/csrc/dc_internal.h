// Host-side structures shared by the translation units of libdc_b200.so.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <string>
#include <vector>

#include "../../include/dc_b200.h"

#define DC_NSTAGE 4
#define DC_WARPS 8
#define DC_STAGE_TARGET 4608  // bytes of weight rows one pipeline stage aims to hold: one warp pass of Q4_K rows

struct dc_weight {
    int type;        // ggml type id
    int64_t K;       // ne[0]: reduction length
    int64_t N;       // ne[1]: rows (outputs) per expert slab
    int64_t E;       // ne[2]: experts (1 for dense tensors)
    size_t row_bytes;
    size_t bytes;
    uint8_t* dev;
};

struct dc_ctx {
    int device = 0;
    int num_sms = 148;
    cudaStream_t stream = nullptr;
    int* d_err = nullptr;          // device error word (bounded waits report here)
    int gemm_tc_min_rows = 32;     // option "gemm_tc_min_rows": token rows from which MUL_MAT runs on the tensor cores
    std::string last_error;
    std::mutex mu;
    std::vector<dc_weight*> weights;
    // op-level scratch (grown on demand, never shrunk)
    uint8_t* scratch = nullptr;
    size_t scratch_bytes = 0;
    void* pinned = nullptr;        // small pinned staging area for host<->device results
    size_t pinned_bytes = 0;
    int use_pdl = 1;
    int route_mode = 0;            // router variant of the op-level MoE calls (DC_ROUTE_*)
};

int dc_fail(dc_ctx* ctx, int status, const char* fmt, ...);
int dc_check_cuda(dc_ctx* ctx, cudaError_t e, const char* what);
uint8_t* dc_scratch(dc_ctx* ctx, size_t bytes);   // returns nullptr on failure (error recorded)
void* dc_pinned(dc_ctx* ctx, size_t bytes);
int dc_check_device_error(dc_ctx* ctx);            // reads d_err after a sync
// One-time, per-device kernel set-up (thread-safe): opt `func` into max_dyn_smem bytes of dynamic shared
// memory on ctx's device; cached occupancy (resident CTAs per SM) of `func` on that device.
int dc_kernel_setup(dc_ctx* ctx, const void* func, int max_dyn_smem, const char* name);
int dc_kernel_occupancy(dc_ctx* ctx, const void* func, int threads, size_t dyn_smem);

// ---- launch helpers implemented in the kernel translation units ----
struct dc_gemv_seg {
    const uint8_t* w;  // first row
    int type;
    int n_rows;
    int row_bytes;
    float* out;        // out[t * ldo + row]
    int ldo;
};
enum { DC_EPI_STORE = 0, DC_EPI_ACC = 1, DC_EPI_SWIGLU = 2 };

// y = W x for T <= 16 tokens whose Q8_K activations are at act_q8 (row stride K/256*292).
// n_seg 1..3 segments share the activations.  DC_EPI_SWIGLU: seg[0]=gate, seg[1]=up,
// result silu(gate.x)*(up.x) stored to seg[0].out.  argmax (optional, [T] u64 keys,
// zeroed by the caller) receives the packed (value,row) maximum of the stored rows.
// dump_I / dump_M (parity checks, single segment): receive the exact int32 block sums the kernel forms,
// [T][n_rows][K/256] (M for Q4_K only).
int dc_launch_gemv(dc_ctx* ctx, const dc_gemv_seg* segs, int n_seg, int epi, const uint8_t* act_q8, int T, int K,
                   unsigned long long* argmax, int32_t* dump_I = nullptr, int32_t* dump_M = nullptr);
// rows x K f32 -> native Q8_K blocks (row stride K/256*292)
int dc_launch_quantize_q8k(dc_ctx* ctx, const float* x, int rows, int K, uint8_t* out);
// Tensor-core MUL_MAT for many token rows (gemm_tc.cu): activations quantised into 64-token tiles, then
// out[slot * ldo + row] for every weight row; tile_expert (optional, device) picks an expert matrix per tile.
size_t dc_gemm_tc_act_bytes(int n_slots, int K);
int dc_gemm_tc_tiles(int n_slots);
bool dc_gemm_tc_supports(const dc_weight* w);
int dc_launch_quantize_q8k_tiled(dc_ctx* ctx, const float* x, int ldx, int n_rows, int K, uint8_t* act, int n_tt,
                                 const int* slot_token);
// pair_tile0 / pair_nset (device, n_pairs entries; needed with tile_expert): the pairs of neighbouring tiles of
// one expert that a CTA works on
int dc_launch_gemm_tc(dc_ctx* ctx, const dc_weight* w, const uint8_t* act, int n_slots, float* out, int ldo,
                      const int* tile_expert = nullptr, const int* slot_row = nullptr, bool accumulate = false,
                      const int* pair_tile0 = nullptr, const int* pair_nset = nullptr, int n_pairs = 0);
// up to three matrices of one type, K and row length in one launch (Q | K | V, gate | up)
int dc_launch_gemm_tc_multi(dc_ctx* ctx, const dc_weight* const* ws, const int* out_off, int nseg, const uint8_t* act,
                            int n_slots, float* out, int ldo, const int* tile_expert = nullptr, const int* slot_row = nullptr,
                            bool accumulate = false, const int* pair_tile0 = nullptr, const int* pair_nset = nullptr,
                            int n_pairs = 0);


// ---- misc.cu ----
int dc_launch_embed(dc_ctx* ctx, const dc_weight* w, const int32_t* tokens, int T, float* x);
// x (+= add) -> RMSNorm * w -> optional f32 copy and Q8_K blocks
int dc_launch_rmsnorm_q8k(dc_ctx* ctx, float* x, const float* add, const float* w, int T, int H, float eps,
                          float* xn_out, uint8_t* q8_out);
int dc_launch_qknorm_rope_kv(dc_ctx* ctx, const float* qkv, const float* qn_w, const float* kn_w,
                             const float* cos_sin, int max_pos, const int32_t* positions, const int32_t* seq_ids,
                             const int32_t* block_tables, int max_blocks, void* k_arena, void* v_arena, int n_head,
                             int n_kv, float eps, int T, float* q_out);
int dc_launch_argmax_finish(dc_ctx* ctx, unsigned long long* keys, int T, int32_t* out_tokens, int32_t* next_tokens,
                            int32_t* positions, int32_t* history, int* history_len, int history_cap);
int dc_launch_argmax_rows(dc_ctx* ctx, const float* logits, int rows, int n, int32_t* out);

// ---- attn.cu ----
struct dc_attn_scratch {
    float* scores;    // [T][n_head][max_blocks*16]
    float* bmax;      // [T][n_head][max_blocks]
    float* part_acc;  // [T][n_head][nsplit][128]
    float* part_d;    // [T][n_head][nsplit]
    int* tickets;     // [T][n_kv], zeroed once
};
size_t dc_attention_scratch_bytes(int T, int n_head, int n_kv, int max_blocks, int nsplit);
void dc_attn_scratch_bind(dc_attn_scratch* sc, uint8_t* base, int T, int n_head, int n_kv, int max_blocks, int nsplit);
int dc_launch_attention(dc_ctx* ctx, const float* q, const void* k_arena, const void* v_arena,
                        const int32_t* block_tables, int max_blocks, const int32_t* seq_ids, const int32_t* positions,
                        int T, int n_head, int n_kv, float scale, int nsplit, const dc_attn_scratch* sc, float* out,
                        uint8_t* q8_out);

// ---- moe.cu ----
// causal attention of a prompt chunk (positions pos0 .. pos0 + n - 1 of one sequence) on the tensor cores
int dc_launch_attention_prefill(dc_ctx* ctx, const float* q, const void* k_arena, const void* v_arena, const int32_t* table,
                                int pos0, int n, int n_head, int n_kv, float scale, float* out);

struct dc_moe_route {
    float* logits;     // [T][E]
    int32_t* ids;      // [T][top_k]
    float* weights;    // [T][top_k]
    int* ticket;       // zeroed once; the router resets it itself
    int* n_active;     // number of distinct local experts hit
    int32_t* uexp;     // [E]
    int32_t* uoff;     // [E+1]
    int32_t* uassign;  // [T*top_k]
};
// mode: DC_ROUTE_STABLE = top-k on the logits with the stable comparator, weights over the picks
// (core/src/llm/moe/native.cpp:610-676); DC_ROUTE_SOFTMAX = softmax over all experts, top-k on the
// probabilities with strict '>', renormalise (core/src/moe/moe_routing.cpp:53-101).
enum { DC_ROUTE_STABLE = 0, DC_ROUTE_SOFTMAX = 1 };
int dc_launch_router(dc_ctx* ctx, const dc_weight* wr, const float* xn, int n_expert, int T, int top_k, float scale,
                     int ep_lo, int ep_hi, const dc_moe_route* rt, int mode = DC_ROUTE_STABLE);
// the same routing for any number of tokens (prompt chunks): logits [T][E], ids and weights [T][top_k]
int dc_launch_router_batched(dc_ctx* ctx, const dc_weight* wr, const float* xn, int T, int top_k, float scale, float* logits,
                             int32_t* ids, float* weights, int mode);
// carves a dc_moe_route for (T, E, top_k) out of a byte buffer; returns bytes used
size_t dc_moe_route_bind(dc_moe_route* rt, uint8_t* base, int T, int E, int top_k);
int dc_launch_moe_mm(dc_ctx* ctx, bool pair, const dc_weight* w0, const dc_weight* w1, const uint8_t* act_q8,
                     int act_rows, int T, int top_k, int e_base, const dc_moe_route* rt, float* out);
int dc_launch_moe_combine(dc_ctx* ctx, const float* dn, const int32_t* ids, const float* weights, int T, int top_k,
                          int H, int ep_lo, int ep_hi, float* out);

// ---- sample.cu ----
// mode 0 greedy / 1 stochastic; result[0] = accepted draft tokens, result[1] = next token
int dc_launch_verify(dc_ctx* ctx, int mode, int gamma, int vocab, const float* target_logits,
                     const int32_t* draft_tokens, const float* draft_probs, const float* u, float temperature,
                     int32_t* argmax_scratch, float* probs_scratch, int32_t* result);
int dc_launch_verify_uniforms(dc_ctx* ctx, unsigned long long seed, uint32_t step, int n, float* u);
int dc_launch_det_softmax(dc_ctx* ctx, const float* logits, int rows, int n, float temperature, float* probs);
// probs = softmax(logits / temperature); *result = inverse-CDF draw with the uniform at u_dev
int dc_launch_sample(dc_ctx* ctx, const float* logits, int n, float temperature, const float* u_dev, float* probs,
                     int32_t* result);
