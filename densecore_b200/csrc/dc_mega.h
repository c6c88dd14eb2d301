// Parameters of the persistent decode kernel (mega.cu).
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

#define MG_THREADS 512
#define MG_WARPS 16
#define MG_NSTAGE 2
#define MG_STAGE 4864   // bytes per pipeline stage of one warp: one pass of four Q4_K rows of 2048, or two gate/up pairs
#define MG_MAX_T 4
#define MG_MAX_E 256
#define MG_MAX_K 16
#define MG_MAX_RANKS 8
#define MG_XCH_FLAG_BYTES 256   // flag array at the head of an exchange buffer
// barrier counter (64 bytes) + 32 phase accumulators + a per-CTA barrier trace (14 x 160) + a per-warp trace
// of MG_WTRACE_POINTS points of the second layer (instrumented builds only; 160 CTAs x 16 warps each)
#define MG_WTRACE_POINTS 18
#define MG_WTRACE_BASE (32 + 14 * 160)
#define DC_MEGA_TIMING_SLOTS (MG_WTRACE_BASE + MG_WTRACE_POINTS * 2560)
#define DC_MEGA_COUNTER_BYTES (64 + DC_MEGA_TIMING_SLOTS * 8)

struct MegaLayer {
    const float *attn_norm, *q_norm, *k_norm, *ffn_norm, *router;
    const uint8_t *wq, *wk, *wv, *wo, *gate, *up, *down;
    int wq_type, wk_type, wv_type, wo_type, gate_type, down_type;
    int wq_rb, wk_rb, wv_rb, wo_rb, gate_rb, down_rb;   // row bytes
    __half *k_arena, *v_arena;                           // this layer's planes
};

struct MegaParams {
    int n_layer, H, n_head, n_kv, vocab, E, top_k, F, T;
    float eps, scale, routed_scale;
    const MegaLayer* layers;       // device array [n_layer]
    const uint8_t* tok_embd;
    int embd_type, embd_row_bytes;
    const float* out_norm;
    const uint8_t* out_w;
    int out_type, out_rb;
    // step inputs / outputs
    int32_t *tokens, *seq_ids, *positions, *out_tokens;
    unsigned long long* argmax_keys;
    int32_t* history;
    int* history_len;
    int history_cap, feedback, n_steps;
    const int32_t* block_tables;
    int max_blocks;
    const float* cos_sin;
    int max_pos;
    // global scratch shared by the CTAs
    float *xa, *xb, *qkv, *h, *dn, *router_logits, *logits;
    float *bmax, *part_acc, *part_d;
    int* tickets;
    uint8_t* q8_attn;
    int32_t* route_ids;            // copies of the last layer's routing, for callers
    float* route_w;
    int nsplit, s_keys;            // attention runs per (token, kv head, head group); keys a run can hold
    int n_hg;                      // head groups a kv head's query heads are split into (1, 2 or 4)
    // expert parallel (ep_size > 1): experts [e_lo, e_hi) live here.  Every rank stores the rows its experts
    // produce in the down projection into all ranks' exchange buffers (peer stores over NVLink), then the ranks
    // meet once per layer through flags in each other's memory; the combine then reads local memory only.
    int ep_rank, ep_size, e_lo, e_hi;
    float* xdn[MG_MAX_RANKS];        // rank r's exchange rows: two halves of [MG_MAX_T * MG_MAX_K][H] floats
    unsigned* xcnt[MG_MAX_RANKS];    // in rank r's memory: the counter this rank's CTAs add their arrivals to
    unsigned* my_xcnt;               // this rank's counter: arrivals of all CTAs of all peers
    unsigned xepoch0;                // exchanges completed before this launch
    int route_mode;                  // DC_ROUTE_STABLE / DC_ROUTE_SOFTMAX
    float* dbg_x;                    // optional capture of every layer's input [n_layer + 1][DC_MAX_T][H]
    unsigned bar_polls;              // poll limit of a grid barrier
    unsigned long long ep_wait_ns;   // time limit of the expert-parallel meeting
    // sync
    unsigned* bar_counter;
    int* err;
    unsigned long long* phase_ns;  // optional [32] phase timing accumulators (CTA 0's view)
    // dynamic shared memory offsets
    uint32_t off_pipe, off_act, off_xs, off_sc, off_v, smem_bytes;
    // rows per pipeline stage
    int rpst_q, rpst_k, rpst_v, rpst_o, rpst_gate, rpst_down, rpst_out;
    uint32_t up_off;
};
