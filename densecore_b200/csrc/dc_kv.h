// Paged KV cache bookkeeping shared by the op-level API and the decoder.
#pragma once
#include <cuda_fp16.h>

#include <vector>

#include "dc_internal.h"

struct dc_kv_seq {
    bool used = false;
    int len = 0;                 // tokens appended so far
    std::vector<int> blocks;     // logical block -> physical block
};

struct dc_kv_cache {
    dc_ctx* ctx = nullptr;
    int n_layer = 0, n_kv = 0, head_dim = 0;
    int max_blocks = 0, max_seqs = 0, max_blocks_per_seq = 0;
    size_t layer_elems = 0;      // fp16 elements per layer in each arena
    __half* k_arena = nullptr;
    __half* v_arena = nullptr;
    int32_t* d_tables = nullptr; // [max_seqs][max_blocks_per_seq]
    std::vector<int> free_list;
    std::vector<int> ref;        // references per physical block (sequences sharing it after a fork)
    std::vector<dc_kv_seq> seqs;
    int stage_off = 0;
};

int dc_kv_init(dc_ctx* ctx, dc_kv_cache* kv, int n_layer, int n_kv_head, int head_dim, int max_blocks, int max_seqs,
               int max_blocks_per_seq);
void dc_kv_release(dc_kv_cache* kv);
int dc_kv_seq_alloc(dc_kv_cache* kv, int* out_seq);
int dc_kv_seq_free(dc_kv_cache* kv, int seq);
int dc_kv_seq_reserve(dc_kv_cache* kv, int seq, int n_tokens);
int dc_kv_seq_fork(dc_kv_cache* kv, int src_seq, int* out_seq);
