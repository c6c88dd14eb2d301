// Paged KV cache bookkeeping shared by the op-level API and the decoder.
#pragma once
#include <cuda_fp16.h>

#include <array>
#include <unordered_map>
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
    // Prefix cache (core/include/densecore/memory/kv_cache.h:176-213): a full block can be registered under
    // the hash of the whole token prefix that ends with it; the cache then holds one reference of its own, so
    // the block outlives its sequence until it is evicted (least recently used first) to satisfy an allocation.
    std::unordered_map<uint64_t, int> prefix;               // cumulative-prefix hash -> physical block
    std::vector<uint64_t> block_hash;                       // hash a block is registered under, 0: none
    std::vector<std::array<int32_t, 16>> block_tokens;      // the block's own tokens (collision check)
    std::vector<uint64_t> block_used;                       // tick of the block's last registration or hit
    uint64_t tick = 0;
    uint64_t prefix_lookups = 0, prefix_hit_blocks = 0, prefix_evictions = 0;
};

int dc_kv_init(dc_ctx* ctx, dc_kv_cache* kv, int n_layer, int n_kv_head, int head_dim, int max_blocks, int max_seqs,
               int max_blocks_per_seq);
void dc_kv_release(dc_kv_cache* kv);
int dc_kv_seq_alloc(dc_kv_cache* kv, int* out_seq);
int dc_kv_seq_free(dc_kv_cache* kv, int seq);
int dc_kv_seq_reserve(dc_kv_cache* kv, int seq, int n_tokens);
int dc_kv_seq_fork(dc_kv_cache* kv, int src_seq, int* out_seq);
uint64_t dc_kv_token_hash(uint64_t h, const int32_t* tokens, int n);
int dc_kv_prefix_attach(dc_kv_cache* kv, int seq, const int32_t* tokens, int n_tokens, int* cached_tokens);
int dc_kv_prefix_register(dc_kv_cache* kv, int seq, const int32_t* tokens, int n_tokens);
int dc_kv_available_blocks(const dc_kv_cache* kv);
