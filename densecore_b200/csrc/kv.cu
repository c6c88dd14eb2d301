// Paged KV cache: fp16 arenas [layer][block][16 slots][kv_head][head_dim] for K
// and V (core/src/runtime/memory/kv_cache_storage.cpp:146-200), a free-list block
// manager and per-sequence block tables (core/include/densecore/memory/kv_cache.h:67-220)
// mirrored in device memory for the kernels.  Host-side bookkeeping only; the
// slot writes and reads are in misc.cu / attn.cu.
#include <string.h>

#include "dc_common.cuh"
#include "dc_internal.h"
#include "dc_kv.h"

int dc_kv_init(dc_ctx* ctx, dc_kv_cache* kv, int n_layer, int n_kv_head, int head_dim, int max_blocks, int max_seqs,
               int max_blocks_per_seq) {
    if (n_layer <= 0 || n_kv_head <= 0 || head_dim != 128 || max_blocks <= 0 || max_seqs <= 0 || max_blocks_per_seq <= 0)
        return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "kv_create: bad shape (head_dim must be 128)");
    kv->ctx = ctx;
    kv->n_layer = n_layer;
    kv->n_kv = n_kv_head;
    kv->head_dim = head_dim;
    kv->max_blocks = max_blocks;
    kv->max_seqs = max_seqs;
    kv->max_blocks_per_seq = max_blocks_per_seq;
    kv->layer_elems = (size_t)max_blocks * DC_KV_BLOCK * n_kv_head * head_dim;
    const size_t bytes = kv->layer_elems * n_layer * sizeof(__half);
    cudaError_t e = cudaMalloc(&kv->k_arena, bytes);
    if (e == cudaSuccess) e = cudaMalloc(&kv->v_arena, bytes);
    if (e == cudaSuccess) e = cudaMalloc(&kv->d_tables, (size_t)max_seqs * max_blocks_per_seq * sizeof(int32_t));
    if (e == cudaSuccess) e = cudaMemsetAsync(kv->k_arena, 0, bytes, ctx->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(kv->v_arena, 0, bytes, ctx->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(kv->d_tables, 0, (size_t)max_seqs * max_blocks_per_seq * sizeof(int32_t), ctx->stream);
    if (e != cudaSuccess) return dc_check_cuda(ctx, e, "kv_create");
    kv->free_list.clear();
    for (int b = max_blocks - 1; b >= 0; --b) kv->free_list.push_back(b);
    kv->ref.assign(max_blocks, 0);
    kv->seqs.assign(max_seqs, dc_kv_seq());
    kv->prefix.clear();
    kv->block_hash.assign(max_blocks, 0);
    kv->block_tokens.assign(max_blocks, std::array<int32_t, 16>());
    kv->block_used.assign(max_blocks, 0);
    return DC_B200_OK;
}

// Blocks an allocation can get: the free list plus cached blocks that only the prefix cache still holds.
int dc_kv_available_blocks(const dc_kv_cache* kv) {
    int n = (int)kv->free_list.size();
    for (int b = 0; b < kv->max_blocks; ++b)
        if (kv->block_hash[b] && kv->ref[b] == 1) ++n;
    return n;
}

// A block for a new owner (reference count 1), evicting the least recently used cached block that no
// sequence holds when the free list is empty; -1 if there is none.
static int take_block(dc_kv_cache* kv) {
    if (kv->free_list.empty()) {
        int victim = -1;
        for (int b = 0; b < kv->max_blocks; ++b)
            if (kv->block_hash[b] && kv->ref[b] == 1 && (victim < 0 || kv->block_used[b] < kv->block_used[victim])) victim = b;
        if (victim < 0) return -1;
        auto it = kv->prefix.find(kv->block_hash[victim]);
        if (it != kv->prefix.end() && it->second == victim) kv->prefix.erase(it);
        kv->block_hash[victim] = 0;
        kv->ref[victim] = 0;
        ++kv->prefix_evictions;
        kv->free_list.push_back(victim);
    }
    const int b = kv->free_list.back();
    kv->free_list.pop_back();
    kv->ref[b] = 1;
    return b;
}

void dc_kv_release(dc_kv_cache* kv) {
    if (kv->k_arena) cudaFree(kv->k_arena);
    if (kv->v_arena) cudaFree(kv->v_arena);
    if (kv->d_tables) cudaFree(kv->d_tables);
    kv->k_arena = kv->v_arena = nullptr;
    kv->d_tables = nullptr;
}

int dc_kv_seq_alloc(dc_kv_cache* kv, int* out_seq) {
    for (int s = 0; s < kv->max_seqs; ++s) {
        if (!kv->seqs[s].used) {
            kv->seqs[s].used = true;
            kv->seqs[s].len = 0;
            kv->seqs[s].blocks.clear();
            *out_seq = s;
            return DC_B200_OK;
        }
    }
    return dc_fail(kv->ctx, DC_B200_OUT_OF_MEMORY, "kv: all %d sequence slots are in use", kv->max_seqs);
}

int dc_kv_seq_free(dc_kv_cache* kv, int seq) {
    if (seq < 0 || seq >= kv->max_seqs || !kv->seqs[seq].used)
        return dc_fail(kv->ctx, DC_B200_INVALID_ARGUMENT, "kv: sequence %d is not allocated", seq);
    // a block returns to the free list when its last reference goes (kv_cache.h:140)
    for (int b : kv->seqs[seq].blocks)
        if (--kv->ref[b] <= 0) {
            kv->ref[b] = 0;
            kv->free_list.push_back(b);
        }
    kv->seqs[seq] = dc_kv_seq();
    return DC_B200_OK;
}

// One block of every layer, K and V: src -> dst.
__global__ void __launch_bounds__(256) k_kv_copy_block(__half* k_arena, __half* v_arena, size_t layer_elems,
                                                       size_t block_elems, int src, int dst) {
    __half* arena = blockIdx.y ? v_arena : k_arena;
    const uint4* s = reinterpret_cast<const uint4*>(arena + layer_elems * blockIdx.x + block_elems * src);
    uint4* d = reinterpret_cast<uint4*>(arena + layer_elems * blockIdx.x + block_elems * dst);
    for (size_t i = threadIdx.x; i < block_elems / 8; i += blockDim.x) d[i] = s[i];
}

// Staged upload of `n` table entries of a sequence starting at logical block `first`.
static int upload_table(dc_kv_cache* kv, int seq, int first, int n) {
    if (n <= 0) return DC_B200_OK;
    int32_t* stage = (int32_t*)dc_pinned(kv->ctx, 64 * 1024);
    if (!stage) return DC_B200_OUT_OF_MEMORY;
    if (n > 16 * 1024) return dc_fail(kv->ctx, DC_B200_UNSUPPORTED, "kv: too many new blocks at once");
    if (kv->stage_off + n > 16 * 1024) {   // a small pinned ring keeps the async copy source valid
        cudaStreamSynchronize(kv->ctx->stream);
        kv->stage_off = 0;
    }
    memcpy(stage + kv->stage_off, kv->seqs[seq].blocks.data() + first, (size_t)n * sizeof(int32_t));
    cudaError_t e = cudaMemcpyAsync(kv->d_tables + (size_t)seq * kv->max_blocks_per_seq + first, stage + kv->stage_off,
                                    (size_t)n * sizeof(int32_t), cudaMemcpyHostToDevice, kv->ctx->stream);
    kv->stage_off += n;
    return dc_check_cuda(kv->ctx, e, "kv: block table upload");
}

// New sequence that shares every block of src (Fork, kv_cache.h:151-156): nothing is copied now; a shared
// block is copied when one of its owners is about to write into it (copy-on-write, :158-161).
int dc_kv_seq_fork(dc_kv_cache* kv, int src_seq, int* out_seq) {
    if (src_seq < 0 || src_seq >= kv->max_seqs || !kv->seqs[src_seq].used)
        return dc_fail(kv->ctx, DC_B200_INVALID_ARGUMENT, "kv: sequence %d is not allocated", src_seq);
    int dst = -1;
    int st = dc_kv_seq_alloc(kv, &dst);
    if (st != DC_B200_OK) return st;
    kv->seqs[dst].blocks = kv->seqs[src_seq].blocks;
    kv->seqs[dst].len = kv->seqs[src_seq].len;
    for (int b : kv->seqs[dst].blocks) ++kv->ref[b];
    st = upload_table(kv, dst, 0, (int)kv->seqs[dst].blocks.size());
    if (st != DC_B200_OK) {
        dc_kv_seq_free(kv, dst);
        return st;
    }
    *out_seq = dst;
    return DC_B200_OK;
}

// Makes sure blocks exist for positions [0, n_tokens), that the blocks the next writes touch (positions
// from the sequence's length on) are not shared with another sequence, and mirrors new table entries to
// the device (ordered on the context's stream).
int dc_kv_seq_reserve(dc_kv_cache* kv, int seq, int n_tokens) {
    if (seq < 0 || seq >= kv->max_seqs || !kv->seqs[seq].used)
        return dc_fail(kv->ctx, DC_B200_INVALID_ARGUMENT, "kv: sequence %d is not allocated", seq);
    dc_kv_seq& s = kv->seqs[seq];
    const int need = (n_tokens + DC_KV_BLOCK - 1) / DC_KV_BLOCK;
    if (need > kv->max_blocks_per_seq)
        return dc_fail(kv->ctx, DC_B200_OUT_OF_MEMORY, "kv: sequence %d needs %d blocks, table holds %d", seq, need,
                       kv->max_blocks_per_seq);
    const int have = (int)s.blocks.size();
    // copy-on-write of shared blocks in the range about to be written
    for (int lb = s.len / DC_KV_BLOCK; lb < have && lb < need; ++lb) {
        const int old = s.blocks[lb];
        if (kv->ref[old] <= 1) continue;
        const int fresh = take_block(kv);
        if (fresh < 0) return dc_fail(kv->ctx, DC_B200_OUT_OF_MEMORY, "kv: out of blocks (copy-on-write)");
        --kv->ref[old];
        const size_t be = (size_t)DC_KV_BLOCK * kv->n_kv * kv->head_dim;
        k_kv_copy_block<<<dim3(kv->n_layer, 2), 256, 0, kv->ctx->stream>>>(kv->k_arena, kv->v_arena, kv->layer_elems, be, old, fresh);
        int st = dc_check_cuda(kv->ctx, cudaGetLastError(), "k_kv_copy_block");
        if (st != DC_B200_OK) return st;
        s.blocks[lb] = fresh;
        st = upload_table(kv, seq, lb, 1);
        if (st != DC_B200_OK) return st;
    }
    if (need <= have) return DC_B200_OK;
    if ((int)kv->free_list.size() < need - have && dc_kv_available_blocks(kv) < need - have)
        return dc_fail(kv->ctx, DC_B200_OUT_OF_MEMORY, "kv: out of blocks (%d free, %d needed)",
                       dc_kv_available_blocks(kv), need - have);
    for (int i = have; i < need; ++i) s.blocks.push_back(take_block(kv));
    return upload_table(kv, seq, have, need - have);
}

// FNV-1a over the token ids, one 64-bit step per token, continued from h (start: 14695981039346656037);
// BlockManager::ComputeTokenHash, core/src/runtime/memory/kv_cache_block_manager.cpp:515-522, without a salt.
uint64_t dc_kv_token_hash(uint64_t h, const int32_t* tokens, int n) {
    for (int i = 0; i < n; ++i) {
        h ^= (uint64_t)(int64_t)tokens[i];
        h *= 1099511628211ULL;
    }
    return h;
}

// Longest cached prefix of whole blocks for a sequence that holds nothing yet
// (FindLongestCachedPrefixWithVerification, kv_cache_block_manager.cpp:364-416): block i is looked up under the
// hash of tokens[0 .. 16 (i + 1)) and accepted only if its stored tokens equal tokens[16 i .. 16 (i + 1)).
// At least one token is always left to run, so that the prompt's last logits are computed as usual.
// The matched blocks join the sequence's table as shared blocks; *cached_tokens of its positions are then filled.
int dc_kv_prefix_attach(dc_kv_cache* kv, int seq, const int32_t* tokens, int n_tokens, int* cached_tokens) {
    *cached_tokens = 0;
    if (seq < 0 || seq >= kv->max_seqs || !kv->seqs[seq].used)
        return dc_fail(kv->ctx, DC_B200_INVALID_ARGUMENT, "kv: sequence %d is not allocated", seq);
    dc_kv_seq& s = kv->seqs[seq];
    if (s.len != 0 || !s.blocks.empty())
        return dc_fail(kv->ctx, DC_B200_INVALID_ARGUMENT, "kv: prefix lookup needs an empty sequence (sequence %d holds %d tokens)", seq, s.len);
    ++kv->prefix_lookups;
    if (!tokens || n_tokens <= DC_KV_BLOCK) return DC_B200_OK;
    int reusable = (n_tokens - 1) / DC_KV_BLOCK * DC_KV_BLOCK;
    if (reusable > kv->max_blocks_per_seq * DC_KV_BLOCK) reusable = kv->max_blocks_per_seq * DC_KV_BLOCK;
    uint64_t h = 14695981039346656037ULL;
    ++kv->tick;
    for (int off = 0; off < reusable; off += DC_KV_BLOCK) {
        h = dc_kv_token_hash(h, tokens + off, DC_KV_BLOCK);
        auto it = kv->prefix.find(h);
        if (it == kv->prefix.end()) break;
        const int b = it->second;
        if (kv->block_hash[b] != h || memcmp(kv->block_tokens[b].data(), tokens + off, sizeof(int32_t) * DC_KV_BLOCK) != 0) break;
        ++kv->ref[b];
        kv->block_used[b] = kv->tick;
        s.blocks.push_back(b);
        ++kv->prefix_hit_blocks;
    }
    s.len = (int)s.blocks.size() * DC_KV_BLOCK;
    *cached_tokens = s.len;
    return upload_table(kv, seq, 0, (int)s.blocks.size());
}

// Registers every whole block of the sequence's first n_tokens positions (whose tokens are `tokens`) under
// its cumulative-prefix hash (RegisterPrefixBlockWithTokens, kv_cache_block_manager.cpp:443-).  A prefix that
// is cached already keeps its block.
int dc_kv_prefix_register(dc_kv_cache* kv, int seq, const int32_t* tokens, int n_tokens) {
    if (seq < 0 || seq >= kv->max_seqs || !kv->seqs[seq].used || !tokens)
        return dc_fail(kv->ctx, DC_B200_INVALID_ARGUMENT, "kv: sequence %d is not allocated", seq);
    dc_kv_seq& s = kv->seqs[seq];
    if (n_tokens > s.len) n_tokens = s.len;
    uint64_t h = 14695981039346656037ULL;
    ++kv->tick;
    for (int lb = 0; (lb + 1) * DC_KV_BLOCK <= n_tokens && lb < (int)s.blocks.size(); ++lb) {
        h = dc_kv_token_hash(h, tokens + lb * DC_KV_BLOCK, DC_KV_BLOCK);
        if (h == 0) continue;
        const int b = s.blocks[lb];
        auto it = kv->prefix.find(h);
        if (it != kv->prefix.end()) {
            kv->block_used[it->second] = kv->tick;
            continue;
        }
        if (kv->block_hash[b]) continue;   // resident under another prefix already
        kv->prefix[h] = b;
        kv->block_hash[b] = h;
        memcpy(kv->block_tokens[b].data(), tokens + lb * DC_KV_BLOCK, sizeof(int32_t) * DC_KV_BLOCK);
        kv->block_used[b] = kv->tick;
        ++kv->ref[b];                       // the cache's own reference
    }
    return DC_B200_OK;
}

extern "C" {

int dc_b200_kv_create(dc_ctx* ctx, int n_layer, int n_kv_head, int head_dim, int max_blocks, int max_seqs,
                      int max_blocks_per_seq, dc_kv_cache** out) {
    if (!ctx || !out) return DC_B200_INVALID_ARGUMENT;
    *out = nullptr;
    cudaSetDevice(ctx->device);
    dc_kv_cache* kv = new dc_kv_cache();
    int st = dc_kv_init(ctx, kv, n_layer, n_kv_head, head_dim, max_blocks, max_seqs, max_blocks_per_seq);
    if (st != DC_B200_OK) {
        dc_kv_release(kv);
        delete kv;
        return st;
    }
    *out = kv;
    return DC_B200_OK;
}

void dc_b200_kv_destroy(dc_kv_cache* kv) {
    if (!kv) return;
    cudaSetDevice(kv->ctx->device);
    cudaStreamSynchronize(kv->ctx->stream);
    dc_kv_release(kv);
    delete kv;
}

int dc_b200_kv_seq_alloc(dc_kv_cache* kv, int* out_seq) {
    if (!kv || !out_seq) return DC_B200_INVALID_ARGUMENT;
    return dc_kv_seq_alloc(kv, out_seq);
}
int dc_b200_kv_seq_free(dc_kv_cache* kv, int seq) { return kv ? dc_kv_seq_free(kv, seq) : DC_B200_INVALID_ARGUMENT; }
int dc_b200_kv_seq_reserve(dc_kv_cache* kv, int seq, int n_tokens) {
    if (!kv) return DC_B200_INVALID_ARGUMENT;
    cudaSetDevice(kv->ctx->device);
    return dc_kv_seq_reserve(kv, seq, n_tokens);
}
int dc_b200_kv_block_table(dc_kv_cache* kv, int seq, int32_t* out_blocks, int capacity, int* out_n) {
    if (!kv || seq < 0 || seq >= kv->max_seqs || !kv->seqs[seq].used || !out_n) return DC_B200_INVALID_ARGUMENT;
    const int n = (int)kv->seqs[seq].blocks.size();
    *out_n = n;
    if (out_blocks)
        for (int i = 0; i < n && i < capacity; ++i) out_blocks[i] = kv->seqs[seq].blocks[i];
    return DC_B200_OK;
}
int dc_b200_kv_seq_fork(dc_kv_cache* kv, int src_seq, int* out_seq) {
    if (!kv || !out_seq) return DC_B200_INVALID_ARGUMENT;
    cudaSetDevice(kv->ctx->device);
    return dc_kv_seq_fork(kv, src_seq, out_seq);
}
int dc_b200_kv_block_refcount(dc_kv_cache* kv, int block) {
    return (kv && block >= 0 && block < kv->max_blocks) ? kv->ref[block] : DC_B200_INVALID_ARGUMENT;
}
int dc_b200_kv_free_blocks(dc_kv_cache* kv) { return kv ? dc_kv_available_blocks(kv) : DC_B200_INVALID_ARGUMENT; }
int dc_b200_kv_prefix_attach(dc_kv_cache* kv, int seq, const int32_t* tokens, int n_tokens, int* cached_tokens) {
    if (!kv || !cached_tokens) return DC_B200_INVALID_ARGUMENT;
    cudaSetDevice(kv->ctx->device);
    return dc_kv_prefix_attach(kv, seq, tokens, n_tokens, cached_tokens);
}
int dc_b200_kv_prefix_register(dc_kv_cache* kv, int seq, const int32_t* tokens, int n_tokens) {
    return kv ? dc_kv_prefix_register(kv, seq, tokens, n_tokens) : DC_B200_INVALID_ARGUMENT;
}
uint64_t dc_b200_kv_prefix_hash(const int32_t* tokens, int n_tokens) {
    return tokens && n_tokens > 0 ? dc_kv_token_hash(14695981039346656037ULL, tokens, n_tokens) : 0;
}
int dc_b200_kv_prefix_stats(dc_kv_cache* kv, uint64_t out[4]) {
    if (!kv || !out) return DC_B200_INVALID_ARGUMENT;
    out[0] = kv->prefix_lookups;
    out[1] = kv->prefix_hit_blocks;
    out[2] = (uint64_t)kv->prefix.size();
    out[3] = kv->prefix_evictions;
    return DC_B200_OK;
}

int dc_b200_kv_read_block(dc_kv_cache* kv, int layer, int block, void* k_host, void* v_host) {
    if (!kv || layer < 0 || layer >= kv->n_layer || block < 0 || block >= kv->max_blocks) return DC_B200_INVALID_ARGUMENT;
    cudaSetDevice(kv->ctx->device);
    const size_t be = (size_t)DC_KV_BLOCK * kv->n_kv * kv->head_dim;
    const size_t off = kv->layer_elems * layer + be * block;
    cudaError_t e = cudaStreamSynchronize(kv->ctx->stream);
    if (e == cudaSuccess && k_host) e = cudaMemcpy(k_host, kv->k_arena + off, be * sizeof(__half), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && v_host) e = cudaMemcpy(v_host, kv->v_arena + off, be * sizeof(__half), cudaMemcpyDeviceToHost);
    return dc_check_cuda(kv->ctx, e, "kv_read_block");
}

}  // extern "C"
