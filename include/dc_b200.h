/*
 * dc_b200.h -- C ABI of libdc_b200.so: DenseCore's quantized decode hot path on
 * one NVIDIA B200 (sm_100a).
 *
 * Every entry point is what a DenseCore ggml custom-op callback (thread
 * ith == 0) or the sampler site would call; each comment names the DenseCore
 * interface it stands in for (path within the DenseCore tree, file:line).
 *
 * Conventions
 *  - Plain C types only.  Tensors follow ggml: ne[0] is the fastest dimension;
 *    a weight W[N_out, K_in] is N_out rows of K_in/256 GGUF super-blocks
 *    (Q4_K 144 B, Q6_K 210 B), copied to the GPU byte for byte.
 *  - Every call returns 0 on success or a negative status that mirrors
 *    DENSECORE_STATUS_* (core/include/densecore.h:143-152).  On failure output
 *    buffers are zero-filled where the callback convention asks for it
 *    (core/src/llm/attention/paged_exec.cpp:358-412, core/src/llm/moe/exec.cpp:397-414)
 *    and dc_b200_last_error() returns one line of text.
 *  - *_host arguments are host pointers (copies happen inside the call, which
 *    returns after the result is in host memory).  *_dev arguments are device
 *    pointers on the context's GPU; those calls only enqueue on the context's
 *    stream (see dc_b200_stream / dc_b200_synchronize).
 *  - A context is bound to one GPU and one stream; calls on one context must
 *    not overlap in time (the ggml graph executor issues ops in order).
 *  - There is no CPU fallback: without a usable GPU dc_b200_init fails.
 */
#ifndef DC_B200_H
#define DC_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DC_B200_API __attribute__((visibility("default")))

/* mirrors DenseCoreStatus, core/include/densecore.h:143-152 */
enum {
    DC_B200_OK = 0,
    DC_B200_INVALID_ARGUMENT = -1,
    DC_B200_MODEL_LOAD_FAILED = -2,
    DC_B200_OUT_OF_MEMORY = -3,
    DC_B200_INTERNAL_ERROR = -5,
    DC_B200_BACKEND_ERROR = -6,
    DC_B200_UNSUPPORTED = -7
};

/* ggml type ids of the tensors this library accepts */
enum { DC_GGML_TYPE_F32 = 0, DC_GGML_TYPE_F16 = 1, DC_GGML_TYPE_Q4_K = 12, DC_GGML_TYPE_Q6_K = 14 };

typedef struct dc_ctx dc_ctx;
typedef struct dc_weight dc_weight;

/* ---- context ---------------------------------------------------------- */
/* Backend bring-up; the role of InitEngine for this path
 * (core/src/runtime/engine.cpp:955) and of CreateBackend in the HAL plugin
 * contract (core/src/backend/backend_registry.cpp:245-374). */
DC_B200_API int dc_b200_init(int device, dc_ctx** out_ctx);
DC_B200_API void dc_b200_destroy(dc_ctx* ctx);
/* DenseCoreGetLastError, core/include/densecore.h:163.  Valid until the next call on ctx. */
DC_B200_API const char* dc_b200_last_error(dc_ctx* ctx);
/* cudaStream_t of the context, as void*. */
DC_B200_API void* dc_b200_stream(dc_ctx* ctx);
/* Waits for the stream and reports any error a kernel recorded (bounded waits
 * that ran out). */
DC_B200_API int dc_b200_synchronize(dc_ctx* ctx);
/* "pdl" 0/1: programmatic dependent launch between consecutive kernels (default 1).
 * "route_mode" 0/1: router of the op-level MoE calls (dc_b200_moe_route, dc_b200_mul_mat_id): 0 = top-k on
 * the logits with the stable comparator, weights over the picks (ComputeQwenNativeMoEStableTopK,
 * core/src/llm/moe/native.cpp:610-676; default); 1 = softmax over all experts, top-k on the probabilities
 * with strict '>', weights renormalised (SoftmaxRow / TopKSelect / NormalizeWeights,
 * core/src/moe/moe_routing.cpp:53-101). */
DC_B200_API int dc_b200_set_option(dc_ctx* ctx, const char* name, int value);

/* cudaProfilerStart (1) / cudaProfilerStop (0): brackets the region a profiler
 * run with --profile-from-start off captures. */
DC_B200_API int dc_b200_profiler_range(int start);

/* ---- weights ---------------------------------------------------------- */
/* Copies a GGUF tensor to HBM verbatim.  ne[0]=K_in (multiple of 256 for
 * K-quants), ne[1]=N_out, ne[2]=experts (1 for a dense tensor), ne[3]=1.  The
 * data a ggml weight tensor's ->data points at (src[1] of the custom op,
 * core/src/llm/matmul/graph_ops.cpp:212-227). */
DC_B200_API int dc_b200_upload_weight(dc_ctx* ctx, int ggml_type, const int64_t ne[4], const void* data_host,
                                      dc_weight** out_weight);
DC_B200_API int dc_b200_free_weight(dc_ctx* ctx, dc_weight* w);
/* Device address and byte size of an uploaded tensor. */
DC_B200_API void* dc_b200_weight_data(const dc_weight* w, size_t* bytes);

/* ---- Q8_K activation quantiser ----------------------------------------- */
/* traits(Q8_K)->from_float as used at core/src/llm/matmul/gemv_exec.cpp:298,321;
 * restated in core/src/kernels/hwy/hwy_moe_quant.cc:103-144.  x: rows x K f32;
 * out: rows x (K/256) blocks of 292 bytes.  Bit-exact with the CPU routine. */
DC_B200_API int dc_b200_quantize_q8k(dc_ctx* ctx, const float* x_host, int rows, int K, void* q8_host);
DC_B200_API int dc_b200_quantize_q8k_dev(dc_ctx* ctx, const float* x_dev, int rows, int K, void* q8_dev);

/* ---- MUL_MAT ----------------------------------------------------------- */
/* y[M, N] = x[M, K] * W[N, K]^T with x quantised to Q8_K first: the body of
 * cb_gemv_custom (M == 1, core/src/llm/matmul/gemv_exec.cpp:99) and
 * cb_gemv_batched_custom (M >= 2, core/src/llm/matmul/batched_exec.cpp:55).
 * Any M >= 1; rows are processed 16 at a time (kMaxSmallBatchColsHard,
 * core/src/llm/matmul/userdata.h:14). */
DC_B200_API int dc_b200_mul_mat(dc_ctx* ctx, const dc_weight* w, const float* x_host, int M, float* y_host);
DC_B200_API int dc_b200_mul_mat_dev(dc_ctx* ctx, const dc_weight* w, const float* x_dev, int M, float* y_dev);
/* The same product for callers that may not allocate (no counterpart in
 * DenseCore; added for hosts that forbid allocator calls on the compute path:
 * op callbacks running under a fixed-buffer graph executor, serving loops that
 * must not take the CUDA allocator lock after warm-up, code inside a stream
 * capture).  x_dev [M, K] and y_dev [M, N] are device buffers of the caller;
 * the Q8_K form of x lives in a 299,008-byte array built into the library
 * (each GPU that loads the library keeps it until exit).  Limits: M <= 16 and
 * K <= 16384, larger shapes are refused with DC_B200_UNSUPPORTED.  No
 * cudaMalloc/cudaFree or allocating routine is called.  The first call on a
 * GPU looks up the array's device address (cudaGetSymbolAddress), and the first
 * call for each row-count class (1, 2-4, 5-8, 9-16) and weight shape also
 * configures its kernel instance (shared-memory opt-in, occupancy query) on
 * that GPU; make one such call before any stream capture begins.  All calls on a GPU share the array
 * and it keeps the previous call's contents (each call overwrites what it
 * reads), so two calls whose kernels can overlap on the GPU, e.g. from two
 * contexts or streams, race: serialise them.  Enqueues on the context's stream. */
DC_B200_API int dc_b200_mul_mat_dev_noalloc(dc_ctx* ctx, const dc_weight* w, const float* x_dev, int M, float* y_dev);
/* Parity aid: the exact int32 block sums the kernel forms, I[M][N][K/256] and
 * (Q4_K only, else may be NULL) Mn[M][N][K/256]; these are the quantities the
 * reference's vec_dot kernels agree on bit for bit
 * (core/src/kernels/hwy/hwy_moe_quant.cc:218-246). */
DC_B200_API int dc_b200_mul_mat_block_sums(dc_ctx* ctx, const dc_weight* w, const float* x_host, int M,
                                           int32_t* I_host, int32_t* Mn_host);

/* ---- device buffers ------------------------------------------------------ */
/* AllocateDevice / FreeDevice / CopyToDevice / CopyFromDevice of the HAL
 * ComputeBackend contract (core/include/densecore/hal/compute_backend.h:308-692). */
DC_B200_API int dc_b200_alloc_device(dc_ctx* ctx, size_t bytes, void** out_dev);
DC_B200_API int dc_b200_free_device(dc_ctx* ctx, void* dev);
DC_B200_API int dc_b200_copy_to_device(dc_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes);
DC_B200_API int dc_b200_copy_from_device(dc_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes);

/* ---- MUL_MAT_ID: one MoE FFN layer ---------------------------------------- */
/* cb_moe_forward (core/src/llm/moe/exec.cpp:813): router logits = x * Wr^T,
 * top-k routing, per-expert SwiGLU FFN, weighted combine.  router: F32
 * [hidden, n_expert]; gate/up: [hidden, ffn, n_expert]; down: [ffn, hidden,
 * n_expert].  x: [T, hidden] f32, T <= 16.  y: [T, hidden].  ids_out [T, top_k]
 * and weights_out [T, top_k] may be NULL.  routed_scale multiplies the routing
 * weights (moe_routed_scaling_factor, core/src/llm/moe/exec.cpp:764-768). */
DC_B200_API int dc_b200_mul_mat_id(dc_ctx* ctx, const dc_weight* router, const dc_weight* gate, const dc_weight* up,
                                   const dc_weight* down, const float* x_host, int T, int top_k, float routed_scale,
                                   float* y_host, int32_t* ids_out, float* weights_out);
/* The same layer on device buffers (x_dev [T, hidden], y_dev [T, hidden], optional ids_dev / weights_dev
 * [T, top_k]): what the body of cb_moe_forward calls when the graph's tensors already live on the GPU.  Only
 * enqueues on the context's stream. */
DC_B200_API int dc_b200_mul_mat_id_dev(dc_ctx* ctx, const dc_weight* router, const dc_weight* gate, const dc_weight* up,
                                       const dc_weight* down, const float* x_dev, int T, int top_k,
                                       float routed_scale, float* y_dev, int32_t* ids_dev, float* weights_dev);
/* cb_moe_forward with its own arguments (core/src/llm/moe/exec.cpp:813: src0 = the routed input, src1 = the
 * router logits the graph computed): routes from gate_logits [T, n_expert] as given, then runs the experts.
 * Fails closed like the callback: y is zero-filled on any error. */
DC_B200_API int dc_b200_moe_forward(dc_ctx* ctx, const dc_weight* gate, const dc_weight* up, const dc_weight* down,
                                    const float* x_host, const float* gate_logits_host, int T, int top_k,
                                    float routed_scale, float* y_host, int32_t* ids_out, float* weights_out);
/* Routing alone from given logits [T, n_expert] (RouteMoESoftmaxTopK, core/src/llm/moe/exec.cpp:734);
 * which of the reference's two routers runs is the context option "route_mode".  1 <= n_expert <= 256,
 * 1 <= top_k <= min(16, n_expert), else DC_B200_UNSUPPORTED with nothing launched. */
DC_B200_API int dc_b200_moe_route(dc_ctx* ctx, const float* logits_host, int T, int n_expert, int top_k,
                                  float routed_scale, int32_t* ids_out, float* weights_out);

/* ---- paged KV cache + FLASH_ATTN (decode) ---------------------------------- */
typedef struct dc_kv_cache dc_kv_cache;
/* PagedKVCache: 16-token blocks, F16, arena [layer][block][slot][kv_head][head_dim]
 * (core/include/densecore/memory/kv_cache.h:50,245-395,
 * core/src/runtime/memory/kv_cache_storage.cpp:146-200). */
DC_B200_API int dc_b200_kv_create(dc_ctx* ctx, int n_layer, int n_kv_head, int head_dim, int max_blocks, int max_seqs,
                                  int max_blocks_per_seq, dc_kv_cache** out);
DC_B200_API void dc_b200_kv_destroy(dc_kv_cache* kv);
/* Sequence slots and their block tables (SequenceBlockTable / BlockManager,
 * kv_cache.h:67-87,92-220).  kv_seq_reserve makes sure blocks exist for
 * positions [0, n_tokens). */
DC_B200_API int dc_b200_kv_seq_alloc(dc_kv_cache* kv, int* out_seq);
DC_B200_API int dc_b200_kv_seq_free(dc_kv_cache* kv, int seq);
DC_B200_API int dc_b200_kv_seq_reserve(dc_kv_cache* kv, int seq, int n_tokens);
DC_B200_API int dc_b200_kv_block_table(dc_kv_cache* kv, int seq, int32_t* out_blocks, int capacity, int* out_n);
DC_B200_API int dc_b200_kv_free_blocks(dc_kv_cache* kv);
/* Fork (BlockManager::Fork / CopyOnWrite, core/include/densecore/memory/kv_cache.h:151-166): a new
 * sequence that shares every block of src_seq and has its length.  Nothing is copied at the fork; when a
 * sequence is about to write into a block that another one still references (kv_seq_reserve, or a model
 * step), that block is first copied to a fresh one on the device (all layers, K and V).  Blocks return
 * to the free list when their last reference goes. */
DC_B200_API int dc_b200_kv_seq_fork(dc_kv_cache* kv, int src_seq, int* out_seq);
DC_B200_API int dc_b200_kv_block_refcount(dc_kv_cache* kv, int block);
/* Prefix cache of the block manager (core/include/densecore/memory/kv_cache.h:176-213,
 * core/src/runtime/memory/kv_cache_block_manager.cpp:364-416,515-522).  A whole block can be registered
 * under the FNV-1a hash of the entire token prefix that ends with it; the cache keeps a reference of its
 * own, so the block outlives its sequence until an allocation has to evict it (least recently used first;
 * only blocks no sequence holds).
 * kv_prefix_attach: for a sequence that holds nothing yet, finds the longest run of cached whole blocks
 * of tokens[0..n_tokens) (each verified token by token, always leaving at least one token to run), makes
 * them the sequence's first blocks (shared, copy-on-write) and sets its length; *cached_tokens = that
 * length.  kv_prefix_register: registers the whole blocks of the sequence's first n_tokens positions,
 * whose tokens the caller passes.  kv_prefix_stats: {lookups, blocks hit, blocks resident, evictions}. */
DC_B200_API int dc_b200_kv_prefix_attach(dc_kv_cache* kv, int seq, const int32_t* tokens, int n_tokens, int* cached_tokens);
DC_B200_API int dc_b200_kv_prefix_register(dc_kv_cache* kv, int seq, const int32_t* tokens, int n_tokens);
DC_B200_API int dc_b200_kv_prefix_stats(dc_kv_cache* kv, uint64_t out[4]);
/* The key a prefix of n_tokens tokens is cached under (BlockManager::ComputeTokenHash without a salt,
 * core/src/runtime/memory/kv_cache_block_manager.cpp:515-522): FNV-1a, one 64-bit step per token id.  Host only. */
DC_B200_API uint64_t dc_b200_kv_prefix_hash(const int32_t* tokens, int n_tokens);
/* cb_paged_attention_decode (core/src/llm/attention/paged_exec.cpp:343): writes
 * the T current tokens' K/V (f32 [T, n_kv, hd]) into the cache at positions[t]
 * of sequence seq_ids[t], then attends q [T, n_head, hd] over keys
 * 0..positions[t].  out: [T, n_head, hd] f32.  scale multiplies q.k. */
DC_B200_API int dc_b200_flash_attn_decode(dc_ctx* ctx, dc_kv_cache* kv, int layer, const float* q_host,
                                          const float* k_host, const float* v_host, const int32_t* seq_ids,
                                          const int32_t* positions, int T, int n_head, float scale, float* out_host);
/* The same op for a prompt chunk: n <= 4096 tokens of one sequence at positions pos0 .. pos0 + n - 1, causal.
 * What the CPU runs for chunks is ggml_flash_attn_ext over the fp16 cache with the query converted to fp16
 * (core/src/llm/attention/exec.cpp:255-275); here scores and P.V run on the tensor cores with fp16
 * operands (the query as a sum of two fp16 terms) and fp32 accumulation. */
DC_B200_API int dc_b200_flash_attn_prefill(dc_ctx* ctx, dc_kv_cache* kv, int layer, const float* q_host,
                                           const float* k_host, const float* v_host, int seq, int pos0, int n,
                                           int n_head, float scale, float* out_host);
/* Raw fp16 contents of one block of one layer (K then V planes), for tests. */
DC_B200_API int dc_b200_kv_read_block(dc_kv_cache* kv, int layer, int block, void* k_host, void* v_host);

/* ---- sampling / speculative verify ----------------------------------------- */
/* Greedy pick, first maximum wins (ArgmaxScalar, core/src/sampler/sampler.cpp:42-57). */
DC_B200_API int dc_b200_argmax(dc_ctx* ctx, const float* logits_host, int rows, int n, int32_t* out_ids);
/* Verify a draft chain of gamma tokens against target logits [gamma+1, vocab].
 * mode 0: greedy prefix match.  mode 1: accept t_i iff u_i*q_i[t_i] < p_i[t_i]
 * with p = softmax(target/temperature); on the first rejection resample from
 * max(0, p-q), else sample the bonus token from p_gamma.  draft_probs
 * [gamma, vocab] (mode 1).  uniforms [gamma+1] or NULL to draw them from
 * Philox4x32-10 keyed by (seed, step).  DenseCore has no such step (its draft
 * model is loaded and unused, core/src/runtime/engine.cpp:593-645). */
DC_B200_API int dc_b200_verify_accept(dc_ctx* ctx, const float* target_logits_host, const int32_t* draft_tokens,
                                      const float* draft_probs_host, const float* uniforms, uint64_t seed,
                                      uint32_t step, int gamma, int vocab, int mode, float temperature,
                                      int32_t* n_accepted, int32_t* next_token);
/* The same step with target logits (and, in mode 1, draft probabilities) already on this GPU, e.g.
 * dc_b200_model_logits_dev after dc_b200_forward_chunk: only the draft ids go in and two ints come out. */
DC_B200_API int dc_b200_verify_accept_dev(dc_ctx* ctx, const float* target_logits_dev, const int32_t* draft_tokens,
                                          const float* draft_probs_dev, const float* uniforms, uint64_t seed,
                                          uint32_t step, int gamma, int vocab, int mode, float temperature,
                                          int32_t* n_accepted, int32_t* next_token);
DC_B200_API int dc_b200_verify_uniforms(dc_ctx* ctx, uint64_t seed, uint32_t step, int n, float* out_host);
/* Temperature sampling of one token from device-resident logits [vocab] (the sampler site,
 * core/src/sampler/sampler.cpp:235-262: v * (1/T), minus max, exp, * 1/sum; here with the verify step's fully
 * specified exp and sums, and an inverse-CDF draw in index order with the uniform u in [0, 1)).  probs_dev
 * [vocab] keeps the distribution: it is the q a later dc_b200_verify_accept_dev (mode 1) needs for this token. */
DC_B200_API int dc_b200_sample_dev(dc_ctx* ctx, const float* logits_dev, int vocab, float temperature, float u,
                                   float* probs_dev, int32_t* token_out);
DC_B200_API int dc_b200_softmax(dc_ctx* ctx, const float* logits_host, int rows, int n, float temperature,
                                float* probs_host);

/* ---- decoder: the ops above chained into one model step --------------------- */
/* The graph BuildTransformerGraph lays out for a Qwen3-style decoder
 * (core/src/llm/graph/decoder.cpp:1085-1100 QKV, :1265-1343 Q/K norm, :1422-1450
 * RoPE, :1846-1872 attention, :2217-2410 MoE, :2662-2730 FFN, :2997 lm_head),
 * captured as a CUDA graph per batch shape. */
typedef struct dc_model dc_model;
typedef struct dc_model_config {
    int n_layer, hidden, n_head, n_kv_head, head_dim, vocab;
    int ffn;             /* dense FFN width (0 for MoE layers) */
    int n_expert;        /* 0 = dense model */
    int n_expert_used;   /* top-k */
    int expert_ffn;
    float rms_eps, rope_theta;
    float routed_scale;  /* 1.0 unless the model says otherwise */
    int tie_embeddings;  /* lm_head = token_embd */
    int qk_norm;         /* per-head RMSNorm on Q and K */
    int max_seqs, max_ctx;
    int ep_rank, ep_size; /* expert-parallel shard of this process (0,1 = all experts) */
} dc_model_config;

DC_B200_API int dc_b200_model_create(dc_ctx* ctx, const dc_model_config* cfg, dc_model** out);
DC_B200_API void dc_b200_model_destroy(dc_model* m);
/* GGUF tensor by name ("token_embd.weight", "blk.3.attn_q.weight",
 * "blk.3.ffn_gate_exps.weight", ...), bytes copied verbatim
 * (LoadGGUFModel, core/src/models/model_loader.cpp:2037). */
DC_B200_API int dc_b200_model_set_tensor(dc_model* m, const char* name, int ggml_type, const int64_t ne[4],
                                         const void* data_host);
/* Fills every tensor on the device from a seeded counter-based generator and
 * this library's own Q4_K / Q6_K quantiser (Q4_K_M-style type mix: attn_v,
 * even-layer ffn_down and the output matrix Q6_K, the rest Q4_K, norms and
 * router F32).  sigma is the weight standard deviation. */
DC_B200_API int dc_b200_model_init_synthetic(dc_model* m, uint64_t seed, float sigma);
/* Looks a tensor up: type, shape, device address, bytes. */
/* The model's configuration (as given to model_create, or as read from a GGUF file). */
DC_B200_API int dc_b200_model_get_config(dc_model* m, dc_model_config* out);
/* Names of all tensors the decoder needs (GGUF names: "token_embd.weight", "blk.0.attn_q.weight" ...).
 * *n_out receives their number; up to `capacity` pointers (owned by the model) are written. */
DC_B200_API int dc_b200_model_tensor_names(dc_model* m, const char** names_out, int capacity, int* n_out);
/* Creates a model from a GGUF v2/v3 file: configuration from the metadata ("<arch>.block_count",
 * ".embedding_length", ".attention.head_count[_kv]", ".attention.key_length",
 * ".attention.layer_norm_rms_epsilon", ".rope.freq_base", ".expert_count", ".expert_used_count",
 * ".expert_feed_forward_length", ".feed_forward_length"; the keys core/src/models/model_loader.cpp:2555-2829
 * reads), tensors uploaded with their file bytes (Q4_K / Q6_K matrices, F32 vectors and router).
 * max_seqs / max_ctx are run-time sizes (0: 4 streams, the file's context_length).  The model still needs
 * dc_b200_model_ep_init (expert-parallel runs) and dc_b200_model_finalize. */
DC_B200_API int dc_b200_model_from_gguf(dc_ctx* ctx, const char* path, int max_seqs, int max_ctx, int ep_rank,
                                        int ep_size, dc_model** out_model);
DC_B200_API int dc_b200_model_get_tensor(dc_model* m, const char* name, int* ggml_type, int64_t ne[4], void** dev,
                                         size_t* bytes);
DC_B200_API int dc_b200_model_finalize(dc_model* m);
DC_B200_API size_t dc_b200_model_weight_bytes(dc_model* m);
/* Sequences (KV slots). */
DC_B200_API int dc_b200_seq_alloc(dc_model* m, int* out_seq);
DC_B200_API int dc_b200_seq_free(dc_model* m, int seq);
/* A new sequence sharing src_seq's KV blocks (a common prompt prefilled once, then several continuations);
 * copy-on-write as dc_b200_kv_seq_fork.  dc_b200_model_free_blocks: blocks not referenced by any sequence. */
DC_B200_API int dc_b200_seq_fork(dc_model* m, int src_seq, int* out_seq);
DC_B200_API int dc_b200_model_free_blocks(dc_model* m);
DC_B200_API int dc_b200_seq_len(dc_model* m, int seq);
DC_B200_API int dc_b200_seq_truncate(dc_model* m, int seq, int new_len);
/* Runs n tokens of one sequence through the model in chunks of <= 16 and
 * appends them to its KV cache.  logits_host (NULL or [vocab]) receives the
 * logits of the last token; next_token its greedy pick. */
DC_B200_API int dc_b200_prefill(dc_model* m, int seq, const int32_t* tokens_host, int n, float* logits_host,
                                int32_t* next_token);
/* One decode step for n_seq sequences: token i is appended to sequence seqs[i].
 * Inputs come from host memory and the picks go back to host memory inside the
 * call.  logits_host: NULL or [n_seq, vocab]. */
DC_B200_API int dc_b200_decode_step(dc_model* m, const int32_t* seqs, int n_seq, const int32_t* tokens_host,
                                    int32_t* next_tokens_host, float* logits_host);
/* n_steps greedy decode steps with the tokens fed back on the device; picks
 * [n_steps, n_seq] are copied to the host once at the end.  ms_out (optional)
 * receives the device time of the steps, measured with events on the stream. */
DC_B200_API int dc_b200_decode_run(dc_model* m, const int32_t* seqs, int n_seq, const int32_t* first_tokens_host,
                                   int n_steps, int32_t* out_tokens_host, float* ms_out);
/* Forward over a chunk of n <= 16 tokens of one sequence with logits for every
 * token ([n, vocab], device-resident; copied to logits_host if not NULL): the
 * batched target forward of a speculative verify step. */
DC_B200_API int dc_b200_forward_chunk(dc_model* m, int seq, const int32_t* tokens_host, int n, float* logits_host);
DC_B200_API void* dc_b200_model_logits_dev(dc_model* m);
/* With model option "phase_timing" = 1 the persistent decode kernel accumulates, per phase
 * boundary, the nanoseconds CTA 0 spent since the previous boundary (work and barrier waits
 * separately); this reads the first n accumulators (32 phases; a library built with
 * -DDC_MEGA_SUBMARKS also fills 14 x 160 more: arrival, then release, time of every CTA at
 * the seven barriers of the second layer; n <= 2272). */
DC_B200_API int dc_b200_model_phase_timing(dc_model* m, uint64_t* ns_out, int n);
/* Per-step counters of the last decode_run / decode_step: kernels launched per
 * step, bytes of weights and KV a step must read (algorithmic). */
DC_B200_API int dc_b200_model_step_stats(dc_model* m, int* kernels_per_step, double* weight_bytes_per_step,
                                         double* kv_bytes_per_token_ctx);

/* One eager decode step with CUDA events around every launch: device time,
 * launches and algorithmic bytes per kernel class (dc_b200_kernel_class_name
 * names class i; pass arrays of at least 16 entries).  The mirror of the
 * reference's per-op profile buckets (moe_route_ns, moe_w1w3_ns, moe_w2_ns,
 * paged_attention_ns ..., core/src/llm/moe/exec.cpp:948-960,
 * core/src/llm/attention/paged_exec.cpp:842-861). */
DC_B200_API int dc_b200_model_profile_step(dc_model* m, const int32_t* seqs, int n_seq, const int32_t* tokens_host,
                                           int n_classes, float* ms_out, int* launches_out, double* bytes_out);
DC_B200_API const char* dc_b200_kernel_class_name(int cls);
/* Parity aids.  With model option "capture_layer_inputs" = 1 every step also stores the hidden state that
 * enters each layer (after the previous layer's MoE/FFN output and residual were added) and the one that
 * enters the output norm; read_layer_input copies layer `layer`'s (layer == n_layer: the output norm's) rows
 * of the last step, [n_tokens, hidden] f32.  read_kv copies the fp16 K and V rows [n_tokens, n_kv_head,
 * head_dim] of positions first .. first + n_tokens of a sequence in one layer.  With these a CPU checker
 * can redo any single layer from exactly the inputs the GPU had. */
DC_B200_API int dc_b200_model_read_layer_input(dc_model* m, int layer, int n_tokens, float* x_host);
DC_B200_API int dc_b200_model_read_kv(dc_model* m, int layer, int seq, int first, int n_tokens, void* k_host,
                                      void* v_host);
/* "graphs" 0/1: replay each step shape as a CUDA graph (default 1).
 * "route_mode" 0/1: which router the MoE layers use (see dc_b200_set_option; default 0).
 * "capture_layer_inputs" 0/1: see dc_b200_model_read_layer_input (steps then run without graphs).
 * "test_barrier_polls" n, "test_ep_wait_us" n: shorten the poll limit of the persistent kernel's grid
 * barrier / the time limit of its expert-parallel meeting (0 restores the defaults), so that a test can
 * make a bounded wait run out and check the status that comes back (DC_B200_BACKEND_ERROR; the kernel drains
 * its copies in flight and returns, the context stays usable).  "test_ep_loopback" 1, before finalize, on
 * a fresh model of ep_size 2: the peer's exchange buffer is a second local buffer that nothing signals, so
 * that the expert-parallel wait can be exercised on one GPU (such a model may only run decode steps).
 * "tc_prefill" 0/1 (default 1): prompts of 32 tokens or more run in chunks through the tensor-core matmuls;
 * "prefill_chunk" 32..4096 (default 2048, fixed once a chunk has run); "prefill_attention" 1 (default) chunk
 * attention on the tensor cores, 0 the decode kernels' exact running-maximum chain; "prefix_cache" 0/1.
 * "persistent" 0/1/2: decode steps of MoE models run in one persistent cooperative kernel with grid
 * barriers between phases: 0 never, 1 for one stream (default: with more streams the per-op kernels are
 * faster), 2 for every stream count it supports (1-4). */
DC_B200_API int dc_b200_model_set_option(dc_model* m, const char* name, int value);
/* Prefix-cache counters of a model (option "prefix_cache" = 1 makes dc_b200_prefill and the scheduler use
 * the cache): {lookups, blocks hit, blocks resident, evictions, prompt tokens run through the decoder}. */
DC_B200_API int dc_b200_model_prefix_stats(dc_model* m, uint64_t out[5]);

/* ---- step scheduler ---------------------------------------------------------- */
/* Continuous batching over one model with DenseCore's CPU-path policy: at most max_num_seqs sequences
 * (0: 4, KVCacheConfig::max_num_seqs, core/src/runtime/engine_internal.h:89), one prefill in flight at a
 * time, prompts run in chunks of max_prefill_chunk tokens (0: 512) that alternate with batched decode
 * steps of all running sequences; admission takes over cached prompt prefixes
 * (core/src/runtime/scheduler.cpp:30-85).  Greedy sampling.  eos_token < 0: none. */
typedef struct dc_sched dc_sched;
typedef struct dc_sched_event {
    int32_t request;  /* id from dc_b200_sched_add */
    int32_t token;    /* the token this step produced for the request */
    int32_t finished; /* 0: continues; 1: reached max_new_tokens; 2: end-of-sequence token; 3: failed */
} dc_sched_event;
DC_B200_API int dc_b200_sched_create(dc_model* m, int max_num_seqs, int max_prefill_chunk, int eos_token, dc_sched** out);
DC_B200_API void dc_b200_sched_destroy(dc_sched* s);
DC_B200_API int dc_b200_sched_add(dc_sched* s, const int32_t* prompt, int n_prompt, int max_new_tokens, int* request_id);
/* One unit of GPU work (a prompt chunk or one batched decode step).  events receives at most capacity
 * entries; *n_events is the number produced (0 with nothing pending: idle). */
DC_B200_API int dc_b200_sched_step(dc_sched* s, dc_sched_event* events, int capacity, int* n_events);
DC_B200_API int dc_b200_sched_pending(dc_sched* s);
/* {steps, prompt chunks, decode steps, decoded tokens, largest decode batch, prompt tokens taken from the cache} */
DC_B200_API int dc_b200_sched_stats(dc_sched* s, uint64_t out[6]);

/* ---- expert parallelism over the GPUs of one node ---------------------------- */
/* One process per GPU.  Experts are split into contiguous ranges (rank r owns
 * experts [r*E/G, (r+1)*E/G)); everything else is replicated; the partial MoE
 * outputs are summed with one NCCL all-reduce per layer.  DenseCore's nearest
 * analogue is NUMA-sticky expert placement (core/src/llm/moe/native.cpp:1196,
 * :1506-1567).  Rank 0 makes the 128-byte id, the launcher hands it to every
 * rank, each rank calls model_ep_init before model_finalize.  nccl_path: path
 * of libnccl.so.2, or NULL to use the loader's search path. */
DC_B200_API int dc_b200_ep_unique_id(dc_ctx* ctx, const char* nccl_path, void* id_out_128);
DC_B200_API int dc_b200_model_ep_init(dc_model* m, const char* nccl_path, const void* id_128);
/* Exchange buffers of the persistent decode kernel's expert-parallel path (one process per GPU of one
 * node).  Each rank exports a 64-byte handle of its buffer (cudaIpcGetMemHandle), the launcher hands
 * every rank's handle to every other rank, and each rank imports its ep_size - 1 peers.  With all peers
 * connected, decode steps the persistent kernel serves (option "persistent") run in it: every GPU stores the rows its
 * experts produce straight into all GPUs' buffers over NVLink and the GPUs meet once per layer through
 * flags in each other's memory, so the weighted combine runs in routing order on local memory and the
 * result is bit-identical to a single GPU's (the NCCL all-reduce of the per-op path is only tolerance-
 * equal).  Every rank must then make the same sequence of decode calls.  A rank whose peers do not
 * arrive gives up after two seconds and the call returns DC_B200_BACKEND_ERROR.  Without these calls
 * expert-parallel decode uses the per-op kernels and NCCL.  No counterpart in the reference (its experts
 * share one address space). */
DC_B200_API int dc_b200_model_ep_export(dc_model* m, void* handle_out_64);
DC_B200_API int dc_b200_model_ep_import(dc_model* m, int rank, const void* handle_64);

#ifdef __cplusplus
}
#endif
#endif /* DC_B200_H */
