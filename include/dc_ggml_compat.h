/* ggml-shaped custom-op callbacks over the dc_b200 C ABI.
 *
 * DenseCore runs its hot ops as GGML_OP_CUSTOM / ggml_map_custom2 nodes whose
 * callbacks receive (dst, ith, nth, userdata) and read their operands from
 * dst->src[] (core/src/llm/matmul/graph_ops.cpp:143-310).  The three callbacks
 * below have those signatures and argument layouts and run the op on the GPU, so
 * that a graph builder only swaps the function pointer and the userdata.
 *
 * Thread contract: the ggml executor calls a callback from nth threads; here the
 * thread with ith == 0 does all the work and returns after the result is in
 * dst->data; the other threads return at once (cb_moe_forward does the same,
 * core/src/llm/moe/exec.cpp:829-831).
 *
 * Failure contract: on a bad node (null data, wrong type, shapes that do not
 * agree) thread 0 zero-fills dst->data, one "CRITICAL" line goes to stderr
 * (core/src/llm/matmul/gemv_exec.cpp:119,138, core/src/llm/moe/exec.cpp:404-414,
 * core/src/llm/attention/paged_exec.cpp:358-412) and the per-process counter
 * dc_b200_shim_fail_closed_count() goes up by one.
 *
 * Inside DenseCore, include ggml.h before this header; without it (tests, other
 * hosts) the few ggml_tensor fields the callbacks read are declared here with
 * ggml's own field names.  That stand-in is NOT layout-compatible with ggml's
 * struct: a program uses one or the other. */
#ifndef DC_GGML_COMPAT_H
#define DC_GGML_COMPAT_H

#include <stddef.h>
#include <stdint.h>

#include "dc_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

#ifndef GGML_FILE_MAGIC /* ggml.h not included */
#define DC_GGML_STANDIN 1
#define GGML_MAX_DIMS 4
#define GGML_MAX_SRC 10
#define GGML_MAX_OP_PARAMS 64
enum ggml_type { GGML_TYPE_F32 = 0, GGML_TYPE_F16 = 1, GGML_TYPE_Q4_K = 12, GGML_TYPE_Q6_K = 14, GGML_TYPE_Q8_K = 15 };
struct ggml_tensor {
    enum ggml_type type;
    int64_t ne[GGML_MAX_DIMS]; /* elements per dimension, ne[0] innermost */
    size_t nb[GGML_MAX_DIMS];  /* stride in bytes per dimension */
    int32_t op_params[GGML_MAX_OP_PARAMS / sizeof(int32_t)];
    struct ggml_tensor* src[GGML_MAX_SRC];
    void* data;
    char name[64];
};
#endif

/* userdata of cb_gemv_b200: stands in for GemvUserData / GemvBatchedUserData
 * (core/src/llm/matmul/userdata.h:17-85).  weight may be left NULL: the first
 * call uploads dst->src[1]->data and keeps the handle here. */
typedef struct dc_b200_gemv_userdata {
    dc_ctx* ctx;
    dc_weight* weight;
} dc_b200_gemv_userdata;

/* userdata of cb_moe_forward_b200: stands in for MoEUserData
 * (core/src/llm/runtime/inference_types_internal.h:60-72).  k = experts per
 * token; the three expert tensors are uploaded once by the model loader. */
typedef struct dc_b200_moe_userdata {
    dc_ctx* ctx;
    const dc_weight* gate_exps; /* [hidden, ffn, n_expert] */
    const dc_weight* up_exps;   /* [hidden, ffn, n_expert] */
    const dc_weight* down_exps; /* [ffn, hidden, n_expert] */
    int k;
    float routed_scaling_factor; /* 0 or 1: none */
} dc_b200_moe_userdata;

/* userdata of cb_paged_attention_decode_b200: stands in for
 * PagedAttentionUserData plus the batch fields the callback reads from the
 * current BatchSpec (seq_id, pos; core/src/llm/attention/paged_exec.cpp:412-470). */
typedef struct dc_b200_attn_userdata {
    dc_ctx* ctx;
    dc_kv_cache* cache;
    int layer;
    int n_head, n_head_kv, head_dim;
    float scale;            /* multiplies q.k; 0: 1/sqrt(head_dim) */
    const int32_t* seq_id;  /* [q_tokens] cache sequence of every token */
    const int32_t* pos;     /* [q_tokens] position of every token */
} dc_b200_attn_userdata;

/* cb_gemv_custom and cb_gemv_batched_custom (core/src/llm/matmul/userdata.h:85-86):
 * dst F32 [K_out, M]; dst->src[0] = input F32 [N_in, M]; dst->src[1] = weight
 * [N_in, K_out] of type Q4_K or Q6_K. */
DC_B200_API void cb_gemv_b200(struct ggml_tensor* dst, int ith, int nth, void* userdata);
/* cb_moe_forward (core/src/llm/moe/exec.cpp:813; node built by ggml_map_custom2 at
 * core/src/llm/graph/decoder.cpp:2404): dst F32 [hidden, T]; src0 = routed input
 * F32 [hidden, T]; src1 = router logits F32 [n_expert, T]. */
DC_B200_API void cb_moe_forward_b200(struct ggml_tensor* dst, const struct ggml_tensor* src0,
                                     const struct ggml_tensor* src1, int ith, int nth, void* userdata);
/* cb_paged_attention_decode (core/src/llm/attention/paged_exec.cpp:343): dst F32
 * [head_dim, n_head, T]; dst->src[0..2] = q [head_dim, n_head, T], k and v
 * [head_dim, n_head_kv, T], all F32 and dense. */
DC_B200_API void cb_paged_attention_decode_b200(struct ggml_tensor* dst, int ith, int nth, void* userdata);

/* Number of fail-closed returns of the three callbacks in this process. */
DC_B200_API uint64_t dc_b200_shim_fail_closed_count(void);

#ifdef __cplusplus
}
#endif
#endif
