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
/* 0/1: programmatic dependent launch between consecutive kernels (default 1). */
DC_B200_API int dc_b200_set_option(dc_ctx* ctx, const char* name, int value);

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
/* Parity aid: the exact int32 block sums the kernel forms, I[M][N][K/256] and
 * (Q4_K only, else may be NULL) Mn[M][N][K/256]; these are the quantities the
 * reference's vec_dot kernels agree on bit for bit
 * (core/src/kernels/hwy/hwy_moe_quant.cc:218-246). */
DC_B200_API int dc_b200_mul_mat_block_sums(dc_ctx* ctx, const dc_weight* w, const float* x_host, int M,
                                           int32_t* I_host, int32_t* Mn_host);

#ifdef __cplusplus
}
#endif
#endif /* DC_B200_H */
