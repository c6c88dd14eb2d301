// Small fused kernels around the matmuls of one decoder step: token-embedding
// row dequantisation (ggml get_rows), RMSNorm fused with the Q8_K quantiser,
// per-head Q/K RMSNorm + RoPE + paged-KV write, and the greedy-token epilogue.
#include "dc_common.cuh"
#include "dc_internal.h"

using namespace dc;

// ------------------------------------------------------------ embedding
// x[t, :] = dequantise(row tokens[t] of token_embd).  Q4_K: d*sc*q - dmin*m with
// the nibble order of core/src/kernels/hwy/hwy_moe_quant.cc:202-211; Q6_K:
// d*scale*(q-32) with the order of core/src/llm/matmul/q6_small_batch.h:52-74.
__global__ void __launch_bounds__(256) k_embed(const uint8_t* __restrict__ w, int type, int row_bytes, int H,
                                               const int32_t* __restrict__ tokens, int vocab,
                                               float* __restrict__ x) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int tok = tokens[t];
    if (tok < 0 || tok >= vocab) tok = 0;
    const uint8_t* row = w + (size_t)tok * row_bytes;
    float* o = x + (size_t)t * H;
    for (int e = threadIdx.x; e < H; e += blockDim.x) {
        const int b = e >> 8, i = e & 255;
        float v;
        if (type == DC_TYPE_Q4_K) {
            const uint8_t* blk = row + b * DC_Q4K_BYTES;
            const float d = fp16_bits_to_float(*reinterpret_cast<const uint16_t*>(blk));
            const float dmin = fp16_bits_to_float(*reinterpret_cast<const uint16_t*>(blk + 2));
            const int j = i >> 5, c = i >> 6, l = i & 31;
            const uint8_t* s = blk + 4;
            int sc, m;
            if (j < 4) {
                sc = s[j] & 63;
                m = s[j + 4] & 63;
            } else {
                sc = (s[j + 4] & 15) | ((s[j - 4] >> 6) << 4);
                m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
            }
            const uint8_t qb = blk[16 + 32 * c + l];
            const int q = (j & 1) ? (qb >> 4) : (qb & 15);
            v = __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)m));
        } else if (type == DC_TYPE_Q6_K) {
            const uint8_t* blk = row + b * DC_Q6K_BYTES;
            const float d = fp16_bits_to_float((uint16_t)(blk[208] | (blk[209] << 8)));
            const int jh = i >> 7, qd = (i >> 5) & 3, l = i & 31;
            const uint8_t ql = blk[64 * jh + 32 * (qd & 1) + l];
            const uint8_t qh = blk[128 + 32 * jh + l];
            const int q = (((qd & 2) ? (ql >> 4) : (ql & 15)) | (((qh >> (2 * qd)) & 3) << 4)) - 32;
            const int sc = (int)(int8_t)blk[192 + (i >> 4)];
            v = __fmul_rn(__fmul_rn(d, (float)sc), (float)q);
        } else if (type == DC_TYPE_F16) {
            v = fp16_bits_to_float(reinterpret_cast<const uint16_t*>(row)[e]);
        } else {
            v = reinterpret_cast<const float*>(row)[e];
        }
        o[e] = v;
    }
}

int dc_launch_embed(dc_ctx* ctx, const dc_weight* w, const int32_t* tokens, int T, float* x) {
    k_embed<<<T, 256, 0, ctx->stream>>>(w->dev, w->type, (int)w->row_bytes, (int)w->K, tokens, (int)w->N, x);
    return dc_check_cuda(ctx, cudaGetLastError(), "k_embed");
}

// ------------------------------------------------------ RMSNorm + Q8_K
// One CTA per token.  x (+= add, if given) -> y = x / sqrt(mean(x^2)+eps) * w
// (core/src/llm/graph/decoder.cpp:268), then Q8_K blocks of y
// (core/src/kernels/hwy/hwy_moe_quant.cc:103-144).  xn_out / q8_out optional.
__global__ void __launch_bounds__(256) k_rmsnorm_q8k(float* __restrict__ x, const float* __restrict__ add,
                                                     const float* __restrict__ w, int H, float eps,
                                                     float* __restrict__ xn_out, uint8_t* __restrict__ q8_out) {
    extern __shared__ __align__(16) float sx[];
    __shared__ double red[8];
    pdl_launch_dependents();
    // the norm weights do not depend on the previous kernel: they are fetched (first touch comes from HBM)
    // while this kernel still waits for it
    float wreg[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int e = threadIdx.x + i * 256;
        wreg[i] = e < H ? w[e] : 0.0f;
    }
    pdl_wait();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* xr = x + (size_t)t * H;
    // sum of squares in double, as ggml_rms_norm does: any summation order then
    // rounds to the same float
    double ss = 0.0;
    for (int e = threadIdx.x; e < H; e += blockDim.x) {
        float v = xr[e];
        if (add) {
            v = __fadd_rn(v, add[(size_t)t * H + e]);
            xr[e] = v;
        }
        sx[e] = v;
        ss += (double)v * (double)v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    double tot = 0.0;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float mean = (float)(tot / (double)H);
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int e = threadIdx.x + i * 256;
        if (e < H) {
            const float v = __fmul_rn(__fmul_rn(sx[e], scale), wreg[i]);
            sx[e] = v;
            if (xn_out) xn_out[(size_t)t * H + e] = v;
        }
    }
    for (int e = threadIdx.x + 8 * 256; e < H; e += 256) {
        const float v = __fmul_rn(__fmul_rn(sx[e], scale), w[e]);
        sx[e] = v;
        if (xn_out) xn_out[(size_t)t * H + e] = v;
    }
    __syncthreads();
    if (q8_out) {
        const int nb = H / DC_QK_K;
        for (int b = warp; b < nb; b += 8)
            quantize_block_q8k_warp(sx + b * DC_QK_K, q8_out + ((size_t)t * nb + b) * DC_Q8K_BYTES, lane);
    }
}

int dc_launch_rmsnorm_q8k(dc_ctx* ctx, float* x, const float* add, const float* w, int T, int H, float eps,
                          float* xn_out, uint8_t* q8_out) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(T);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = (size_t)H * 4;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->use_pdl ? 1 : 0;
    return dc_check_cuda(ctx, cudaLaunchKernelEx(&cfg, k_rmsnorm_q8k, x, add, w, H, eps, xn_out, q8_out),
                         "k_rmsnorm_q8k");
}

// ------------------------------------ per-head Q/K norm + RoPE + KV write
// One warp per (token, head) over the fused QKV projection output
// qkv[t] = [n_head*128 | n_kv*128 | n_kv*128].  Q heads: optional RMSNorm over the
// head (core/src/llm/graph/decoder.cpp:1287-1343), RoPE on interleaved pairs
// (core/src/kernels/hwy/hwy_rope.cc:96-104), stored f32 to q_out.  K heads: same,
// then fp16 into slot pos%16 of block table[pos/16]; V heads: fp16 into the V
// arena (core/src/runtime/memory/kv_cache_storage.cpp:146-200, :436).
__global__ void __launch_bounds__(256) k_qknorm_rope_kv(const float* __restrict__ qkv, const float* __restrict__ qn_w,
                                                        const float* __restrict__ kn_w,
                                                        const float* __restrict__ cos_sin, int max_pos,
                                                        const int32_t* __restrict__ positions,
                                                        const int32_t* __restrict__ seq_ids,
                                                        const int32_t* __restrict__ block_tables, int max_blocks,
                                                        __half* __restrict__ k_arena, __half* __restrict__ v_arena,
                                                        int n_head, int n_kv, float eps, int T,
                                                        float* __restrict__ q_out) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int heads = n_head + 2 * n_kv;
    const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (gw >= T * heads) return;
    const int t = gw / heads, h = gw % heads;
    const float4 v4 = reinterpret_cast<const float4*>(qkv + ((size_t)t * heads + h) * 128)[lane];
    float v[4] = {v4.x, v4.y, v4.z, v4.w};
    int pos = positions[t];
    pos = pos < 0 ? 0 : ((max_pos > 0 && pos >= max_pos) ? max_pos - 1 : pos);
    const bool is_q = h < n_head, is_k = !is_q && h < n_head + n_kv;
    if (is_q || is_k) {
        const float* nw = is_q ? qn_w : kn_w;
        if (nw) {
            double ss = (double)v[0] * v[0] + (double)v[1] * v[1] + (double)v[2] * v[2] + (double)v[3] * v[3];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float mean = (float)(ss / 128.0);
            const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
            const float4 w4 = reinterpret_cast<const float4*>(nw)[lane];
            v[0] = __fmul_rn(__fmul_rn(v[0], scale), w4.x);
            v[1] = __fmul_rn(__fmul_rn(v[1], scale), w4.y);
            v[2] = __fmul_rn(__fmul_rn(v[2], scale), w4.z);
            v[3] = __fmul_rn(__fmul_rn(v[3], scale), w4.w);
        }
        if (cos_sin) {
            const float4 cs = reinterpret_cast<const float4*>(cos_sin + (size_t)pos * 128)[lane];
            const float a0 = __fsub_rn(__fmul_rn(v[0], cs.x), __fmul_rn(v[1], cs.y));
            const float a1 = __fadd_rn(__fmul_rn(v[0], cs.y), __fmul_rn(v[1], cs.x));
            const float b0 = __fsub_rn(__fmul_rn(v[2], cs.z), __fmul_rn(v[3], cs.w));
            const float b1 = __fadd_rn(__fmul_rn(v[2], cs.w), __fmul_rn(v[3], cs.z));
            v[0] = a0; v[1] = a1; v[2] = b0; v[3] = b1;
        }
    }
    if (is_q) {
        reinterpret_cast<float4*>(q_out + ((size_t)t * n_head + h) * 128)[lane] = make_float4(v[0], v[1], v[2], v[3]);
    } else {
        const int kvh = is_k ? h - n_head : h - n_head - n_kv;
        const int blk = block_tables[(size_t)seq_ids[t] * max_blocks + pos / DC_KV_BLOCK];
        __half* dst = (is_k ? k_arena : v_arena) +
                      (((size_t)blk * DC_KV_BLOCK + pos % DC_KV_BLOCK) * n_kv + kvh) * 128 + 4 * lane;
        __half2 lo = __halves2half2(__float2half_rn(v[0]), __float2half_rn(v[1]));
        __half2 hi = __halves2half2(__float2half_rn(v[2]), __float2half_rn(v[3]));
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&lo);
        pk.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(dst) = pk;
    }
}

int dc_launch_qknorm_rope_kv(dc_ctx* ctx, const float* qkv, const float* qn_w, const float* kn_w,
                             const float* cos_sin, int max_pos, const int32_t* positions, const int32_t* seq_ids,
                             const int32_t* block_tables, int max_blocks, void* k_arena, void* v_arena, int n_head,
                             int n_kv, float eps, int T, float* q_out) {
    const int warps = T * (n_head + 2 * n_kv);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((warps + 7) / 8);
    cfg.blockDim = dim3(256);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->use_pdl ? 1 : 0;
    return dc_check_cuda(ctx,
                         cudaLaunchKernelEx(&cfg, k_qknorm_rope_kv, qkv, qn_w, kn_w, cos_sin, max_pos, positions,
                                            seq_ids, block_tables, max_blocks, (__half*)k_arena, (__half*)v_arena,
                                            n_head, n_kv, eps, T, q_out),
                         "k_qknorm_rope_kv");
}

// ------------------------------------------------------ greedy epilogue
// Decodes the packed argmax keys (first maximum wins, core/src/sampler/sampler.cpp:42-57)
// into token ids; optionally feeds them back as the next step's inputs and
// advances the positions, and clears the keys for the next step.
__global__ void k_argmax_finish(unsigned long long* __restrict__ keys, int T, int32_t* __restrict__ out_tokens,
                                int32_t* __restrict__ next_tokens, int32_t* __restrict__ positions,
                                int32_t* __restrict__ history, int* __restrict__ history_len, int history_cap) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = threadIdx.x;
    if (t < T) {
        const unsigned long long k = keys[t];
        const int32_t tok = (int32_t)(0xFFFFFFFFu - (uint32_t)(k & 0xFFFFFFFFull));
        out_tokens[t] = tok;
        if (next_tokens) next_tokens[t] = tok;
        if (positions) positions[t] += 1;
        if (history) {
            const int n = *history_len;
            if (n < history_cap) history[(size_t)n * T + t] = tok;
        }
        keys[t] = 0ull;
    }
    __syncthreads();
    if (t == 0 && history) *history_len += 1;
}

int dc_launch_argmax_finish(dc_ctx* ctx, unsigned long long* keys, int T, int32_t* out_tokens, int32_t* next_tokens,
                            int32_t* positions, int32_t* history, int* history_len, int history_cap) {
    k_argmax_finish<<<1, 32, 0, ctx->stream>>>(keys, T, out_tokens, next_tokens, positions, history, history_len,
                                               history_cap);
    return dc_check_cuda(ctx, cudaGetLastError(), "k_argmax_finish");
}

// Plain argmax over rows of logits (used by the verify step and by callers that
// already hold logits).  One CTA per row.
__global__ void __launch_bounds__(1024) k_argmax_rows(const float* __restrict__ logits, int n, int32_t* __restrict__ out) {
    __shared__ unsigned long long red[32];
    const float* v = logits + (size_t)blockIdx.x * n;
    unsigned long long best = 0ull;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float f = v[i];
        uint32_t u = __float_as_uint(f);
        u = (f != f) ? 0u : ((u & 0x80000000u) ? ~u : (u | 0x80000000u));
        const unsigned long long k = ((unsigned long long)u << 32) | (0xFFFFFFFFu - (uint32_t)i);
        best = k > best ? k : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long ok = __shfl_xor_sync(0xffffffffu, best, o);
        best = ok > best ? ok : best;
    }
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x < 32) {
        best = red[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long ok = __shfl_xor_sync(0xffffffffu, best, o);
            best = ok > best ? ok : best;
        }
        if (threadIdx.x == 0) out[blockIdx.x] = (int32_t)(0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFull));
    }
}

int dc_launch_argmax_rows(dc_ctx* ctx, const float* logits, int rows, int n, int32_t* out) {
    k_argmax_rows<<<rows, 1024, 0, ctx->stream>>>(logits, n, out);
    return dc_check_cuda(ctx, cudaGetLastError(), "k_argmax_rows");
}
