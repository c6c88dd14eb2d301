// Speculative-decoding verify/accept on the device.  DenseCore has no
// counterpart (core/src/runtime/engine.cpp:593-645 loads a draft model that
// nothing consumes); this follows the standard draft-verify rule: greedy prefix
// match, or accept draft token t_i iff u_i * q_i[t_i] < p_i[t_i] with residual
// max(0, p - q) resampling, uniforms from a seeded Philox4x32-10 stream.
// Softmax follows the sampler's temperature softmax
// (core/src/sampler/sampler.cpp:235-262) with a fully specified exp and fixed
// summation shapes so that every decision is reproducible bit for bit.
#include "dc_common.cuh"
#include "dc_internal.h"
#include "dc_launch.cuh"

using namespace dc;

#define DET_LANES 1024

// exp for x <= 0: y = x*log2e, r = rint(y), f = y - r, 2^r * P(f); only *, fma, rint.
__device__ __forceinline__ float det_exp(float x) {
    if (x < -87.0f) return 0.0f;
    if (x > 0.0f) x = 0.0f;
    const float y = __fmul_rn(x, 1.4426950408889634f);
    const float r = rintf(y);
    const float f = __fsub_rn(y, r);
    float p = 1.5403530e-4f;
    p = __fmaf_rn(p, f, 1.3333558e-3f);
    p = __fmaf_rn(p, f, 9.6181291e-3f);
    p = __fmaf_rn(p, f, 5.5504109e-2f);
    p = __fmaf_rn(p, f, 2.4022651e-1f);
    p = __fmaf_rn(p, f, 6.9314718e-1f);
    p = __fmaf_rn(p, f, 1.0f);
    return __fmul_rn(p, __int_as_float(((int)r + 127) << 23));
}

// Philox4x32-10 (Salmon et al., SC'11).
__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                              uint32_t k1, uint32_t out[4]) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t h0 = __umulhi(0xD2511F53u, c0), l0 = 0xD2511F53u * c0;
        const uint32_t h1 = __umulhi(0xCD9E8D57u, c2), l1 = 0xCD9E8D57u * c2;
        const uint32_t n0 = h1 ^ c1 ^ k0, n2 = h0 ^ c3 ^ k1;
        c0 = n0; c1 = l1; c2 = n2; c3 = l0;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// Uniforms of one verify step: counter (step, i/4, 0, 0), key = seed; u = (r>>8) * 2^-24.
__global__ void k_verify_uniforms(unsigned long long seed, uint32_t step, int n, float* __restrict__ u) {
    const int i = threadIdx.x;
    if (i >= n) return;
    uint32_t o[4];
    philox4x32_10(step, (uint32_t)(i / 4), 0u, 0u, (uint32_t)seed, (uint32_t)(seed >> 32), o);
    u[i] = (float)(o[i & 3] >> 8) * (1.0f / 16777216.0f);
}

// One CTA (1024 threads) per row: p = softmax(logits / T).  Lane j sums elements
// j, j+1024, ... in index order; the 1024 lane sums are added by a pairwise tree
// (stride 512, 256, ... 1).
__global__ void __launch_bounds__(DET_LANES) k_det_softmax(const float* __restrict__ logits, int n, float inv_t,
                                                           float* __restrict__ probs) {
    __shared__ float red[DET_LANES];
    const float* l = logits + (size_t)blockIdx.x * n;
    float* p = probs + (size_t)blockIdx.x * n;
    const int j = threadIdx.x;
    float mx = -INFINITY;
    for (int i = j; i < n; i += DET_LANES) mx = fmaxf(mx, __fmul_rn(l[i], inv_t));
    red[j] = mx;
    __syncthreads();
    for (int st = DET_LANES / 2; st > 0; st >>= 1) {
        if (j < st) red[j] = fmaxf(red[j], red[j + st]);
        __syncthreads();
    }
    mx = red[0];
    __syncthreads();
    float s = 0.0f;
    for (int i = j; i < n; i += DET_LANES) {
        const float e = det_exp(__fsub_rn(__fmul_rn(l[i], inv_t), mx));
        p[i] = e;
        s = __fadd_rn(s, e);
    }
    red[j] = s;
    __syncthreads();
    for (int st = DET_LANES / 2; st > 0; st >>= 1) {
        if (j < st) red[j] = __fadd_rn(red[j], red[j + st]);
        __syncthreads();
    }
    const float inv = __fdiv_rn(1.0f, red[0]);
    for (int i = j; i < n; i += DET_LANES) p[i] = __fmul_rn(p[i], inv);
}

#define CDF_MAX_RUNS 8192  // vocab <= 262144

// Inverse CDF in index order over w[i] = residual ? max(0, p[i]-q[i]) : p[i].
// Fixed sum shapes: run = 32 consecutive elements added in order from 0; chunk =
// 32 run sums added in order; total = chunk sums added in order.  Returns -1 if
// total <= 0.  Called by the whole CTA; result valid in thread 0.
__device__ int det_inverse_cdf_cta(const float* __restrict__ p, const float* __restrict__ q, int n, float u,
                                   float* runsum, float* chunksum) {
    const int n_runs = (n + 31) / 32, n_chunks = (n_runs + 31) / 32;
    for (int r = threadIdx.x; r < n_runs; r += blockDim.x) {
        float s = 0.0f;
        const int hi = min(n, 32 * r + 32);
        for (int i = 32 * r; i < hi; ++i) {
            float w = p[i];
            if (q) w = fmaxf(__fsub_rn(w, q[i]), 0.0f);
            s = __fadd_rn(s, w);
        }
        runsum[r] = s;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < n_chunks; c += blockDim.x) {
        float s = 0.0f;
        const int hi = min(n_runs, 32 * c + 32);
        for (int r = 32 * c; r < hi; ++r) s = __fadd_rn(s, runsum[r]);
        chunksum[c] = s;
    }
    __syncthreads();
    int result = -1;
    if (threadIdx.x == 0) {
        float total = 0.0f;
        for (int c = 0; c < n_chunks; ++c) total = __fadd_rn(total, chunksum[c]);
        if (total > 0.0f) {
            const float target = __fmul_rn(u, total);
            float base = 0.0f;
            for (int c = 0; c < n_chunks && result < 0; ++c) {
                const float cs = chunksum[c];
                if (!(__fadd_rn(base, cs) > target)) {
                    base = __fadd_rn(base, cs);
                    continue;
                }
                float cbase = base;
                const int rhi = min(n_runs, 32 * c + 32);
                for (int r = 32 * c; r < rhi && result < 0; ++r) {
                    const float rs = runsum[r];
                    if (__fadd_rn(cbase, rs) > target) {
                        float prefix = 0.0f;
                        const int hi = min(n, 32 * r + 32);
                        for (int i = 32 * r; i < hi; ++i) {
                            float w = p[i];
                            if (q) w = fmaxf(__fsub_rn(w, q[i]), 0.0f);
                            prefix = __fadd_rn(prefix, w);
                            if (__fadd_rn(cbase, prefix) > target) {
                                result = i;
                                break;
                            }
                        }
                    }
                    cbase = __fadd_rn(cbase, rs);
                }
                base = __fadd_rn(base, cs);
            }
            if (result < 0) {  // rounding left nothing above target: last positive weight
                for (int i = n - 1; i >= 0; --i) {
                    float w = p[i];
                    if (q) w = fmaxf(__fsub_rn(w, q[i]), 0.0f);
                    if (w > 0.0f) {
                        result = i;
                        break;
                    }
                }
            }
        }
    }
    return result;
}

// mode 0 (greedy): argmax_ids[gamma+1] precomputed.  mode 1 (stochastic):
// probs[gamma+1][vocab] precomputed by k_det_softmax.  result[0] = n_accepted,
// result[1] = next token.
__global__ void __launch_bounds__(1024) k_verify_accept(int mode, int gamma, int vocab,
                                                        const int32_t* __restrict__ draft_tokens,
                                                        const int32_t* __restrict__ argmax_ids,
                                                        const float* __restrict__ probs,
                                                        const float* __restrict__ draft_probs,
                                                        const float* __restrict__ u, int32_t* __restrict__ result) {
    __shared__ float runsum[CDF_MAX_RUNS];
    __shared__ float chunksum[CDF_MAX_RUNS / 32];
    __shared__ int s_n, s_tok;
    if (mode == 0) {
        if (threadIdx.x == 0) {
            int n = 0;
            while (n < gamma && argmax_ids[n] == draft_tokens[n]) ++n;
            result[0] = n;
            result[1] = argmax_ids[n];
        }
        return;
    }
    if (threadIdx.x == 0) {
        int n = 0;
        for (; n < gamma; ++n) {
            const int t = draft_tokens[n];
            const float q = draft_probs[(size_t)n * vocab + t], p = probs[(size_t)n * vocab + t];
            if (!(__fmul_rn(u[n], q) < p)) break;
        }
        s_n = n;
    }
    __syncthreads();
    const int n = s_n;
    const float* p = probs + (size_t)n * vocab;
    const float* q = n < gamma ? draft_probs + (size_t)n * vocab : nullptr;
    int tok = det_inverse_cdf_cta(p, q, vocab, u[gamma], runsum, chunksum);
    __syncthreads();
    if (q) {
        if (threadIdx.x == 0) s_tok = tok;
        __syncthreads();
        if (s_tok < 0) {  // p == q everywhere: sample from p itself
            tok = det_inverse_cdf_cta(p, nullptr, vocab, u[gamma], runsum, chunksum);
        }
    }
    if (threadIdx.x == 0) {
        result[0] = n;
        result[1] = tok;
    }
}

int dc_launch_verify(dc_ctx* ctx, int mode, int gamma, int vocab, const float* target_logits,
                     const int32_t* draft_tokens, const float* draft_probs, const float* u, float temperature,
                     int32_t* argmax_scratch, float* probs_scratch, int32_t* result) {
    if (vocab > CDF_MAX_RUNS * 32) return dc_fail(ctx, DC_B200_UNSUPPORTED, "verify: vocab %d too large", vocab);
    if (mode == 0) {
        int st = dc_launch_argmax_rows(ctx, target_logits, gamma + 1, vocab, argmax_scratch);
        if (st != DC_B200_OK) return st;
    } else {
        if (!(temperature > 0.0f)) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "verify: temperature must be > 0");
        k_det_softmax<<<gamma + 1, DET_LANES, 0, ctx->stream>>>(target_logits, vocab, 1.0f / temperature, probs_scratch);
        int st = dc_check_cuda(ctx, cudaGetLastError(), "k_det_softmax");
        if (st != DC_B200_OK) return st;
    }
    k_verify_accept<<<1, 1024, 0, ctx->stream>>>(mode, gamma, vocab, draft_tokens, argmax_scratch, probs_scratch,
                                                 draft_probs, u, result);
    return dc_check_cuda(ctx, cudaGetLastError(), "k_verify_accept");
}

// One draw from probabilities p[n] (not necessarily normalised) by the same fixed-shape inverse CDF the
// verify step uses for its resampling; *u is the uniform.
__global__ void __launch_bounds__(1024) k_sample_cdf(const float* __restrict__ p, int n, const float* __restrict__ u,
                                                     int32_t* __restrict__ result) {
    __shared__ float runsum[CDF_MAX_RUNS];
    __shared__ float chunksum[CDF_MAX_RUNS / 32];
    const int tok = det_inverse_cdf_cta(p, nullptr, n, *u, runsum, chunksum);
    if (threadIdx.x == 0) *result = tok;
}

int dc_launch_sample(dc_ctx* ctx, const float* logits, int n, float temperature, const float* u_dev, float* probs,
                     int32_t* result) {
    if (n > CDF_MAX_RUNS * 32) return dc_fail(ctx, DC_B200_UNSUPPORTED, "sample: vocab %d too large", n);
    if (!(temperature > 0.0f)) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "sample: temperature must be > 0");
    k_det_softmax<<<1, DET_LANES, 0, ctx->stream>>>(logits, n, 1.0f / temperature, probs);
    int st = dc_check_cuda(ctx, cudaGetLastError(), "k_det_softmax");
    if (st != DC_B200_OK) return st;
    k_sample_cdf<<<1, 1024, 0, ctx->stream>>>(probs, n, u_dev, result);
    return dc_check_cuda(ctx, cudaGetLastError(), "k_sample_cdf");
}

int dc_launch_verify_uniforms(dc_ctx* ctx, unsigned long long seed, uint32_t step, int n, float* u) {
    k_verify_uniforms<<<1, 32, 0, ctx->stream>>>(seed, step, n, u);
    return dc_check_cuda(ctx, cudaGetLastError(), "k_verify_uniforms");
}

int dc_launch_det_softmax(dc_ctx* ctx, const float* logits, int rows, int n, float temperature, float* probs) {
    k_det_softmax<<<rows, DET_LANES, 0, ctx->stream>>>(logits, n, 1.0f / temperature, probs);
    return dc_check_cuda(ctx, cudaGetLastError(), "k_det_softmax");
}
