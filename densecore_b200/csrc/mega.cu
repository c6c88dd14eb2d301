// Persistent decode kernel: one cooperative launch runs whole decode steps of
// the MoE decoder for 1..4 streams.  One CTA per SM stays resident; the phases
// of a layer (norm + QKV, attention scores, attention P.V, output projection,
// norm + router, top-k + gate/up, down) are separated by grid-wide barriers
// instead of kernel launches, the hidden state is normalised and quantised to
// Q8_K in shared memory by every CTA instead of round-tripping through global
// memory, and every warp asks for the next phase's weight rows (bulk async
// copies into its shared-memory ring) before it arrives at the barrier, so the
// HBM stream keeps running while the barrier and the small phases execute.
//
// The arithmetic is the same code as the stand-alone kernels (dc_stream.cuh,
// dc_common.cuh): same Q8_K quantiser, same block decoders, same reference
// running-maximum chain in attention.  Every wait is bounded: a barrier or
// mbarrier that does not complete within its poll limit records an error code
// and the kernel carries on to its end.
#include <cooperative_groups.h>

#include "dc_common.cuh"
#include "dc_internal.h"
#include "dc_mega.h"
#include "dc_model.h"
#include "dc_stream.cuh"

using namespace dc;

#define MG_BAR_LIMIT (1u << 21)
#define DC_ERR_GRID_BARRIER 2

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// All CTAs of the (co-resident) grid meet here.  counter only grows during a
// launch; the host zeroes it before the launch.
__device__ __forceinline__ void grid_barrier(const MegaParams& p, unsigned& epoch) {
    __syncthreads();
    ++epoch;
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(p.bar_counter, 1u);
        const unsigned target = epoch * gridDim.x;
        unsigned polls = 0;
        while (ld_acquire_u32(p.bar_counter) < target) {
            if (++polls > MG_BAR_LIMIT) {
                atomicExch(p.err, DC_ERR_GRID_BARRIER);
                break;
            }
            __nanosleep(32);
        }
        __threadfence();
    }
    __syncthreads();
}

// ---- token embedding element (same decode as k_embed) ----
__device__ __forceinline__ float embed_elem(const uint8_t* row, int type, int e) {
    const int b = e >> 8, i = e & 255;
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
        return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)m));
    }
    if (type == DC_TYPE_Q6_K) {
        const uint8_t* blk = row + b * DC_Q6K_BYTES;
        const float d = fp16_bits_to_float((uint16_t)(blk[208] | (blk[209] << 8)));
        const int jh = i >> 7, qd = (i >> 5) & 3, l = i & 31;
        const uint8_t ql = blk[64 * jh + 32 * (qd & 1) + l];
        const uint8_t qh = blk[128 + 32 * jh + l];
        const int q = (((qd & 2) ? (ql >> 4) : (ql & 15)) | (((qh >> (2 * qd)) & 3) << 4)) - 32;
        const int sc = (int)(int8_t)blk[192 + (i >> 4)];
        return __fmul_rn(__fmul_rn(d, (float)sc), (float)q);
    }
    if (type == DC_TYPE_F16) return fp16_bits_to_float(reinterpret_cast<const uint16_t*>(row)[e]);
    return reinterpret_cast<const float*>(row)[e];
}

// Shared state of one CTA that outlives a phase.
struct MegaShared {
    int32_t ids[MG_MAX_T * MG_MAX_K];      // routing of the current layer (kept for the combine in the next P0)
    float w[MG_MAX_T * MG_MAX_K];
    int32_t uexp[MG_MAX_E];
    int32_t uoff[MG_MAX_E + 1];
    int32_t uassign[MG_MAX_T * MG_MAX_K];
    int n_active;
    int have_moe;                          // a MoE output is pending (added when x is next assembled)
    double red[MG_WARPS][MG_MAX_T];
    float scale[MG_MAX_T];
    int wsum_a[MG_WARPS], wsum_c[MG_WARPS];
    // attention
    float sq[8][128];
    float p[8][DC_KV_BLOCK];
    float m[8], d[8], alpha[8], suffix[8];
    int last;
};

// x <- (layer 0: embedding rows) or (x_in + pending MoE combine), into shared xs[T][H];
// this CTA also writes its interleaved share of x to x_out.  The combine adds the
// assignments of a token one at a time in routing order into a zeroed sum
// (core/src/backend/cpu_backend_moe_ops.cpp:1578-1597), then the residual add.
__device__ __forceinline__ void assemble_x(const MegaParams& p, MegaShared& sh, float* xs, const float* x_in,
                                           float* x_out, bool first_layer) {
    const int H = p.H, T = p.T;
    for (int e = threadIdx.x; e < T * H; e += MG_THREADS) {
        const int t = e / H, dd = e - t * H;
        float v;
        if (first_layer) {
            int tok = __ldcg(p.tokens + t);
            if (tok < 0 || tok >= p.vocab) tok = 0;
            v = embed_elem(p.tok_embd + (size_t)tok * p.embd_row_bytes, p.embd_type, dd);
        } else {
            v = __ldcg(x_in + e);
            if (sh.have_moe) {
                float sum = 0.0f;
                for (int k = 0; k < p.top_k; ++k) {
                    const int a = t * p.top_k + k;
                    const float w = sh.w[a];
                    if (w == 0.0f) continue;
                    sum = __fadd_rn(sum, __fmul_rn(w, __ldcg(p.dn + (size_t)a * H + dd)));
                }
                v = __fadd_rn(v, sum);
            }
        }
        xs[e] = v;
        if (x_out && (e % (int)gridDim.x) == (int)blockIdx.x) x_out[e] = v;
    }
    __syncthreads();
}

// RMSNorm of xs[T][H] in place (xs becomes the normed rows) and Q8_K blocks into act
// (core/src/llm/graph/decoder.cpp:268; core/src/kernels/hwy/hwy_moe_quant.cc:103-144).
__device__ __forceinline__ void norm_quant(const MegaParams& p, MegaShared& sh, float* xs, const float* w,
                                           const ActSmem& act) {
    const int H = p.H, T = p.T, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    double ss[MG_MAX_T];
#pragma unroll
    for (int t = 0; t < MG_MAX_T; ++t) ss[t] = 0.0;
    for (int e = threadIdx.x; e < H; e += MG_THREADS) {
#pragma unroll
        for (int t = 0; t < MG_MAX_T; ++t)
            if (t < T) {
                const float v = xs[t * H + e];
                ss[t] += (double)v * (double)v;
            }
    }
#pragma unroll
    for (int t = 0; t < MG_MAX_T; ++t) {
        if (t < T) {
            double s = ss[t];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (lane == 0) sh.red[warp][t] = s;
        }
    }
    __syncthreads();
    if (threadIdx.x < T) {
        double tot = 0.0;
        for (int i = 0; i < MG_WARPS; ++i) tot += sh.red[i][threadIdx.x];
        const float mean = (float)(tot / (double)H);
        sh.scale[threadIdx.x] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, p.eps)));
    }
    __syncthreads();
    for (int e = threadIdx.x; e < T * H; e += MG_THREADS) {
        const int t = e / H, dd = e - t * H;
        xs[e] = __fmul_rn(__fmul_rn(xs[e], sh.scale[t]), w[dd]);
    }
    __syncthreads();
    const int nb = H / DC_QK_K;
    for (int i = warp; i < T * nb; i += MG_WARPS) {
        const int t = i / nb, b = i - t * nb;
        const float4 a = reinterpret_cast<const float4*>(xs + t * H + b * DC_QK_K)[2 * lane];
        const float4 c = reinterpret_cast<const float4*>(xs + t * H + b * DC_QK_K)[2 * lane + 1];
        const float v[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
        quantize_block_q8k_to_act(v, act, t, b, lane);
    }
    __syncthreads();
}

// ------------------------------------------------------------ attention
struct AttnItem {
    bool valid;
    int t, kvh, split, pos, ctx_len, n_blk, b0, b1;
    const int32_t* table;
};

__device__ __forceinline__ AttnItem attn_item(const MegaParams& p) {
    AttnItem it;
    const int items = p.T * p.n_kv * p.nsplit, item = blockIdx.x;
    it.valid = item < items;
    const int i = it.valid ? item : 0;
    it.t = i / (p.n_kv * p.nsplit);
    it.kvh = (i / p.nsplit) % p.n_kv;
    it.split = i % p.nsplit;
    it.pos = __ldcg(p.positions + it.t);
    it.ctx_len = it.pos + 1;
    it.n_blk = (it.ctx_len + DC_KV_BLOCK - 1) / DC_KV_BLOCK;
    const int bps = (it.n_blk + p.nsplit - 1) / p.nsplit;
    it.b0 = min(it.n_blk, it.split * bps);
    it.b1 = min(it.n_blk, it.b0 + bps);
    it.table = p.block_tables + (size_t)p.seq_ids[it.t] * p.max_blocks;
    return it;
}

// One warp: RMSNorm over a 128-wide head (optional), RoPE on interleaved pairs.
// Same steps as k_qknorm_rope_kv (core/src/llm/graph/decoder.cpp:1287-1343,
// core/src/kernels/hwy/hwy_rope.cc:96-104).
__device__ __forceinline__ void head_norm_rope(float (&v)[4], const float* nw, const float* cos_sin_row, float eps,
                                               int lane, bool rope) {
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
    if (rope) {
        const float4 cs = reinterpret_cast<const float4*>(cos_sin_row)[lane];
        const float a0 = __fsub_rn(__fmul_rn(v[0], cs.x), __fmul_rn(v[1], cs.y));
        const float a1 = __fadd_rn(__fmul_rn(v[0], cs.y), __fmul_rn(v[1], cs.x));
        const float b0 = __fsub_rn(__fmul_rn(v[2], cs.z), __fmul_rn(v[3], cs.w));
        const float b1 = __fadd_rn(__fmul_rn(v[2], cs.w), __fmul_rn(v[3], cs.z));
        v[0] = a0; v[1] = a1; v[2] = b0; v[3] = b1;
    }
}

// Phase 1: Q/K norm + RoPE, K/V of the new token into the paged cache (by the run
// that owns its block), scores of this run into shared memory, block maxima to global.
__device__ __forceinline__ void attn_scores_phase(const MegaParams& p, const MegaLayer& L, MegaShared& sh,
                                                  float* s_sc) {
    const AttnItem it = attn_item(p);
    if (!it.valid) return;
    const int g = p.n_head / p.n_kv, heads = p.n_head + 2 * p.n_kv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = min(it.pos, p.max_pos - 1);
    const float* cs_row = p.cos_sin + (size_t)pos * 128;
    const float* qkv_t = p.qkv + (size_t)it.t * heads * 128;
    const bool owner = (it.pos / DC_KV_BLOCK) >= it.b0 && (it.pos / DC_KV_BLOCK) < it.b1;
    if (warp < g) {
        const float4 v4 = __ldcg(reinterpret_cast<const float4*>(qkv_t + (size_t)(it.kvh * g + warp) * 128) + lane);
        float v[4] = {v4.x, v4.y, v4.z, v4.w};
        head_norm_rope(v, L.q_norm, cs_row, p.eps, lane, true);
        reinterpret_cast<float4*>(&sh.sq[warp][0])[lane] = make_float4(v[0], v[1], v[2], v[3]);
    } else if (owner && (warp == g || warp == g + 1)) {
        const bool is_k = warp == g;
        const int hh = is_k ? p.n_head + it.kvh : p.n_head + p.n_kv + it.kvh;
        const float4 v4 = __ldcg(reinterpret_cast<const float4*>(qkv_t + (size_t)hh * 128) + lane);
        float v[4] = {v4.x, v4.y, v4.z, v4.w};
        if (is_k) head_norm_rope(v, L.k_norm, cs_row, p.eps, lane, true);
        const int blk = it.table[it.pos / DC_KV_BLOCK];
        __half* dst = (is_k ? L.k_arena : L.v_arena) +
                      (((size_t)blk * DC_KV_BLOCK + it.pos % DC_KV_BLOCK) * p.n_kv + it.kvh) * 128 + 4 * lane;
        __half2 lo = __halves2half2(__float2half_rn(v[0]), __float2half_rn(v[1]));
        __half2 hi = __halves2half2(__float2half_rn(v[2]), __float2half_rn(v[3]));
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&lo);
        pk.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(dst) = pk;
    }
    __syncthreads();   // sq ready; this CTA's K/V stores are visible to its own loads
    const int n_keys = (it.b1 - it.b0) * DC_KV_BLOCK;
    for (int k0 = 0; k0 < n_keys; k0 += MG_WARPS * 8) {
        const int kk = k0 + warp * 8 + (lane >> 2), sub = lane & 3;
        const int blk = it.b0 + kk / DC_KV_BLOCK, kpos = blk * DC_KV_BLOCK + kk % DC_KV_BLOCK;
        const bool valid = kk < n_keys && kpos < it.ctx_len;
        float kf[32];
        if (valid) {
            const int pb = it.table[blk];
            const uint4* kp = reinterpret_cast<const uint4*>(
                L.k_arena + (((size_t)pb * DC_KV_BLOCK + kk % DC_KV_BLOCK) * p.n_kv + it.kvh) * 128 + sub * 32);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 u = __ldcg(kp + i);
                const __half2* h2 = reinterpret_cast<const __half2*>(&u);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __half22float2(h2[j]);
                    kf[i * 8 + 2 * j] = f.x;
                    kf[i * 8 + 2 * j + 1] = f.y;
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) kf[i] = 0.0f;
        }
        for (int h = 0; h < g; ++h) {
            float dot = 0.0f;
            const float4* qp = reinterpret_cast<const float4*>(&sh.sq[h][sub * 32]);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float4 qq = qp[i];
                dot = fmaf(qq.x, kf[4 * i], dot);
                dot = fmaf(qq.y, kf[4 * i + 1], dot);
                dot = fmaf(qq.z, kf[4 * i + 2], dot);
                dot = fmaf(qq.w, kf[4 * i + 3], dot);
            }
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            if (sub == 0 && kk < n_keys) s_sc[h * p.s_keys + kk] = valid ? __fmul_rn(dot, p.scale) : -INFINITY;
        }
    }
    __syncthreads();
    const int nb_run = it.b1 - it.b0;
    for (int i = threadIdx.x; i < g * nb_run; i += MG_THREADS) {
        const int h = i / nb_run, bb = i - h * nb_run;
        float mx = -1e30f;
#pragma unroll
        for (int k = 0; k < DC_KV_BLOCK; ++k) mx = fmaxf(mx, s_sc[h * p.s_keys + bb * DC_KV_BLOCK + k]);
        p.bmax[((size_t)it.t * p.n_head + it.kvh * g + h) * p.max_blocks + it.b0 + bb] = mx;
    }
}

// Phase 2: the reference's running-maximum chain from all block maxima, this run's
// blocks accumulated as the reference walks them, partial scaled by the alphas of
// all later blocks; the last run of a (token, kv head) sums the partials and emits
// the Q8_K blocks of the attention output (hwy_paged_attention.cc:428-629).
__device__ __forceinline__ void attn_pv_phase(const MegaParams& p, const MegaLayer& L, MegaShared& sh,
                                              const float* s_sc) {
    const AttnItem it = attn_item(p);
    if (!it.valid) return;
    const int g = p.n_head / p.n_kv;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int h = warp; h < g; h += MG_WARPS) {
        const float* bm = p.bmax + ((size_t)it.t * p.n_head + it.kvh * g + h) * p.max_blocks;
        float m_start = -1e30f;
        for (int b = lane; b < it.b0; b += 32) m_start = fmaxf(m_start, __ldcg(bm + b));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m_start = fmaxf(m_start, __shfl_xor_sync(0xffffffffu, m_start, o));
        float m_run = m_start;
        for (int b = it.b0 + lane; b < it.b1; b += 32) m_run = fmaxf(m_run, __ldcg(bm + b));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m_run = fmaxf(m_run, __shfl_xor_sync(0xffffffffu, m_run, o));
        float carry = m_run, suffix = 1.0f;
        for (int c0 = it.b1; c0 < it.n_blk; c0 += 32) {
            const int c = c0 + lane;
            const float v = c < it.n_blk ? __ldcg(bm + c) : -1e30f;
            float incl = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float u = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl = fmaxf(incl, u);
            }
            float excl = __shfl_up_sync(0xffffffffu, incl, 1);
            if (lane == 0) excl = -1e30f;
            const float m_prev = fmaxf(carry, excl), m_new = fmaxf(carry, incl);
            float a = c < it.n_blk ? fast_exp_fma(m_prev - m_new) : 1.0f;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) a *= __shfl_xor_sync(0xffffffffu, a, o);
            suffix *= a;
            carry = fmaxf(carry, __shfl_sync(0xffffffffu, incl, 31));
        }
        if (lane == 0) {
            sh.suffix[h] = suffix;
            sh.m[h] = m_start;
            sh.d[h] = 0.0f;
        }
    }
    // thread -> (dim, two heads): heads hq and hq + 4
    const int dim = tid & 127, hq = tid >> 7;
    float acc0 = 0.0f, acc1 = 0.0f;
    __syncthreads();
    for (int blk = it.b0; blk < it.b1; ++blk) {
        const int pb = it.table[blk];
        const int nk = min(DC_KV_BLOCK, it.ctx_len - blk * DC_KV_BLOCK);
        if (tid < 128) {
            const int h = tid >> 4, key = tid & 15;
            float s = -INFINITY;
            if (h < g && key < nk) s = s_sc[h * p.s_keys + (blk - it.b0) * DC_KV_BLOCK + key];
            float mx = fmaxf(s, -1e30f);
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float m_prev = h < g ? sh.m[h] : -1e30f;
            const float m_new = fmaxf(m_prev, mx);
            const float pr = (s == -INFINITY) ? 0.0f : fast_exp_fma(s - m_new);
            float ps = pr;
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
            if (h < g) sh.p[h][key] = pr;
            __syncwarp();
            if (h < g && key == 0) {
                const float alpha = fast_exp_fma(m_prev - m_new);
                sh.alpha[h] = alpha;
                sh.d[h] = sh.d[h] * alpha + ps;
                sh.m[h] = m_new;
            }
        }
        __syncthreads();
        const bool h0 = hq < g, h1 = hq + 4 < g;
        if (h0 && sh.alpha[hq] != 1.0f) acc0 *= sh.alpha[hq];
        if (h1 && sh.alpha[hq + 4] != 1.0f) acc1 *= sh.alpha[hq + 4];
        const __half* vb = L.v_arena + ((size_t)pb * DC_KV_BLOCK * p.n_kv + it.kvh) * 128 + dim;
        for (int key = 0; key < nk; ++key) {
            const float v = __half2float(
                __ushort_as_half(__ldcg(reinterpret_cast<const unsigned short*>(vb + (size_t)key * p.n_kv * 128))));
            if (h0) acc0 = fmaf(sh.p[hq][key], v, acc0);
            if (h1) acc1 = fmaf(sh.p[hq + 4][key], v, acc1);
        }
        __syncthreads();
    }
    if (hq < g) {
        const size_t idx = ((size_t)it.t * p.n_head + it.kvh * g + hq) * p.nsplit + it.split;
        p.part_acc[idx * 128 + dim] = acc0 * sh.suffix[hq];
        if (dim == 0) p.part_d[idx] = sh.d[hq] * sh.suffix[hq];
    }
    if (hq + 4 < g) {
        const size_t idx = ((size_t)it.t * p.n_head + it.kvh * g + hq + 4) * p.nsplit + it.split;
        p.part_acc[idx * 128 + dim] = acc1 * sh.suffix[hq + 4];
        if (dim == 0) p.part_d[idx] = sh.d[hq + 4] * sh.suffix[hq + 4];
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) sh.last = (atomicAdd(p.tickets + it.t * p.n_kv + it.kvh, 1) == p.nsplit - 1);
    __syncthreads();
    if (!sh.last) return;
    __threadfence();
    if (tid == 0) p.tickets[it.t * p.n_kv + it.kvh] = 0;
    for (int pb2 = warp; pb2 < g / 2; pb2 += MG_WARPS) {
        const int head = it.kvh * g + 2 * pb2 + (lane >> 4), d0 = (lane & 15) * 8;
        const size_t base = ((size_t)it.t * p.n_head + head) * p.nsplit;
        float v[8] = {0, 0, 0, 0, 0, 0, 0, 0}, den = 0.0f;
        for (int s = 0; s < p.nsplit; ++s) {
            den += __ldcg(p.part_d + base + s);
            const float4 a = __ldcg(reinterpret_cast<const float4*>(p.part_acc + (base + s) * 128 + d0));
            const float4 c = __ldcg(reinterpret_cast<const float4*>(p.part_acc + (base + s) * 128 + d0 + 4));
            v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
            v[4] += c.x; v[5] += c.y; v[6] += c.z; v[7] += c.w;
        }
        const float inv = (den > 0.0f && isfinite(den)) ? __fdiv_rn(1.0f, __fadd_rn(den, 1e-6f)) : 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] *= inv;
        quantize_block_q8k_regs(v, p.q8_attn + ((size_t)it.t * (p.n_head / 2) + it.kvh * (g / 2) + pb2) * DC_Q8K_BYTES, lane);
    }
}

// ------------------------------------------------------------- routing
__device__ __forceinline__ unsigned long long mg_route_key(float v, int id) {
    uint32_t u;
    if (v != v) u = 0u;
    else {
        if (v == 0.0f) v = 0.0f;
        u = __float_as_uint(v);
        u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    }
    return ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)id);
}

// Router logits of this CTA's expert (expert id = blockIdx.x): each warp dots one
// 1/16 of the F32 router row with the normed hidden state in shared memory.
__device__ __forceinline__ void router_logits_phase(const MegaParams& p, const MegaLayer& L, MegaShared& sh,
                                                    const float* xn) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int e = blockIdx.x; e < p.E; e += gridDim.x) {
        const int seg = p.H / MG_WARPS;  // floats per warp
        const float* w = L.router + (size_t)e * p.H + warp * seg;
        float acc[MG_MAX_T];
#pragma unroll
        for (int t = 0; t < MG_MAX_T; ++t) acc[t] = 0.0f;
        for (int i = lane * 4; i < seg; i += 128) {
            const float4 wv = *reinterpret_cast<const float4*>(w + i);
#pragma unroll
            for (int t = 0; t < MG_MAX_T; ++t) {
                if (t < p.T) {
                    const float4 xv = *reinterpret_cast<const float4*>(xn + t * p.H + warp * seg + i);
                    acc[t] = fmaf(wv.x, xv.x, acc[t]);
                    acc[t] = fmaf(wv.y, xv.y, acc[t]);
                    acc[t] = fmaf(wv.z, xv.z, acc[t]);
                    acc[t] = fmaf(wv.w, xv.w, acc[t]);
                }
            }
        }
#pragma unroll
        for (int t = 0; t < MG_MAX_T; ++t) {
            if (t < p.T) {
                float v = acc[t];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0) sh.red[warp][t] = (double)v;
            }
        }
        __syncthreads();
        if (threadIdx.x < p.T) {
            float s = 0.0f;
            for (int i = 0; i < MG_WARPS; ++i) s += (float)sh.red[i][threadIdx.x];
            p.router_logits[(size_t)threadIdx.x * p.E + e] = s;
        }
        __syncthreads();
    }
}

// Every CTA routes all tokens itself from the logits in global memory: stable top-k
// on logits, weights over the selected experts (core/src/llm/moe/native.cpp:610-676),
// then the expert-grouped assignment map (core/src/moe/moe_routing.cpp:534-603).
__device__ __forceinline__ void route_phase(const MegaParams& p, MegaShared& sh) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int t = warp; t < p.T; t += MG_WARPS) {
        float lv[MG_MAX_E / 32];
        bool taken[MG_MAX_E / 32];
#pragma unroll
        for (int j = 0; j < MG_MAX_E / 32; ++j) {
            const int id = j * 32 + lane;
            lv[j] = id < p.E ? __ldcg(p.router_logits + (size_t)t * p.E + id) : 0.0f;
            taken[j] = id >= p.E;
        }
        float mine = 0.0f;  // lane k keeps the logit of the k-th pick
        for (int k = 0; k < p.top_k; ++k) {
            unsigned long long best = 0ull;
#pragma unroll
            for (int j = 0; j < MG_MAX_E / 32; ++j) {
                if (!taken[j]) {
                    const unsigned long long key = mg_route_key(lv[j], j * 32 + lane);
                    best = key > best ? key : best;
                }
            }
            unsigned long long win = best;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const unsigned long long ok = __shfl_xor_sync(0xffffffffu, win, o);
                win = ok > win ? ok : win;
            }
            const int wid = (int)(0xFFFFFFFFu - (uint32_t)(win & 0xFFFFFFFFull));
            float wl = 0.0f;
#pragma unroll
            for (int j = 0; j < MG_MAX_E / 32; ++j)
                if (j * 32 + lane == wid) {
                    taken[j] = true;
                    wl = lv[j];
                }
            wl = __shfl_sync(0xffffffffu, wl, wid & 31);
            if (lane == k) mine = wl;
            if (lane == 0) sh.ids[t * p.top_k + k] = wid;
        }
        // weights, sequentially by lane 0 as the reference does
        float sel[MG_MAX_K];
#pragma unroll
        for (int k = 0; k < MG_MAX_K; ++k) sel[k] = __shfl_sync(0xffffffffu, mine, k);
        if (lane == 0) {
            float mx = -INFINITY;
            bool finite = true;
#pragma unroll
            for (int k = 0; k < MG_MAX_K; ++k)
                if (k < p.top_k) {
                    finite = finite && isfinite(sel[k]);
                    if (isfinite(sel[k]) && sel[k] > mx) mx = sel[k];
                }
            float den = 0.0f, wv[MG_MAX_K];
#pragma unroll
            for (int k = 0; k < MG_MAX_K; ++k) {
                wv[k] = 0.0f;
                if (k < p.top_k && finite && isfinite(mx)) {
                    wv[k] = expf(sel[k] - mx);
                    den += wv[k];
                }
            }
            const bool ok = den > 0.0f && isfinite(den);
#pragma unroll
            for (int k = 0; k < MG_MAX_K; ++k)
                if (k < p.top_k) {
                    const float w = ok ? __fdiv_rn(wv[k], den) : __fdiv_rn(1.0f, (float)p.top_k);
                    sh.w[t * p.top_k + k] = __fmul_rn(w, p.routed_scale);
                }
        }
    }
    __syncthreads();
    // bucketing: thread e owns expert e (E <= 256 < 512 threads)
    const int A = p.T * p.top_k, me = threadIdx.x;
    int cnt = 0;
    if (me < p.E)
        for (int i = 0; i < A; ++i) cnt += (sh.ids[i] == me);
    const int act = cnt > 0 ? 1 : 0;
    int sa = act, scn = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int a2 = __shfl_up_sync(0xffffffffu, sa, o), c2 = __shfl_up_sync(0xffffffffu, scn, o);
        if (lane >= o) {
            sa += a2;
            scn += c2;
        }
    }
    if (lane == 31) {
        sh.wsum_a[warp] = sa;
        sh.wsum_c[warp] = scn;
    }
    __syncthreads();
    int base_a = 0, base_c = 0, tot_a = 0, tot_c = 0;
#pragma unroll
    for (int w = 0; w < MG_WARPS; ++w) {
        if (w < warp) {
            base_a += sh.wsum_a[w];
            base_c += sh.wsum_c[w];
        }
        tot_a += sh.wsum_a[w];
        tot_c += sh.wsum_c[w];
    }
    if (act) {
        const int u = base_a + sa - 1, off = base_c + scn - cnt;
        sh.uexp[u] = me;
        sh.uoff[u] = off;
        int o = off;
        for (int i = 0; i < A; ++i)
            if (sh.ids[i] == me) sh.uassign[o++] = i;
    }
    if (threadIdx.x == 0) {
        sh.n_active = tot_a;
        sh.uoff[tot_a] = tot_c;
        sh.have_moe = 1;
    }
    if (blockIdx.x == 0 && threadIdx.x < A) {
        if (p.route_ids) p.route_ids[threadIdx.x] = sh.ids[threadIdx.x];
        if (p.route_w) p.route_w[threadIdx.x] = sh.w[threadIdx.x];
    }
    __syncthreads();
}

// ------------------------------------------------------------ the kernel
__device__ __forceinline__ unsigned long long mg_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Optional phase timing as seen by CTA 0: slot i accumulates the nanoseconds between
// mark i-1 and mark i over all layers and steps.
#define MG_MARK(i)                                              \
    do {                                                        \
        if (p.phase_ns && blockIdx.x == 0 && tid == 0) {        \
            const unsigned long long _n = mg_now();             \
            p.phase_ns[i] += _n - t_last;                       \
            t_last = _n;                                        \
        }                                                       \
    } while (0)

__device__ __forceinline__ GemvParams mg_qkv(const MegaParams& p, const MegaLayer& L) {
    GemvParams g = {};
    const int QD = p.n_head * 128, KD = p.n_kv * 128, QKV = QD + 2 * KD;
    g.seg[0] = dc_gemv_seg{L.wq, L.wq_type, QD, L.wq_rb, p.qkv, QKV};
    g.seg[1] = dc_gemv_seg{L.wk, L.wk_type, KD, L.wk_rb, p.qkv + QD, QKV};
    g.seg[2] = dc_gemv_seg{L.wv, L.wv_type, KD, L.wv_rb, p.qkv + QD + KD, QKV};
    g.n_seg = 3;
    g.rpst[0] = p.rpst_q;
    g.rpst[1] = p.rpst_k;
    g.rpst[2] = p.rpst_v;
    g.total_rows = QKV;
    g.epi = DC_EPI_STORE;
    g.T = p.T;
    g.K = p.H;
    g.stage_bytes = MG_STAGE;
    g.err = p.err;
    return g;
}
__device__ __forceinline__ GemvParams mg_single(const MegaParams& p, const uint8_t* w, int type, int rb, int rows,
                                                int rpst, int K, int epi, float* out, int ldo,
                                                unsigned long long* argmax) {
    GemvParams g = {};
    g.seg[0] = dc_gemv_seg{w, type, rows, rb, out, ldo};
    g.n_seg = 1;
    g.rpst[0] = rpst;
    g.total_rows = rows;
    g.epi = epi;
    g.T = p.T;
    g.K = K;
    g.stage_bytes = MG_STAGE;
    g.argmax = argmax;
    g.err = p.err;
    return g;
}
__device__ __forceinline__ MoeMMParams mg_experts(const MegaParams& p, const MegaShared& sh, const uint8_t* w0,
                                                  const uint8_t* w1, int type, int rb, int N, int K, int rpst,
                                                  float* out) {
    MoeMMParams m = {};
    m.w0 = w0;
    m.w1 = w1;
    m.type = type;
    m.row_bytes = rb;
    m.N = N;
    m.K = K;
    m.top_k = p.top_k;
    m.e_base = 0;
    m.uexp = sh.uexp;
    m.uoff = sh.uoff;
    m.uassign = sh.uassign;
    m.out = out;
    m.rpst = rpst;
    m.stage_bytes = MG_STAGE;
    m.up_off = p.up_off;
    m.err = p.err;
    return m;
}

template <int NT>
__global__ void __launch_bounds__(MG_THREADS, 1) k_decode_mega(const MegaParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ MegaShared sh;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gw = blockIdx.x * MG_WARPS + warp, nw = gridDim.x * MG_WARPS;
    WarpPipe<MG_NSTAGE> pipe;
    pipe.init(smem + p.off_pipe + (size_t)warp * MG_NSTAGE * MG_STAGE, reinterpret_cast<uint64_t*>(smem) + warp * MG_NSTAGE,
              MG_STAGE, p.err);
    float* xs = reinterpret_cast<float*>(smem + p.off_xs);
    float* s_sc = reinterpret_cast<float*>(smem + p.off_sc);
    uint8_t* act_base = smem + p.off_act;
    const int QD = p.n_head * 128, A = p.T * p.top_k;
    unsigned epoch = 0;
    unsigned long long t_last = mg_now();
    if (tid == 0) sh.have_moe = 0;
    __syncthreads();

    for (int step = 0; step < p.n_steps; ++step) {
        GemvParams gq = mg_qkv(p, p.layers[0]);
        GemvStream<MG_NSTAGE> sq;
        sq.begin(gq, gw, nw);
        sq.prefill(gq, pipe, lane);
        GemvParams glm = {};
        GemvStream<MG_NSTAGE> slm;
        for (int l = 0; l < p.n_layer; ++l) {
            const MegaLayer& L = p.layers[l];
            const float* xin = (l & 1) ? p.xb : p.xa;
            float* xout = (l & 1) ? p.xa : p.xb;
            // ---- P0: hidden state, attn_norm, Q8_K, QKV rows
            MG_MARK(0);
            assemble_x(p, sh, xs, xin, xout, l == 0);
            if (tid == 0) sh.have_moe = 0;
            MG_MARK(1);
            ActSmem act;
            act.bind(act_base, p.T, p.H);
            norm_quant(p, sh, xs, L.attn_norm, act);
            MG_MARK(2);
            sq.template consume<NT>(gq, pipe, act, lane);
            MG_MARK(3);
            GemvParams go = mg_single(p, L.wo, L.wo_type, L.wo_rb, p.H, p.rpst_o, QD, DC_EPI_ACC, xout, p.H, nullptr);
            GemvStream<MG_NSTAGE> so;
            so.begin(go, gw, nw);
            so.prefill(go, pipe, lane);   // output-projection rows stream in during attention
            grid_barrier(p, epoch);
            MG_MARK(4);
            // ---- P1 / P2: attention
            attn_scores_phase(p, L, sh, s_sc);
            MG_MARK(5);
            grid_barrier(p, epoch);
            MG_MARK(6);
            attn_pv_phase(p, L, sh, s_sc);
            MG_MARK(7);
            grid_barrier(p, epoch);
            MG_MARK(8);
            // ---- P3: output projection, x += Wo . attn
            act.bind(act_base, p.T, QD);
            act.template fill<true>(p.q8_attn, p.T);
            __syncthreads();
            MG_MARK(9);
            so.template consume<NT>(go, pipe, act, lane);
            MG_MARK(10);
            grid_barrier(p, epoch);
            MG_MARK(11);
            // ---- P4: ffn_norm, Q8_K, router logits
            for (int e = tid; e < p.T * p.H; e += MG_THREADS) xs[e] = __ldcg(xout + e);
            __syncthreads();
            act.bind(act_base, p.T, p.H);
            norm_quant(p, sh, xs, L.ffn_norm, act);
            MG_MARK(12);
            router_logits_phase(p, L, sh, xs);
            MG_MARK(13);
            grid_barrier(p, epoch);
            MG_MARK(14);
            // ---- P5: routing, gate/up + SwiGLU
            route_phase(p, sh);
            MG_MARK(15);
            MoeMMParams mgu = mg_experts(p, sh, L.gate, L.up, L.gate_type, L.gate_rb, p.F, p.H, p.rpst_gate, p.h);
            MoeStream<MG_NSTAGE, true> sg;
            sg.begin(mgu, sh.n_active, gw, nw);
            sg.prefill(mgu, pipe, lane);
            sg.template consume<NT>(mgu, pipe, act, lane);
            MG_MARK(16);
            MoeMMParams mdn = mg_experts(p, sh, L.down, nullptr, L.down_type, L.down_rb, p.H, p.F, p.rpst_down, p.dn);
            MoeStream<MG_NSTAGE, false> sd;
            sd.begin(mdn, sh.n_active, gw, nw);
            sd.prefill(mdn, pipe, lane);  // down rows stream in across the barrier
            grid_barrier(p, epoch);
            MG_MARK(17);
            // ---- P6: h -> Q8_K, down rows
            ActSmem acth;
            acth.bind(act_base, A, p.F);
            {
                const int nbh = p.F / DC_QK_K;
                for (int i = warp; i < A * nbh; i += MG_WARPS) {
                    const int a = i / nbh, b = i - a * nbh;
                    const float4* src = reinterpret_cast<const float4*>(p.h + (size_t)a * p.F + b * DC_QK_K) + 2 * lane;
                    const float4 v0 = __ldcg(src), v1 = __ldcg(src + 1);
                    const float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
                    quantize_block_q8k_to_act(v, acth, a, b, lane);
                }
            }
            __syncthreads();
            MG_MARK(18);
            sd.template consume<NT>(mdn, pipe, acth, lane);
            MG_MARK(19);
            if (l + 1 < p.n_layer) {
                gq = mg_qkv(p, p.layers[l + 1]);
                sq.begin(gq, gw, nw);
                sq.prefill(gq, pipe, lane);
            } else {
                glm = mg_single(p, p.out_w, p.out_type, p.out_rb, p.vocab, p.rpst_out, p.H, DC_EPI_STORE, p.logits,
                                p.vocab, p.argmax_keys);
                slm.begin(glm, gw, nw);
                slm.prefill(glm, pipe, lane);
            }
            grid_barrier(p, epoch);
            MG_MARK(20);
        }
        // ---- final: last MoE output + residual, output norm, lm_head with arg-max keys
        assemble_x(p, sh, xs, (p.n_layer & 1) ? p.xb : p.xa, nullptr, false);
        if (tid == 0) sh.have_moe = 0;
        ActSmem act;
        act.bind(act_base, p.T, p.H);
        norm_quant(p, sh, xs, p.out_norm, act);
        slm.template consume<NT>(glm, pipe, act, lane);
        grid_barrier(p, epoch);
        MG_MARK(21);
        // greedy pick: first maximum wins (core/src/sampler/sampler.cpp:42-57)
        if (blockIdx.x == 0 && tid < p.T) {
            const unsigned long long k = __ldcg(p.argmax_keys + tid);
            const int32_t tok = (int32_t)(0xFFFFFFFFu - (uint32_t)(k & 0xFFFFFFFFull));
            p.out_tokens[tid] = tok;
            if (p.feedback) {
                p.tokens[tid] = tok;
                p.positions[tid] = __ldcg(p.positions + tid) + 1;
                if (p.history) {
                    const int n = *p.history_len;
                    if (n < p.history_cap) p.history[(size_t)n * p.T + tid] = tok;
                }
            }
            p.argmax_keys[tid] = 0ull;
        }
        if (blockIdx.x == 0) {
            __syncthreads();
            if (tid == 0 && p.feedback && p.history) *p.history_len += 1;
        }
        if (step + 1 < p.n_steps) grid_barrier(p, epoch);
    }
}

// ------------------------------------------------------------------ host
static int mg_rows_per_stage(int type, int K, int row_bytes) {
    const int G = dc::lanes_per_row(type, K);
    const int per_pass = 32 / G;
    int r = DC_STAGE_TARGET / row_bytes;
    r = r / per_pass * per_pass;
    return r < per_pass ? per_pass : r;
}

// Decides whether the persistent kernel can run this model for T streams and fills
// the parameter block.  Returns false (with a reason) when the shapes do not fit
// its fixed shared-memory plan; the caller then uses the per-op kernels.
bool dc_mega_plan(dc_model* m, int T, MegaParams* out, const char** why) {
    const dc_model_config& c = m->cfg;
    static const char* reason = "";
    *why = reason;
#define NO(msg)        \
    do {               \
        *why = msg;    \
        return false;  \
    } while (0)
    if (c.n_expert <= 0) NO("dense FFN models use the per-op kernels");
    if (c.ep_size > 1) NO("expert-parallel runs use the per-op kernels");
    if (T < 1 || T > MG_MAX_T || T * c.n_expert_used > MG_MAX_T * 8) NO("more than 4 streams or 32 assignments");
    if (c.n_expert > MG_MAX_E || c.n_expert_used > MG_MAX_K) NO("too many experts");
    const int g = c.n_head / c.n_kv_head;
    if (g > 8 || (g & 1)) NO("query-head group must be even and <= 8");
    if (c.hidden % (MG_WARPS * 4)) NO("hidden size");
    MegaParams p = {};
    const int G = m->ctx->num_sms;
    p.n_layer = c.n_layer; p.H = c.hidden; p.n_head = c.n_head; p.n_kv = c.n_kv_head; p.vocab = c.vocab;
    p.E = c.n_expert; p.top_k = c.n_expert_used; p.F = c.expert_ffn; p.T = T;
    p.eps = c.rms_eps; p.scale = 1.0f / sqrtf((float)c.head_dim); p.routed_scale = c.routed_scale;
    p.nsplit = G / (T * c.n_kv_head);
    if (p.nsplit < 1) NO("fewer SMs than (stream, kv head) pairs");
    const int max_blocks = m->kv.max_blocks_per_seq;
    if (p.nsplit > max_blocks) p.nsplit = max_blocks;
    if (p.nsplit > m->nsplit) p.nsplit = m->nsplit;   // partial buffers are sized for the per-op split count
    p.s_keys = ((max_blocks + p.nsplit - 1) / p.nsplit) * DC_KV_BLOCK;
    // stage plan: every stage must fit MG_STAGE
    const dc_layer& L0 = m->layers[0];
    auto fits = [&](const dc_weight* w, int K, int* rpst) {
        *rpst = mg_rows_per_stage(w->type, K, (int)w->row_bytes);
        return (size_t)*rpst * w->row_bytes + 32 <= MG_STAGE;
    };
    const int QD = c.n_head * 128;
    bool ok = fits(L0.wq, c.hidden, &p.rpst_q) && fits(L0.wk, c.hidden, &p.rpst_k) && fits(L0.wv, c.hidden, &p.rpst_v) &&
              fits(L0.wo, QD, &p.rpst_o) && fits(c.tie_embeddings ? m->tok_embd : m->output, c.hidden, &p.rpst_out);
    // expert tensors: the widest row type over the layers decides
    p.rpst_gate = 1 << 30;
    p.rpst_down = 1 << 30;
    for (const dc_layer& L : m->layers) {
        int rg, rd;
        ok = ok && fits(L.down_exps, c.expert_ffn, &rd);
        rg = mg_rows_per_stage(L.gate_exps->type, c.hidden, (int)L.gate_exps->row_bytes);
        if (L.gate_exps->type != L.up_exps->type) NO("gate and up tensors differ in type");
        if (rg < p.rpst_gate) p.rpst_gate = rg;
        if (rd < p.rpst_down) p.rpst_down = rd;
        if (L.wq->type != L0.wq->type || L.wk->type != L0.wk->type || L.wv->type != L0.wv->type || L.wo->type != L0.wo->type)
            NO("attention tensor types vary by layer");
    }
    if (!ok) NO("a weight row does not fit a pipeline stage");
    // gate/up pairs: halve the rows per stage until two halves fit
    {
        const int per_pass = 32 / dc::lanes_per_row(L0.gate_exps->type, c.hidden);
        int r = p.rpst_gate;
        uint32_t half = 0;
        for (;;) {
            half = ((uint32_t)r * (uint32_t)L0.gate_exps->row_bytes + 32 + 127) & ~127u;
            if (2 * half <= MG_STAGE || r <= per_pass) break;
            r -= per_pass;
        }
        if (2 * half > MG_STAGE) NO("a gate/up row pair does not fit a pipeline stage");
        p.rpst_gate = r;
        p.up_off = half;
    }
    // shared memory plan
    size_t act_bytes = ActSmem::bytes(T, QD);
    const size_t a2 = ActSmem::bytes(T * c.n_expert_used, c.expert_ffn), a3 = ActSmem::bytes(T, c.hidden);
    if (a2 > act_bytes) act_bytes = a2;
    if (a3 > act_bytes) act_bytes = a3;
    uint32_t off = 512;
    p.off_pipe = off;
    off += MG_WARPS * MG_NSTAGE * MG_STAGE;
    p.off_act = off;
    off += (uint32_t)((act_bytes + 127) & ~(size_t)127);
    p.off_xs = off;
    off += (uint32_t)(T * c.hidden * 4);
    p.off_sc = off;
    off += (uint32_t)((8 * p.s_keys * 4 + 127) & ~127);
    p.smem_bytes = off;
    if (off > 218 * 1024) NO("shared memory plan exceeds the 227 KB of an SM");
    *out = p;
    return true;
#undef NO
}

template <int NT>
static int mg_launch(dc_model* m, MegaParams& p) {
    dc_ctx* ctx = m->ctx;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(k_decode_mega<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 218 * 1024);
        if (e != cudaSuccess) return dc_check_cuda(ctx, e, "cudaFuncSetAttribute(k_decode_mega)");
        configured = true;
    }
    int per_sm = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_decode_mega<NT>, MG_THREADS, p.smem_bytes);
    if (e != cudaSuccess) return dc_check_cuda(ctx, e, "occupancy query");
    if (per_sm < 1) return dc_fail(ctx, DC_B200_UNSUPPORTED, "persistent decode kernel does not fit on an SM");
    void* args[] = {&p};
    e = cudaLaunchCooperativeKernel((void*)k_decode_mega<NT>, dim3(ctx->num_sms), dim3(MG_THREADS), args, p.smem_bytes,
                                    ctx->stream);
    return dc_check_cuda(ctx, e, "k_decode_mega");
}

// Runs n_steps decode steps for the T streams whose inputs are already in the step buffers.
int dc_mega_run(dc_model* m, int T, int n_steps, bool feedback) {
    MegaParams p;
    const char* why = "";
    if (!dc_mega_plan(m, T, &p, &why)) return dc_fail(m->ctx, DC_B200_UNSUPPORTED, "persistent decode: %s", why);
    dc_step_buffers& b = m->buf;
    p.layers = (const MegaLayer*)m->mega_layers;
    p.tok_embd = m->tok_embd->dev;
    p.embd_type = m->tok_embd->type;
    p.embd_row_bytes = (int)m->tok_embd->row_bytes;
    p.out_norm = (const float*)m->out_norm->dev;
    const dc_weight* ow = m->cfg.tie_embeddings ? m->tok_embd : m->output;
    p.out_w = ow->dev;
    p.out_type = ow->type;
    p.out_rb = (int)ow->row_bytes;
    p.tokens = b.tokens; p.seq_ids = b.seq_ids; p.positions = b.positions; p.out_tokens = b.out_tokens;
    p.argmax_keys = b.argmax_keys;
    p.history = feedback ? b.history : nullptr;
    p.history_len = b.history_len;
    p.history_cap = DC_HISTORY_CAP;
    p.feedback = feedback ? 1 : 0;
    p.n_steps = n_steps;
    p.block_tables = m->kv.d_tables;
    p.max_blocks = m->kv.max_blocks_per_seq;
    p.cos_sin = b.cos_sin;
    p.max_pos = m->cfg.max_ctx;
    p.xa = b.x; p.xb = b.xn; p.qkv = b.qkv; p.h = b.h; p.dn = b.dn;
    p.router_logits = b.route.logits;
    p.logits = b.logits;
    p.bmax = b.attn.bmax; p.part_acc = b.attn.part_acc; p.part_d = b.attn.part_d; p.tickets = b.attn.tickets;
    p.q8_attn = b.q8_attn;
    p.route_ids = b.route.ids;
    p.route_w = b.route.weights;
    p.bar_counter = m->mega_counter;
    p.err = m->ctx->d_err;
    p.phase_ns = m->mega_timing ? (unsigned long long*)((uint8_t*)m->mega_counter + 64) : nullptr;
    int st = dc_check_cuda(m->ctx, cudaMemsetAsync(m->mega_counter, 0, sizeof(unsigned), m->ctx->stream), "memset");
    if (st != DC_B200_OK) return st;
    m->last_launches = 1;
    return T == 1 ? mg_launch<1>(m, p) : mg_launch<MG_MAX_T>(m, p);
}

// Device copy of the per-layer pointer table; called once when the model is finalized.
int dc_mega_prepare(dc_model* m) {
    if (m->cfg.n_expert <= 0) return DC_B200_OK;
    std::vector<MegaLayer> v(m->cfg.n_layer);
    for (int il = 0; il < m->cfg.n_layer; ++il) {
        const dc_layer& L = m->layers[il];
        MegaLayer& d = v[il];
        d.attn_norm = (const float*)L.attn_norm->dev;
        d.q_norm = L.q_norm ? (const float*)L.q_norm->dev : nullptr;
        d.k_norm = L.k_norm ? (const float*)L.k_norm->dev : nullptr;
        d.ffn_norm = (const float*)L.ffn_norm->dev;
        d.router = (const float*)L.router->dev;
        d.wq = L.wq->dev; d.wk = L.wk->dev; d.wv = L.wv->dev; d.wo = L.wo->dev;
        d.gate = L.gate_exps->dev; d.up = L.up_exps->dev; d.down = L.down_exps->dev;
        d.wq_type = L.wq->type; d.wk_type = L.wk->type; d.wv_type = L.wv->type; d.wo_type = L.wo->type;
        d.gate_type = L.gate_exps->type; d.down_type = L.down_exps->type;
        d.wq_rb = (int)L.wq->row_bytes; d.wk_rb = (int)L.wk->row_bytes; d.wv_rb = (int)L.wv->row_bytes;
        d.wo_rb = (int)L.wo->row_bytes; d.gate_rb = (int)L.gate_exps->row_bytes; d.down_rb = (int)L.down_exps->row_bytes;
        d.k_arena = m->kv.k_arena + m->kv.layer_elems * il;
        d.v_arena = m->kv.v_arena + m->kv.layer_elems * il;
    }
    cudaError_t e = cudaMalloc(&m->mega_layers, v.size() * sizeof(MegaLayer));
    if (e == cudaSuccess) e = cudaMalloc((void**)&m->mega_counter, 512);
    if (e == cudaSuccess) e = cudaMemcpy(m->mega_layers, v.data(), v.size() * sizeof(MegaLayer), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemset(m->mega_counter, 0, 512);
    return dc_check_cuda(m->ctx, e, "persistent decode set-up");
}
