// Paged-KV split-K flash-decode attention.  Replaces cb_paged_attention_decode
// (core/src/llm/attention/paged_exec.cpp:343) and its kernel PagedAttentionImpl
// (core/src/kernels/hwy/hwy_paged_attention.cc:367-630).
//
// The reference walks a sequence's 16-token KV blocks in order with an online
// softmax: m_b = max(m_{b-1}, block max), alpha_b = fastexp(m_{b-1} - m_b),
// acc = acc*alpha_b + sum_t fastexp(s_t - m_b) v_t, and finally acc/(d + 1e-6).
// fastexp is a cubic polynomial, so the result depends on which maximum each
// exponent is taken against.  To stay on the reference's numbers while cutting
// the sequence into parallel runs, the work is split in two kernels:
//   k_attn_scores  every run computes its scores s_t and per-block maxima;
//   k_attn_pv      every run rebuilds the reference's running-maximum chain from
//                  ALL block maxima (so its exponents are taken against exactly
//                  the reference's m_b), accumulates its blocks as the reference
//                  does, scales its partial by the product of the alphas of all
//                  later blocks, and the last run to finish (a ticket, no
//                  waiting) adds the partials and emits f32 and Q8_K output.
// Only float summation order differs from the sequential walk.
#include "dc_common.cuh"
#include "dc_internal.h"
#include "dc_launch.cuh"

using namespace dc;

#define ATT_MAX_GROUP 8  // query heads per kv head
#define ATT_TILE 32      // keys per score tile (two KV blocks)

struct AttnParams {
    const float* q;              // [T][n_head][128]
    const __half* k_arena;       // this layer
    const __half* v_arena;
    const int32_t* block_tables; // [max_seqs][max_blocks]
    int max_blocks;
    const int32_t* seq_ids;      // [T]
    const int32_t* positions;    // [T]
    int n_head, n_kv, T, nsplit;
    float scale;
    float* scores;               // [T][n_head][max_blocks*16]
    float* bmax;                 // [T][n_head][max_blocks]
    float* part_acc;             // [T][n_head][nsplit][128]
    float* part_d;               // [T][n_head][nsplit]
    int* tickets;                // [T][n_kv], zeroed once, self-resetting
    float* out;                  // optional [T][n_head][128]
    uint8_t* q8_out;             // optional Q8_K rows of out
};

__device__ __forceinline__ void split_range(int pos, int split, int nsplit, int& n_blk, int& b0, int& b1) {
    n_blk = (pos + 1 + DC_KV_BLOCK - 1) / DC_KV_BLOCK;
    const int bps = (n_blk + nsplit - 1) / nsplit;
    b0 = min(n_blk, split * bps);
    b1 = min(n_blk, b0 + bps);
}

__global__ void __launch_bounds__(128) k_attn_scores(const AttnParams p) {
    // a q head as four 32-dim quarters 36 floats apart: the four lanes of a key read the same offset of
    // different quarters, which then fall into different banks
    __shared__ __align__(16) float sq[ATT_MAX_GROUP][4 * 36];
    __shared__ float sc[ATT_MAX_GROUP][ATT_TILE];
    __shared__ int s_blk[ATT_TILE / DC_KV_BLOCK];
    pdl_launch_dependents();
    const int split = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
    const int g = p.n_head / p.n_kv;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // positions, sequence ids and block tables were settled before this step began, and K rows of earlier
    // positions are not written during it: the first tile's history rows are fetched while this kernel
    // still waits for the one that writes the new token's row and the q heads
    // (in an eager chain of steps the position may still be the previous step's here: everything is
    // recomputed after the wait and the early rows are dropped if the run moved)
    const int32_t* table = p.block_tables + (size_t)p.seq_ids[t] * p.max_blocks;
    uint4 kr0[4];
    bool pre = false;
    int pre_b0;
    {
        const int pos0 = p.positions[t];
        // rows written during this step: this token's, and those of earlier tokens of the same sequence
        // in a multi-token chunk; only rows before the first of them are safe to read early
        int stable = pos0;
        const int sid = p.seq_ids[t];
        for (int u = 0; u < p.T; ++u)
            if (p.seq_ids[u] == sid) stable = min(stable, p.positions[u]);
        int nb0, e1;
        split_range(pos0, split, p.nsplit, nb0, pre_b0, e1);
        const int key = warp * 8 + (lane >> 2), sub = lane & 3, blk = pre_b0 + key / DC_KV_BLOCK;
        const int kpos = pre_b0 * DC_KV_BLOCK + key;
        if (pos0 >= 0 && blk < e1 && kpos < stable) {
            const uint4* kp = reinterpret_cast<const uint4*>(
                p.k_arena + (((size_t)table[blk] * DC_KV_BLOCK + key % DC_KV_BLOCK) * p.n_kv + kvh) * 128 + sub * 32);
#pragma unroll
            for (int i = 0; i < 4; ++i) kr0[i] = kp[i];
            pre = true;
        }
    }
    pdl_wait();
    const int pos = *reinterpret_cast<const volatile int32_t*>(p.positions + t), ctx_len = pos + 1;
    int n_blk, b0, b1;
    split_range(pos, split, p.nsplit, n_blk, b0, b1);
    if (b0 != pre_b0) pre = false;
    if (b0 >= b1) return;
    for (int i = tid; i < g * 128; i += 128)
        sq[i >> 7][((i & 127) >> 5) * 36 + (i & 31)] = p.q[((size_t)t * p.n_head + kvh * g + (i >> 7)) * 128 + (i & 127)];
    __syncthreads();
    const size_t ctx_pad = (size_t)p.max_blocks * DC_KV_BLOCK;
    for (int blk = b0; blk < b1; blk += ATT_TILE / DC_KV_BLOCK) {
        if (tid < ATT_TILE / DC_KV_BLOCK) s_blk[tid] = (blk + tid < b1) ? table[blk + tid] : -1;
        __syncthreads();
        {   // 4 lanes per key, 32 dims per lane
            const int key = warp * 8 + (lane >> 2), sub = lane & 3;
            const int kpos = blk * DC_KV_BLOCK + key;
            const int pb = s_blk[key / DC_KV_BLOCK];
            const bool valid = pb >= 0 && kpos < ctx_len;
            float kf[32];
            if (valid) {
                const uint4* kp = reinterpret_cast<const uint4*>(
                    p.k_arena + (((size_t)pb * DC_KV_BLOCK + key % DC_KV_BLOCK) * p.n_kv + kvh) * 128 + sub * 32);
                const bool have = pre && blk == b0;   // fetched before the wait
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint4 u = have ? kr0[i] : kp[i];
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
                const float4* qp = reinterpret_cast<const float4*>(&sq[h][sub * 36]);
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
                if (sub == 0) sc[h][key] = valid ? __fmul_rn(dot, p.scale) : -INFINITY;
            }
        }
        __syncthreads();
        // scores out (32 consecutive keys per head) and the two block maxima
        for (int i = tid; i < g * ATT_TILE; i += 128) {
            const int h = i / ATT_TILE, key = i % ATT_TILE;
            if (blk + key / DC_KV_BLOCK < b1)
                p.scores[((size_t)t * p.n_head + kvh * g + h) * ctx_pad + (size_t)blk * DC_KV_BLOCK + key] = sc[h][key];
        }
        if (tid < g * (ATT_TILE / DC_KV_BLOCK)) {
            const int h = tid / (ATT_TILE / DC_KV_BLOCK), bb = tid % (ATT_TILE / DC_KV_BLOCK);
            if (blk + bb < b1) {
                float mx = -1e30f;  // the reference's m_block starts at -1e30
#pragma unroll
                for (int k = 0; k < DC_KV_BLOCK; ++k) mx = fmaxf(mx, sc[h][bb * DC_KV_BLOCK + k]);
                p.bmax[((size_t)t * p.n_head + kvh * g + h) * p.max_blocks + blk + bb] = mx;
            }
        }
        __syncthreads();
    }
}

// Tail of both P.V kernels: the run's partials are in global memory; the last run of the (token, kv head)
// to get here sums all runs in run order, normalises and emits (no run waits for another).
__device__ __forceinline__ void attn_merge_tail(const AttnParams& p, int t, int kvh, int g, int tid, int warp, int lane,
                                                int& s_last) {
    // release: the CTA barrier puts every thread's partial before thread 0's ticket, whose release half publishes
    // them; acquire: the last run's thread 0 sees the other runs' partials through the ticket's acquire half, and
    // the CTA barrier passes that on
    __syncthreads();
    if (tid == 0) {
        int old;
        asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], %2;" : "=r"(old) : "l"(p.tickets + t * p.n_kv + kvh), "r"(1) : "memory");
        const int last = old == p.nsplit - 1;
        if (last) p.tickets[t * p.n_kv + kvh] = 0;
        s_last = last;
    }
    __syncthreads();
    if (!s_last) return;
    // ---- last run of this (token, kv head): sum the runs in run order, normalise, emit.
    // One warp per 256 outputs (two heads) = one Q8_K block of the o-projection input.
    for (int pb2 = warp; pb2 < g / 2; pb2 += 4) {
        const int head = kvh * g + 2 * pb2 + (lane >> 4), d0 = (lane & 15) * 8;
        const size_t base = ((size_t)t * p.n_head + head) * p.nsplit;
        float v[8] = {0, 0, 0, 0, 0, 0, 0, 0}, den = 0.0f;
        for (int s0 = 0; s0 < p.nsplit; s0 += 8) {
            float dd[8];
            float4 a[8], c[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {   // eight runs' loads in flight, then added in run order
                const size_t bi = base + (s0 + j < p.nsplit ? s0 + j : 0);
                dd[j] = __ldcg(p.part_d + bi);
                a[j] = __ldcg(reinterpret_cast<const float4*>(p.part_acc + bi * 128 + d0));
                c[j] = __ldcg(reinterpret_cast<const float4*>(p.part_acc + bi * 128 + d0 + 4));
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (s0 + j < p.nsplit) {
                    den += dd[j];
                    v[0] += a[j].x; v[1] += a[j].y; v[2] += a[j].z; v[3] += a[j].w;
                    v[4] += c[j].x; v[5] += c[j].y; v[6] += c[j].z; v[7] += c[j].w;
                }
            }
        }
        const float inv = (den > 0.0f && isfinite(den)) ? __fdiv_rn(1.0f, __fadd_rn(den, 1e-6f)) : 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] *= inv;
        if (p.out) {
            float* o = p.out + ((size_t)t * p.n_head + head) * 128 + d0;
            *reinterpret_cast<float4*>(o) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4*>(o + 4) = make_float4(v[4], v[5], v[6], v[7]);
        }
        if (p.q8_out)
            quantize_block_q8k_regs(v, p.q8_out + ((size_t)t * (p.n_head / 2) + kvh * (g / 2) + pb2) * DC_Q8K_BYTES, lane);
    }
}

__global__ void __launch_bounds__(128) k_attn_pv(const AttnParams p) {
    __shared__ float s_p[ATT_MAX_GROUP][DC_KV_BLOCK];
    __shared__ float s_suffix[ATT_MAX_GROUP];
    __shared__ float s_m[ATT_MAX_GROUP], s_d[ATT_MAX_GROUP], s_alpha[ATT_MAX_GROUP];
    __shared__ int s_last;
    pdl_launch_dependents();
    pdl_wait();
    const int split = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
    const int g = p.n_head / p.n_kv;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int pos = p.positions[t], ctx_len = pos + 1;
    int n_blk, b0, b1;
    split_range(pos, split, p.nsplit, n_blk, b0, b1);
    const int32_t* table = p.block_tables + (size_t)p.seq_ids[t] * p.max_blocks;
    const size_t ctx_pad = (size_t)p.max_blocks * DC_KV_BLOCK;

    // ---- the reference's chain from all block maxima: m before this run, and the
    //      product of alpha_c over every block c >= b1 (blocks after this run)
    for (int h = warp; h < g; h += 4) {
        const float* bm = p.bmax + ((size_t)t * p.n_head + kvh * g + h) * p.max_blocks;
        float m_start = -1e30f;
        for (int b = lane; b < b0; b += 256) {   // eight loads in flight per lane
            float vb8[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) vb8[k] = b + 32 * k < b0 ? bm[b + 32 * k] : -1e30f;
#pragma unroll
            for (int k = 0; k < 8; ++k) m_start = fmaxf(m_start, vb8[k]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m_start = fmaxf(m_start, __shfl_xor_sync(0xffffffffu, m_start, o));
        float m_run = m_start;
        for (int b = b0 + lane; b < b1; b += 32) m_run = fmaxf(m_run, bm[b]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m_run = fmaxf(m_run, __shfl_xor_sync(0xffffffffu, m_run, o));
        // later blocks in chunks of 32: inclusive prefix max by shuffles, alpha per block, product
        float carry = m_run, suffix = 1.0f;
        for (int c0 = b1; c0 < n_blk; c0 += 32) {
            const int c = c0 + lane;
            float v = c < n_blk ? bm[c] : -1e30f;
            float incl = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float u = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl = fmaxf(incl, u);
            }
            float excl = __shfl_up_sync(0xffffffffu, incl, 1);
            if (lane == 0) excl = -1e30f;
            const float m_prev = fmaxf(carry, excl), m_new = fmaxf(carry, incl);
            float a = c < n_blk ? fast_exp_fma(m_prev - m_new) : 1.0f;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) a *= __shfl_xor_sync(0xffffffffu, a, o);
            suffix *= a;
            carry = fmaxf(carry, __shfl_sync(0xffffffffu, incl, 31));
        }
        if (lane == 0) {
            s_suffix[h] = suffix;
            s_m[h] = m_start;
            s_d[h] = 0.0f;
        }
    }
    float acc[ATT_MAX_GROUP];
#pragma unroll
    for (int h = 0; h < ATT_MAX_GROUP; ++h) acc[h] = 0.0f;
    __syncthreads();

    // ---- own blocks, one 16-key block at a time exactly as the reference walks them
    for (int blk = b0; blk < b1; ++blk) {
        const int pb = table[blk];
        const int nk = min(DC_KV_BLOCK, ctx_len - blk * DC_KV_BLOCK);
        {
            const int h = tid >> 4, key = tid & 15;  // 128 threads = 8 heads x 16 keys
            float s = -INFINITY;
            if (h < g && key < nk)
                s = p.scores[((size_t)t * p.n_head + kvh * g + h) * ctx_pad + (size_t)blk * DC_KV_BLOCK + key];
            float mx = fmaxf(s, -1e30f);
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float m_prev = h < g ? s_m[h] : -1e30f;
            const float m_new = fmaxf(m_prev, mx);
            const float pr = (s == -INFINITY) ? 0.0f : fast_exp_fma(s - m_new);
            float ps = pr;
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
            if (h < g) s_p[h][key] = pr;
            __syncwarp();
            if (h < g && key == 0) {
                const float alpha = fast_exp_fma(m_prev - m_new);
                s_alpha[h] = alpha;
                s_d[h] = s_d[h] * alpha + ps;
                s_m[h] = m_new;
            }
        }
        __syncthreads();
#pragma unroll
        for (int h = 0; h < ATT_MAX_GROUP; ++h)
            if (h < g && s_alpha[h] != 1.0f) acc[h] *= s_alpha[h];
        const __half* vb = p.v_arena + ((size_t)pb * DC_KV_BLOCK * p.n_kv + kvh) * 128 + tid;
        // the block's 16 V values are requested together (rows beyond nk exist in the arena and are not used)
        __half vv[DC_KV_BLOCK];
#pragma unroll
        for (int key = 0; key < DC_KV_BLOCK; ++key) vv[key] = vb[(size_t)key * p.n_kv * 128];
#pragma unroll
        for (int key = 0; key < DC_KV_BLOCK; ++key) {
            if (key < nk) {
                const float v = __half2float(vv[key]);
#pragma unroll
                for (int h = 0; h < ATT_MAX_GROUP; ++h)
                    if (h < g) acc[h] = fmaf(s_p[h][key], v, acc[h]);
            }
        }
        __syncthreads();
    }
    // ---- partials scaled by the alphas of all later blocks
#pragma unroll
    for (int h = 0; h < ATT_MAX_GROUP; ++h) {
        if (h < g) {
            const size_t idx = ((size_t)t * p.n_head + kvh * g + h) * p.nsplit + split;
            p.part_acc[idx * 128 + tid] = acc[h] * s_suffix[h];
            if (tid == 0) p.part_d[idx] = s_d[h] * s_suffix[h];
        }
    }
    attn_merge_tail(p, t, kvh, g, tid, warp, lane, s_last);
}

// Same result as k_attn_pv for runs of at most ATT_MAX_RUN KV blocks, organised for latency: every
// block's running maximum and rescale factor follow from the block maxima alone, so they are computed
// for the whole run first (one batched load, prefix maxima by shuffles); then all exponentials of the
// run at once; then one pass over the keys with no CTA barrier inside.
#define ATT_MAX_RUN 64
__global__ void __launch_bounds__(128) k_attn_pv_run(const AttnParams p) {
    __shared__ __align__(16) float s_pw[ATT_MAX_GROUP * ATT_MAX_RUN * DC_KV_BLOCK];   // scores of the run, then exponentials
    __shared__ float s_mnew[ATT_MAX_GROUP][ATT_MAX_RUN], s_alpha[ATT_MAX_GROUP][ATT_MAX_RUN], s_ps[ATT_MAX_GROUP][ATT_MAX_RUN];
    __shared__ float s_suffix[ATT_MAX_GROUP];
    __shared__ int s_blk[ATT_MAX_RUN];
    __shared__ int s_last;
    pdl_launch_dependents();
    pdl_wait();
    const int split = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
    const int g = p.n_head / p.n_kv;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int pos = p.positions[t], ctx_len = pos + 1;
    int n_blk, b0, b1;
    split_range(pos, split, p.nsplit, n_blk, b0, b1);
    const int32_t* table = p.block_tables + (size_t)p.seq_ids[t] * p.max_blocks;
    const size_t ctx_pad = (size_t)p.max_blocks * DC_KV_BLOCK;
    const int nb = b1 - b0, stride = nb * DC_KV_BLOCK;
    for (int i = tid; i < g * stride; i += 128) {
        const int h = i / stride, k = i - h * stride;
        s_pw[i] = p.scores[((size_t)t * p.n_head + kvh * g + h) * ctx_pad + (size_t)b0 * DC_KV_BLOCK + k];
    }
    for (int i = tid; i < nb; i += 128) s_blk[i] = table[b0 + i];
    for (int h = warp; h < g; h += 4) {
        const float* bm = p.bmax + ((size_t)t * p.n_head + kvh * g + h) * p.max_blocks;
        float carry = -1e30f, suffix = 1.0f;
        for (int s0 = 0; s0 < n_blk; s0 += 256) {
            float vb[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int c = s0 + 32 * k + lane;
                vb[k] = c < n_blk ? bm[c] : -1e30f;
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int c0 = s0 + 32 * k, c = c0 + lane;
                if (c0 >= n_blk) break;
                if (c0 + 32 <= b0) {   // wholly before the run: only the running maximum
                    float mx = vb[k];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                    carry = fmaxf(carry, mx);
                    continue;
                }
                float incl = vb[k];
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const float u = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl = fmaxf(incl, u);
                }
                float excl = __shfl_up_sync(0xffffffffu, incl, 1);
                if (lane == 0) excl = -1e30f;
                const float m_prev = fmaxf(carry, excl), m_new = fmaxf(carry, incl);
                const float a = (c >= b0 && c < n_blk) ? fast_exp_fma(m_prev - m_new) : 1.0f;
                if (c >= b0 && c < b1) {
                    s_mnew[h][c - b0] = m_new;
                    s_alpha[h][c - b0] = a;
                }
                if (c0 + 32 > b1) {   // the chunk reaches past the run: those factors go into the suffix
                    float later = c >= b1 ? a : 1.0f;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) later *= __shfl_xor_sync(0xffffffffu, later, o);
                    suffix *= later;
                }
                carry = fmaxf(carry, __shfl_sync(0xffffffffu, incl, 31));
            }
        }
        if (lane == 0) s_suffix[h] = suffix;
    }
    __syncthreads();
    // exponentials: 16 lanes per (head, block)
    for (int base = 0; base < g * nb; base += 8) {
        const int pair = base + (tid >> 4), key = tid & 15;
        const bool in = pair < g * nb;
        const int h = in ? pair / nb : 0, bl = in ? pair - h * nb : 0;
        const int nk = min(DC_KV_BLOCK, ctx_len - (b0 + bl) * DC_KV_BLOCK);
        const float s = (in && key < nk) ? s_pw[h * stride + bl * DC_KV_BLOCK + key] : -INFINITY;
        const float pr = (s == -INFINITY) ? 0.0f : fast_exp_fma(s - s_mnew[h][bl]);
        float ps = pr;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        if (in) {
            s_pw[h * stride + bl * DC_KV_BLOCK + key] = pr;
            if (key == 0) s_ps[h][bl] = ps;
        }
    }
    __syncthreads();
    // thread = dim; one accumulator per head; thread h also carries head h's denominator
    float acc[ATT_MAX_GROUP];
#pragma unroll
    for (int h = 0; h < ATT_MAX_GROUP; ++h) acc[h] = 0.0f;
    float den = 0.0f;
    // a block's 16 V values are requested together, one block ahead of the FMAs (rows beyond nk exist in
    // the arena and are not used)
    __half vn[DC_KV_BLOCK];
    if (nb > 0) {
        const __half* vb = p.v_arena + ((size_t)s_blk[0] * DC_KV_BLOCK * p.n_kv + kvh) * 128 + tid;
#pragma unroll
        for (int key = 0; key < DC_KV_BLOCK; ++key) vn[key] = vb[(size_t)key * p.n_kv * 128];
    }
    for (int bl = 0; bl < nb; ++bl) {
        const int nk = min(DC_KV_BLOCK, ctx_len - (b0 + bl) * DC_KV_BLOCK);
        __half vv[DC_KV_BLOCK];
#pragma unroll
        for (int key = 0; key < DC_KV_BLOCK; ++key) vv[key] = vn[key];
        if (bl + 1 < nb) {
            const __half* vb = p.v_arena + ((size_t)s_blk[bl + 1] * DC_KV_BLOCK * p.n_kv + kvh) * 128 + tid;
#pragma unroll
            for (int key = 0; key < DC_KV_BLOCK; ++key) vn[key] = vb[(size_t)key * p.n_kv * 128];
        }
        if (tid < g) den = den * s_alpha[tid][bl] + s_ps[tid][bl];
#pragma unroll
        for (int h = 0; h < ATT_MAX_GROUP; ++h)
            if (h < g && s_alpha[h][bl] != 1.0f) acc[h] *= s_alpha[h][bl];
        float vf[DC_KV_BLOCK];
#pragma unroll
        for (int key = 0; key < DC_KV_BLOCK; ++key) vf[key] = __half2float(vv[key]);
        // per head: the block's 16 exponentials in four 128-bit loads, then the FMA chain in key order
#pragma unroll
        for (int h = 0; h < ATT_MAX_GROUP; ++h) {
            if (h < g) {
                float pp[DC_KV_BLOCK];
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    *reinterpret_cast<float4*>(&pp[4 * q]) =
                        *reinterpret_cast<const float4*>(&s_pw[h * stride + bl * DC_KV_BLOCK + 4 * q]);
#pragma unroll
                for (int key = 0; key < DC_KV_BLOCK; ++key)
                    if (key < nk) acc[h] = fmaf(pp[key], vf[key], acc[h]);
            }
        }
    }
#pragma unroll
    for (int h = 0; h < ATT_MAX_GROUP; ++h) {
        if (h < g) {
            const size_t idx = ((size_t)t * p.n_head + kvh * g + h) * p.nsplit + split;
            p.part_acc[idx * 128 + tid] = acc[h] * s_suffix[h];
        }
    }
    if (tid < g) p.part_d[((size_t)t * p.n_head + kvh * g + tid) * p.nsplit + split] = den * s_suffix[tid];
    attn_merge_tail(p, t, kvh, g, tid, warp, lane, s_last);
}

size_t dc_attention_scratch_bytes(int T, int n_head, int n_kv, int max_blocks, int nsplit) {
    size_t n = 0;
    n += (size_t)T * n_head * max_blocks * DC_KV_BLOCK * 4 + 256;  // scores
    n += (size_t)T * n_head * max_blocks * 4 + 256;                // bmax
    n += (size_t)T * n_head * nsplit * 128 * 4 + 256;              // part_acc
    n += (size_t)T * n_head * nsplit * 4 + 256;                    // part_d
    n += (size_t)T * n_head * 4 + 256;                             // tickets (one per merge group)
    return n;
}

// scratch: dc_attention_scratch_bytes() bytes whose ticket area (the last
// T*n_kv ints) was zeroed once.
int dc_launch_attention(dc_ctx* ctx, const float* q, const void* k_arena, const void* v_arena,
                        const int32_t* block_tables, int max_blocks, const int32_t* seq_ids, const int32_t* positions,
                        int T, int n_head, int n_kv, float scale, int nsplit, const dc_attn_scratch* sc, float* out,
                        uint8_t* q8_out) {
    const int g = n_kv > 0 ? n_head / n_kv : 0;
    if (n_kv < 1 || n_head % n_kv || g > ATT_MAX_GROUP || (g & 1))
        return dc_fail(ctx, DC_B200_UNSUPPORTED, "attention: n_head=%d n_kv=%d not supported (group must be even, <= 8)", n_head, n_kv);
    AttnParams p = {};
    p.q = q;
    p.k_arena = (const __half*)k_arena;
    p.v_arena = (const __half*)v_arena;
    p.block_tables = block_tables;
    p.max_blocks = max_blocks;
    p.seq_ids = seq_ids;
    p.positions = positions;
    p.n_head = n_head;
    p.n_kv = n_kv;
    p.T = T;
    p.nsplit = nsplit;
    p.scale = scale;
    p.scores = sc->scores;
    p.bmax = sc->bmax;
    p.part_acc = sc->part_acc;
    p.part_d = sc->part_d;
    p.tickets = sc->tickets;
    p.out = out;
    p.q8_out = q8_out;
    int st = dc_launch(ctx, "k_attn_scores", k_attn_scores, dim3(nsplit, n_kv, T), dim3(128), 0, p);
    if (st != DC_B200_OK) return st;
    // runs short enough for the kernel that keeps a whole run's scores in shared memory
    if ((max_blocks + nsplit - 1) / nsplit <= ATT_MAX_RUN)
        return dc_launch(ctx, "k_attn_pv_run", k_attn_pv_run, dim3(nsplit, n_kv, T), dim3(128), 0, p);
    return dc_launch(ctx, "k_attn_pv", k_attn_pv, dim3(nsplit, n_kv, T), dim3(128), 0, p);
}

void dc_attn_scratch_bind(dc_attn_scratch* sc, uint8_t* base, int T, int n_head, int n_kv, int max_blocks, int nsplit) {
    size_t off = 0;
    auto take = [&](size_t bytes) {
        uint8_t* p = base + off;
        off += (bytes + 255) & ~(size_t)255;
        return p;
    };
    sc->scores = (float*)take((size_t)T * n_head * max_blocks * DC_KV_BLOCK * 4);
    sc->bmax = (float*)take((size_t)T * n_head * max_blocks * 4);
    sc->part_acc = (float*)take((size_t)T * n_head * nsplit * 128 * 4);
    sc->part_d = (float*)take((size_t)T * n_head * nsplit * 4);
    sc->tickets = (int*)take((size_t)T * n_head * 4);
}
