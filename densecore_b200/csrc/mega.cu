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
#include <string.h>

#include "dc_common.cuh"
#include "dc_internal.h"
#include "dc_mega.h"
#include "dc_model.h"
#include "dc_stream.cuh"

using namespace dc;

#define MG_BAR_LIMIT (1u << 21)
#define MG_MAX_RUN_BLOCKS 64
#define DC_ERR_GRID_BARRIER 2
#ifndef MG_BAR_SLEEP
#define MG_BAR_SLEEP 32   // nanoseconds between polls of the barrier counter
#endif

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// All CTAs of the (co-resident) grid meet here.  counter only grows during a
// launch; the host zeroes it before the launch.
__device__ __forceinline__ unsigned long long mg_now();
// Split in two so that work that does not depend on the other CTAs (asking for the next phase's weight rows,
// prefetches) runs between a CTA's arrival and its release instead of in front of the arrival: issuing those
// copies takes a warp longer than the barrier's own release latency.
__device__ __forceinline__ void ep_arrive(const MegaParams& p);
__device__ __noinline__ void grid_arrive(const MegaParams& p, unsigned& epoch, bool sys_scope = false) {
    __syncthreads();
    ++epoch;
#ifdef DC_MEGA_SUBMARKS
    // arrival and release time of every CTA at the seven barriers of the second layer
    const bool trace = threadIdx.x == 0 && p.phase_ns && epoch > 7 && epoch <= 14;
    if (trace) p.phase_ns[32 + (epoch - 8) * 160 + blockIdx.x] = mg_now();
#endif
    if (sys_scope) ep_arrive(p);                 // this CTA's stores to other GPUs are performed first
    if (threadIdx.x == 0)   // one instruction: the release covers what the CTA barrier above ordered before this thread
        asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p.bar_counter), "r"(1u) : "memory");
}
// Returns true if this CTA's wait ran out: the caller then leaves the kernel (drains its copies in flight and
// returns) instead of computing on data that other CTAs may not have written yet.  The CTAs that did arrive
// run out at their next barrier, since this one never arrives there.
__device__ __noinline__ bool grid_wait(const MegaParams& p, unsigned epoch) {
    __shared__ int s_gave_up;
    if (threadIdx.x == 0) {
        const unsigned target = epoch * gridDim.x;
        unsigned polls = 0;
        int gave_up = 0;
        while (ld_acquire_u32(p.bar_counter) < target) {
            if (++polls > p.bar_polls) {
                atomicExch(p.err, DC_ERR_GRID_BARRIER);
                gave_up = 1;
                break;
            }
            if (MG_BAR_SLEEP) __nanosleep(MG_BAR_SLEEP);
        }
        s_gave_up = gave_up;
        // (no fence here: the acquire load above orders this thread after the arrivals it observed, and the CTA
        // barrier below passes that on to the other threads; a fence cost 0.4 us per barrier)
    }
#ifdef DC_MEGA_SUBMARKS
    if (threadIdx.x == 0 && p.phase_ns && epoch > 7 && epoch <= 14) p.phase_ns[32 + (7 + epoch - 8) * 160 + blockIdx.x] = mg_now();
#endif
    __syncthreads();
    return s_gave_up != 0;
}
__device__ __forceinline__ bool grid_barrier(const MegaParams& p, unsigned& epoch, bool sys_scope = false) {
    grid_arrive(p, epoch, sys_scope);
    return grid_wait(p, epoch);
}

// Expert-parallel meeting point, once per layer, folded into the grid barrier that ends the down projection:
// a CTA that arrives (its rows are stored in every GPU's exchange buffer) also adds one to an arrival counter
// in every peer's memory (red.release.sys after a system-scope fence; lane r of warp 0 talks to rank r, so the
// peers are signalled side by side), and after the local barrier every CTA waits until all CTAs of all peers
// have arrived here.  The remote arrivals travel while the local barrier and the next phase's prefetch run.
// The wait gives up after two seconds, or at once if an error is already recorded, and records DC_ERR_EP_WAIT.
#define DC_ERR_EP_WAIT 3
#define MG_EP_WAIT_NS 2000000000ull
#define MG_XCNT_WORD 32          // word index of the arrival counter in an exchange buffer's flag area
__device__ __forceinline__ void red_release_sys_add(unsigned* p, unsigned v) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// after the CTA's __syncthreads (grid_arrive): tell the peers
__device__ __forceinline__ void ep_arrive(const MegaParams& p) {
    const int r = threadIdx.x;
    // (the release half of the reduction orders the rows stored before the CTA barrier ahead of the arrival: no
    // separate system-scope fence)
    if (r < p.ep_size && r != p.ep_rank) red_release_sys_add(p.xcnt[r], 1u);
}
// exchanges: how many have completed once this one has (all ranks count alike)
__device__ __noinline__ bool ep_wait(const MegaParams& p, unsigned exchanges) {
    __shared__ int s_gave_up;
    if (threadIdx.x == 0) {
        const unsigned target = exchanges * (unsigned)(p.ep_size - 1) * gridDim.x;
        const unsigned long long t0 = mg_now();
        int gave_up = 0;
        // the counter only grows; the difference is taken modulo 2^32
        while ((int)(ld_acquire_sys_u32(p.my_xcnt) - target) < 0) {
            if (*reinterpret_cast<volatile int*>(p.err) != 0 || mg_now() - t0 > p.ep_wait_ns) {
                atomicExch(p.err, DC_ERR_EP_WAIT);
                gave_up = 1;
                break;
            }
            __nanosleep(32);
        }
        s_gave_up = gave_up;
    }
    __syncthreads();
    return s_gave_up != 0;
}

// Every CTA reads the same small arrays (hidden state, expert outputs, attention
// output) at the same moment; walking them from a CTA-dependent starting point keeps
// the 148 SMs off the same L2 lines.  Returns a multiple of 32 in [0, n).
__device__ __forceinline__ int cta_rotation(int n) {
    const int step = max(32, (n / (int)gridDim.x) & ~31);
    return (int)(((long long)blockIdx.x * step) % n) & ~31;
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

// Eight consecutive elements of a token-embedding row; out of line and rolled, since it runs
// once per step and its decode is long.
struct Float8 {
    float v[8];
};
__device__ __noinline__ Float8 embed_row8(const uint8_t* row, int type, int e0) {
    Float8 r;
#pragma unroll 1
    for (int i = 0; i < 8; ++i) {
        const float x = embed_elem(row, type, e0 + i);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (j == i) r.v[j] = x;
    }
    return r;
}

// A q head sits in shared memory as four 32-dim quarters 36 floats apart: the four lanes of a
// key read the same offset of different quarters, which then fall into different banks.
#define MG_SQ_QUARTER 36

// Shared state of one CTA that outlives a phase.
struct MegaShared {
    int32_t ids[MG_MAX_T * MG_MAX_K];      // routing of the current layer (kept for the combine in the next P0)
    float w[MG_MAX_T * MG_MAX_K];
    int32_t uexp[MG_MAX_E];
    int32_t uoff[MG_MAX_E + 1];
    int32_t uassign[MG_MAX_T * MG_MAX_K];
    int n_active;
    alignas(8) double red[MG_WARPS][MG_MAX_T];
    alignas(8) double red2[32];            // sum of squares per (token, block)
    int wsum_a[MG_WARPS], wsum_c[MG_WARPS];
    // attention
    alignas(16) float sq[8][4 * MG_SQ_QUARTER];   // q heads; each 32-dim quarter padded (bank spread)
    float suffix[8];
    int last;
    MegaLayer layer[2];                    // descriptor of the current layer and the next one
    // parameter blocks of the streaming phases (shared, so that no thread keeps a private copy)
    GemvParams g_qkv, g_o, g_lm;
    MoeMMParams m_gu, m_dn;
    // per-step constants of this CTA's attention item
    int32_t tbl[MG_MAX_RUN_BLOCKS];        // physical ids of the run's KV blocks
    alignas(16) float cs[128];             // RoPE cos/sin row of the item's token
    alignas(8) unsigned long long rkeys[MG_MAX_T][MG_MAX_E];   // routing keys (rank selection)
    float sel[MG_MAX_T][MG_MAX_K];         // logits (or probabilities) of the picks, in pick order
    float prob[MG_MAX_T][MG_MAX_E];        // generic router: exponentials of all experts
    int rng[MG_WARPS][2];                  // row range of each warp's stream between its prefill and its consume
};

// Dynamic shared memory the kernel may ask for: what the SM offers a CTA (227 KB) less the
// kernel's static shared memory (MegaShared and its copy of the parameters).
static constexpr uint32_t MG_DYN_LIMIT =
    (227u * 1024u - (uint32_t)sizeof(MegaShared) - (uint32_t)sizeof(MegaParams) - 256u) & ~127u;

// Hidden state -> RMSNorm -> Q8_K, one warp per (token, 256-value block), values held
// in registers (lane l: 8 consecutive values).
//   src 0: token-embedding rows (first layer)
//   src 1: x_in + the pending MoE output: the token's assignments are added one at a time
//          in routing order into a zeroed sum (core/src/backend/cpu_backend_moe_ops.cpp:1578-1597),
//          then the residual add
//   src 2: x_in as it is
// The block's owner CTA also writes the assembled values to x_out.  Norm:
// y = x / sqrt(mean(x^2) + eps) * w with the sum of squares in double
// (core/src/llm/graph/decoder.cpp:268), then the Q8_K quantiser
// (core/src/kernels/hwy/hwy_moe_quant.cc:103-144) straight into the activation layout;
// xn (optional) receives the normed f32 rows in shared memory.  T * H/256 <= 32.
// NPI (token, block) pairs per warp: T * H/256 <= 16 * NPI.
template <int NPI>
__device__ __noinline__ void x_norm_phase(const MegaParams& p, MegaShared& sh, int src, const float* x_in, float* x_out,
                                          const float* w, const ActSmem& act, float* xn, const float* dn) {
    const int H = p.H, nb = H / DC_QK_K, pairs = p.T * nb;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float v[NPI][8];
    float4 wv[NPI][2];
#pragma unroll
    for (int pi = 0; pi < NPI; ++pi) {
        const int pr = warp + pi * MG_WARPS;
        if (pr >= pairs) continue;
        const int t = pr / nb, b = pr - t * nb, dd = b * DC_QK_K + 8 * lane;
        // norm weights first: their load overlaps everything below
        wv[pi][0] = *reinterpret_cast<const float4*>(w + dd);
        wv[pi][1] = *reinterpret_cast<const float4*>(w + dd + 4);
        if (src == 0) {
            int tok = __ldcg(p.tokens + t);
            if (tok < 0 || tok >= p.vocab) tok = 0;
            const uint8_t* row = p.tok_embd + (size_t)tok * p.embd_row_bytes;
            const Float8 e8 = embed_row8(row, p.embd_type, dd);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[pi][i] = e8.v[i];
        } else {
            const float4 x0 = __ldcg(reinterpret_cast<const float4*>(x_in + (size_t)t * H + dd));
            const float4 x1 = __ldcg(reinterpret_cast<const float4*>(x_in + (size_t)t * H + dd + 4));
            v[pi][0] = x0.x; v[pi][1] = x0.y; v[pi][2] = x0.z; v[pi][3] = x0.w;
            v[pi][4] = x1.x; v[pi][5] = x1.y; v[pi][6] = x1.z; v[pi][7] = x1.w;
            if (src == 1) {
                float sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                for (int k0 = 0; k0 < p.top_k; k0 += 4) {
                    float4 d0[4], d1[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {   // four experts' rows in flight
                        const int k = min(k0 + j, p.top_k - 1);
                        const float* dr = dn + (size_t)(t * p.top_k + k) * H + dd;
                        d0[j] = __ldcg(reinterpret_cast<const float4*>(dr));
                        d1[j] = __ldcg(reinterpret_cast<const float4*>(dr + 4));
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (k0 + j < p.top_k) {
                            const float wk = sh.w[t * p.top_k + k0 + j];
                            if (wk != 0.0f) {
                                sum[0] = __fadd_rn(sum[0], __fmul_rn(wk, d0[j].x));
                                sum[1] = __fadd_rn(sum[1], __fmul_rn(wk, d0[j].y));
                                sum[2] = __fadd_rn(sum[2], __fmul_rn(wk, d0[j].z));
                                sum[3] = __fadd_rn(sum[3], __fmul_rn(wk, d0[j].w));
                                sum[4] = __fadd_rn(sum[4], __fmul_rn(wk, d1[j].x));
                                sum[5] = __fadd_rn(sum[5], __fmul_rn(wk, d1[j].y));
                                sum[6] = __fadd_rn(sum[6], __fmul_rn(wk, d1[j].z));
                                sum[7] = __fadd_rn(sum[7], __fmul_rn(wk, d1[j].w));
                            }
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) v[pi][i] = __fadd_rn(v[pi][i], sum[i]);
            }
        }
        if (x_out && src != 2 && (pr % (int)gridDim.x) == (int)blockIdx.x) {
            float* o = x_out + (size_t)t * H + dd;
            *reinterpret_cast<float4*>(o) = make_float4(v[pi][0], v[pi][1], v[pi][2], v[pi][3]);
            *reinterpret_cast<float4*>(o + 4) = make_float4(v[pi][4], v[pi][5], v[pi][6], v[pi][7]);
        }
        double ss = 0.0;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += (double)v[pi][i] * (double)v[pi][i];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) sh.red2[pr] = ss;
    }
    __syncthreads();
#pragma unroll
    for (int pi = 0; pi < NPI; ++pi) {
        const int pr = warp + pi * MG_WARPS;
        if (pr >= pairs) continue;
        const int t = pr / nb, b = pr - t * nb;
        double tot = 0.0;
        for (int i = 0; i < nb; ++i) tot += sh.red2[t * nb + i];
        // (a power-of-two width divides exactly either way; the multiplication spares a double-precision division)
        const float mean = (H & (H - 1)) == 0 ? (float)(tot * (1.0 / (double)H)) : (float)(tot / (double)H);
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, p.eps)));
        const float ww[8] = {wv[pi][0].x, wv[pi][0].y, wv[pi][0].z, wv[pi][0].w,
                             wv[pi][1].x, wv[pi][1].y, wv[pi][1].z, wv[pi][1].w};
        float y[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = __fmul_rn(__fmul_rn(v[pi][i], scale), ww[i]);
        if (xn) {
            float* o = xn + t * H + b * DC_QK_K + 8 * lane;
            *reinterpret_cast<float4*>(o) = make_float4(y[0], y[1], y[2], y[3]);
            *reinterpret_cast<float4*>(o + 4) = make_float4(y[4], y[5], y[6], y[7]);
        }
        quantize_block_q8k_to_act(y, act, t, b, lane);
    }
    __syncthreads();
}

// Parity capture: the CTAs that own a (token, 256-value block) of the hidden state copy the rows they have
// just written to x into capture slot `slot`.  Out of line: it only runs when a test asked for it.
__device__ __noinline__ void mg_capture_x(const MegaParams& p, const float* x, int slot) {
    const int nb = p.H / DC_QK_K, pairs = p.T * nb;
    float* dst = p.dbg_x + (size_t)slot * DC_MAX_T * p.H;
    for (int pr = blockIdx.x; pr < pairs; pr += gridDim.x) {
        const int t = pr / nb, b = pr - t * nb;
        if (threadIdx.x < 64) {
            const size_t o = (size_t)t * p.H + b * DC_QK_K + 4 * threadIdx.x;
            *reinterpret_cast<float4*>(dst + o) = __ldcg(reinterpret_cast<const float4*>(x + o));
        }
    }
}

// ------------------------------------------------------------ attention
__device__ __forceinline__ unsigned long long mg_now();
#ifdef DC_MEGA_SUBMARKS
#define MG_SUB(i)                                                             \
    do {                                                                      \
        if (p.phase_ns && blockIdx.x == 0 && threadIdx.x == 0) {              \
            const unsigned long long _n = mg_now();                           \
            p.phase_ns[i] += _n - sub_t;                                      \
            sub_t = _n;                                                       \
        }                                                                     \
    } while (0)
#define MG_SUB_BEGIN unsigned long long sub_t = mg_now()
// when every warp of every CTA passes point i of the second layer in the first step of a launch
#define MG_WTRACE(i)                                                                                       \
    do {                                                                                                   \
        if (p.phase_ns && lane == 0 && l == 1 && step == 0)                                                \
            p.phase_ns[MG_WTRACE_BASE + (i) * 2560 + blockIdx.x * MG_WARPS + warp] = mg_now();             \
    } while (0)
#else
#define MG_WTRACE(i) do {} while (0)
#define MG_SUB(i) do {} while (0)
#define MG_SUB_BEGIN do {} while (0)
#endif
// One attention run: token t, kv head kvh, head group hg (gh query heads starting at head hb of the
// kv head's group), KV blocks [b0, b1).
struct AttnItem {
    bool valid;
    int t, kvh, hg, hb, gh, split, pos, ctx_len, n_blk, b0, b1;
    const int32_t* table;
};

__device__ __forceinline__ AttnItem attn_item(const MegaParams& p) {
    AttnItem it;
    const int items = p.T * p.n_kv * p.n_hg * p.nsplit, item = blockIdx.x;
    it.valid = item < items;
    const int i = it.valid ? item : 0;
    it.split = i % p.nsplit;
    it.hg = (i / p.nsplit) % p.n_hg;
    it.kvh = (i / (p.nsplit * p.n_hg)) % p.n_kv;
    it.t = i / (p.nsplit * p.n_hg * p.n_kv);
    it.gh = (p.n_head / p.n_kv) / p.n_hg;
    it.hb = it.hg * it.gh;
    it.pos = __ldcg(p.positions + it.t);
    it.ctx_len = it.pos + 1;
    it.n_blk = (it.ctx_len + DC_KV_BLOCK - 1) / DC_KV_BLOCK;
    const int bps = (it.n_blk + p.nsplit - 1) / p.nsplit;
    it.b0 = min(it.n_blk, it.split * bps);
    it.b1 = min(it.n_blk, it.b0 + bps);
    it.table = p.block_tables + (size_t)p.seq_ids[it.t] * p.max_blocks;
    return it;
}

// Once per step: the item of this CTA, the physical ids of its KV blocks and the
// RoPE row of its token go to registers / shared memory, so the attention phases
// of all layers start without dependent global loads.
__device__ __forceinline__ AttnItem attn_step_setup(const MegaParams& p, MegaShared& sh) {
    const AttnItem it = attn_item(p);
    if (it.valid) {
        for (int i = threadIdx.x; i < it.b1 - it.b0; i += MG_THREADS) sh.tbl[i] = it.table[it.b0 + i];
        const int pos = min(it.pos, p.max_pos - 1);
        if (threadIdx.x < 128) sh.cs[threadIdx.x] = p.cos_sin[(size_t)pos * 128 + threadIdx.x];
    }
    __syncthreads();
    return it;
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

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

// One K row slice (32 of 128 dims) of key kk of the run, as loaded (fp16 pairs).  The row of the
// token being decoded (kpos == pos) is written by this CTA during the phase: it is flagged `late`
// and fetched after the CTA barrier instead.  Keys outside the run or the context read as zeros.
__device__ __forceinline__ void mg_load_k_raw(const MegaParams& p, const MegaLayer& L, const MegaShared& sh,
                                              const AttnItem& it, int n_keys, int kk, int sub, uint4 (&kr)[4],
                                              bool& valid, bool& late) {
    const int blk = kk / DC_KV_BLOCK, kpos = (it.b0 + blk) * DC_KV_BLOCK + kk % DC_KV_BLOCK;
    valid = kk < n_keys && kpos < it.ctx_len;
    late = valid && kpos == it.pos;
    if (valid && !late) {
        const uint4* kp = reinterpret_cast<const uint4*>(
            L.k_arena + (((size_t)sh.tbl[blk] * DC_KV_BLOCK + kk % DC_KV_BLOCK) * p.n_kv + it.kvh) * 128 + sub * 32);
#pragma unroll
        for (int i = 0; i < 4; ++i) kr[i] = __ldcg(kp + i);
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) kr[i] = make_uint4(0u, 0u, 0u, 0u);
    }
}
__device__ __forceinline__ void mg_k_to_float(const uint4 (&kr)[4], float (&kf)[32]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2* h2 = reinterpret_cast<const __half2*>(&kr[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(h2[j]);
            kf[i * 8 + 2 * j] = f.x;
            kf[i * 8 + 2 * j + 1] = f.y;
        }
    }
}

// Phase 1: Q/K norm + RoPE, K/V of the new token into the paged cache (by the run
// that owns its block), scores of this run into shared memory, block maxima to global.
// The run's V rows are requested here (16-byte async copies into vbuf) so that the
// P.V phase finds them in shared memory.
__device__ DC_HOT void attn_scores_phase(const MegaParams& p, const MegaLayer& L, MegaShared& sh,
                                                  const AttnItem& it, float* s_sc, uint8_t* vbuf, int vcap_blocks) {
    if (!it.valid) return;
    // g: query heads of this run (a head group of the kv head); head0: the first of them
    const int g = it.gh, head0 = it.kvh * (p.n_head / p.n_kv) + it.hb, heads = p.n_head + 2 * p.n_kv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float* qkv_t = p.qkv + (size_t)it.t * heads * 128;
    const bool owner = (it.pos / DC_KV_BLOCK) >= it.b0 && (it.pos / DC_KV_BLOCK) < it.b1;
    const int nb_run = it.b1 - it.b0, n_keys = nb_run * DC_KV_BLOCK;
    MG_SUB_BEGIN;
    // ---- V rows of the run: block bb, slot s, 16 chunks of 16 bytes
    {
        const int nst = min(nb_run, vcap_blocks) * DC_KV_BLOCK * 16;
        const uint32_t vb = smem_u32(vbuf);
        for (int i = threadIdx.x; i < nst; i += MG_THREADS) {
            const int bb = i >> 8, slot = (i >> 4) & 15, ch = i & 15;
            const __half* src = L.v_arena + (((size_t)sh.tbl[bb] * DC_KV_BLOCK + slot) * p.n_kv + it.kvh) * 128 + ch * 8;
            cp_async16(vb + (uint32_t)i * 16, src);
        }
        cp_async_commit();
    }
    MG_SUB(22);
    // ---- first pass of K rows: history keys are loaded before anything else
    // warp -> (group of 8 keys, group of heads): with few keys in the run the heads are spread
    // over the warps instead, so that all 16 warps share the work
    int KG = 1;
    while (KG < MG_WARPS && KG * 8 < n_keys) KG <<= 1;
    const int HG = MG_WARPS / KG, kgi = warp & (KG - 1), hgi = warp / KG;
    const int hpg = (g + HG - 1) / HG, h0 = min(g, hgi * hpg), h1 = min(g, h0 + hpg);
    uint4 kr[4];
    bool valid = false, late = false;
    if (h0 < h1) mg_load_k_raw(p, L, sh, it, n_keys, kgi * 8 + (lane >> 2), lane & 3, kr, valid, late);
    MG_SUB(23);
    // ---- q heads, and the new token's K/V rows
    if (warp < g) {
        const float4 v4 = __ldcg(reinterpret_cast<const float4*>(qkv_t + (size_t)(head0 + warp) * 128) + lane);
        float v[4] = {v4.x, v4.y, v4.z, v4.w};
        head_norm_rope(v, L.q_norm, sh.cs, p.eps, lane, true);
        *reinterpret_cast<float4*>(&sh.sq[warp][(lane >> 3) * MG_SQ_QUARTER + (lane & 7) * 4]) = make_float4(v[0], v[1], v[2], v[3]);
    } else if (owner && (warp == g || warp == g + 1)) {
        const bool is_k = warp == g;
        const int hh = is_k ? p.n_head + it.kvh : p.n_head + p.n_kv + it.kvh;
        const float4 v4 = __ldcg(reinterpret_cast<const float4*>(qkv_t + (size_t)hh * 128) + lane);
        float v[4] = {v4.x, v4.y, v4.z, v4.w};
        if (is_k) head_norm_rope(v, L.k_norm, sh.cs, p.eps, lane, true);
        const int blk = sh.tbl[it.pos / DC_KV_BLOCK - it.b0];
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
    MG_SUB(24);
    if (h0 < h1) {
        float kf[32];
        for (int k0 = 0; k0 + kgi * 8 < n_keys; k0 += KG * 8) {
            const int kk = k0 + kgi * 8 + (lane >> 2), sub = lane & 3;
            if (late) {   // this CTA wrote the row before the barrier above
                const int blk = kk / DC_KV_BLOCK;
                const uint4* kp = reinterpret_cast<const uint4*>(
                    L.k_arena + (((size_t)sh.tbl[blk] * DC_KV_BLOCK + kk % DC_KV_BLOCK) * p.n_kv + it.kvh) * 128 + sub * 32);
#pragma unroll
                for (int i = 0; i < 4; ++i) kr[i] = __ldcg(kp + i);
            }
            mg_k_to_float(kr, kf);
            const bool cur_valid = valid;
            // the next pass's rows are requested before this pass's dot products
            if (k0 + KG * 8 + kgi * 8 < n_keys) mg_load_k_raw(p, L, sh, it, n_keys, kk + KG * 8, sub, kr, valid, late);
            // one head at a time, rolled: the loop body is small and stays in the instruction cache
#pragma unroll 1
            for (int h = h0; h < h1; ++h) {
                const float4* qp = reinterpret_cast<const float4*>(&sh.sq[h][sub * MG_SQ_QUARTER]);
                float dot = 0.0f;
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
                if (sub == 0 && kk < n_keys) s_sc[h * p.s_keys + kk] = cur_valid ? __fmul_rn(dot, p.scale) : -INFINITY;
            }
        }
    }
    __syncthreads();
    MG_SUB(25);
    for (int i = threadIdx.x; i < g * nb_run; i += MG_THREADS) {
        const int h = i / nb_run, bb = i - h * nb_run;
        float mx = -1e30f;
#pragma unroll
        for (int k = 0; k < DC_KV_BLOCK; ++k) mx = fmaxf(mx, s_sc[h * p.s_keys + bb * DC_KV_BLOCK + k]);
        p.bmax[((size_t)it.t * p.n_head + head0 + h) * p.max_blocks + it.b0 + bb] = mx;
    }
}

// Phase 2: the reference's running-maximum chain from all block maxima, this run's
// blocks accumulated as the reference walks them, partial scaled by the alphas of
// all later blocks; the last run of a (token, kv head, head group) sums the partials and
// emits the Q8_K blocks of the attention output (hwy_paged_attention.cc:428-629).
// Every block's running maximum and rescale factor follow from the block maxima alone, so
// they are computed for the whole run first (one warp per head); then all exponentials in
// parallel; then one pass over the keys with no barrier inside.
__device__ DC_HOT void attn_pv_phase(const MegaParams& p, const MegaLayer& L, MegaShared& sh,
                                              const AttnItem& it, const float* s_sc, const uint8_t* vbuf,
                                              int vcap_blocks) {
#ifdef DC_MEGA_SUBMARKS
    const unsigned long long pv_t0 = mg_now();
#endif
    cp_async_wait_all();   // this thread's V copies of the scores phase have landed
    if (!it.valid) return;
    const int g = it.gh, head0 = it.kvh * (p.n_head / p.n_kv) + it.hb;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nb_run = it.b1 - it.b0;
    // per (head, block of the run): running maximum after the block, rescale factor, sum of the
    // block's exponentials (the routing keys' space is idle during attention)
    static_assert(sizeof(sh.rkeys) >= 3 * 8 * MG_MAX_RUN_BLOCKS * sizeof(float), "per-block attention state");
    float* bl_mnew = reinterpret_cast<float*>(sh.rkeys);
    float* bl_alpha = bl_mnew + 8 * MG_MAX_RUN_BLOCKS;
    float* bl_ps = bl_alpha + 8 * MG_MAX_RUN_BLOCKS;
    float* pw = const_cast<float*>(s_sc);   // scores become exponentials in place
    for (int h = warp; h < g; h += MG_WARPS) {
        const float* bm = p.bmax + ((size_t)it.t * p.n_head + head0 + h) * p.max_blocks;
        // blocks before the run only feed the running maximum; the run's blocks get their maximum and
        // rescale factor; the factors of later blocks multiply into the suffix.  The block maxima are
        // fetched 256 at a time so that their loads overlap.
        float carry = -1e30f, suffix = 1.0f;
        for (int s0 = 0; s0 < it.n_blk; s0 += 256) {
            float vb[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int c = s0 + 32 * k + lane;
                vb[k] = c < it.n_blk ? __ldcg(bm + c) : -1e30f;
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int c0 = s0 + 32 * k, c = c0 + lane;
                if (c0 >= it.n_blk) break;
                if (c0 + 32 <= it.b0) {   // wholly before the run
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
                const float a = (c >= it.b0 && c < it.n_blk) ? fast_exp_fma(m_prev - m_new) : 1.0f;
                if (c >= it.b0 && c < it.b1) {
                    bl_mnew[h * MG_MAX_RUN_BLOCKS + c - it.b0] = m_new;
                    bl_alpha[h * MG_MAX_RUN_BLOCKS + c - it.b0] = a;
                }
                if (c0 + 32 > it.b1) {   // the chunk reaches past the run
                    float later = c >= it.b1 ? a : 1.0f;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) later *= __shfl_xor_sync(0xffffffffu, later, o);
                    suffix *= later;
                }
                carry = fmaxf(carry, __shfl_sync(0xffffffffu, incl, 31));
            }
        }
        if (lane == 0) sh.suffix[h] = suffix;
    }
    __syncthreads();   // every thread's async copies are complete and visible; block state is set
    {
        // the new token's V row was written during the scores phase, possibly after its
        // async copy was issued: the owning run copies that one row again
        const int pb_new = it.pos / DC_KV_BLOCK - it.b0;
        if (pb_new >= 0 && pb_new < nb_run && pb_new < vcap_blocks && tid < 16) {
            const int slot = it.pos % DC_KV_BLOCK;
            const uint4* src = reinterpret_cast<const uint4*>(
                L.v_arena + (((size_t)sh.tbl[pb_new] * DC_KV_BLOCK + slot) * p.n_kv + it.kvh) * 128) + tid;
            reinterpret_cast<uint4*>(const_cast<uint8_t*>(vbuf))[(pb_new * DC_KV_BLOCK + slot) * 16 + tid] = __ldcg(src);
        }
    }
    // exponentials: 16 lanes per (head, block)
    for (int base = 0; base < g * nb_run; base += MG_THREADS / 16) {
        const int pair = base + (tid >> 4), key = tid & 15;
        const bool in = pair < g * nb_run;
        const int h = in ? pair / nb_run : 0, bl = in ? pair - h * nb_run : 0;
        const int nk = min(DC_KV_BLOCK, it.ctx_len - (it.b0 + bl) * DC_KV_BLOCK);
        const float s = (in && key < nk) ? pw[h * p.s_keys + bl * DC_KV_BLOCK + key] : -INFINITY;
        const float pr = (s == -INFINITY) ? 0.0f : fast_exp_fma(s - bl_mnew[h * MG_MAX_RUN_BLOCKS + bl]);
        float ps = pr;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        if (in) {
            pw[h * p.s_keys + bl * DC_KV_BLOCK + key] = pr;
            if (key == 0) bl_ps[h * MG_MAX_RUN_BLOCKS + bl] = ps;
        }
    }
    __syncthreads();
    // thread -> (dim, two heads): heads hq and hq + 4
    const int dim = tid & 127, hq = tid >> 7;
    const bool h0 = hq < g, h1 = hq + 4 < g;
    float acc0 = 0.0f, acc1 = 0.0f, d0 = 0.0f, d1 = 0.0f;
    const __half* vs = reinterpret_cast<const __half*>(vbuf);
    const float* p0 = pw + hq * p.s_keys;
    const float* p1 = pw + (hq + 4) * p.s_keys;
    for (int bl = 0; bl < nb_run; ++bl) {
        const int nk = min(DC_KV_BLOCK, it.ctx_len - (it.b0 + bl) * DC_KV_BLOCK);
        if (h0) {
            const float a = bl_alpha[hq * MG_MAX_RUN_BLOCKS + bl];
            if (a != 1.0f) acc0 *= a;
            if (dim == 0) d0 = d0 * a + bl_ps[hq * MG_MAX_RUN_BLOCKS + bl];
        }
        if (h1) {
            const float a = bl_alpha[(hq + 4) * MG_MAX_RUN_BLOCKS + bl];
            if (a != 1.0f) acc1 *= a;
            if (dim == 0) d1 = d1 * a + bl_ps[(hq + 4) * MG_MAX_RUN_BLOCKS + bl];
        }
        if (bl < vcap_blocks) {
            // all 16 V values and exponentials of the block are fetched first, then added in key order
            const __half* vrow = vs + (size_t)bl * DC_KV_BLOCK * 128 + dim;
            float vv[DC_KV_BLOCK];
#pragma unroll
            for (int key = 0; key < DC_KV_BLOCK; ++key) vv[key] = __half2float(vrow[key * 128]);
            if (h0) {
                float pp[DC_KV_BLOCK];
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    *reinterpret_cast<float4*>(&pp[4 * q]) = *reinterpret_cast<const float4*>(p0 + bl * DC_KV_BLOCK + 4 * q);
#pragma unroll
                for (int key = 0; key < DC_KV_BLOCK; ++key)
                    if (key < nk) acc0 = fmaf(pp[key], vv[key], acc0);
            }
            if (h1) {
                float pp[DC_KV_BLOCK];
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    *reinterpret_cast<float4*>(&pp[4 * q]) = *reinterpret_cast<const float4*>(p1 + bl * DC_KV_BLOCK + 4 * q);
#pragma unroll
                for (int key = 0; key < DC_KV_BLOCK; ++key)
                    if (key < nk) acc1 = fmaf(pp[key], vv[key], acc1);
            }
        } else {
            const __half* vb = L.v_arena + ((size_t)sh.tbl[bl] * DC_KV_BLOCK * p.n_kv + it.kvh) * 128 + dim;
#pragma unroll 4
            for (int key = 0; key < nk; ++key) {
                const float v = __half2float(
                    __ushort_as_half(__ldcg(reinterpret_cast<const unsigned short*>(vb + (size_t)key * p.n_kv * 128))));
                if (h0) acc0 = fmaf(p0[bl * DC_KV_BLOCK + key], v, acc0);
                if (h1) acc1 = fmaf(p1[bl * DC_KV_BLOCK + key], v, acc1);
            }
        }
    }
    if (h0) {
        const size_t idx = ((size_t)it.t * p.n_head + head0 + hq) * p.nsplit + it.split;
        p.part_acc[idx * 128 + dim] = acc0 * sh.suffix[hq];
        if (dim == 0) p.part_d[idx] = d0 * sh.suffix[hq];
    }
    if (h1) {
        const size_t idx = ((size_t)it.t * p.n_head + head0 + hq + 4) * p.nsplit + it.split;
        p.part_acc[idx * 128 + dim] = acc1 * sh.suffix[hq + 4];
        if (dim == 0) p.part_d[idx] = d1 * sh.suffix[hq + 4];
    }
    // release: the CTA barrier puts every thread's partial before thread 0's ticket, whose release half publishes
    // them; acquire: the last run's thread 0 sees the other runs' partials through the ticket's acquire half, and the
    // CTA barrier passes that on
    __syncthreads();
    int* ticket = p.tickets + (it.t * p.n_kv + it.kvh) * p.n_hg + it.hg;
    if (tid == 0) {
        int old;
        asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], %2;" : "=r"(old) : "l"(ticket), "r"(1) : "memory");
        const bool last = old == p.nsplit - 1;
        if (last) *ticket = 0;
        sh.last = last;
    }
    __syncthreads();
    if (!sh.last) return;
#ifdef DC_MEGA_SUBMARKS
    const unsigned long long merge_t0 = mg_now();
#endif
    // every thread sums two neighbouring outputs of one head over the runs in run order, with 16 runs'
    // loads in flight at a time; the sums meet in shared memory (the score buffer is idle by now) and
    // one warp per 256-value block quantises them
    float* merged = const_cast<float*>(s_sc);
    for (int o2 = tid; o2 < g * 64; o2 += MG_THREADS) {
        const int h = o2 >> 6, d0 = (o2 & 63) * 2;
        const size_t base = ((size_t)it.t * p.n_head + head0 + h) * p.nsplit;
        float v0 = 0.0f, v1 = 0.0f, den = 0.0f;
        for (int s0 = 0; s0 < p.nsplit; s0 += 16) {
            float dd[16];
            float2 a[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const bool in = s0 + j < p.nsplit;
                const size_t bi = base + (in ? s0 + j : 0);
                dd[j] = __ldcg(p.part_d + bi);
                a[j] = __ldcg(reinterpret_cast<const float2*>(p.part_acc + bi * 128 + d0));
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                if (s0 + j < p.nsplit) {
                    den += dd[j];
                    v0 += a[j].x;
                    v1 += a[j].y;
                }
            }
        }
        const float inv = (den > 0.0f && isfinite(den)) ? __fdiv_rn(1.0f, __fadd_rn(den, 1e-6f)) : 0.0f;
        *reinterpret_cast<float2*>(merged + h * 128 + d0) = make_float2(v0 * inv, v1 * inv);
    }
    __syncthreads();
    for (int pb2 = warp; pb2 < g / 2; pb2 += MG_WARPS) {
        const float4 x0 = *reinterpret_cast<const float4*>(merged + pb2 * 256 + lane * 8);
        const float4 x1 = *reinterpret_cast<const float4*>(merged + pb2 * 256 + lane * 8 + 4);
        const float v[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
        quantize_block_q8k_regs(v, p.q8_attn + ((size_t)it.t * (p.n_head / 2) + head0 / 2 + pb2) * DC_Q8K_BYTES, lane);
    }
#ifdef DC_MEGA_SUBMARKS
    if (p.phase_ns && tid == 0 && it.t == 0 && it.kvh == 0 && it.hg == 0) {
        p.phase_ns[26] += mg_now() - merge_t0;      // the merge itself
        p.phase_ns[27] += merge_t0 - pv_t0;         // from the start of the phase to the ticket
    }
#endif
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
__device__ DC_HOT void router_logits_phase(const MegaParams& p, const MegaLayer& L, MegaShared& sh,
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

// Generic router, first half: softmax over all experts (expf(x - max), sum in index order, times 1/sum:
// core/include/densecore/simd/simd_ops.h:1171-1195); the ranks are then taken on the probabilities.  The
// exponential is the double-precision one rounded to float, which is what the host's expf returns.  Out of
// line: the double-precision code would otherwise weigh on the registers of every phase inlined next to it.
__device__ __noinline__ void mg_softmax_keys(const MegaParams& p, MegaShared& sh) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp >= p.T) return;
    const int t = warp;
    float mx = -INFINITY;
    for (int e = lane; e < p.E; e += 32) mx = fmaxf(mx, __ldcg(p.router_logits + t * p.E + e));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    for (int e = lane; e < p.E; e += 32)
        sh.prob[t][e] = (float)exp((double)__fsub_rn(__ldcg(p.router_logits + t * p.E + e), mx));
    __syncwarp();
    float sum = 0.0f;
    if (lane == 0)
        for (int e = 0; e < p.E; ++e) sum = __fadd_rn(sum, sh.prob[t][e]);
    sum = __shfl_sync(0xffffffffu, sum, 0);
    const float inv = __fdiv_rn(1.0f, sum);
    for (int e = lane; e < p.E; e += 32) sh.rkeys[t][e] = mg_route_key(__fmul_rn(sh.prob[t][e], inv), e);
}

// Every CTA routes all tokens itself from the logits in global memory: stable top-k
// on logits, weights over the selected experts (core/src/llm/moe/native.cpp:610-676),
// then the expert-grouped assignment map (core/src/moe/moe_routing.cpp:534-603).
__device__ DC_HOT void route_phase(const MegaParams& p, MegaShared& sh) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // rank selection: thread (t, e) counts the candidates that precede its own
    // ("larger logit first, then lower id, NaN last"); the k best have ranks 0..k-1
    if (p.route_mode == DC_ROUTE_SOFTMAX) {
        mg_softmax_keys(p, sh);
    } else {
        for (int i = threadIdx.x; i < p.T * p.E; i += MG_THREADS) {
            const int t = i / p.E, e = i - t * p.E;
            sh.rkeys[t][e] = mg_route_key(__ldcg(p.router_logits + i), e);
        }
    }
    __syncthreads();
    {
        // Q neighbouring lanes share one candidate: each counts part of the row, a shuffle adds up
        const int TE = p.T * p.E;
        int Q = 1;
        while (Q < 32 && TE * Q * 2 <= MG_THREADS) Q <<= 1;
        for (int base = 0; base < TE; base += MG_THREADS / Q) {
            const int i = base + (int)threadIdx.x / Q, part = (int)threadIdx.x % Q;
            const bool in = i < TE;
            const int t = in ? i / p.E : 0, e = in ? i - t * p.E : 0;
            const unsigned long long mine = sh.rkeys[t][e];
            int rank = 0;
            if (in)
                for (int j = part; j < p.E; j += Q) rank += (sh.rkeys[t][j] > mine);
            for (int o = Q >> 1; o > 0; o >>= 1) rank += __shfl_xor_sync(0xffffffffu, rank, o);
            if (in && part == 0 && rank < p.top_k) {
                sh.ids[t * p.top_k + rank] = e;
                // the logit back out of the key (NaN stays NaN; -0 was made +0, which exp treats alike)
                const uint32_t u = (uint32_t)(mine >> 32);
                sh.sel[t][rank] = __uint_as_float((u & 0x80000000u) ? (u & 0x7FFFFFFFu) : ~u);
            }
        }
    }
    __syncthreads();
    if (warp < p.T) {
        // weights over the selected experts (native.cpp:649-674): exponentials side by side, the sum in
        // pick order as the reference adds them
        const int t = warp;
        const float v = lane < p.top_k ? sh.sel[t][lane] : -INFINITY;
        if (p.route_mode == DC_ROUTE_SOFTMAX) {
            // renormalise over the picks in pick order, w * (1 / sum) (core/src/moe/moe_routing.cpp:90-101)
            float sum = 0.0f;
            for (int k = 0; k < p.top_k; ++k) sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, v, k));
            if (lane < p.top_k) {
                const float w = sum > 0.0f ? __fmul_rn(v, __fdiv_rn(1.0f, sum)) : v;
                sh.w[t * p.top_k + lane] = __fmul_rn(w, p.routed_scale);
            }
        } else {
        const bool fin_l = lane >= p.top_k || isfinite(v);
        const bool finite = __all_sync(0xffffffffu, fin_l);
        float mx = (lane < p.top_k && isfinite(v)) ? v : -INFINITY;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const bool use = finite && isfinite(mx);
        const float ev = (use && lane < p.top_k) ? expf(v - mx) : 0.0f;
        float den = 0.0f;
        for (int k = 0; k < p.top_k; ++k) den += __shfl_sync(0xffffffffu, ev, k);
        const bool ok = den > 0.0f && isfinite(den);
        if (lane < p.top_k) {
            const float w = ok ? __fdiv_rn(ev, den) : __fdiv_rn(1.0f, (float)p.top_k);
            sh.w[t * p.top_k + lane] = __fmul_rn(w, p.routed_scale);
        }
        }
    }
    __syncthreads();
    const int A = p.T * p.top_k, me = threadIdx.x;
    if (p.T == 1) {
        // one token: its experts are distinct, so each local one is a unit of its own; units are ordered by
        // expert id (position = number of local picks with a smaller id)
        if (me < p.top_k) {
            const int e = sh.ids[me];
            const bool local = e >= p.e_lo && e < p.e_hi;
            int posn = 0, n_local = 0;
            for (int j = 0; j < p.top_k; ++j) {
                const int ej = sh.ids[j];
                const bool lj = ej >= p.e_lo && ej < p.e_hi;
                n_local += lj;
                posn += (lj && ej < e);
            }
            if (local) {
                sh.uexp[posn] = e;
                sh.uoff[posn] = posn;
                sh.uassign[posn] = me;
            }
            if (me == 0) {
                sh.n_active = n_local;
                sh.uoff[n_local] = n_local;
            }
        }
        if (blockIdx.x == 0 && me < A) {
            if (p.route_ids) p.route_ids[me] = sh.ids[me];
            if (p.route_w) p.route_w[me] = sh.w[me];
        }
        __syncthreads();
        return;
    }
    // bucketing: thread e owns expert e (E <= 256 < 512 threads)
    int cnt = 0;
    if (me >= p.e_lo && me < p.e_hi)   // experts stored on this GPU
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
    }
    if (blockIdx.x == 0 && threadIdx.x < A) {
        if (p.route_ids) p.route_ids[threadIdx.x] = sh.ids[threadIdx.x];
        if (p.route_w) p.route_w[threadIdx.x] = sh.w[threadIdx.x];
    }
    __syncthreads();
}

// ------------------------------------------------------------ the kernel
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
// The whole CTA asks L2 for a small vector that a later phase will read (norm weights,
// this CTA's router row), 128 bytes per thread.
__device__ __forceinline__ void prefetch_vec(const void* base, size_t bytes) {
    if (!base) return;
    for (size_t o = (size_t)threadIdx.x * 128; o < bytes; o += (size_t)MG_THREADS * 128)
        prefetch_l2(reinterpret_cast<const uint8_t*>(base) + o);
}
// Copies one layer descriptor from global memory into shared slot `slot`.
__device__ __forceinline__ void load_layer(const MegaParams& p, MegaShared& sh, int l, int slot) {
    const uint32_t* src = reinterpret_cast<const uint32_t*>(p.layers + l);
    uint32_t* dst = reinterpret_cast<uint32_t*>(&sh.layer[slot]);
    for (int i = threadIdx.x; i < (int)(sizeof(MegaLayer) / 4); i += MG_THREADS) dst[i] = src[i];
}

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
    m.e_base = p.e_lo;
    m.n_peer = 0;
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

// The streaming matmul bodies are large; each is kept out of line and shared by all of its
// call sites so that one layer's instruction footprint stays small (the kernel runs the same
// code once per layer, and an instruction-cache miss costs a round trip to L2).
// A stream's row range is worked out once, when its first stages are requested, and kept in shared memory
// until the consuming phase picks it up (the partition arithmetic costs as much as a weight row).
__device__ __noinline__ void mg_gemv_prefill(const GemvParams& g, WarpPipe<MG_NSTAGE>& pipe, MegaShared& sh, int gw,
                                             int nw, int lane) {
    GemvStream<MG_NSTAGE> st;
    int r0, r1;
    GemvStream<MG_NSTAGE>::range(g, gw, nw, r0, r1);
    st.resume_range(g, r0, r1, 0);
    st.prefill(g, pipe, lane);
    if (lane == 0) {
        sh.rng[gw % MG_WARPS][0] = r0;
        sh.rng[gw % MG_WARPS][1] = r1;
    }
    __syncwarp();
}
template <int NT>
__device__ __noinline__ void mg_gemv_consume(const GemvParams& g, WarpPipe<MG_NSTAGE>& pipe, const ActSmem& act,
                                             const MegaShared& sh, int gw, int lane) {
    GemvStream<MG_NSTAGE> st;
    st.resume_range(g, sh.rng[gw % MG_WARPS][0], sh.rng[gw % MG_WARPS][1], (int)(pipe.issued - pipe.consumed));
    st.template consume<NT, false>(g, pipe, act, lane);
}
__device__ __noinline__ void mg_moe_prefill(const MoeMMParams& m, int U, WarpPipe<MG_NSTAGE>& pipe, MegaShared& sh, int gw,
                                            int nw, int lane) {
    MoeStream<MG_NSTAGE, 2> st;
    int r0, r1;
    MoeStream<MG_NSTAGE, 2>::range(m, U, gw, nw, r0, r1);
    st.resume_range(m, r0, r1, 0);
    st.prefill(m, pipe, lane);
    if (lane == 0) {
        sh.rng[gw % MG_WARPS][0] = r0;
        sh.rng[gw % MG_WARPS][1] = r1;
    }
    __syncwarp();
}
template <int NT>
__device__ __noinline__ void mg_moe_consume(const MoeMMParams& m, WarpPipe<MG_NSTAGE>& pipe, const ActSmem& act,
                                            const MegaShared& sh, int gw, int lane) {
    MoeStream<MG_NSTAGE, 2> st;
    st.resume_range(m, sh.rng[gw % MG_WARPS][0], sh.rng[gw % MG_WARPS][1], (int)(pipe.issued - pipe.consumed));
    st.template consume<NT>(m, pipe, act, lane);
}

// Expert activations h [A][F] (written by all CTAs in the gate/up phase) -> Q8_K in shared memory,
// one warp per 256-value block, two blocks per pass so that both loads are in flight together.
__device__ __noinline__ void mg_h_quant(const MegaParams& p, const ActSmem& acth, int A) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nbh = p.F / DC_QK_K;
    const int rotb = (int)(blockIdx.x % (unsigned)(A * nbh));
    for (int il = warp; il < A * nbh; il += 2 * MG_WARPS) {
        const int i0 = (il + rotb) % (A * nbh), il1 = il + MG_WARPS;
        const bool two = il1 < A * nbh;
        const int i1 = two ? (il1 + rotb) % (A * nbh) : i0;
        const int a0 = i0 / nbh, b0 = i0 - a0 * nbh, a1 = i1 / nbh, b1 = i1 - a1 * nbh;
        const float4* s0 = reinterpret_cast<const float4*>(p.h + (size_t)a0 * p.F + b0 * DC_QK_K) + 2 * lane;
        const float4* s1 = reinterpret_cast<const float4*>(p.h + (size_t)a1 * p.F + b1 * DC_QK_K) + 2 * lane;
        const float4 v0 = __ldcg(s0), v1 = __ldcg(s0 + 1), w0 = __ldcg(s1), w1 = __ldcg(s1 + 1);
        const float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        quantize_block_q8k_to_act(v, acth, a0, b0, lane);
        if (two) {
            const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
            quantize_block_q8k_to_act(w, acth, a1, b1, lane);
        }
    }
}

template <int NT>
__global__ void __launch_bounds__(MG_THREADS, 1) k_decode_mega(const __grid_constant__ MegaParams gp) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(16) MegaShared sh;
    // the parameter block is read through references by out-of-line phase functions: keep it in
    // shared memory so that those reads are cheap shared loads rather than a per-thread local copy
    __shared__ __align__(16) MegaParams sp;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int i = tid; i < (int)(sizeof(MegaParams) / 4); i += MG_THREADS)
        reinterpret_cast<uint32_t*>(&sp)[i] = reinterpret_cast<const uint32_t*>(&gp)[i];
    __syncthreads();
    const MegaParams& p = sp;
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

    // scores and the V rows of an attention run live where the activations and the hidden state live in the
    // other phases (both are idle during attention)
    uint8_t* vbuf = smem + p.off_v;
    const int vcap_blocks = (int)((p.smem_bytes - p.off_v) / (DC_KV_BLOCK * 256));
    // expert parallel: rows of the down projection go to the exchange buffers, alternating halves by layer
    const bool ep = p.ep_size > 1;
    const size_t xhalf = (size_t)MG_MAX_T * MG_MAX_K * p.H;
    unsigned xe = p.xepoch0;           // exchanges done so far (all ranks count alike)
    const float* dn_r = p.dn;          // where the pending MoE output is read from
    for (int step = 0; step < p.n_steps; ++step) {
        const AttnItem item = attn_step_setup(p, sh);
        load_layer(p, sh, 0, 0);
        __syncthreads();
        if (tid == 0) sh.g_qkv = mg_qkv(p, sh.layer[0]);
        __syncthreads();
        const GemvParams& gq = sh.g_qkv;
        mg_gemv_prefill(gq, pipe, sh, gw, nw, lane);
        const GemvParams& glm = sh.g_lm;
        const GemvParams& go = sh.g_o;
        for (int l = 0; l < p.n_layer; ++l) {
            const MegaLayer& L = sh.layer[l & 1];
            if (l + 1 < p.n_layer) load_layer(p, sh, l + 1, (l + 1) & 1);   // read long before it is used
            const float* xin = (l & 1) ? p.xb : p.xa;
            float* xout = (l & 1) ? p.xa : p.xb;
            // ---- P0: hidden state, attn_norm, Q8_K, QKV rows
            MG_MARK(0);
            MG_WTRACE(0);
            ActSmem act;
            act.bind(act_base, p.T, p.H);
            // the output projection's parameter block is written now (the barriers inside the norm phase publish
            // it), so that every warp can ask for its first rows the moment it is done with its QKV rows
            if (tid == 0) sh.g_o = mg_single(p, L.wo, L.wo_type, L.wo_rb, p.H, p.rpst_o, QD, DC_EPI_ACC, xout, p.H, nullptr);
            x_norm_phase<(NT > 1 ? 2 : 1)>(p, sh, l == 0 ? 0 : 1, xin, xout, L.attn_norm, act, nullptr, dn_r);
            if (p.dbg_x) mg_capture_x(p, xout, l);
            MG_MARK(2);
            MG_WTRACE(1);
            mg_gemv_consume<NT>(gq, pipe, act, sh, gw, lane);
            MG_MARK(3);
            MG_WTRACE(2);
            grid_arrive(p, epoch);
            mg_gemv_prefill(go, pipe, sh, gw, nw, lane);   // output-projection rows stream in during attention
            prefetch_vec(L.ffn_norm, (size_t)p.H * 4);
            if ((int)blockIdx.x < p.E) prefetch_vec(L.router + (size_t)blockIdx.x * p.H, (size_t)p.H * 4);
            if (grid_wait(p, epoch)) goto gave_up;
            MG_MARK(4);
            MG_WTRACE(3);
            // ---- P1 / P2: attention
            attn_scores_phase(p, L, sh, item, s_sc, vbuf, vcap_blocks);
            MG_MARK(5);
            MG_WTRACE(4);
            if (grid_barrier(p, epoch)) goto gave_up;
            MG_MARK(6);
            MG_WTRACE(5);
            attn_pv_phase(p, L, sh, item, s_sc, vbuf, vcap_blocks);
            MG_MARK(7);
            MG_WTRACE(6);
            if (grid_barrier(p, epoch)) goto gave_up;
            MG_MARK(8);
            MG_WTRACE(7);
            // ---- P3: output projection, x += Wo . attn
            act.bind(act_base, p.T, QD);
            act.template fill<true>(p.q8_attn, p.T);
            __syncthreads();
            MG_MARK(9);
            mg_gemv_consume<NT>(go, pipe, act, sh, gw, lane);
            MG_MARK(10);
            MG_WTRACE(8);
            if (grid_barrier(p, epoch)) goto gave_up;
            MG_MARK(11);
            MG_WTRACE(9);
            // ---- P4: ffn_norm, Q8_K, router logits
            act.bind(act_base, p.T, p.H);
            x_norm_phase<(NT > 1 ? 2 : 1)>(p, sh, 2, xout, nullptr, L.ffn_norm, act, xs, nullptr);
            MG_MARK(12);
            router_logits_phase(p, L, sh, xs);
            MG_MARK(13);
            MG_WTRACE(10);
            // parameter blocks of the two expert phases: they depend on the layer, not on the routing, so
            // they are built while this CTA would otherwise wait at the barrier
            float* dn_w = ep ? p.xdn[p.ep_rank] + (xe & 1u) * xhalf : p.dn;
            grid_arrive(p, epoch);
            if (tid == 0) {
                sh.m_gu = mg_experts(p, sh, L.gate, L.up, L.gate_type, L.gate_rb, p.F, p.H, p.rpst_gate, p.h);
                sh.m_dn = mg_experts(p, sh, L.down, nullptr, L.down_type, L.down_rb, p.H, p.F, p.rpst_down, dn_w);
                if (ep) {   // the same rows in every peer's exchange buffer
                    int q = 0;
                    for (int r = 0; r < p.ep_size; ++r)
                        if (r != p.ep_rank) sh.m_dn.peer_out[q++] = p.xdn[r] + (xe & 1u) * xhalf;
                    sh.m_dn.n_peer = q;
                }
            }
            if (grid_wait(p, epoch)) goto gave_up;
            MG_MARK(14);
            MG_WTRACE(11);
            // ---- P5: routing, gate/up + SwiGLU
            route_phase(p, sh);   // ends with a CTA barrier: the blocks above are visible too
            MG_MARK(15);
            MG_WTRACE(12);
            const MoeMMParams& mgu = sh.m_gu;
            mg_moe_prefill(mgu, sh.n_active, pipe, sh, gw, nw, lane);
            mg_moe_consume<NT>(mgu, pipe, act, sh, gw, lane);
            MG_MARK(16);
            MG_WTRACE(13);
            const MoeMMParams& mdn = sh.m_dn;
            grid_arrive(p, epoch);
            mg_moe_prefill(mdn, sh.n_active, pipe, sh, gw, nw, lane);  // down rows stream in across the barrier
            if (l + 1 < p.n_layer) {
                const MegaLayer& Ln = sh.layer[(l + 1) & 1];
                prefetch_vec(Ln.attn_norm, (size_t)p.H * 4);
                prefetch_vec(Ln.q_norm, 512);
                prefetch_vec(Ln.k_norm, 512);
            } else {
                prefetch_vec(p.out_norm, (size_t)p.H * 4);
            }
            if (grid_wait(p, epoch)) goto gave_up;
            MG_MARK(17);
            MG_WTRACE(14);
            // ---- P6: h -> Q8_K, down rows
            ActSmem acth;
            acth.bind(act_base, A, p.F);
            // the parameter block of the stream that follows the down rows (next layer's QKV, or the lm_head) is
            // written now: the barrier below publishes it, and no warp has to wait for the others before it asks
            // for that stream's first rows
            if (tid == 0) {
                if (l + 1 < p.n_layer) sh.g_qkv = mg_qkv(p, sh.layer[(l + 1) & 1]);
                else
                    sh.g_lm = mg_single(p, p.out_w, p.out_type, p.out_rb, p.vocab, p.rpst_out, p.H, DC_EPI_STORE, p.logits,
                                        p.vocab, p.argmax_keys);
            }
            mg_h_quant(p, acth, A);
            __syncthreads();
            MG_MARK(18);
            MG_WTRACE(15);
            mg_moe_consume<NT>(mdn, pipe, acth, sh, gw, lane);
            MG_MARK(19);
            MG_WTRACE(16);
            grid_arrive(p, epoch, ep);
            mg_gemv_prefill(l + 1 < p.n_layer ? gq : glm, pipe, sh, gw, nw, lane);
            if (grid_wait(p, epoch)) goto gave_up;
            if (ep && ep_wait(p, xe + 1)) goto gave_up;
            ++xe;
            dn_r = dn_w;
            MG_MARK(20);
            MG_WTRACE(17);
        }
        // ---- final: last MoE output + residual, output norm, lm_head with arg-max keys
        ActSmem act;
        act.bind(act_base, p.T, p.H);
        // (parity capture on: the assembled final hidden state goes straight to its capture slot)
        x_norm_phase<(NT > 1 ? 2 : 1)>(p, sh, 1, (p.n_layer & 1) ? p.xb : p.xa,
                                       p.dbg_x ? p.dbg_x + (size_t)p.n_layer * DC_MAX_T * p.H : nullptr, p.out_norm, act,
                                       nullptr, dn_r);
        mg_gemv_consume<NT>(glm, pipe, act, sh, gw, lane);
        if (grid_barrier(p, epoch)) goto gave_up;
        MG_MARK(21);
        // greedy pick: first maximum wins (core/src/sampler/sampler.cpp:42-57)
        if (blockIdx.x == 0 && tid < p.T) {
            const unsigned long long k = __ldcg(p.argmax_keys + tid);
            int32_t tok = (int32_t)(0xFFFFFFFFu - (uint32_t)(k & 0xFFFFFFFFull));
            // (a step cut short by a wait that ran out may leave no key behind: the id must stay a valid row index)
            if ((uint32_t)tok >= (uint32_t)p.vocab) tok = 0;
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
        if (step + 1 < p.n_steps && grid_barrier(p, epoch)) goto gave_up;
    }
    return;
gave_up:
    // a bounded wait ran out (the error word is set): wait, again with a limit, for this warp's weight copies
    // still in flight, then leave; nothing is computed on data that may not be there
    pipe.drain();
}

// ------------------------------------------------------------------ host
static int mg_rows_per_stage(int type, int K, int row_bytes) {
    const int G = dc::lanes_per_row(type, K);
    const int per_pass = 32 / G;
    int r = (MG_STAGE - 32) / row_bytes;
    r = r / per_pass * per_pass;
    return r < per_pass ? per_pass : r;
}

// Score buffer of an attention run: 8 heads x s_keys floats, and at least 8 x 128 floats because
// the merging run reuses it for the merged heads.
static uint32_t mg_sc_bytes(int s_keys) {
    const int keys = s_keys < 128 ? 128 : s_keys;
    return (uint32_t)((8 * keys * 4 + 127) & ~127);
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
    if (c.ep_size > 1 && (c.ep_size > MG_MAX_RANKS || m->xch_connected != c.ep_size - 1))
        NO("expert-parallel exchange buffers are not connected (dc_b200_model_ep_export / _import)");
    if (T < 1 || T > MG_MAX_T || T * c.n_expert_used > MG_MAX_T * 8) NO("more than 4 streams or 32 assignments");
    if (c.n_expert > MG_MAX_E || c.n_expert_used > MG_MAX_K) NO("too many experts");
    const int g = c.n_head / c.n_kv_head;
    if (g > 8 || (g & 1)) NO("query-head group must be even and <= 8");
    if (c.hidden % MG_THREADS || T * (c.hidden / DC_QK_K) > 2 * MG_WARPS) NO("hidden size x streams");
    MegaParams p = {};
    const int G = m->ctx->num_sms;
    p.n_layer = c.n_layer; p.H = c.hidden; p.n_head = c.n_head; p.n_kv = c.n_kv_head; p.vocab = c.vocab;
    p.E = c.n_expert; p.top_k = c.n_expert_used; p.F = c.expert_ffn; p.T = T;
    p.eps = c.rms_eps; p.scale = 1.0f / sqrtf((float)c.head_dim); p.routed_scale = c.routed_scale;
    // attention runs: (stream, kv head, head group, split).  More head groups mean fewer, longer runs per
    // group and a shorter merge (the merging CTA adds nsplit partials per output); K/V rows are then read
    // once per head group (from L2).  Groups hold an even number of heads (a Q8_K block spans two).
    p.n_hg = 1;
    while (p.n_hg < 4 && G / (T * c.n_kv_head * p.n_hg) > 20 && (g / (2 * p.n_hg)) % 2 == 0 && g / (2 * p.n_hg) >= 2) p.n_hg *= 2;
    p.nsplit = G / (T * c.n_kv_head * p.n_hg);
    // at most 16 runs per group: the merging run then fetches all partials in one round of loads, and the merge is
    // the tail of the phase (measured: the second round costs more than the 12 % longer runs)
    if (p.nsplit > 16) p.nsplit = 16;
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
    // gate/up pairs: a pass takes gate rows in the lower half of its lane groups and the up rows of the same
    // outputs in the upper half, so a stage holds a multiple of (rows per pass) / 2 outputs in each of its halves
    {
        const int G = dc::lanes_per_row(L0.gate_exps->type, c.hidden);
        const int rpp = 32 / G, step = rpp >= 2 ? rpp / 2 : 1;
        int r = step;
        uint32_t half = ((uint32_t)r * (uint32_t)L0.gate_exps->row_bytes + 32 + 127) & ~127u;
        if (2 * half > MG_STAGE) NO("a gate/up row pair does not fit a pipeline stage");
        for (;;) {   // more passes per stage while they fit
            const uint32_t h2 = ((uint32_t)(r + step) * (uint32_t)L0.gate_exps->row_bytes + 32 + 127) & ~127u;
            if (2 * h2 > MG_STAGE) break;
            r += step;
            half = h2;
        }
        p.rpst_gate = r;
        p.up_off = half;
    }
    // Shared memory plan.  After the warps' pipelines comes one region that every phase lays out for itself:
    // norm phases put the Q8_K hidden state first and (before the router) the normed f32 rows behind it; the
    // output projection and the down projection put their Q8_K inputs there; attention puts its scores there
    // and stages the run's V rows behind them.  The region is as large as its largest user, and is grown to
    // hold a whole attention run's V rows if the SM has room left.
    const size_t a_x = (ActSmem::bytes(T, c.hidden) + 127) & ~(size_t)127;
    size_t region = a_x + (size_t)T * c.hidden * 4;
    const size_t a_o = ActSmem::bytes(T, QD), a_h = ActSmem::bytes(T * c.n_expert_used, c.expert_ffn);
    if (a_o > region) region = a_o;
    if (a_h > region) region = a_h;
    const uint32_t sc_bytes = mg_sc_bytes(p.s_keys);
    const size_t v_run = (size_t)(p.s_keys / DC_KV_BLOCK) * DC_KV_BLOCK * 256;
    uint32_t off = 512;
    p.off_pipe = off;
    off += MG_WARPS * MG_NSTAGE * MG_STAGE;
    p.off_act = off;
    p.off_xs = off + (uint32_t)a_x;
    p.off_sc = off;
    p.off_v = off + sc_bytes;
    if (region < sc_bytes + 4096) region = sc_bytes + 4096;
    if (region < sc_bytes + v_run) {
        const size_t room = off + region < MG_DYN_LIMIT ? MG_DYN_LIMIT - off - region : 0;
        const size_t want = sc_bytes + v_run - region;
        region += want < room ? want : (room & ~(size_t)4095);
    }
    region = (region + 127) & ~(size_t)127;
    off += (uint32_t)region;
    p.smem_bytes = off;
    if (off > MG_DYN_LIMIT) NO("shared memory plan exceeds the 227 KB of an SM");
    if (p.s_keys / DC_KV_BLOCK > MG_MAX_RUN_BLOCKS) NO("attention run longer than 64 KV blocks");
    *out = p;
    return true;
#undef NO
}

template <int NT>
static int mg_launch(dc_model* m, MegaParams& p) {
    dc_ctx* ctx = m->ctx;
    int st = dc_kernel_setup(ctx, (const void*)k_decode_mega<NT>, MG_DYN_LIMIT, "cudaFuncSetAttribute(k_decode_mega)");
    if (st != DC_B200_OK) return st;
    const int per_sm = dc_kernel_occupancy(ctx, (const void*)k_decode_mega<NT>, MG_THREADS, p.smem_bytes);
    cudaError_t e;
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
    p.ep_rank = m->cfg.ep_rank; p.ep_size = m->cfg.ep_size; p.e_lo = m->ep_lo; p.e_hi = m->ep_hi;
    if (p.ep_size > 1) {
        for (int r = 0; r < p.ep_size; ++r) {
            p.xdn[r] = (float*)(m->xch_peer[r] + MG_XCH_FLAG_BYTES);
            p.xcnt[r] = (unsigned*)m->xch_peer[r] + MG_XCNT_WORD;
        }
        p.my_xcnt = (unsigned*)m->xch + MG_XCNT_WORD;
        p.xepoch0 = m->xepoch;
        m->xepoch += (unsigned)(m->cfg.n_layer * n_steps);
    }
    p.route_mode = m->route_mode;
    p.dbg_x = m->dbg_x;
    p.bar_polls = m->test_barrier_polls ? m->test_barrier_polls : MG_BAR_LIMIT;
    p.ep_wait_ns = m->test_ep_wait_ns ? m->test_ep_wait_ns : MG_EP_WAIT_NS;
    p.bar_counter = m->mega_counter;
    p.err = m->ctx->d_err;
    p.phase_ns = m->mega_timing ? (unsigned long long*)((uint8_t*)m->mega_counter + 64) : nullptr;
    int st = dc_check_cuda(m->ctx, cudaMemsetAsync(m->mega_counter, 0, sizeof(unsigned), m->ctx->stream), "memset");
    if (st != DC_B200_OK) return st;
    // the merge tickets reset themselves when a merge completes; a launch that gave up may have left some behind
    st = dc_check_cuda(m->ctx, cudaMemsetAsync(b.attn.tickets, 0, (size_t)DC_MAX_T * m->cfg.n_head * sizeof(int), m->ctx->stream), "memset");
    if (st != DC_B200_OK) return st;
    m->last_launches = 1;
    return (T == 1 && m->cfg.hidden <= 4096) ? mg_launch<1>(m, p) : mg_launch<MG_MAX_T>(m, p);
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
    if (e == cudaSuccess) e = cudaMalloc((void**)&m->mega_counter, DC_MEGA_COUNTER_BYTES);
    if (e == cudaSuccess) e = cudaMemcpy(m->mega_layers, v.data(), v.size() * sizeof(MegaLayer), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemset(m->mega_counter, 0, DC_MEGA_COUNTER_BYTES);
    return dc_check_cuda(m->ctx, e, "persistent decode set-up");
}

// ---- expert-parallel exchange buffers (one process per GPU; handles travel through the caller) ----
size_t dc_mega_xch_bytes(const dc_model* m) {
    return MG_XCH_FLAG_BYTES + 2 * (size_t)MG_MAX_T * MG_MAX_K * m->cfg.hidden * sizeof(float);
}

extern "C" {

int dc_b200_model_ep_export(dc_model* m, void* handle_out_64) {
    if (!m || !handle_out_64) return DC_B200_INVALID_ARGUMENT;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    cudaSetDevice(m->ctx->device);
    if (!m->xch) {
        cudaError_t e = cudaMalloc((void**)&m->xch, dc_mega_xch_bytes(m));
        if (e == cudaSuccess) e = cudaMemset(m->xch, 0, dc_mega_xch_bytes(m));
        if (e != cudaSuccess) return dc_check_cuda(m->ctx, e, "exchange buffer");
        m->xch_peer[m->cfg.ep_rank] = m->xch;
    }
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, m->xch);
    if (e != cudaSuccess) return dc_check_cuda(m->ctx, e, "cudaIpcGetMemHandle");
    memcpy(handle_out_64, &h, 64);
    return DC_B200_OK;
}

int dc_b200_model_ep_import(dc_model* m, int rank, const void* handle_64) {
    if (!m || !handle_64 || rank < 0 || rank >= m->cfg.ep_size || rank >= MG_MAX_RANKS || rank == m->cfg.ep_rank)
        return DC_B200_INVALID_ARGUMENT;
    if (!m->xch) return dc_fail(m->ctx, DC_B200_INVALID_ARGUMENT, "ep_import before ep_export");
    if (m->xch_peer[rank]) return dc_fail(m->ctx, DC_B200_INVALID_ARGUMENT, "rank %d is already connected", rank);
    cudaSetDevice(m->ctx->device);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle_64, 64);
    void* ptr = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return dc_check_cuda(m->ctx, e, "cudaIpcOpenMemHandle");
    m->xch_peer[rank] = (uint8_t*)ptr;
    m->xch_connected++;
    return DC_B200_OK;
}

}  // extern "C"

// Test hook for the exchange's bounded wait on ONE GPU: a rank of a two-rank model whose "peer" is a second
// local buffer that nothing ever signals.  The persistent kernel then stores its rows into that buffer, adds its
// arrivals to a counter nobody reads, and its own wait for the peer's arrivals runs out.  No communicator exists:
// only decode steps through the persistent kernel may run on such a model.
int dc_mega_test_loopback(dc_model* m) {
    if (m->cfg.ep_size != 2 || m->xch || m->ep_ready)
        return dc_fail(m->ctx, DC_B200_INVALID_ARGUMENT, "test_ep_loopback needs a fresh two-rank model");
    cudaSetDevice(m->ctx->device);
    uint8_t* fake = nullptr;
    cudaError_t e = cudaMalloc((void**)&m->xch, dc_mega_xch_bytes(m));
    if (e == cudaSuccess) e = cudaMemset(m->xch, 0, dc_mega_xch_bytes(m));
    if (e == cudaSuccess) e = cudaMalloc((void**)&fake, dc_mega_xch_bytes(m));
    if (e == cudaSuccess) e = cudaMemset(fake, 0, dc_mega_xch_bytes(m));
    if (e != cudaSuccess) return dc_check_cuda(m->ctx, e, "loopback exchange buffers");
    m->xch_peer[m->cfg.ep_rank] = m->xch;
    m->xch_peer[1 - m->cfg.ep_rank] = fake;
    m->xch_connected = 1;
    m->xch_loopback = true;
    m->ep_ready = true;
    return DC_B200_OK;
}

void dc_mega_release_xch(dc_model* m) {
    for (int r = 0; r < 8; ++r) {
        if (m->xch_peer[r] && m->xch_peer[r] != m->xch) {
            if (m->xch_loopback) cudaFree(m->xch_peer[r]);
            else cudaIpcCloseMemHandle(m->xch_peer[r]);
        }
        m->xch_peer[r] = nullptr;
    }
    if (m->xch) cudaFree(m->xch);
    m->xch = nullptr;
    m->xch_connected = 0;
}
