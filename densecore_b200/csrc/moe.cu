// Fused MoE layer (MUL_MAT_ID).  Replaces cb_moe_forward
// (core/src/llm/moe/exec.cpp:813) -> RouteMoESoftmaxTopK (:734) ->
// CpuBackend::ForwardMoE (core/src/backend/cpu_backend_moe_ops.cpp:1195):
//   k_router      router logits (F32 matmul, core/src/llm/graph/decoder.cpp:2265),
//                 stable top-k + weights (core/src/llm/moe/native.cpp:610-676),
//                 token->expert bucketing (core/src/moe/moe_routing.cpp:534-603)
//   k_moe_mm<PAIR> gate/up + SwiGLU for every (distinct expert, row), each expert's
//                 weights read once for all its tokens (native.cpp:3929-4345)
//   k_moe_mm      down projection per assignment (native.cpp:3051-3295)
//   k_moe_combine weighted sum in the reference's order
//                 (cpu_backend_moe_ops.cpp:1578-1597, moe_routing.cpp:647-676)
#include "dc_common.cuh"
#include "dc_internal.h"
#include "dc_launch.cuh"
#include "dc_stream.cuh"

using namespace dc;

#define MOE_MAX_E 256
#define MOE_MAX_K 16

// ------------------------------------------------------------------ router
struct RouterParams {
    const float* wr;      // [E][H] f32
    const float* xn;      // [T][H] f32 (normed hidden state)
    int E, H, T, top_k;
    float scale;          // moe_routed_scaling_factor
    int mode;             // DC_ROUTE_STABLE (top-k on logits) or DC_ROUTE_SOFTMAX (softmax over all experts first)
    int ep_lo, ep_hi;     // experts owned by this GPU
    float* logits;        // [T][E]
    int32_t* ids;         // [T][top_k]
    float* weights;       // [T][top_k]
    int* ticket;          // zero-initialised, self-resetting
    int* n_active;        // U
    int32_t* uexp;        // [E]   distinct local experts, ascending
    int32_t* uoff;        // [E+1] offsets into uassign
    int32_t* uassign;     // [T*top_k] assignment indices t*top_k+k, grouped by expert, routing order inside
};

__device__ __forceinline__ unsigned long long route_key(float v, int id) {
    uint32_t u;
    if (v != v) u = 0u;
    else {
        if (v == 0.0f) v = 0.0f;  // -0 == +0 for the comparator
        u = __float_as_uint(v);
        u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    }
    return ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)id);
}

// expf rounded as the host library rounds it: the double-precision exponential (1 ulp of double) rounded once
// to float is the correctly rounded float result except on a 2^-29 sliver of arguments, and so is glibc's expf.
// The generic router compares probabilities for equality (ties go to the lower expert id), so its
// exponentials must be the CPU's bit for bit.
__device__ __forceinline__ float expf_cr(float x) { return (float)exp((double)x); }

// Routing of token t by one warp: stable top-k on the logits (native router) or on the softmax probabilities
// (generic router), then the routing weights.  s_prob: MOE_MAX_E floats of shared memory owned by this warp;
// s_ids (optional): shared copy of the ids for the bucketing that follows in k_router.
__device__ __forceinline__ void route_token(const RouterParams& p, int t, int lane, float* s_prob, int32_t* s_ids) {
    float lv[MOE_MAX_E / 32];
    bool taken[MOE_MAX_E / 32];
#pragma unroll
    for (int j = 0; j < MOE_MAX_E / 32; ++j) {
        const int id = j * 32 + lane;
        lv[j] = id < p.E ? __ldcg(p.logits + (size_t)t * p.E + id) : 0.0f;
        taken[j] = id >= p.E;
    }
    if (p.mode == DC_ROUTE_SOFTMAX) {
        // softmax over all experts: expf(x - max), sum in index order, times 1/sum
        // (core/include/densecore/simd/simd_ops.h:1171-1195); selection then runs on the probabilities
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < MOE_MAX_E / 32; ++j)
            if (!taken[j]) mx = fmaxf(mx, lv[j]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
#pragma unroll
        for (int j = 0; j < MOE_MAX_E / 32; ++j) {
            if (!taken[j]) {
                lv[j] = expf_cr(__fsub_rn(lv[j], mx));
                s_prob[j * 32 + lane] = lv[j];
            }
        }
        __syncwarp();
        float sum = 0.0f;
        if (lane == 0)
            for (int e = 0; e < p.E; ++e) sum = __fadd_rn(sum, s_prob[e]);
        sum = __shfl_sync(0xffffffffu, sum, 0);
        const float inv = __fdiv_rn(1.0f, sum);
#pragma unroll
        for (int j = 0; j < MOE_MAX_E / 32; ++j)
            if (!taken[j]) lv[j] = __fmul_rn(lv[j], inv);
        __syncwarp();
    }
    float sel_l[MOE_MAX_K];
    for (int k = 0; k < p.top_k; ++k) {
        unsigned long long best = 0ull;
#pragma unroll
        for (int j = 0; j < MOE_MAX_E / 32; ++j) {
            if (!taken[j]) {
                const unsigned long long key = route_key(lv[j], j * 32 + lane);
                best = key > best ? key : best;
            }
        }
        // a real candidate's key is never 0 (its low word is 0xFFFFFFFF - id), so 0 means "none"
        unsigned long long win = best;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long ok = __shfl_xor_sync(0xffffffffu, win, o);
            win = ok > win ? ok : win;
        }
        const int wid = (int)(0xFFFFFFFFu - (uint32_t)(win & 0xFFFFFFFFull));
#pragma unroll
        for (int j = 0; j < MOE_MAX_E / 32; ++j)
            if (j * 32 + lane == wid) taken[j] = true;
        // the winner's value back out of its key (NaN stays NaN; -0 was made +0, which exp treats alike):
        // no load per round
        const uint32_t ku = (uint32_t)(win >> 32);
        const float wl = __uint_as_float((ku & 0x80000000u) ? (ku & 0x7FFFFFFFu) : ~ku);
        if (k < MOE_MAX_K) sel_l[k] = wl;
        if (lane == 0) {
            p.ids[t * p.top_k + k] = wid;
            if (s_ids) s_ids[t * p.top_k + k] = wid;
        }
    }
    if (lane == 0 && p.mode == DC_ROUTE_SOFTMAX) {
        // renormalise over the picks in pick order: w * (1 / sum) (core/src/moe/moe_routing.cpp:90-101),
        // then the routed scaling factor (core/src/llm/moe/exec.cpp:764-768)
        float sum = 0.0f;
        for (int k = 0; k < p.top_k; ++k) sum = __fadd_rn(sum, sel_l[k]);
        const float is = sum > 0.0f ? __fdiv_rn(1.0f, sum) : 1.0f;
        for (int k = 0; k < p.top_k; ++k)
            p.weights[t * p.top_k + k] = __fmul_rn(sum > 0.0f ? __fmul_rn(sel_l[k], is) : sel_l[k], p.scale);
    } else if (lane == 0) {
        // weights over the selected experts only (native.cpp:649-674)
        float mx = -INFINITY;
        bool finite = true;
        for (int k = 0; k < p.top_k; ++k) {
            finite = finite && isfinite(sel_l[k]);
            if (isfinite(sel_l[k]) && sel_l[k] > mx) mx = sel_l[k];
        }
        float den = 0.0f, wv[MOE_MAX_K];
        if (finite && isfinite(mx)) {
            for (int k = 0; k < p.top_k; ++k) {
                wv[k] = expf(sel_l[k] - mx);
                den += wv[k];
            }
        }
        const bool ok = den > 0.0f && isfinite(den);
        for (int k = 0; k < p.top_k; ++k) {
            const float w = ok ? __fdiv_rn(wv[k], den) : __fdiv_rn(1.0f, (float)p.top_k);
            p.weights[t * p.top_k + k] = __fmul_rn(w, p.scale);
        }
    }
}

__global__ void __launch_bounds__(256) k_router(const RouterParams p) {
    __shared__ int s_last;
    __shared__ float s_prob[8][MOE_MAX_E];
    __shared__ int32_t s_ids[DC_MAX_T * MOE_MAX_K];
    __shared__ int s_wsum_a[8], s_wsum_c[8];
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // logits: two experts per CTA, four warps per expert, each warp a quarter of the row
    // with all of its loads issued before the first use.  The router weights do not depend on the
    // previous kernel: the first batch is fetched while this kernel still waits for it.
    float4 wv0[4];
    {
        const int e = blockIdx.x * 2 + (warp >> 2), quarter = warp & 3, seg = p.H / 4;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = j * 32 + lane;
            wv0[j] = (p.wr && e < p.E && i < seg / 4)
                         ? reinterpret_cast<const float4*>(p.wr + (size_t)e * p.H + quarter * seg)[i]
                         : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    pdl_wait();
    if (p.wr) {
        __shared__ float s_part[8][DC_MAX_T];
        const int e = blockIdx.x * 2 + (warp >> 2), quarter = warp & 3;
        const int seg = p.H / 4;  // H is a multiple of 256
        float acc[DC_MAX_T];
#pragma unroll
        for (int t = 0; t < DC_MAX_T; ++t) acc[t] = 0.0f;
        if (e < p.E) {
            const float4* w4 = reinterpret_cast<const float4*>(p.wr + (size_t)e * p.H + quarter * seg);
            for (int i0 = 0; i0 < seg / 4; i0 += 128) {
                float4 wv[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = i0 + j * 32 + lane;
                    wv[j] = i0 == 0 ? wv0[j] : (i < seg / 4 ? w4[i] : make_float4(0.f, 0.f, 0.f, 0.f));
                }
#pragma unroll
                for (int t = 0; t < DC_MAX_T; ++t) {
                    if (t < p.T) {
                        const float4* x4 = reinterpret_cast<const float4*>(p.xn + (size_t)t * p.H + quarter * seg);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int i = i0 + j * 32 + lane;
                            if (i < seg / 4) {
                                const float4 xv = x4[i];
                                acc[t] = fmaf(wv[j].x, xv.x, acc[t]);
                                acc[t] = fmaf(wv[j].y, xv.y, acc[t]);
                                acc[t] = fmaf(wv[j].z, xv.z, acc[t]);
                                acc[t] = fmaf(wv[j].w, xv.w, acc[t]);
                            }
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int t = 0; t < DC_MAX_T; ++t) {
            if (t < p.T) {
                float v = acc[t];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0) s_part[warp][t] = v;
            }
        }
        __syncthreads();
        if (threadIdx.x < 2 * p.T) {
            const int which = threadIdx.x / p.T, t = threadIdx.x % p.T, ee = blockIdx.x * 2 + which;
            if (ee < p.E)
                p.logits[(size_t)t * p.E + ee] = (s_part[which * 4][t] + s_part[which * 4 + 1][t]) +
                                                 (s_part[which * 4 + 2][t] + s_part[which * 4 + 3][t]);
        }
    }
    // release: the CTA barrier puts this CTA's logits before thread 0's ticket, whose release half publishes them;
    // acquire: the last CTA's thread 0 sees the others' logits through the ticket's acquire half, and the CTA
    // barrier passes that on
    __syncthreads();
    if (threadIdx.x == 0) {
        int old;
        asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], %2;" : "=r"(old) : "l"(p.ticket), "r"(1) : "memory");
        s_last = old == (int)gridDim.x - 1;
        if (s_last) *p.ticket = 0;
    }
    __syncthreads();
    if (!s_last) return;

    // ---- stable top-k per token, one warp per token
    for (int t = warp; t < p.T; t += 8) route_token(p, t, lane, s_prob[warp], s_ids);
    __syncthreads();
    // ---- bucketing: thread e owns expert e
    const int A = p.T * p.top_k;
    const int me = threadIdx.x;
    int cnt = 0;
    if (me < p.E && me >= p.ep_lo && me < p.ep_hi)
        for (int i = 0; i < A; ++i) cnt += (s_ids[i] == me);
    int act = cnt > 0 ? 1 : 0;
    // inclusive scans of (act, cnt) over the 256 threads
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
        s_wsum_a[warp] = sa;
        s_wsum_c[warp] = scn;
    }
    __syncthreads();
    int base_a = 0, base_c = 0, tot_a = 0, tot_c = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        if (w < warp) {
            base_a += s_wsum_a[w];
            base_c += s_wsum_c[w];
        }
        tot_a += s_wsum_a[w];
        tot_c += s_wsum_c[w];
    }
    if (act) {
        const int u = base_a + sa - 1, off = base_c + scn - cnt;
        p.uexp[u] = me;
        p.uoff[u] = off;
        int o = off;
        for (int i = 0; i < A; ++i)
            if (s_ids[i] == me) p.uassign[o++] = i;
    }
    if (threadIdx.x == 0) {
        *p.n_active = tot_a;
        p.uoff[tot_a] = tot_c;
    }
}

// ------------------------------------------- router over a prompt chunk
// The same arithmetic as k_router for any number of tokens: logits by CTAs of two experts x sixteen tokens
// (four warps per expert, a quarter of the row each, lane partials chained by fma in the same element order,
// butterfly sum, quarters added pairwise), then one warp per token for the selection.  No bucketing: the
// chunk's assignments are grouped by k_moe_group.
__global__ void __launch_bounds__(256) k_router_logits_batched(const RouterParams p) {
    __shared__ float s_part[8][DC_MAX_T];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.x * 2 + (warp >> 2), quarter = warp & 3, seg = p.H / 4;
    const int t0 = blockIdx.y * DC_MAX_T, tn = min(DC_MAX_T, p.T - t0);
    float acc[DC_MAX_T];
#pragma unroll
    for (int t = 0; t < DC_MAX_T; ++t) acc[t] = 0.0f;
    if (e < p.E) {
        const float4* w4 = reinterpret_cast<const float4*>(p.wr + (size_t)e * p.H + quarter * seg);
        for (int i0 = 0; i0 < seg / 4; i0 += 128) {
            float4 wv[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int i = i0 + j * 32 + lane;
                wv[j] = i < seg / 4 ? w4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int t = 0; t < DC_MAX_T; ++t) {
                if (t < tn) {
                    const float4* x4 = reinterpret_cast<const float4*>(p.xn + (size_t)(t0 + t) * p.H + quarter * seg);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int i = i0 + j * 32 + lane;
                        if (i < seg / 4) {
                            const float4 xv = x4[i];
                            acc[t] = fmaf(wv[j].x, xv.x, acc[t]);
                            acc[t] = fmaf(wv[j].y, xv.y, acc[t]);
                            acc[t] = fmaf(wv[j].z, xv.z, acc[t]);
                            acc[t] = fmaf(wv[j].w, xv.w, acc[t]);
                        }
                    }
                }
            }
        }
    }
#pragma unroll
    for (int t = 0; t < DC_MAX_T; ++t) {
        if (t < tn) {
            float v = acc[t];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) s_part[warp][t] = v;
        }
    }
    __syncthreads();
    if (threadIdx.x < 2 * tn) {
        const int which = threadIdx.x / tn, t = threadIdx.x % tn, ee = blockIdx.x * 2 + which;
        if (ee < p.E)
            p.logits[(size_t)(t0 + t) * p.E + ee] = (s_part[which * 4][t] + s_part[which * 4 + 1][t]) +
                                                    (s_part[which * 4 + 2][t] + s_part[which * 4 + 3][t]);
    }
}

__global__ void __launch_bounds__(256) k_router_select_batched(const RouterParams p) {
    __shared__ float s_prob[8][MOE_MAX_E];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 8 + warp;
    if (t < p.T) route_token(p, t, lane, s_prob[warp], nullptr);
}

// Router of a prompt chunk: logits [T][E], ids and weights [T][top_k] for any T.
int dc_launch_router_batched(dc_ctx* ctx, const dc_weight* wr, const float* xn, int T, int top_k, float scale, float* logits,
                             int32_t* ids, float* weights, int mode) {
    if (!wr || wr->type != DC_TYPE_F32) return dc_fail(ctx, DC_B200_UNSUPPORTED, "router weight must be F32");
    const int E = (int)wr->N;
    if (E < 1 || E > MOE_MAX_E || top_k < 1 || top_k > MOE_MAX_K || top_k > E || T < 1)
        return dc_fail(ctx, DC_B200_UNSUPPORTED, "router: E=%d top_k=%d T=%d out of range", E, top_k, T);
    RouterParams p = {};
    p.wr = (const float*)wr->dev;
    p.xn = xn;
    p.E = E;
    p.H = (int)wr->K;
    p.T = T;
    p.top_k = top_k;
    p.scale = scale;
    p.mode = mode;
    p.ep_lo = 0;
    p.ep_hi = E;
    p.logits = logits;
    p.ids = ids;
    p.weights = weights;
    k_router_logits_batched<<<dim3((E + 1) / 2, (T + DC_MAX_T - 1) / DC_MAX_T), 256, 0, ctx->stream>>>(p);
    {
        const int st = dc_check_cuda(ctx, cudaGetLastError(), "k_router_logits_batched");
        if (st != DC_B200_OK) return st;
    }
    k_router_select_batched<<<(T + 7) / 8, 256, 0, ctx->stream>>>(p);
    return dc_check_cuda(ctx, cudaGetLastError(), "k_router_select_batched");
}

// --------------------------------------------------- expert matmul kernel
// NSTAGE: pipeline depth per warp.  Fewer, smaller rings let more CTAs share an SM: the row decode is
// bound by instruction issue, so resident warps matter more than bytes in flight per warp.
template <int NT, bool PAIR, int NSTAGE>
__global__ void __launch_bounds__(DC_WARPS * 32) k_moe_mm(const MoeMMParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem) + warp * NSTAGE;
    uint8_t* act_base = smem + DC_WARPS * DC_NSTAGE * 8;
    const size_t act_bytes = (ActSmem::bytes(p.act_rows, p.K) + 127) & ~(size_t)127;
    uint8_t* bufs = act_base + act_bytes + (size_t)warp * NSTAGE * p.stage_bytes;
    WarpPipe<NSTAGE> pipe;
    pipe.init(bufs, bars, p.stage_bytes, p.err);
    pdl_launch_dependents();
    MoeStream<NSTAGE, PAIR> st;
    if (PAIR) {
        pdl_wait();  // expert ids come from the router kernel just before: nothing can be fetched earlier
        st.begin(p, *p.n_active, blockIdx.x * DC_WARPS + warp, gridDim.x * DC_WARPS);
        st.prefill(p, pipe, lane);
    } else {
        // down projection: the routing was final before the gate/up kernel ran, and the kernel just before
        // this one (the quantiser of h, an ordinary launch) started only after gate/up had completed, so
        // the expert rows can be requested while this kernel still waits for the quantiser's output
        st.begin(p, *p.n_active, blockIdx.x * DC_WARPS + warp, gridDim.x * DC_WARPS);
        st.prefill(p, pipe, lane);
        pdl_wait();
    }
    ActSmem act;
    act.bind(act_base, p.act_rows, p.K);
    act.fill(p.act_q8, p.act_rows);
    __syncthreads();
    st.template consume<NT>(p, pipe, act, lane);
}

template <int NT, bool PAIR, int NSTAGE>
static int launch_moe_mm_ns(dc_ctx* ctx, const MoeMMParams& p, int grid, size_t smem) {
    int st = dc_kernel_setup(ctx, (const void*)k_moe_mm<NT, PAIR, NSTAGE>, 200 * 1024, "cudaFuncSetAttribute(k_moe_mm)");
    if (st != DC_B200_OK) return st;
    return dc_launch(ctx, "k_moe_mm", k_moe_mm<NT, PAIR, NSTAGE>, dim3(grid), dim3(DC_WARPS * 32), smem, p);
}

// Shared memory of one CTA with `ns` stages per warp.
static size_t moe_smem(size_t act_bytes, uint32_t stage, int ns) {
    return DC_WARPS * DC_NSTAGE * 8 + act_bytes + (size_t)DC_WARPS * ns * stage;
}
// CTAs of that size an SM holds (227 KB of shared memory, 1 KB reserved per CTA), at most 4.
static int moe_ctas_per_sm(size_t smem) {
    const int n = (int)((227u * 1024u) / (smem + 1024));
    return n > 4 ? 4 : n;
}

template <int NT, bool PAIR>
static int launch_moe_mm(dc_ctx* ctx, const MoeMMParams& p, size_t act_bytes) {
    // two stages per warp wherever that puts more CTAs on an SM, else the full depth
    const size_t s4 = moe_smem(act_bytes, p.stage_bytes, DC_NSTAGE), s2 = moe_smem(act_bytes, p.stage_bytes, 2);
    // resident CTAs per SM by shared memory, then by the kernel's registers (asked once per device and instance)
    int reg_limit4 = dc_kernel_occupancy(ctx, (const void*)k_moe_mm<NT, PAIR, DC_NSTAGE>, DC_WARPS * 32, 0);
    int reg_limit2 = dc_kernel_occupancy(ctx, (const void*)k_moe_mm<NT, PAIR, 2>, DC_WARPS * 32, 0);
    if (reg_limit4 < 1) reg_limit4 = 1;
    if (reg_limit2 < 1) reg_limit2 = 1;
    int n4 = s4 <= 200 * 1024 ? moe_ctas_per_sm(s4) : 0, n2 = s2 <= 200 * 1024 ? moe_ctas_per_sm(s2) : 0;
    if (n4 > reg_limit4) n4 = reg_limit4;
    if (n2 > reg_limit2) n2 = reg_limit2;
    if (n4 < 1 && n2 < 1) return dc_fail(ctx, DC_B200_UNSUPPORTED, "moe: shared memory need %zu too large", s2);
    if (n2 > n4) return launch_moe_mm_ns<NT, PAIR, 2>(ctx, p, ctx->num_sms * n2, s2);
    return launch_moe_mm_ns<NT, PAIR, DC_NSTAGE>(ctx, p, ctx->num_sms * n4, s4);
}

static int rows_per_stage_moe(int type, int K, int row_bytes) {
    const int G = dc::lanes_per_row(type, K);
    const int per_pass = 32 / G;
    int r = DC_STAGE_TARGET / row_bytes;
    r = r / per_pass * per_pass;
    return r < per_pass ? per_pass : r;
}

// w0/w1: expert tensors [K, N, E].  pair: gate/up + SwiGLU, activations are the T
// token rows; else down, activations are the T*top_k assignment rows.
int dc_launch_moe_mm(dc_ctx* ctx, bool pair, const dc_weight* w0, const dc_weight* w1, const uint8_t* act_q8,
                     int act_rows, int T, int top_k, int e_base, const dc_moe_route* rt, float* out) {
    MoeMMParams p = {};
    p.e_base = e_base;
    p.w0 = w0->dev;
    p.w1 = pair ? w1->dev : nullptr;
    p.type = w0->type;
    p.row_bytes = (int)w0->row_bytes;
    p.N = (int)w0->N;
    p.K = (int)w0->K;
    if (p.type != DC_TYPE_Q4_K && p.type != DC_TYPE_Q6_K)
        return dc_fail(ctx, DC_B200_UNSUPPORTED, "moe: expert weight type %d is not Q4_K/Q6_K", p.type);
    if (pair && (w1->type != w0->type || w1->N != w0->N || w1->K != w0->K))
        return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "moe: gate and up tensors differ in type or shape");
    p.act_q8 = act_q8;
    p.act_rows = act_rows;
    p.top_k = top_k;
    p.n_active = rt->n_active;
    p.uexp = rt->uexp;
    p.uoff = rt->uoff;
    p.uassign = rt->uassign;
    p.out = out;
    p.rpst = rows_per_stage_moe(p.type, p.K, p.row_bytes);
    uint32_t stage = ((uint32_t)p.rpst * p.row_bytes + 32 + 127) & ~127u;
    if (pair) {
        p.up_off = stage;
        stage *= 2;
    }
    p.stage_bytes = stage;
    p.err = ctx->d_err;
    const size_t act_bytes = (ActSmem::bytes(act_rows, p.K) + 127) & ~(size_t)127;
    if (pair) {
        if (T == 1) return launch_moe_mm<1, true>(ctx, p, act_bytes);
        if (T <= 4) return launch_moe_mm<4, true>(ctx, p, act_bytes);
        if (T <= 8) return launch_moe_mm<8, true>(ctx, p, act_bytes);
        return launch_moe_mm<16, true>(ctx, p, act_bytes);
    }
    if (T == 1) return launch_moe_mm<1, false>(ctx, p, act_bytes);
    if (T <= 4) return launch_moe_mm<4, false>(ctx, p, act_bytes);
    if (T <= 8) return launch_moe_mm<8, false>(ctx, p, act_bytes);
    return launch_moe_mm<16, false>(ctx, p, act_bytes);
}

int dc_launch_router(dc_ctx* ctx, const dc_weight* wr, const float* xn, int n_expert, int T, int top_k, float scale,
                     int ep_lo, int ep_hi, const dc_moe_route* rt, int mode) {
    // wr == nullptr: rt->logits already holds the router logits (routing only)
    if (wr && wr->type != DC_TYPE_F32) return dc_fail(ctx, DC_B200_UNSUPPORTED, "router weight must be F32");
    const int E = wr ? (int)wr->N : n_expert;
    if (E < 1 || E > MOE_MAX_E || top_k < 1 || top_k > MOE_MAX_K || top_k > E || T < 1 || T > DC_MAX_T)
        return dc_fail(ctx, DC_B200_UNSUPPORTED, "router: E=%d top_k=%d T=%d out of range", E, top_k, T);
    RouterParams p = {};
    p.wr = wr ? (const float*)wr->dev : nullptr;
    p.xn = xn;
    p.E = E;
    p.H = wr ? (int)wr->K : 0;
    p.T = T;
    p.top_k = top_k;
    p.scale = scale;
    p.mode = mode;
    p.ep_lo = ep_lo;
    p.ep_hi = ep_hi;
    p.logits = rt->logits;
    p.ids = rt->ids;
    p.weights = rt->weights;
    p.ticket = rt->ticket;
    p.n_active = rt->n_active;
    p.uexp = rt->uexp;
    p.uoff = rt->uoff;
    p.uassign = rt->uassign;
    return dc_launch(ctx, "k_router", k_router, dim3(wr ? (p.E + 1) / 2 : 1), dim3(256), 0, p);
}

// ------------------------------------------------------------ combine
// out[t][d] = sum over the token's assignments of w * down[assignment][d],
// added one at a time into a zeroed accumulator.  Order: routing order when
// T <= 4 and T*top_k <= 32 (cpu_backend_moe_ops.cpp:66,1247-1248,1578-1597),
// otherwise ascending expert id (moe_routing.cpp:647-676).  Assignments whose
// expert lives on another GPU are skipped (their share arrives by all-reduce).
__global__ void __launch_bounds__(256) k_moe_combine(const float* __restrict__ dn, const int32_t* __restrict__ ids,
                                                     const float* __restrict__ weights, int T, int top_k, int H,
                                                     int ep_lo, int ep_hi, float* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.y;
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= H) return;
    int order[MOE_MAX_K];
    for (int k = 0; k < top_k; ++k) order[k] = k;
    if (!(T <= 4 && T * top_k <= 32)) {
        for (int i = 1; i < top_k; ++i) {
            const int o = order[i], e = ids[t * top_k + o];
            int j = i - 1;
            while (j >= 0 && ids[t * top_k + order[j]] > e) {
                order[j + 1] = order[j];
                --j;
            }
            order[j + 1] = o;
        }
    }
    float sum = 0.0f;
    for (int k = 0; k < top_k; ++k) {
        const int a = t * top_k + order[k], e = ids[a];
        const float w = weights[a];
        if (e < ep_lo || e >= ep_hi || w == 0.0f) continue;
        sum = __fadd_rn(sum, __fmul_rn(w, dn[(size_t)a * H + d]));
    }
    out[(size_t)t * H + d] = sum;
}

int dc_launch_moe_combine(dc_ctx* ctx, const float* dn, const int32_t* ids, const float* weights, int T, int top_k,
                          int H, int ep_lo, int ep_hi, float* out) {
    return dc_launch(ctx, "k_moe_combine", k_moe_combine, dim3((H + 255) / 256, T), dim3(256), 0, dn, ids, weights, T,
                     top_k, H, ep_lo, ep_hi, out);
}
