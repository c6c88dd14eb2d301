// Row-streaming matmul bodies shared by the stand-alone kernels (k_gemv,
// k_moe_mm) and the persistent decode kernel: each warp walks a contiguous
// range of weight rows through its bulk-copy pipeline, decodes them against the
// Q8_K activations in shared memory and writes one float per (row, token).
#pragma once
#include "dc_common.cuh"
#include "dc_internal.h"

namespace dc {

struct GemvParams {
    dc_gemv_seg seg[3];
    int n_seg;
    int rpst[3];      // rows per pipeline stage, per segment
    int total_rows;   // flattened over segments (pairs count once for SwiGLU)
    int epi;
    const uint8_t* act_q8;
    int T, K;
    uint32_t stage_bytes;
    uint32_t up_off;  // SwiGLU: offset of the up rows inside a stage
    unsigned long long* argmax;
    int* err;
    BlockSumDump dump;   // parity checks only: where the exact block sums go (I == nullptr: nowhere)
};

// Walks a warp's contiguous flattened row range stage by stage.
struct StageIter {
    int cur, end;
    __device__ __forceinline__ bool next(const GemvParams& p, int& seg, int& local, int& n) {
        if (cur >= end) return false;
        int s = 0, base = 0;
        const int nseg = p.epi == DC_EPI_SWIGLU ? 1 : p.n_seg;
        while (s + 1 < nseg && cur >= base + p.seg[s].n_rows) {
            base += p.seg[s].n_rows;
            ++s;
        }
        seg = s;
        local = cur - base;
        int lim = min(end, base + p.seg[s].n_rows);
        n = min(p.rpst[s], lim - cur);
        cur += n;
        return true;
    }
};

__device__ __forceinline__ unsigned long long argmax_key(float v, int row) {
    uint32_t u = __float_as_uint(v);
    if (v != v) u = 0;  // NaN never wins
    else u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)row);
}

template <int NSTAGE>
struct GemvStream {
    StageIter prod, cons;
    // A Q6_K row takes about twice the instructions of a Q4_K row of the same K.
    __device__ __forceinline__ static int row_weight(int type) { return type == DC_TYPE_Q6_K ? 2 : 1; }
    // Flattened row index at weighted position x (segments in order, each row weighing row_weight).
    __device__ __forceinline__ static int row_at(const GemvParams& p, int nseg, unsigned x) {
        unsigned cum = 0;
        int base = 0;
        for (int s = 0; s < nseg; ++s) {
            const unsigned w = (unsigned)row_weight(p.seg[s].type);
            const unsigned span = (unsigned)p.seg[s].n_rows * w;
            if (x < cum + span) return base + (int)((x - cum) / w);
            cum += span;
            base += p.seg[s].n_rows;
        }
        return base;
    }
    // gw * total / nw without 64-bit division where the product fits 32 bits (every shape of a decoder step;
    // the wide form is kept for safety)
    __device__ __forceinline__ static unsigned share(unsigned gw, unsigned total, unsigned nw) {
        if ((unsigned long long)nw * total < 0xFFFFFFFFull) return gw * total / nw;
        return (unsigned)((unsigned long long)gw * total / nw);
    }
    // Each warp takes a contiguous range of rows; with segments of different types the ranges are balanced
    // by weight, so that the warps holding the costlier rows are not the last to finish.
    __device__ __forceinline__ static void range(const GemvParams& p, int gw, int nw, int& r0, int& r1) {
        const int nseg = p.epi == DC_EPI_SWIGLU ? 1 : p.n_seg;
        bool mixed = false;
        unsigned total_w = 0;
        for (int s = 0; s < nseg; ++s) {
            mixed |= p.seg[s].type != p.seg[0].type;
            total_w += (unsigned)p.seg[s].n_rows * (unsigned)row_weight(p.seg[s].type);
        }
        if (!mixed) {
            r0 = (int)share((unsigned)gw, (unsigned)p.total_rows, (unsigned)nw);
            r1 = (int)share((unsigned)gw + 1u, (unsigned)p.total_rows, (unsigned)nw);
        } else {
            r0 = row_at(p, nseg, share((unsigned)gw, total_w, (unsigned)nw));
            r1 = gw + 1 == nw ? p.total_rows : row_at(p, nseg, share((unsigned)gw + 1u, total_w, (unsigned)nw));
        }
    }
    __device__ __forceinline__ void begin(const GemvParams& p, int gw, int nw) {
        int r0, r1;
        range(p, gw, nw, r0, r1);
        prod = StageIter{r0, r1};
        cons = StageIter{r0, r1};
    }
    // Rebuilds the iterators of a stream whose first `inflight` stages were already issued
    // (by prefill in an earlier phase), so that no iterator has to stay live in between.
    __device__ __forceinline__ void resume(const GemvParams& p, int gw, int nw, int inflight) {
        begin(p, gw, nw);
        int sg, lr, n;
        for (int i = 0; i < inflight; ++i) prod.next(p, sg, lr, n);
    }
    // The same from a row range the caller kept (no partition arithmetic).
    __device__ __forceinline__ void resume_range(const GemvParams& p, int r0, int r1, int inflight) {
        prod = StageIter{r0, r1};
        cons = StageIter{r0, r1};
        int sg, lr, n;
        for (int i = 0; i < inflight; ++i) prod.next(p, sg, lr, n);
    }
    // lane 0 only
    __device__ __forceinline__ void issue_next(const GemvParams& p, WarpPipe<NSTAGE>& pipe) {
        int sg, lr, n;
        if (!prod.next(p, sg, lr, n)) return;
        const dc_gemv_seg& s = p.seg[sg];
        const uint32_t bytes = (uint32_t)n * s.row_bytes;
        if (p.epi == DC_EPI_SWIGLU)
            pipe.issue2(s.w + (size_t)lr * s.row_bytes, p.seg[1].w + (size_t)lr * s.row_bytes, bytes, p.up_off);
        else
            pipe.issue(s.w + (size_t)lr * s.row_bytes, bytes);
    }
    __device__ __forceinline__ void prefill(const GemvParams& p, WarpPipe<NSTAGE>& pipe, int lane) {
        if (lane == 0) {
#pragma unroll 1
            for (int s = 0; s < NSTAGE; ++s) issue_next(p, pipe);
        }
    }
    // SWIGLU = false leaves the paired gate/up path out of the generated code (callers that
    // never stream pairs).
    // SWIGLU = false leaves the paired gate/up path out of the generated code (callers that never stream
    // pairs).  DUMP = true also stores the exact block sums (parity checks; never in the decoder's launches).
    // A warp pass runs 32 / G rows side by side, one per lane group.  Gate/up pairs: the lower half of the
    // groups takes gate rows, the upper half the up rows of the same outputs, and the two halves swap
    // results 16 lanes across (one group per row, G = 32: gate row, then up row).
    template <int NT, bool SWIGLU = true, bool DUMP = false>
    __device__ DC_HOT void consume(const GemvParams& p, WarpPipe<NSTAGE>& pipe, const ActSmem& act, int lane) {
        int tok[NT];
#pragma unroll
        for (int s = 0; s < NT; ++s) tok[s] = s;
        unsigned long long best[NT];
#pragma unroll
        for (int s = 0; s < NT; ++s) best[s] = 0ull;
        const bool pair = SWIGLU && p.epi == DC_EPI_SWIGLU;
        int sg, lr, n;
        while (cons.next(p, sg, lr, n)) {
            const dc_gemv_seg& s = p.seg[sg];
            const uint32_t buf = pipe.wait();
            const int G = lanes_per_row(s.type, p.K);
            const int rpp = 32 / G;                       // rows per pass
            const int grp = lane / G, lig = lane % G;
            const bool split = pair && rpp >= 2;          // gate and up rows in one pass
            const int opp = split ? rpp / 2 : rpp;        // outputs per pass
            const bool up_half = split && grp >= opp;
            const uint32_t skew = (uint32_t)(((uintptr_t)s.w + (size_t)lr * s.row_bytes) & 15);
            const uint32_t skew_up = pair ? (uint32_t)(((uintptr_t)p.seg[1].w + (size_t)lr * s.row_bytes) & 15) : 0u;
            const uint32_t base = up_half ? buf + p.up_off + skew_up : buf + skew;
            const BlockSumDump* dump = DUMP ? &p.dump : nullptr;
            for (int r = 0; r < n; r += opp) {
                const int rr = r + (split ? grp % opp : grp);
                const bool active = rr < n;
                float acc[NT], acc2[NT];
                if (NT == 1 && !DUMP) acc[0] = rows_dot1_typed(s.type, base + rr * s.row_bytes, active, lane, G, act, 0);
                else rows_dot_typed<NT>(s.type, base + rr * s.row_bytes, active, lane, G, act, p.T, tok, acc, dump, lr + rr);
                if (pair) {
                    if (split) {
#pragma unroll
                        for (int t = 0; t < NT; ++t) acc2[t] = __shfl_xor_sync(0xffffffffu, acc[t], 16);
                    } else {
                        const uint32_t urow = buf + p.up_off + skew_up + rr * s.row_bytes;
                        if (NT == 1 && !DUMP) acc2[0] = rows_dot1_typed(s.type, urow, active, lane, G, act, 0);
                        else rows_dot_typed<NT>(s.type, urow, active, lane, G, act, p.T, tok, acc2);
                    }
                }
                // every lane of a row's group holds the row's results; lane (t mod G) of the group stores token t
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    if (t < p.T) {
                        float v = acc[t];
                        if (pair) v = __fmul_rn(silu_fast(v), acc2[t]);
                        if (active && !up_half && lig == (t & (G - 1))) {
                            const int row = lr + rr;
                            float* o = s.out + (size_t)t * s.ldo + row;
                            if (p.epi == DC_EPI_ACC) *o = __ldcg(o) + v;  // L2 read: another SM may have written it
                            else *o = v;
                            if (p.argmax) {
                                const unsigned long long k = argmax_key(v, row);
                                best[t] = k > best[t] ? k : best[t];
                            }
                        }
                    }
                }
            }
            pipe.release();
            if (lane == 0) issue_next(p, pipe);
        }
        if (p.argmax) {
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                if (t < p.T) {
                    unsigned long long k = best[t];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        const unsigned long long ok = __shfl_xor_sync(0xffffffffu, k, o);
                        k = ok > k ? ok : k;
                    }
                    if (lane == 0 && k) atomicMax(p.argmax + t, k);
                }
            }
        }
    }
};

// ------------------------------------------------------------ expert rows
struct MoeMMParams {
    const uint8_t* w0;    // gate (PAIR) or down
    const uint8_t* w1;    // up (PAIR)
    int type, row_bytes, N /*rows per expert*/, K;
    const uint8_t* act_q8;  // Q8_K rows: tokens (PAIR) or assignments (down)
    int act_rows, top_k;
    int e_base;           // first expert stored in w0/w1 (expert-parallel shard)
    const int* n_active;
    const int32_t* uexp;
    const int32_t* uoff;
    const int32_t* uassign;
    float* out;           // [assignment][N]
    float* peer_out[7];   // the same array in other GPUs' memory: results are stored there too
    int n_peer;
    int rpst;
    uint32_t stage_bytes, up_off;
    int* err;
};

// Walks a flattened range of (unit, row) pairs stage by stage; the unit and the row inside it are carried
// along (one division when the walk starts, none per stage).
struct MoeIter {
    int cur, end, N, rpst, cu, cr;
    __device__ __forceinline__ static MoeIter make(int r0, int r1, int N, int rpst) {
        const int u = r0 / N;
        return MoeIter{r0, r1, N, rpst, u, r0 - u * N};
    }
    __device__ __forceinline__ bool next(int& u, int& r, int& n) {
        if (cur >= end) return false;
        u = cu;
        r = cr;
        n = min(rpst, min(N - cr, end - cur));
        cur += n;
        cr += n;
        if (cr == N) {
            cr = 0;
            ++cu;
        }
        return true;
    }
};

// PAIRMODE: 0 = single rows (down), 1 = gate/up pairs with SwiGLU, 2 = decided at run time
// by p.w1 (one body serves both uses).
template <int NSTAGE, int PAIRMODE>
struct MoeStream {
    __device__ __forceinline__ static bool is_pair(const MoeMMParams& p) {
        return PAIRMODE == 2 ? p.w1 != nullptr : PAIRMODE == 1;
    }
    MoeIter prod, cons;
    size_t estride;
    // Flattened row index (unit * N + row) at weighted position x, where a row of a unit with nt
    // tokens weighs 1 + nt (one decode plus one dot per token).
    __device__ __forceinline__ static int row_at(const MoeMMParams& p, int U, unsigned x) {
        unsigned cum = 0;
        for (int u = 0; u < U; ++u) {
            const unsigned w = 1u + (unsigned)(p.uoff[u + 1] - p.uoff[u]);
            const unsigned span = (unsigned)p.N * w;
            if (x < cum + span) return u * p.N + (int)((x - cum) / w);
            cum += span;
        }
        return U * p.N;
    }
    // (rows x weights of one MoE layer stay far below 2^32 / warps: 32-bit arithmetic throughout)
    __device__ __forceinline__ static void range(const MoeMMParams& p, int U, int gw, int nw, int& r0, int& r1) {
        const int A = p.uoff[U];   // assignments in all units
        if (A == U) {              // one token per expert everywhere: plain even split
            const unsigned total = (unsigned)(U * p.N);
            r0 = (int)((unsigned)gw * total / (unsigned)nw);
            r1 = (int)(((unsigned)gw + 1u) * total / (unsigned)nw);
        } else {
            const unsigned total_w = (unsigned)p.N * (unsigned)(U + A);
            r0 = row_at(p, U, (unsigned)gw * total_w / (unsigned)nw);
            r1 = gw + 1 == nw ? U * p.N : row_at(p, U, ((unsigned)gw + 1u) * total_w / (unsigned)nw);
        }
    }
    // Each warp takes a contiguous range of the active experts' rows; ranges are balanced by weight so
    // that experts serving several tokens do not make their warps the last to finish.
    __device__ __forceinline__ void begin(const MoeMMParams& p, int U, int gw, int nw) {
        int r0, r1;
        range(p, U, gw, nw, r0, r1);
        prod = MoeIter::make(r0, r1, p.N, p.rpst);
        cons = prod;
        estride = (size_t)p.N * p.row_bytes;
    }
    __device__ __forceinline__ void resume(const MoeMMParams& p, int U, int gw, int nw, int inflight) {
        begin(p, U, gw, nw);
        int u, r, n;
        for (int i = 0; i < inflight; ++i) prod.next(u, r, n);
    }
    __device__ __forceinline__ void resume_range(const MoeMMParams& p, int r0, int r1, int inflight) {
        prod = MoeIter::make(r0, r1, p.N, p.rpst);
        cons = prod;
        estride = (size_t)p.N * p.row_bytes;
        int u, r, n;
        for (int i = 0; i < inflight; ++i) prod.next(u, r, n);
    }
    __device__ __forceinline__ void issue_next(const MoeMMParams& p, WarpPipe<NSTAGE>& pipe) {
        int u, r, n;
        if (!prod.next(u, r, n)) return;
        const size_t off = (size_t)(p.uexp[u] - p.e_base) * estride + (size_t)r * p.row_bytes;
        if (is_pair(p)) pipe.issue2(p.w0 + off, p.w1 + off, (uint32_t)n * p.row_bytes, p.up_off);
        else pipe.issue(p.w0 + off, (uint32_t)n * p.row_bytes);
    }
    __device__ __forceinline__ void prefill(const MoeMMParams& p, WarpPipe<NSTAGE>& pipe, int lane) {
        if (lane == 0) {
#pragma unroll 1
            for (int s = 0; s < NSTAGE; ++s) issue_next(p, pipe);
        }
    }
    // The rows of one stage for the first NTT token slots of tok/asg (see GemvStream::consume for the
    // layout of a pass).
    template <int NTT>
    __device__ __forceinline__ static void stage_rows(const MoeMMParams& p, const ActSmem& act, uint32_t buf, uint32_t skew0,
                                                      uint32_t skew1, bool pair, int r, int n, int nt, const int* tok_in,
                                                      const int* asg_in, int G, int lane) {
        const int rpp = 32 / G, grp = lane / G, lig = lane % G;
        const bool split = pair && rpp >= 2;
        const int opp = split ? rpp / 2 : rpp;
        const bool up_half = split && grp >= opp;
        const uint32_t base = buf + (up_half ? skew1 : skew0);
        int tok[NTT], asg[NTT];
#pragma unroll
        for (int s = 0; s < NTT; ++s) {
            tok[s] = tok_in[s];
            asg[s] = asg_in[s];
        }
        for (int rr0 = 0; rr0 < n; rr0 += opp) {
            const int rr = rr0 + (split ? grp % opp : grp);
            const bool active = rr < n;
            float v[NTT], u[NTT];
            if (NTT == 1) v[0] = rows_dot1_typed(p.type, base + rr * p.row_bytes, active, lane, G, act, tok[0]);
            else rows_dot_typed<NTT>(p.type, base + rr * p.row_bytes, active, lane, G, act, nt, tok, v);
            if (pair) {
                if (split) {
#pragma unroll
                    for (int s = 0; s < NTT; ++s) u[s] = __shfl_xor_sync(0xffffffffu, v[s], 16);
                } else {
                    const uint32_t urow = buf + skew1 + rr * p.row_bytes;
                    if (NTT == 1) u[0] = rows_dot1_typed(p.type, urow, active, lane, G, act, tok[0]);
                    else rows_dot_typed<NTT>(p.type, urow, active, lane, G, act, nt, tok, u);
                }
#pragma unroll
                for (int s = 0; s < NTT; ++s)
                    if (s < nt) v[s] = __fmul_rn(silu_fast(v[s]), u[s]);
            }
#pragma unroll
            for (int s = 0; s < NTT; ++s)
                if (s < nt && active && !up_half && lig == (s & (G - 1))) {
                    const size_t oi = (size_t)asg[s] * p.N + r + rr;
                    p.out[oi] = v[s];
                    for (int q = 0; q < p.n_peer; ++q) p.peer_out[q][oi] = v[s];
                }
        }
    }

    template <int NT>
    __device__ DC_HOT void consume(const MoeMMParams& p, WarpPipe<NSTAGE>& pipe, const ActSmem& act, int lane) {
        const bool pair = is_pair(p);
        const int G = lanes_per_row(p.type, p.K);
        int u, r, n;
        while (cons.next(u, r, n)) {
            const uint32_t buf = pipe.wait();
            const size_t off = (size_t)(p.uexp[u] - p.e_base) * estride + (size_t)r * p.row_bytes;
            const uint32_t skew0 = (uint32_t)(((uintptr_t)p.w0 + off) & 15);
            const uint32_t skew1 = pair ? p.up_off + (uint32_t)(((uintptr_t)p.w1 + off) & 15) : 0u;
            const int a0 = p.uoff[u], nt = min(NT, p.uoff[u + 1] - a0);
            int tok[NT], asg[NT];
#pragma unroll
            for (int s = 0; s < NT; ++s) {
                asg[s] = s < nt ? p.uassign[a0 + s] : 0;
                tok[s] = pair ? asg[s] / p.top_k : asg[s];
            }
            // most experts of a step serve a single token: that case runs the one-token body
            // and at 8 or 16 tokens per step few experts serve more than four
            if (NT > 1 && nt == 1) stage_rows<1>(p, act, buf, skew0, skew1, pair, r, n, nt, tok, asg, G, lane);
            else if (NT > 4 && nt <= 4) stage_rows<4>(p, act, buf, skew0, skew1, pair, r, n, nt, tok, asg, G, lane);
            else stage_rows<NT>(p, act, buf, skew0, skew1, pair, r, n, nt, tok, asg, G, lane);
            pipe.release();
            if (lane == 0) issue_next(p, pipe);
        }
    }
};

}  // namespace dc
