// MUL_MAT over Q4_K / Q6_K weights for 1..16 activation rows, and the Q8_K
// activation quantiser.  Replaces cb_gemv_custom / cb_gemv_batched_custom
// (core/src/llm/matmul/gemv_exec.cpp:99, core/src/llm/matmul/batched_exec.cpp:55).
//
// Weights stay in their GGUF-native 144-byte / 210-byte super-blocks.  Every
// warp streams a contiguous range of weight rows HBM -> shared memory through
// its own ring of bulk async copies, decodes the 4/6-bit codes from shared
// memory and forms exact int32 block sums against the Q8_K activations with
// dp4a; the fp32 scaling and the cross-block sum are the only float steps.
#include <stdarg.h>
#include <stdio.h>

#include "dc_common.cuh"
#include "dc_internal.h"
#include "dc_stream.cuh"

using namespace dc;

__global__ void __launch_bounds__(256) k_quantize_q8k(const float* __restrict__ x, int n_blocks,
                                                      uint8_t* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const int nw = (gridDim.x * blockDim.x) >> 5;
    for (int b = gw; b < n_blocks; b += nw)
        quantize_block_q8k_warp(x + (size_t)b * DC_QK_K, out + (size_t)b * DC_Q8K_BYTES, lane);
}

int dc_launch_quantize_q8k(dc_ctx* ctx, const float* x, int rows, int K, uint8_t* out) {
    const int n_blocks = rows * (K / DC_QK_K);
    const int grid = (n_blocks + 7) / 8;
    k_quantize_q8k<<<grid < 1 ? 1 : grid, 256, 0, ctx->stream>>>(x, n_blocks, out);
    return dc_check_cuda(ctx, cudaGetLastError(), "k_quantize_q8k");
}

// ------------------------------------------------------------------- GEMV
// NSTAGE: pipeline depth per warp (2 where that lets more CTAs share an SM: the row decode is bound by
// instruction issue, so resident warps matter more than bytes in flight per warp).
template <int NT, int NSTAGE, bool DUMP = false>
__global__ void __launch_bounds__(DC_WARPS * 32) k_gemv(const GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem) + warp * NSTAGE;
    uint8_t* act_base = smem + DC_WARPS * DC_NSTAGE * 8;
    const size_t act_bytes = (ActSmem::bytes(p.T, p.K) + 127) & ~(size_t)127;
    uint8_t* bufs = act_base + act_bytes + (size_t)warp * NSTAGE * p.stage_bytes;

    WarpPipe<NSTAGE> pipe;
    pipe.init(bufs, bars, p.stage_bytes, p.err);
    GemvStream<NSTAGE> st;
    st.begin(p, blockIdx.x * DC_WARPS + warp, gridDim.x * DC_WARPS);
    // Weights do not depend on the previous kernel: start streaming before waiting for it.
    st.prefill(p, pipe, lane);
    pdl_launch_dependents();
    pdl_wait();

    ActSmem act;
    act.bind(act_base, p.T, p.K);
    act.fill(p.act_q8, p.T);
    __syncthreads();
    st.template consume<NT, true, DUMP>(p, pipe, act, lane);
}

static int rows_per_stage(int type, int K, int row_bytes) {
    const int G = dc::lanes_per_row(type, K);
    const int per_pass = 32 / G;
    int r = DC_STAGE_TARGET / row_bytes;
    r = r / per_pass * per_pass;
    return r < per_pass ? per_pass : r;
}

template <int NT, int NSTAGE, bool DUMP = false>
static int launch_gemv_ns(dc_ctx* ctx, const GemvParams& p, int grid, size_t smem) {
    int st = dc_kernel_setup(ctx, (const void*)k_gemv<NT, NSTAGE, DUMP>, 200 * 1024, "cudaFuncSetAttribute(k_gemv)");
    if (st != DC_B200_OK) return st;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(DC_WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->use_pdl ? 1 : 0;
    return dc_check_cuda(ctx, cudaLaunchKernelEx(&cfg, k_gemv<NT, NSTAGE, DUMP>, p), "k_gemv");
}

static size_t gemv_smem(size_t act_bytes, uint32_t stage, int ns) {
    return DC_WARPS * DC_NSTAGE * 8 + act_bytes + (size_t)DC_WARPS * ns * stage;
}
// CTAs of that size an SM holds (227 KB of shared memory, 1 KB reserved per CTA), at most 4.
static int gemv_ctas_per_sm(size_t smem) {
    if (smem > 200 * 1024) return 0;
    const int n = (int)((227u * 1024u) / (smem + 1024));
    return n > 4 ? 4 : n;
}

// Grid: a multiple of the SM count, no more warps than row groups; two stages per warp wherever that
// puts more CTAs on an SM.
template <int NT>
static int launch_gemv_nt(dc_ctx* ctx, const GemvParams& p, size_t act_bytes, int total_rows) {
    const size_t s4 = gemv_smem(act_bytes, p.stage_bytes, DC_NSTAGE), s2 = gemv_smem(act_bytes, p.stage_bytes, 2);
    // resident CTAs per SM by shared memory, then by the kernel's registers (asked once per device and instance)
    int reg_limit4 = dc_kernel_occupancy(ctx, (const void*)k_gemv<NT, DC_NSTAGE>, DC_WARPS * 32, 0);
    int reg_limit2 = dc_kernel_occupancy(ctx, (const void*)k_gemv<NT, 2>, DC_WARPS * 32, 0);
    if (reg_limit4 < 1) reg_limit4 = 1;
    if (reg_limit2 < 1) reg_limit2 = 1;
    int n4 = gemv_ctas_per_sm(s4), n2 = gemv_ctas_per_sm(s2);
    if (n4 > reg_limit4) n4 = reg_limit4;
    if (n2 > reg_limit2) n2 = reg_limit2;
    // parity capture of the block sums: the same kernel compiled with the stores in (never in a decoder step)
    if (p.dump.I) {
        const int max_useful = (total_rows + DC_WARPS - 1) / DC_WARPS;
        return launch_gemv_ns<NT, DC_NSTAGE, true>(ctx, p, ctx->num_sms < max_useful ? ctx->num_sms : max_useful, s4);
    }
    const bool two = n2 > n4;
    int grid = ctx->num_sms * (two ? n2 : n4);
    const int max_useful = (total_rows + DC_WARPS - 1) / DC_WARPS;
    if (grid > max_useful) grid = max_useful < 1 ? 1 : max_useful;
    return two ? launch_gemv_ns<NT, 2>(ctx, p, grid, s2) : launch_gemv_ns<NT, DC_NSTAGE>(ctx, p, grid, s4);
}

int dc_launch_gemv(dc_ctx* ctx, const dc_gemv_seg* segs, int n_seg, int epi, const uint8_t* act_q8, int T, int K,
                   unsigned long long* argmax, int32_t* dump_I, int32_t* dump_M) {
    if (n_seg < 1 || n_seg > 3 || T < 1 || T > DC_MAX_T || K % DC_QK_K)
        return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "gemv: bad shape (n_seg=%d T=%d K=%d)", n_seg, T, K);
    GemvParams p = {};
    p.n_seg = n_seg;
    p.epi = epi;
    p.act_q8 = act_q8;
    p.T = T;
    p.K = K;
    p.argmax = argmax;
    p.err = ctx->d_err;
    if (dump_I) {
        if (n_seg != 1 || epi != DC_EPI_STORE) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "gemv: block-sum capture takes one plain segment");
        p.dump = BlockSumDump{dump_I, dump_M, segs[0].n_rows};
    }
    uint32_t stage = 0;
    int total = 0;
    for (int i = 0; i < n_seg; ++i) {
        p.seg[i] = segs[i];
        if (segs[i].type != DC_TYPE_Q4_K && segs[i].type != DC_TYPE_Q6_K)
            return dc_fail(ctx, DC_B200_UNSUPPORTED, "gemv: weight type %d is not Q4_K/Q6_K", segs[i].type);
        p.rpst[i] = rows_per_stage(segs[i].type, K, segs[i].row_bytes);
        const uint32_t need = (uint32_t)p.rpst[i] * segs[i].row_bytes + 32;
        stage = need > stage ? need : stage;
        total += segs[i].n_rows;
    }
    stage = (stage + 127) & ~127u;
    if (epi == DC_EPI_SWIGLU) {
        if (n_seg != 2 || segs[0].n_rows != segs[1].n_rows || segs[0].type != segs[1].type)
            return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "gemv: SwiGLU needs matching gate/up segments");
        total = segs[0].n_rows;
        p.up_off = stage;
        stage *= 2;
    }
    p.total_rows = total;
    p.stage_bytes = stage;
    const size_t act_bytes = (ActSmem::bytes(T, K) + 127) & ~(size_t)127;
    if (gemv_smem(act_bytes, stage, 2) > 200 * 1024) {
        // activations of all T tokens do not fit beside the weight pipeline: run the tokens in two halves
        if (T == 1 || argmax || dump_I)
            return dc_fail(ctx, DC_B200_UNSUPPORTED, "gemv: shared memory need %zu too large", gemv_smem(act_bytes, stage, 2));
        const int T0 = T / 2;
        dc_gemv_seg second[3];
        for (int i = 0; i < n_seg; ++i) {
            second[i] = segs[i];
            second[i].out = segs[i].out + (size_t)T0 * segs[i].ldo;
        }
        int st = dc_launch_gemv(ctx, segs, n_seg, epi, act_q8, T0, K, nullptr);
        if (st != DC_B200_OK) return st;
        return dc_launch_gemv(ctx, second, n_seg, epi, act_q8 + (size_t)T0 * (K / DC_QK_K) * DC_Q8K_BYTES, T - T0, K, nullptr);
    }
    if (T == 1) return launch_gemv_nt<1>(ctx, p, act_bytes, total);
    if (T <= 4) return launch_gemv_nt<4>(ctx, p, act_bytes, total);
    if (T <= 8) return launch_gemv_nt<8>(ctx, p, act_bytes, total);
    return launch_gemv_nt<16>(ctx, p, act_bytes, total);
}

