// Device-side building blocks shared by every kernel of the library:
// block layouts, exact scalar helpers, the per-warp bulk-copy pipeline that
// streams weight rows HBM -> shared memory, and the K-quant row-dot decoders.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define DC_QK_K 256
#define DC_Q4K_BYTES 144
#define DC_Q6K_BYTES 210
#define DC_Q8K_BYTES 292
#define DC_KV_BLOCK 16   // core/include/densecore/memory/kv_cache.h:50
#define DC_MAX_T 16      // tokens per step (kMaxSmallBatchColsHard, core/src/llm/matmul/userdata.h:14)
#define DC_TYPE_F32 0
#define DC_TYPE_F16 1
#define DC_TYPE_Q4_K 12
#define DC_TYPE_Q6_K 14

// Hot bodies (row dots, stream loops, phases of the persistent kernel) are inlined into their callers;
// the callers that several sites share are the ones kept out of line (measured: outlining per row costs
// 12 %, outlining per phase is free and shrinks the code).
#define DC_HOT __forceinline__
// Bounded waits: every wait on an mbarrier gives up after this many polls,
// records an error code in the context's device error word and carries on, so
// no kernel can hang the GPU.
#define DC_WAIT_LIMIT (1u << 22)
#define DC_ERR_MBAR_TIMEOUT 1

namespace dc {

__device__ __forceinline__ float fp16_bits_to_float(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// core/src/kernels/hwy/hwy_fastexp.h:50-84 (fused multiply-add Horner form).
__device__ __forceinline__ float fast_exp_fma(float x) {
    x = fmaxf(fminf(x, 50.0f), -50.0f);
    const float y = __fmul_rn(x, 1.4426950408889634f);
    const float i_f = floorf(y);
    const float f = __fsub_rn(y, i_f);
    float p = __fmaf_rn(0.07944023841053369f, f, 0.224494337302845f);
    p = __fmaf_rn(p, f, 0.6960656421638072f);
    p = __fmaf_rn(p, f, 1.0f);
    return __fmul_rn(p, __int_as_float(((int)i_f + 127) << 23));
}
// core/src/backend/cpu_backend_internal.h:99-114 (separate multiply and add).
__device__ __forceinline__ float fast_exp(float x) {
    x = fmaxf(fminf(x, 50.0f), -50.0f);
    const float y = __fmul_rn(x, 1.4426950408889634f);
    const int i = (int)floorf(y);
    const float f = __fsub_rn(y, (float)i);
    float p = __fadd_rn(0.224494337302845f, __fmul_rn(f, 0.07944023841053369f));
    p = __fadd_rn(0.6960656421638072f, __fmul_rn(f, p));
    p = __fadd_rn(1.0f, __fmul_rn(f, p));
    return __fmul_rn(__int_as_float((i + 127) << 23), p);
}
// SiLU of the production SwiGLU kernels: g / (1 + fast_exp(-g))
// (core/src/backend/cpu_backend_moe_quant_projection.inl:710-802).
__device__ __forceinline__ float silu_fast(float g) { return __fdiv_rn(g, __fadd_rn(1.0f, fast_exp(-g))); }

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait; returns false (and records the error) if the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* err_word) {
    for (uint32_t i = 0; i < DC_WAIT_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    if (err_word) atomicExch(err_word, DC_ERR_MBAR_TIMEOUT);
    return false;
}
// Untiled bulk copy global -> this CTA's shared memory (no multicast).
// dst, src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
// Programmatic dependent launch: let the next kernel in the stream start its
// prologue, and wait for the previous kernel's results.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ------------------------------------------------- per-warp row pipeline
// Each warp owns NSTAGE shared-memory buffers and one mbarrier per buffer.
// Lane 0 issues one bulk copy per stage covering a byte range of the weight
// tensor (rounded out to 16-byte boundaries); all lanes wait on the stage's
// barrier, decode from shared memory, __syncwarp, and lane 0 refills.
template <int NSTAGE>
struct WarpPipe {
    uint32_t buf0;       // shared address of stage 0
    uint32_t bar0;       // shared address of barrier 0
    uint32_t stage_bytes;
    uint32_t issued, consumed;
    int* err;

    __device__ __forceinline__ void init(uint8_t* smem_bufs, uint64_t* smem_bars, uint32_t stage_bytes_, int* err_word) {
        buf0 = smem_u32(smem_bufs);
        bar0 = smem_u32(smem_bars);
        stage_bytes = stage_bytes_;
        issued = consumed = 0;
        err = err_word;
        if ((threadIdx.x & 31) == 0) {
            for (int s = 0; s < NSTAGE; ++s) mbar_init(bar0 + 8 * s, 1);
            mbar_fence_init();
        }
        __syncwarp();
    }
    // Lane 0 only.  Copies [src, src+bytes) (any alignment) as the enclosing
    // 16-byte aligned range; returns nothing, the consumer recomputes the skew.
    __device__ __forceinline__ void issue(const uint8_t* src, uint32_t bytes) {
        const uint32_t s = issued % NSTAGE;
        const uintptr_t a = (uintptr_t)src;
        const uintptr_t a0 = a & ~(uintptr_t)15;
        const uint32_t len = (uint32_t)(((a + bytes + 15) & ~(uintptr_t)15) - a0);
        mbar_expect_tx(bar0 + 8 * s, len);
        bulk_g2s(buf0 + s * stage_bytes, (const void*)a0, len, bar0 + 8 * s);
        ++issued;
    }
    // Two ranges into one stage (gate row + up row).  Second lands at offset off2.
    __device__ __forceinline__ void issue2(const uint8_t* src1, const uint8_t* src2, uint32_t bytes, uint32_t off2) {
        const uint32_t s = issued % NSTAGE;
        const uintptr_t a = (uintptr_t)src1, b = (uintptr_t)src2;
        const uintptr_t a0 = a & ~(uintptr_t)15, b0 = b & ~(uintptr_t)15;
        const uint32_t la = (uint32_t)(((a + bytes + 15) & ~(uintptr_t)15) - a0);
        const uint32_t lb = (uint32_t)(((b + bytes + 15) & ~(uintptr_t)15) - b0);
        mbar_expect_tx(bar0 + 8 * s, la + lb);
        bulk_g2s(buf0 + s * stage_bytes, (const void*)a0, la, bar0 + 8 * s);
        bulk_g2s(buf0 + s * stage_bytes + off2, (const void*)b0, lb, bar0 + 8 * s);
        ++issued;
    }
    // All lanes.  Returns the shared address of the stage's buffer.
    __device__ __forceinline__ uint32_t wait() {
        const uint32_t s = consumed % NSTAGE;
        mbar_wait(bar0 + 8 * s, (consumed / NSTAGE) & 1, err);
        return buf0 + s * stage_bytes;
    }
    __device__ __forceinline__ void release() {
        ++consumed;
        __syncwarp();
    }
    // Leaving early: lane 0 (the only lane that counts issues) waits, bounded, for the copies still in flight.
    __device__ __forceinline__ void drain() {
        if ((threadIdx.x & 31) == 0)
            for (; consumed < issued; ++consumed) mbar_wait(bar0 + 8 * (consumed % NSTAGE), (consumed / NSTAGE) & 1, nullptr);
        __syncwarp();
    }
};

// ------------------------------------------------------- shared loads
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t a) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds8(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ int lds_s8(uint32_t a) {
    int v;
    asm volatile("ld.shared.s8 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
// 32-bit load from a 2-byte aligned shared address.
__device__ __forceinline__ uint32_t lds32_a2(uint32_t a) { return lds16(a) | (lds16(a + 2) << 16); }

// ------------------------------------------------------------ Q8_K quantise
// One warp per 256-element block; lane l holds elements 8l..8l+7.
// Follows core/src/kernels/hwy/hwy_moe_quant.cc:103-144 step by step:
// first element of largest magnitude keeps its sign; iscale = -127/max;
// q = min(127, rne(iscale*x)); bsums per 16; d = 1/iscale.
// Core of the block quantiser: every lane gets its two packed words of codes,
// the bsums word it may own (lanes with lane%4==0: groups lane/2 and lane/2+1)
// and the block scale d (0 for an all-zero block).
__device__ __forceinline__ void q8k_block_core(const float (&v)[8], int lane, uint32_t& w0, uint32_t& w1,
                                               uint32_t& bsum_word, float& d) {
    float amax = 0.0f, mx = 0.0f;
    int idx = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float ax = fabsf(v[j]);
        if (ax > amax) {
            amax = ax;
            mx = v[j];
            idx = 8 * lane + j;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, amax, o);
        const float om = __shfl_xor_sync(0xffffffffu, mx, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (oa > amax || (oa == amax && oi < idx)) {
            amax = oa;
            mx = om;
            idx = oi;
        }
    }
    if (amax == 0.0f) {
        w0 = w1 = bsum_word = 0u;
        d = 0.0f;
        return;
    }
    const float iscale = __fdiv_rn(-127.0f, mx);
    int q[8], sum = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        q[j] = min(127, __float2int_rn(__fmul_rn(iscale, v[j])));
        sum += q[j];
    }
    w0 = (q[0] & 0xFF) | ((q[1] & 0xFF) << 8) | ((q[2] & 0xFF) << 16) | ((uint32_t)(q[3] & 0xFF) << 24);
    w1 = (q[4] & 0xFF) | ((q[5] & 0xFF) << 8) | ((q[6] & 0xFF) << 16) | ((uint32_t)(q[7] & 0xFF) << 24);
    // bsums: group g = lanes 2g, 2g+1
    const int pair = sum + __shfl_xor_sync(0xffffffffu, sum, 1);
    const int other = __shfl_xor_sync(0xffffffffu, pair, 2);  // neighbouring group's sum
    bsum_word = (uint32_t)(pair & 0xFFFF) | ((uint32_t)(other & 0xFFFF) << 16);
    d = __fdiv_rn(1.0f, iscale);
}
// Writes the native 292-byte block.
__device__ __forceinline__ void quantize_block_q8k_regs(const float (&v)[8], uint8_t* __restrict__ out, int lane) {
    uint32_t w0, w1, bw;
    float d;
    q8k_block_core(v, lane, w0, w1, bw, d);
    uint32_t* o32 = reinterpret_cast<uint32_t*>(out);
    o32[1 + 2 * lane] = w0;
    o32[2 + 2 * lane] = w1;
    if ((lane & 3) == 0) o32[65 + (lane >> 2)] = bw;
    if (lane == 0) o32[0] = __float_as_uint(d);
}
__device__ __forceinline__ void quantize_block_q8k_warp(const float* __restrict__ x, uint8_t* __restrict__ out,
                                                        int lane) {
    float v[8];
    const float4 a = reinterpret_cast<const float4*>(x)[2 * lane];
    const float4 b = reinterpret_cast<const float4*>(x)[2 * lane + 1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    quantize_block_q8k_regs(v, out, lane);
}

// ------------------------------------------------------- activations
// Q8_K activations of the step's tokens in shared memory, laid out for the dot kernels, where one lane
// works on one whole super-block: per (token, block) 256 int8 codes 272 bytes apart, the f32 scale, and
// the 16 int16 sums 48 bytes apart.  The lanes of a quarter warp read the same offset of neighbouring
// blocks with 128-bit loads: 272 bytes = 68 words and 48 bytes = 12 words put those eight accesses on
// disjoint bank quads.  Filled from the native 292-byte blocks in global memory.
struct ActSmem {
    uint32_t qs, d, bs;  // shared addresses
    int K, nb;
    static constexpr uint32_t QS = 272, BS = 48;
    __host__ __device__ __forceinline__ static size_t bytes(int T, int K) {
        const size_t n = (size_t)T * (K / DC_QK_K);
        return n * QS + ((n * 4 + 15) & ~(size_t)15) + n * BS;
    }
    __device__ __forceinline__ void bind(uint8_t* base, int T, int K_) {
        K = K_;
        nb = K_ / DC_QK_K;
        const uint32_t n = (uint32_t)(T * nb);
        qs = smem_u32(base);
        d = qs + n * QS;
        bs = d + ((n * 4 + 15) & ~15u);
    }
    __device__ __forceinline__ uint32_t qblk(int t, int b) const { return qs + (uint32_t)(t * nb + b) * QS; }
    __device__ __forceinline__ uint32_t dptr(int t, int b) const { return d + (uint32_t)(t * nb + b) * 4; }
    __device__ __forceinline__ uint32_t bsptr(int t, int b) const { return bs + (uint32_t)(t * nb + b) * BS; }
    // Cooperative fill by the whole CTA from native Q8_K rows (row stride nb*292).
    // CG: read through L2 (the rows were written by other SMs during this kernel).
    template <bool CG = false>
    __device__ __forceinline__ void fill(const uint8_t* q8, int T) {
        const int words_per_row = nb * 73;  // 292/4
        const uint32_t* src = reinterpret_cast<const uint32_t*>(q8);
        // CG readers are many CTAs reading the same rows at once: each starts somewhere else
        const int total = T * words_per_row, rot = CG ? (int)((blockIdx.x * 97u) % (unsigned)total) : 0;
        for (int il = threadIdx.x; il < total; il += blockDim.x) {
            const int i = CG ? (il + rot) % total : il;
            const int t = i / words_per_row, w = i - t * words_per_row;
            const int b = w / 73, o = w - b * 73;
            const uint32_t v = CG ? __ldcg(src + i) : src[i];
            uint32_t dst;
            if (o == 0) dst = dptr(t, b);
            else if (o <= 64) dst = qblk(t, b) + (o - 1) * 4;
            else dst = bsptr(t, b) + (o - 65) * 4;
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(dst), "r"(v));
        }
    }
};

// Quantises one 256-element block held in registers (lane l: elements 8l..8l+7)
// straight into the shared-memory activation layout: row t, block b.
__device__ __forceinline__ void quantize_block_q8k_to_act(const float (&v)[8], const ActSmem& act, int t, int b, int lane) {
    uint32_t w0, w1, bw;
    float d;
    q8k_block_core(v, lane, w0, w1, bw, d);
    const uint32_t qa = act.qblk(t, b) + 8 * lane;
    asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(qa), "r"(w0), "r"(w1));
    if ((lane & 3) == 0) asm volatile("st.shared.u32 [%0], %1;" ::"r"(act.bsptr(t, b) + (lane >> 2) * 4), "r"(bw));
    if (lane == 0) asm volatile("st.shared.f32 [%0], %1;" ::"r"(act.dptr(t, b)), "f"(d));
}

// ---------------------------------------------------------------- row dots
// One lane works on one whole super-block (Q4_K) or one half of one (Q6_K), so a row of K values takes
// G lanes and a warp runs 32 / G rows side by side: the reductions, the block-order float chain and the
// loop overhead are paid once per pass of 32 / G rows.  (The earlier form, one 64-value chunk per lane
// and one row per warp pass, took 418 warp instructions per Q4_K row of 2048 and 700 per Q6_K row,
// measured, against a budget of about 200 at the HBM roofline.)
__host__ __device__ inline int pow2_at_least(int n) {
    int g = 1;
    while (g < n) g <<= 1;
    return g;
}
// Lanes that cooperate on one row.
__host__ __device__ inline int lanes_per_row(int type, int K) {
    const int g = pow2_at_least(K / DC_QK_K) * (type == DC_TYPE_Q6_K ? 2 : 1);
    return g > 32 ? 32 : g;
}
// Four unsigned bytes of a times four signed bytes of b, added to c.
__device__ __forceinline__ int dp4a_u8s8(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// Two int16 of a times bytes (0,1) / (2,3) of b, added to c.
__device__ __forceinline__ int dp2a_lo(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp2a.lo.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp2a_hi(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp2a.hi.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Optional capture of the exact per-block integer sums a row dot forms (parity checks):
// I[(t * N + row) * nb + b], M likewise (Q4_K only).  Null in production launches.
struct BlockSumDump {
    int32_t* I;
    int32_t* M;
    int N;   // rows of the whole matrix (stride of a token)
};

// Q4_K super-block at shared address blk (16-byte aligned) against block b of NT token rows: the exact
// integers I = sum_s scale_s * (q . y)_s and M = sum_g bsums_g * min_(g/2)
// (core/src/kernels/hwy/hwy_moe_quant.cc:202-246); low nibbles of 32 bytes are sub-block 2c, high
// nibbles sub-block 2c+1 (:202-211); scales and mins from the 12 packed bytes as :90-101.
template <int NT>
__device__ __forceinline__ void q4k_block_ints(uint32_t blk, const ActSmem& act, int b, int nt, const int (&tok)[NT],
                                               int (&I)[NT], int (&M)[NT], float& d, float& dmin) {
    const uint32_t dd = lds32(blk);
    d = fp16_bits_to_float((uint16_t)(dd & 0xFFFF));
    dmin = fp16_bits_to_float((uint16_t)(dd >> 16));
    const uint32_t u0 = lds32(blk + 4), u1 = lds32(blk + 8), u2 = lds32(blk + 12);
    const uint32_t sc_a = u0 & 0x3f3f3f3fu, sc_b = (u2 & 0x0f0f0f0fu) | (((u0 >> 6) & 0x03030303u) << 4);
    const uint32_t mn_a = u1 & 0x3f3f3f3fu, mn_b = ((u2 >> 4) & 0x0f0f0f0fu) | (((u1 >> 6) & 0x03030303u) << 4);
#pragma unroll
    for (int s = 0; s < NT; ++s) I[s] = 0;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint4 w0 = lds128(blk + 16 + 32 * c), w1 = lds128(blk + 32 + 32 * c);
        const uint32_t scw = c < 2 ? sc_a : sc_b;
        const int sc_lo = (int)((scw >> (16 * (c & 1))) & 0xFFu), sc_hi = (int)((scw >> (16 * (c & 1) + 8)) & 0xFFu);
#pragma unroll
        for (int s = 0; s < NT; ++s) {
            if (s < nt) {
                const uint32_t yq = act.qblk(tok[s], b) + 64 * c;
                const uint4 y0 = lds128(yq), y1 = lds128(yq + 16), y2 = lds128(yq + 32), y3 = lds128(yq + 48);
                int lo = 0, hi16 = 0;
                lo = __dp4a((int)(w0.x & 0x0F0F0F0Fu), (int)y0.x, lo);
                lo = __dp4a((int)(w0.y & 0x0F0F0F0Fu), (int)y0.y, lo);
                lo = __dp4a((int)(w0.z & 0x0F0F0F0Fu), (int)y0.z, lo);
                lo = __dp4a((int)(w0.w & 0x0F0F0F0Fu), (int)y0.w, lo);
                lo = __dp4a((int)(w1.x & 0x0F0F0F0Fu), (int)y1.x, lo);
                lo = __dp4a((int)(w1.y & 0x0F0F0F0Fu), (int)y1.y, lo);
                lo = __dp4a((int)(w1.z & 0x0F0F0F0Fu), (int)y1.z, lo);
                lo = __dp4a((int)(w1.w & 0x0F0F0F0Fu), (int)y1.w, lo);
                // high nibbles stay in place (bytes 16*q, taken as unsigned): their dot is 16 times the wanted
                // one, exactly, so one shift at the end replaces a shift per word
                hi16 = dp4a_u8s8(w0.x & 0xF0F0F0F0u, y2.x, hi16);
                hi16 = dp4a_u8s8(w0.y & 0xF0F0F0F0u, y2.y, hi16);
                hi16 = dp4a_u8s8(w0.z & 0xF0F0F0F0u, y2.z, hi16);
                hi16 = dp4a_u8s8(w0.w & 0xF0F0F0F0u, y2.w, hi16);
                hi16 = dp4a_u8s8(w1.x & 0xF0F0F0F0u, y3.x, hi16);
                hi16 = dp4a_u8s8(w1.y & 0xF0F0F0F0u, y3.y, hi16);
                hi16 = dp4a_u8s8(w1.z & 0xF0F0F0F0u, y3.z, hi16);
                hi16 = dp4a_u8s8(w1.w & 0xF0F0F0F0u, y3.w, hi16);
                I[s] += sc_lo * lo + sc_hi * (hi16 >> 4);
            }
        }
    }
    // mins: word k of the sums holds groups 2k and 2k+1, both of sub-block k
    const uint32_t m01 = __byte_perm(mn_a, 0, 0x1100), m23 = __byte_perm(mn_a, 0, 0x3322);
    const uint32_t m45 = __byte_perm(mn_b, 0, 0x1100), m67 = __byte_perm(mn_b, 0, 0x3322);
#pragma unroll
    for (int s = 0; s < NT; ++s) {
        M[s] = 0;
        if (s < nt) {
            const uint32_t bp = act.bsptr(tok[s], b);
            const uint4 b0 = lds128(bp), b1 = lds128(bp + 16);
            int m = dp2a_lo(b0.x, m01, 0);
            m = dp2a_hi(b0.y, m01, m);
            m = dp2a_lo(b0.z, m23, m);
            m = dp2a_hi(b0.w, m23, m);
            m = dp2a_lo(b1.x, m45, m);
            m = dp2a_hi(b1.y, m45, m);
            m = dp2a_lo(b1.z, m67, m);
            m = dp2a_hi(b1.w, m67, m);
            M[s] = m;
        }
    }
}

// per byte: q in 0..63 -> q - 32 as a signed byte.  With bit 7 set no byte borrows from its
// neighbour, so one 32-bit subtraction does all four: ((q | 0x80) - 0x20) ^ 0x80.
__device__ __forceinline__ uint32_t q6_signed(uint32_t q) { return ((q | 0x80808080u) - 0x20202020u) ^ 0x80808080u; }

// NW consecutive 32-bit words starting at a 2-byte aligned shared address: NW + 1 aligned loads and a
// funnel shift each (the shift is 0 or 16 bits, the same for the whole block).
template <int NW>
__device__ __forceinline__ void lds_words_a2(uint32_t a, uint32_t (&out)[NW]) {
    const uint32_t base = a & ~3u, sh = (a & 2u) * 8u;
    uint32_t prev = lds32(base);
#pragma unroll
    for (int i = 0; i < NW; ++i) {
        const uint32_t next = lds32(base + 4 * (i + 1));
        out[i] = __funnelshift_r(prev, next, sh);
        prev = next;
    }
}

// Half j (128 values) of the Q6_K super-block at shared address blk (2-byte aligned) against block b of
// TT token rows: P[s][L], the exact int32 partial that collects bytes 4L..4L+3 of each of the half's four
// 32-value quadrants times the group scales (core/src/llm/matmul/q6_small_batch.h:52-83; element order
// :52-74).  The block's partials are the sums of the two halves'.
template <int TT>
__device__ __forceinline__ void q6k_half_ints(uint32_t blk, int j, const ActSmem& act, int b, int nt, const int* tok,
                                              int (&P)[TT][8], float& d) {
    uint32_t ql[16], qh[8], scw[2];
    lds_words_a2<16>(blk + 64 * j, ql);
    lds_words_a2<8>(blk + 128 + 32 * j, qh);
    lds_words_a2<2>(blk + 192 + 8 * j, scw);
    d = fp16_bits_to_float((uint16_t)lds16(blk + 208));
    int sc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) sc[i] = (int)(int8_t)((scw[i >> 2] >> (8 * (i & 3))) & 0xFFu);
#pragma unroll
    for (int s = 0; s < TT; ++s)
#pragma unroll
        for (int L = 0; L < 8; ++L) P[s][L] = 0;
#pragma unroll
    for (int wq = 0; wq < 2; ++wq) {
        uint32_t q[4][4];   // [quadrant][word]: signed bytes q - 32
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t a = ql[4 * wq + k], c = ql[8 + 4 * wq + k], h = qh[4 * wq + k];
            q[0][k] = q6_signed((a & 0x0F0F0F0Fu) | ((h << 4) & 0x30303030u));
            q[1][k] = q6_signed((c & 0x0F0F0F0Fu) | ((h << 2) & 0x30303030u));
            q[2][k] = q6_signed(((a >> 4) & 0x0F0F0F0Fu) | (h & 0x30303030u));
            q[3][k] = q6_signed(((c >> 4) & 0x0F0F0F0Fu) | ((h >> 2) & 0x30303030u));
        }
#pragma unroll
        for (int s = 0; s < TT; ++s) {
            if (s < nt) {
                const uint32_t yh = act.qblk(tok[s], b) + 128 * j + 16 * wq;
#pragma unroll
                for (int qd = 0; qd < 4; ++qd) {
                    const uint4 y = lds128(yh + 32 * qd);
                    const int scale = sc[2 * qd + wq];
                    P[s][4 * wq + 0] += scale * __dp4a((int)q[qd][0], (int)y.x, 0);
                    P[s][4 * wq + 1] += scale * __dp4a((int)q[qd][1], (int)y.y, 0);
                    P[s][4 * wq + 2] += scale * __dp4a((int)q[qd][2], (int)y.z, 0);
                    P[s][4 * wq + 3] += scale * __dp4a((int)q[qd][3], (int)y.w, 0);
                }
            }
        }
    }
}

// Row dots for up to NT tokens in the float order of the CPU kernels they stand in for, so that the result
// is bit-identical to them:
//   Q4_K (core/src/kernels/hwy/hwy_moe_quant.cc:218-253): per super-block the exact int32 sums I and M,
//     then in block order  sumf += (d * yd) * float(I);  sumf -= (dmin * yd) * float(M).
//   Q6_K (core/src/llm/matmul/q6_small_batch.h:62-103): per super-block eight int32 partials, then per
//     partial acc[L] = fma(yd * d, float(partial L), acc[L]) in block order, and at the end
//     ((a0 + a4) + (a2 + a6)) + ((a1 + a5) + (a3 + a7)).
// `row` is the shared address of THIS lane's row (the groups of a warp run different rows), G =
// lanes_per_row; all 32 lanes of the warp must call (the exchanges are full-warp shuffles that stay inside a
// group); `active` = this lane's row exists.  On return every lane of a group holds its row's results.
// tok[s] = activation row of token slot s (slots >= nt are skipped).
template <int NT, int TYPE>
__device__ DC_HOT void rows_dot(uint32_t row, bool active, int lane, int G, const ActSmem& act, int nt,
                                const int (&tok)[NT], float (&out)[NT], const BlockSumDump* dump = nullptr,
                                int dump_row = 0) {
    const int nb = act.nb;
    const int lig = lane & (G - 1), gbase = lane & ~(G - 1);
    if (TYPE == DC_TYPE_Q4_K) {
        float acc[NT];
#pragma unroll
        for (int s = 0; s < NT; ++s) acc[s] = 0.0f;
#pragma unroll 1
        for (int b0 = 0; b0 < nb; b0 += G) {
            const int b = b0 + lig;
            const bool on = active && b < nb;
            float tI[NT], tM[NT];
#pragma unroll
            for (int s = 0; s < NT; ++s) tI[s] = tM[s] = 0.0f;
            if (on) {
                int I[NT], M[NT];
                float d, dmin;
                q4k_block_ints<NT>(row + b * DC_Q4K_BYTES, act, b, nt, tok, I, M, d, dmin);
#pragma unroll
                for (int s = 0; s < NT; ++s) {
                    if (s < nt) {
                        const float yd = __int_as_float(lds32(act.dptr(tok[s], b)));
                        tI[s] = __fmul_rn(__fmul_rn(d, yd), (float)I[s]);
                        tM[s] = __fmul_rn(__fmul_rn(dmin, yd), (float)M[s]);
                        if (dump) {
                            const size_t di = ((size_t)tok[s] * dump->N + dump_row) * nb + b;
                            dump->I[di] = I[s];
                            if (dump->M) dump->M[di] = M[s];
                        }
                    }
                }
            }
            // block order: every lane of the group adds the pass's blocks one by one
            const int nbb = min(G, nb - b0);
#pragma unroll 1
            for (int bb = 0; bb < nbb; ++bb) {
#pragma unroll
                for (int s = 0; s < NT; ++s) {
                    if (s < nt) {
                        const float a = __shfl_sync(0xffffffffu, tI[s], gbase + bb);
                        const float m = __shfl_sync(0xffffffffu, tM[s], gbase + bb);
                        acc[s] = __fsub_rn(__fadd_rn(acc[s], a), m);
                    }
                }
            }
        }
#pragma unroll
        for (int s = 0; s < NT; ++s) out[s] = acc[s];
    } else {
        // lane -> (block lig / 2, half lig % 2).  After the integer exchange both lanes of a block hold its
        // eight partials; the lane of half j then carries the block-order chains of partials 4j .. 4j+3.
        constexpr int TT = NT < 4 ? NT : 4;   // tokens per decode of the weights (registers)
        const int j = lig & 1, bpp = G >> 1;
#pragma unroll 1
        for (int s0 = 0; s0 < NT; s0 += TT) {
            if (s0 >= nt) break;
            float ac[TT][4];
#pragma unroll
            for (int s = 0; s < TT; ++s)
#pragma unroll
                for (int k = 0; k < 4; ++k) ac[s][k] = 0.0f;
#pragma unroll 1
            for (int b0 = 0; b0 < nb; b0 += bpp) {
                const int b = b0 + (lig >> 1);
                const bool on = active && b < nb;
                int P[TT][8];
                float sf[TT];
#pragma unroll
                for (int s = 0; s < TT; ++s) {
                    sf[s] = 0.0f;
#pragma unroll
                    for (int L = 0; L < 8; ++L) P[s][L] = 0;
                }
                if (on) {
                    float d;
                    q6k_half_ints<TT>(row + b * DC_Q6K_BYTES, j, act, b, nt - s0, &tok[s0], P, d);
#pragma unroll
                    for (int s = 0; s < TT; ++s)
                        if (s0 + s < nt) sf[s] = __fmul_rn(__int_as_float(lds32(act.dptr(tok[s0 + s], b))), d);
                }
                int x[TT][4];
#pragma unroll
                for (int s = 0; s < TT; ++s) {
                    if (s0 + s < nt) {
#pragma unroll
                        for (int L = 0; L < 8; ++L) P[s][L] += __shfl_xor_sync(0xffffffffu, P[s][L], 1);
                        if (dump && on && j == 0) {
                            int tot = 0;
#pragma unroll
                            for (int L = 0; L < 8; ++L) tot += P[s][L];
                            dump->I[((size_t)tok[s0 + s] * dump->N + dump_row) * nb + b] = tot;
                        }
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) x[s][k] = j ? P[s][4 + k] : P[s][k];
                }
                const int nbb = min(bpp, nb - b0);
#pragma unroll 1
                for (int bb = 0; bb < nbb; ++bb) {
                    const int src = gbase + 2 * bb + j;
#pragma unroll
                    for (int s = 0; s < TT; ++s) {
                        if (s0 + s < nt) {
                            const float f = __shfl_sync(0xffffffffu, sf[s], src);
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                const int v = __shfl_sync(0xffffffffu, x[s][k], src);
                                ac[s][k] = __fmaf_rn(f, (float)v, ac[s][k]);
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int s = 0; s < TT; ++s) {
                if (s0 + s < nt) {
                    // the lane of half 0 holds a0..a3, its neighbour a4..a7
                    float r[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) r[k] = __fadd_rn(ac[s][k], __shfl_xor_sync(0xffffffffu, ac[s][k], 1));
                    const float res = __fadd_rn(__fadd_rn(r[0], r[2]), __fadd_rn(r[1], r[3]));
#pragma unroll
                    for (int q = 0; q < NT; ++q)
                        if (q == s0 + s) out[q] = res;
                }
            }
        }
    }
}

// The single-token form as an out-of-line leaf with scalar arguments (everything travels in registers):
// (qs_t, d_t, bs_t) are the shared-memory addresses of the token's codes, block scales and block sums.
// Inside the persistent kernel the inlined form costs the surrounding phases their registers (the kernel and
// its out-of-line phase functions share one register file along each call chain, and spill what does not
// fit: measured 24 % of the step time); one call serves all the rows of a warp pass.
template <int TYPE>
__device__ __noinline__ float rows_dot1(uint32_t row, int active, int lane, int G, uint32_t qs_t, uint32_t d_t,
                                        uint32_t bs_t, int nb) {
    ActSmem a;
    a.qs = qs_t;
    a.d = d_t;
    a.bs = bs_t;
    a.nb = nb;
    a.K = nb * DC_QK_K;
    const int tok[1] = {0};
    float out[1];
    rows_dot<1, TYPE>(row, active != 0, lane, G, a, 1, tok, out);
    return out[0];
}
// Token row t of an activation layout, by either decoder.
__device__ __forceinline__ float rows_dot1_typed(int type, uint32_t row, bool active, int lane, int G, const ActSmem& act,
                                                 int t) {
    const uint32_t qs_t = act.qblk(t, 0), d_t = act.dptr(t, 0), bs_t = act.bsptr(t, 0);
    return type == DC_TYPE_Q4_K ? rows_dot1<DC_TYPE_Q4_K>(row, active, lane, G, qs_t, d_t, bs_t, act.nb)
                                : rows_dot1<DC_TYPE_Q6_K>(row, active, lane, G, qs_t, d_t, bs_t, act.nb);
}
// Any token count, type decided at run time.
template <int NT>
__device__ __forceinline__ void rows_dot_typed(int type, uint32_t row, bool active, int lane, int G, const ActSmem& act,
                                               int nt, const int (&tok)[NT], float (&out)[NT],
                                               const BlockSumDump* dump = nullptr, int dump_row = 0) {
    if (type == DC_TYPE_Q4_K) rows_dot<NT, DC_TYPE_Q4_K>(row, active, lane, G, act, nt, tok, out, dump, dump_row);
    else rows_dot<NT, DC_TYPE_Q6_K>(row, active, lane, G, act, nt, tok, out, dump, dump_row);
}

// Generic-width lane-group sum (G a power of two <= 32, runtime value).
__device__ __forceinline__ float group_sum_rt(float v, int G) {
    for (int o = G >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

}  // namespace dc
