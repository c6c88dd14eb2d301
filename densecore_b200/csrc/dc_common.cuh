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
// Q8_K activations of the step's tokens, laid out in shared memory for the
// dot kernels: qs[T][K] int8 (16-byte aligned rows), d[T][nb] f32,
// bs[T][nb][16] int16.  Filled from the native 292-byte blocks in global memory.
struct ActSmem {
    uint32_t qs, d, bs;  // shared addresses
    int K, nb;
    uint32_t rs;         // bytes between the int8 rows of two tokens
    // The int8 codes are stored in 64-byte chunks 80 bytes apart: the lanes of a warp read
    // chunks that are multiples of 64 values apart, and a stride of 80 bytes (20 banks) spreads
    // those reads over all 32 banks instead of piling them onto two.
    __host__ __device__ __forceinline__ static size_t row_stride(int K) { return (size_t)(K / 64) * 80; }
    __host__ __device__ __forceinline__ static size_t bytes(int T, int K) {
        const int nb = K / DC_QK_K;
        return (size_t)T * row_stride(K) + (size_t)T * nb * 4 + (size_t)T * nb * 32;
    }
    __device__ __forceinline__ void bind(uint8_t* base, int T, int K_) {
        K = K_;
        nb = K_ / DC_QK_K;
        rs = (uint32_t)row_stride(K_);
        qs = smem_u32(base);
        d = qs + T * rs;
        bs = d + T * nb * 4;
    }
    // shared address of code e (0 <= e < K) of token row t
    __device__ __forceinline__ uint32_t q(int t, int e) const { return qs + t * rs + (e >> 6) * 80 + (e & 63); }
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
            if (o == 0) dst = d + (t * nb + b) * 4;
            else if (o <= 64) dst = q(t, b * 256 + (o - 1) * 4);
            else dst = bs + (t * nb + b) * 32 + (o - 65) * 4;
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
    const uint32_t qa = act.q(t, b * 256 + 8 * lane);
    asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(qa), "r"(w0), "r"(w1));
    if ((lane & 3) == 0) asm volatile("st.shared.u32 [%0], %1;" ::"r"(act.bs + (t * act.nb + b) * 32 + (lane >> 2) * 4), "r"(bw));
    if (lane == 0) asm volatile("st.shared.f32 [%0], %1;" ::"r"(act.d + (t * act.nb + b) * 4), "f"(d));
}

// ------------------------------------------------------- Q4_K row dot
// One "item" = (super-block b, chunk c): 32 bytes of qs = sub-blocks 2c (low
// nibbles) and 2c+1 (high nibbles) (core/src/kernels/hwy/hwy_moe_quant.cc:202-211).
// Returns the lane's exact integer partials: I = sc_lo*dot_lo + sc_hi*dot_hi,
// M = m_lo*(bsums[4c]+bsums[4c+1]) + m_hi*(bsums[4c+2]+bsums[4c+3]).
// Four unsigned bytes of a times four signed bytes of b, added to c.
__device__ __forceinline__ int dp4a_u8s8(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
struct Q4Item {
    uint32_t q[8];
    int sc_lo, sc_hi, m_lo, m_hi;
    float d, dmin;
};
__device__ __forceinline__ void q4k_load_item(uint32_t row, int b, int c, Q4Item& it) {
    const uint32_t blk = row + b * DC_Q4K_BYTES;
    const uint4 a = lds128(blk + 16 + 32 * c), e = lds128(blk + 32 + 32 * c);
    it.q[0] = a.x; it.q[1] = a.y; it.q[2] = a.z; it.q[3] = a.w;
    it.q[4] = e.x; it.q[5] = e.y; it.q[6] = e.z; it.q[7] = e.w;
    const uint32_t dd = lds32(blk);
    it.d = fp16_bits_to_float((uint16_t)(dd & 0xFFFF));
    it.dmin = fp16_bits_to_float((uint16_t)(dd >> 16));
    // 6-bit scale/min unpack, scalar form of hwy_moe_quant.cc:90-101
    // (per sub-block j: j<4: sc=s[j]&63, m=s[j+4]&63; else sc=(s[j+4]&15)|((s[j-4]>>6)<<4),
    //  m=(s[j+4]>>4)|((s[j]>>6)<<4)), for j = 2c and 2c+1.
    const uint32_t s = blk + 4;
    const int j = 2 * c;
    if (c < 2) {
        const uint32_t p = lds16(s + j), m = lds16(s + j + 4);
        it.sc_lo = p & 63; it.sc_hi = (p >> 8) & 63;
        it.m_lo = m & 63; it.m_hi = (m >> 8) & 63;
    } else {
        const uint32_t hi = lds16(s + j + 4), lo = lds16(s + j - 4), mid = lds16(s + j);
        it.sc_lo = (hi & 15) | (((lo >> 6) & 3) << 4);
        it.sc_hi = ((hi >> 8) & 15) | (((lo >> 14) & 3) << 4);
        it.m_lo = ((hi >> 4) & 15) | (((mid >> 6) & 3) << 4);
        it.m_hi = ((hi >> 12) & 15) | (((mid >> 14) & 3) << 4);
    }
}
__device__ __forceinline__ void q4k_item_ints(const Q4Item& it, uint32_t yq /*shared addr of 64 int8*/,
                                              uint32_t ybs /*shared addr of 4 int16*/, int& I, int& M) {
    // high nibbles stay in place (bytes 16*q, taken as unsigned): their dot is 16 times the wanted one,
    // exactly, so one shift at the end replaces a shift per word
    int lo = 0, hi16 = 0;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint4 y0 = lds128(yq + 16 * h), y1 = lds128(yq + 32 + 16 * h);
        const uint32_t* w = &it.q[4 * h];
        lo = __dp4a((int)(w[0] & 0x0F0F0F0F), (int)y0.x, lo);
        lo = __dp4a((int)(w[1] & 0x0F0F0F0F), (int)y0.y, lo);
        lo = __dp4a((int)(w[2] & 0x0F0F0F0F), (int)y0.z, lo);
        lo = __dp4a((int)(w[3] & 0x0F0F0F0F), (int)y0.w, lo);
        hi16 = dp4a_u8s8(w[0] & 0xF0F0F0F0u, y1.x, hi16);
        hi16 = dp4a_u8s8(w[1] & 0xF0F0F0F0u, y1.y, hi16);
        hi16 = dp4a_u8s8(w[2] & 0xF0F0F0F0u, y1.z, hi16);
        hi16 = dp4a_u8s8(w[3] & 0xF0F0F0F0u, y1.w, hi16);
    }
    const int hi = hi16 >> 4;
    const uint32_t b01 = lds32(ybs), b23 = lds32(ybs + 4);
    const int s_lo = (int)(short)(b01 & 0xFFFF) + (int)(short)(b01 >> 16);
    const int s_hi = (int)(short)(b23 & 0xFFFF) + (int)(short)(b23 >> 16);
    I = it.sc_lo * lo + it.sc_hi * hi;
    M = it.m_lo * s_lo + it.m_hi * s_hi;
}

// ------------------------------------------------------- Q6_K row dot
// One "item" = (super-block b, half j, eighth t): 8 bytes of ql at 64j+8t, 8 at
// 64j+32+8t, 8 of qh at 32j+8t -> 4 quadrants x 8 elements
// (core/src/llm/matmul/q6_small_batch.h:52-74).  Block bytes are only 2-byte
// aligned in shared memory.
__device__ __forceinline__ uint32_t q6_signed(uint32_t q) { return ((q | 0x80808080u) - 0x20202020u) ^ 0x80808080u; }
struct Q6Item {
    uint32_t q[8];  // signed bytes (q-32), quadrant-major: q[2*quad + w]
    int sc[4];
    float d;
};
// Eight consecutive bytes from a 2-byte aligned shared address as two 32-bit words: two aligned
// 64-bit loads and funnel shifts (instead of four 16-bit loads).  Reads up to a + 15.
__device__ __forceinline__ uint2 lds64_a2(uint32_t a) {
    const uint32_t a0 = a & ~7u, o = a & 7u;   // o in {0, 2, 4, 6}
    const uint2 lo = lds64(a0), hi = lds64(a0 + 8);
    const uint32_t sh = (o & 3u) * 8u;         // 0 or 16 bits
    const bool up = o >= 4u;
    const uint32_t w0 = up ? lo.y : lo.x, w1 = up ? hi.x : lo.y, w2 = up ? hi.y : hi.x;
    return make_uint2(__funnelshift_r(w0, w1, sh), __funnelshift_r(w1, w2, sh));
}
__device__ __forceinline__ void q6k_load_item(uint32_t row, int b, int j, int t, Q6Item& it) {
    const uint32_t blk = row + b * DC_Q6K_BYTES;
    const uint32_t ql0 = blk + 64 * j + 8 * t, ql1 = ql0 + 32, qh = blk + 128 + 32 * j + 8 * t;
    // every range read below ends at most 15 bytes after its start, inside the 210-byte block
    const uint2 A = lds64_a2(ql0), C = lds64_a2(ql1), H = lds64_a2(qh);
#pragma unroll
    for (int w = 0; w < 2; ++w) {
        const uint32_t a = w ? A.y : A.x, c = w ? C.y : C.x, h = w ? H.y : H.x;
        // per byte: q in 0..63 -> q - 32 as a signed byte.  With bit 7 set no byte borrows from its
        // neighbour, so one 32-bit subtraction does all four: ((q | 0x80) - 0x20) ^ 0x80.
        it.q[0 + w] = q6_signed((a & 0x0F0F0F0F) | ((h << 4) & 0x30303030));
        it.q[2 + w] = q6_signed((c & 0x0F0F0F0F) | ((h << 2) & 0x30303030));
        it.q[4 + w] = q6_signed(((a >> 4) & 0x0F0F0F0F) | (h & 0x30303030));
        it.q[6 + w] = q6_signed(((c >> 4) & 0x0F0F0F0F) | ((h >> 2) & 0x30303030));
    }
    const uint32_t s = blk + 192 + 8 * j + (t >> 1);
#pragma unroll
    for (int qd = 0; qd < 4; ++qd) it.sc[qd] = lds_s8(s + 2 * qd);
    it.d = fp16_bits_to_float((uint16_t)lds16(blk + 208));
}
// yq: shared address of the activation code at element 256b + 128j + 8t.  Quadrant qd
// is 32*qd elements further on: same 64-value chunk for odd qd, next chunk (80 bytes on) for qd >= 2.
// I0 takes bytes 8t..8t+3 of every quadrant, I1 bytes 8t+4..8t+7: they belong to the partials 2t and
// 2t+1 of core/src/llm/matmul/q6_small_batch.h:62-83.
__device__ __forceinline__ void q6k_item_ints(const Q6Item& it, uint32_t yq, int& I0, int& I1) {
    I0 = I1 = 0;
#pragma unroll
    for (int qd = 0; qd < 4; ++qd) {
        const uint32_t a = yq + (qd >> 1) * 80 + (qd & 1) * 32;
        const uint2 y = lds64(a);
        I0 += it.sc[qd] * __dp4a((int)it.q[2 * qd], (int)y.x, 0);
        I1 += it.sc[qd] * __dp4a((int)it.q[2 * qd + 1], (int)y.y, 0);
    }
}

// Sum over the G lanes of a power-of-two lane group (all 32 lanes call it).
template <int G>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Optional capture of the exact per-block integer sums a row dot forms (parity checks):
// I[(t * N + row) * nb + b], M likewise (Q4_K only).  Null in production launches.
struct BlockSumDump {
    int32_t* I;
    int32_t* M;
    int N;   // rows of the whole matrix (stride of a token)
};

// Row dot for up to NT tokens, in the float order of the CPU kernels it stands in for, so that the
// result is bit-identical to them:
//   Q4_K (core/src/kernels/hwy/hwy_moe_quant.cc:218-253): per super-block the exact int32 sums
//     I = sum_s scale_s * dot_s and M = sum_g bsums_g * min_(g/2), then in block order
//     sumf += (d * yd) * float(I);  sumf -= (dmin * yd) * float(M).
//   Q6_K (core/src/llm/matmul/q6_small_batch.h:62-103): per super-block eight int32 partials (partial L
//     collects bytes 4L..4L+3 of every 32-value quadrant, times the group scales), then per partial
//     acc[L] = fma(yd * d, float(partial L), acc[L]) in block order, and at the end
//     ((a0 + a4) + (a2 + a6)) + ((a1 + a5) + (a3 + a7)).
// Weights are decoded once per item and reused for every token.  G lanes cooperate on one row and ALL 32
// lanes of the warp must call (the exchanges are full-warp shuffles); `active` = this lane's row exists.
// On return lane row_dot_owner(type, s) of the group (among others) holds the row's result for token slot s.
// tok[s] = row of the activation arrays in shared memory used by token slot s (slots >= nt are skipped).
// Lane of a row's group that ends up with token t's result (see row_dot_exact).
__device__ __forceinline__ int row_dot_owner(int type, int t) { return type == DC_TYPE_Q4_K ? (t & 3) : 4 * (t & 1); }

// v[base + sub] for a lane-dependent sub < N (0 beyond the array): register arrays cannot be indexed by a
// run-time value, so the pick is a chain of selects.
template <int N, int LEN, typename T>
__device__ __forceinline__ T pick_slot(const T (&v)[LEN], int base, int sub) {
    T r = base < LEN ? v[base < LEN ? base : 0] : T(0);
#pragma unroll
    for (int j = 1; j < N; ++j)
        if (base + j < LEN && sub == j) r = v[base + j < LEN ? base + j : 0];
    return r;
}

template <int NT>
__device__ DC_HOT void row_dot_exact(int type, uint32_t row, bool active, int lane, int G, const ActSmem& act, int nt,
                                     const int (&tok)[NT], float (&out)[NT], const BlockSumDump* dump = nullptr,
                                     int dump_row = 0) {
    const int nb = act.nb;
    const int lig = lane & (G - 1), gbase = lane & ~(G - 1);
    if (type == DC_TYPE_Q4_K) {
        // The four lanes of a block hold the same block sums after the integer exchange; lane `sub` of them
        // carries the block-order chain of the tokens sub, sub + 4, ...: one pair of shuffles per block then
        // serves four tokens.
        constexpr int NG = (NT + 3) / 4;
        const int sub = lig & 3;
        float acc[NG];
#pragma unroll
        for (int g = 0; g < NG; ++g) acc[g] = 0.0f;
        const int n_items = nb * 4, bpp = G >> 2;   // blocks per pass
        for (int i0 = 0; i0 < n_items; i0 += G) {
            const int i = i0 + lig, b = i >> 2, c = i & 3;
            const bool on = active && i < n_items;
            Q4Item it;
            if (on) q4k_load_item(row, b, c, it);
            float tI[NT], tM[NT];
#pragma unroll
            for (int s = 0; s < NT; ++s) {
                tI[s] = tM[s] = 0.0f;
                if (s < nt) {
                    const int t = tok[s];
                    int I = 0, M = 0;
                    float yd = 0.0f;
                    if (on) {
                        q4k_item_ints(it, act.q(t, b * 256 + 64 * c), act.bs + (t * nb + b) * 32 + 8 * c, I, M);
                        yd = __int_as_float(lds32(act.d + (t * nb + b) * 4));
                    }
                    // the block's four chunks sit in four neighbouring lanes
                    I += __shfl_xor_sync(0xffffffffu, I, 1);
                    M += __shfl_xor_sync(0xffffffffu, M, 1);
                    I += __shfl_xor_sync(0xffffffffu, I, 2);
                    M += __shfl_xor_sync(0xffffffffu, M, 2);
                    if (on) {
                        tI[s] = __fmul_rn(__fmul_rn(it.d, yd), (float)I);
                        tM[s] = __fmul_rn(__fmul_rn(it.dmin, yd), (float)M);
                        if (dump && c == 0) {
                            const size_t di = ((size_t)t * dump->N + dump_row) * nb + b;
                            dump->I[di] = I;
                            if (dump->M) dump->M[di] = M;
                        }
                    }
                }
            }
            float xi[NG], xm[NG];
#pragma unroll
            for (int g = 0; g < NG; ++g) {
                xi[g] = pick_slot<4>(tI, 4 * g, sub);
                xm[g] = pick_slot<4>(tM, 4 * g, sub);
            }
            // block order: the terms of the pass's blocks are fetched side by side, then added one by one
#pragma unroll 1
            for (int bb = 0; bb < bpp; ++bb) {
                if ((i0 >> 2) + bb >= nb) break;
                const int src = gbase + 4 * bb + sub;
#pragma unroll
                for (int g = 0; g < NG; ++g) {
                    const float a = __shfl_sync(0xffffffffu, xi[g], src);
                    const float m = __shfl_sync(0xffffffffu, xm[g], src);
                    acc[g] = __fsub_rn(__fadd_rn(acc[g], a), m);
                }
            }
        }
#pragma unroll
        for (int s = 0; s < NT; ++s) out[s] = acc[s >> 2];   // valid on the lanes with sub == s % 4
    } else {
        // lane -> (block, half j, eighth tq).  After the integer exchange both halves hold the block's partials
        // 2tq and 2tq+1; half j then carries the chains of the tokens j, j + 2, ...
        constexpr int NG = (NT + 1) / 2;
        const int jj = (lig >> 2) & 1;
        float a0[NG], a1[NG];
#pragma unroll
        for (int g = 0; g < NG; ++g) a0[g] = a1[g] = 0.0f;
        const int n_items = nb * 8, bpp = G >> 3;
        for (int i0 = 0; i0 < n_items; i0 += G) {
            const int i = i0 + lig, b = i >> 3, j = (i >> 2) & 1, tq = i & 3;
            const bool on = active && i < n_items;
            Q6Item it;
            if (on) q6k_load_item(row, b, j, tq, it);
            int I0[NT], I1[NT];
            float sc[NT];
#pragma unroll
            for (int s = 0; s < NT; ++s) {
                I0[s] = I1[s] = 0;
                sc[s] = 0.0f;
                if (s < nt) {
                    const int t = tok[s];
                    if (on) {
                        q6k_item_ints(it, act.q(t, b * 256 + 128 * j + 8 * tq), I0[s], I1[s]);
                        sc[s] = __fmul_rn(__int_as_float(lds32(act.d + (t * nb + b) * 4)), it.d);
                    }
                    // the two halves of a block are four lanes apart
                    I0[s] += __shfl_xor_sync(0xffffffffu, I0[s], 4);
                    I1[s] += __shfl_xor_sync(0xffffffffu, I1[s], 4);
                    if (dump) {
                        int tot = I0[s] + I1[s];
                        tot += __shfl_xor_sync(0xffffffffu, tot, 1);
                        tot += __shfl_xor_sync(0xffffffffu, tot, 2);
                        if (on && j == 0 && tq == 0) dump->I[((size_t)t * dump->N + dump_row) * nb + b] = tot;
                    }
                }
            }
            float xf[NG];
            int x0[NG], x1[NG];
#pragma unroll
            for (int g = 0; g < NG; ++g) {
                xf[g] = pick_slot<2>(sc, 2 * g, jj);
                x0[g] = pick_slot<2>(I0, 2 * g, jj);
                x1[g] = pick_slot<2>(I1, 2 * g, jj);
            }
#pragma unroll 1
            for (int bb = 0; bb < bpp; ++bb) {
                if ((i0 >> 3) + bb >= nb) break;
                const int src = gbase + 8 * bb + (lig & 7);
#pragma unroll
                for (int g = 0; g < NG; ++g) {
                    const float f = __shfl_sync(0xffffffffu, xf[g], src);
                    const int v0 = __shfl_sync(0xffffffffu, x0[g], src);
                    const int v1 = __shfl_sync(0xffffffffu, x1[g], src);
                    a0[g] = __fmaf_rn(f, (float)v0, a0[g]);
                    a1[g] = __fmaf_rn(f, (float)v1, a1[g]);
                }
            }
        }
        float r[NG];
#pragma unroll
        for (int g = 0; g < NG; ++g) {
            // lanes tq = 0..3 (of one half) hold (a0,a1), (a2,a3), (a4,a5), (a6,a7) of their token
            const float x0s = __fadd_rn(a0[g], __shfl_xor_sync(0xffffffffu, a0[g], 2));   // a0+a4 | a2+a6
            const float x1s = __fadd_rn(a1[g], __shfl_xor_sync(0xffffffffu, a1[g], 2));   // a1+a5 | a3+a7
            const float y0 = __fadd_rn(x0s, __shfl_xor_sync(0xffffffffu, x0s, 1));        // (a0+a4)+(a2+a6)
            const float y1 = __fadd_rn(x1s, __shfl_xor_sync(0xffffffffu, x1s, 1));        // (a1+a5)+(a3+a7)
            r[g] = __fadd_rn(y0, y1);
        }
#pragma unroll
        for (int s = 0; s < NT; ++s) out[s] = r[s >> 1];   // valid on the lanes of half s % 2
    }
}
// The single-token row dot as an out-of-line leaf with scalar arguments (everything travels in registers):
// (qs_t, d_t, bs_t) are the shared-memory addresses of the token's codes, block scales and block sums.
// Inside the persistent kernel the inlined form costs the surrounding phases their registers (the kernel and
// its out-of-line phase functions share one register file along each call chain, and spill what does not
// fit: measured 24 % of the step time), and a call per row of the 32-register leaf costs 3 %.
template <int TYPE>
__device__ __noinline__ float row_dot_exact1(uint32_t row, int active, int lane, int G, uint32_t qs_t, uint32_t d_t,
                                             uint32_t bs_t, int nb) {
    ActSmem a;
    a.qs = qs_t;
    a.d = d_t;
    a.bs = bs_t;
    a.nb = nb;
    a.K = nb * DC_QK_K;
    a.rs = 0;
    const int tok[1] = {0};
    float out[1];
    row_dot_exact<1>(TYPE, row, active != 0, lane, G, a, 1, tok, out);
    return out[0];
}
// Token row t of an activation layout, by either decoder.
__device__ __forceinline__ float row_dot_exact1_typed(int type, uint32_t row, bool active, int lane, int G,
                                                      const ActSmem& act, int t) {
    const uint32_t qs_t = act.qs + t * act.rs, d_t = act.d + t * act.nb * 4, bs_t = act.bs + t * act.nb * 32;
    return type == DC_TYPE_Q4_K ? row_dot_exact1<DC_TYPE_Q4_K>(row, active, lane, G, qs_t, d_t, bs_t, act.nb)
                                : row_dot_exact1<DC_TYPE_Q6_K>(row, active, lane, G, qs_t, d_t, bs_t, act.nb);
}

// Generic-width lane-group sum (G a power of two <= 32, runtime value).
__device__ __forceinline__ float group_sum_rt(float v, int G) {
    for (int o = G >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Lanes that cooperate on one row for a given type and K: one item per lane where the row
// has that many items (measured: two items per lane and half-warp rows were ~30 % slower).
__host__ __device__ inline int lanes_per_row(int type, int K) {
    const int items = (K / DC_QK_K) * (type == DC_TYPE_Q4_K ? 4 : 8);
    int g = 4;
    while (g < items && g < 32) g <<= 1;
    return g;
}

}  // namespace dc
