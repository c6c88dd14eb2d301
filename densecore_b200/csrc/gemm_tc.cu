// Batched MUL_MAT for prompt chunks (M >= 32 token rows): K-quant weights x Q8_K activations on the
// 5th-generation tensor cores (tcgen05.mma kind::i8, accumulators in tensor memory), with the block sums
// kept as exact integers so that the float steps per 256-value block are the CPU kernels' own
// (core/src/llm/matmul/batched_exec.cpp:1040-1240 serves these shapes on the CPU; per block
// sumf += (d*yd)*float(I); sumf -= (dmin*yd)*float(M), core/src/kernels/hwy/hwy_moe_quant.cc:248-253).
//
// One CTA per SM owns 128 weight rows x two 64-token tiles over the whole reduction length; its warps split
// the three jobs of a 256-value block and overlap them (see k_gemm_tc below):
//   1. expanders turn the raw quants of the 128 rows into 8-bit operand planes in shared memory, K-major rows
//      of 128 bytes with the 128-byte swizzle the tensor core reads at full rate (a half block is exactly one
//      such row):
//        Q4_K: q4 * (sc >> 3), q4 * (sc & 7) and the sub-block minimum m broadcast (3 planes, unsigned),
//              so that I = 8 * acc0 + acc1 = sum sc_j * sum q4*q8 and M = acc2 = sum m_j * sum q8;
//        Q6_K: sign(sc) * digit_i(|sc|) * (q6 - 32) for the four base-4 digits of |sc| (4 planes, signed),
//              so that I = acc0 + 4 acc1 + 16 acc2 + 64 acc3;
//      every plane entry fits 8 bits and the 32-bit accumulators are exact;
//   2. one thread issues the UMMAs (128 rows x 128 tokens x 32 values each), two halves of 128 values per block;
//   3. read-out warps fetch the accumulators (tcgen05.ld) and add the block's float terms in block order.
// The token side is prepared once per activation matrix by k_quantize_q8k_tiled: the Q8_K codes of every
// (block, 64-token tile) stored as the B operand (two halves of 64 swizzled 128-byte rows), followed by the
// 64 block scales, so that a tile half is one contiguous bulk copy.  No multicast load anywhere.
//
// Q4_K results are bit-equal to the GEMV path and the CPU oracle.  Q6_K adds one float term per block
// instead of the CPU small-batch kernel's eight lane partials (q6_small_batch.h:62-103): equal integers,
// a different float order, relative difference ~1e-7.
#include <cstdio>
#include <cstdlib>

#include "dc_common.cuh"
#include "dc_gemm_tc.h"
#include "dc_internal.h"

#define DC_TRY(expr)                       \
    do {                                   \
        int st_ = (expr);                  \
        if (st_ != DC_B200_OK) return st_; \
    } while (0)

namespace dc {

constexpr int TC_ROWS = 128;
constexpr int TC_PLANE = TC_ROWS * 128;               // one operand plane of a half block: 128 rows of 128 bytes

struct GemmTcSeg {
    const uint8_t* w;      // rows of the matrix (expert 0)
    int N;                 // its rows
    int out_off;           // column offset of its outputs in a row of out
};

struct GemmTcParams {
    GemmTcSeg seg[3];      // matrices of one shape family (same K, row bytes, type) run in one launch: Q | K | V, gate | up
    int nseg;
    int row_bytes, K;
    const uint8_t* act;    // [K / 256][n_tt][TC_ACT_TILE]
    int n_tt;
    int n_slots;           // token slots that hold data (stores beyond are skipped)
    float* out;            // out[slot * ldo + row]
    int ldo;
    const int* tile_expert;   // optional [n_tt]: weights of tile t start at w + tile_expert[t] * estride; < 0: tile unused
    size_t estride;
    const int* slot_row;      // optional [n_tt * 64]: output row of every slot instead of the slot itself; < 0: none
    const int* pair_tile0;    // optional [grid.x]: first tile of the CTA's pair of neighbouring tiles (< 0: none) ...
    const int* pair_nset;     // ... and how many tiles of the pair exist (1 or 2); without it CTA i owns tiles 2i, 2i + 1
    int accumulate;           // out += result (one float add) instead of out = result
    int* err;
};

// ---- tcgen05 wrappers -------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[128 x N] (+)= A[128 x 32] * B[32 x N], 8-bit operands from shared memory, int32 accumulators in TMEM.
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Shared-memory operand descriptor, K-major rows of 128 bytes with the 128-byte swizzle (8-row groups of 1024
// bytes, 1024-byte aligned; chunk c of row r at chunk position c ^ (r % 8)).  saddr = the tile's base plus the
// K offset of the instruction in bytes (32 per K-step); sbo = byte distance between 8-row groups.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr, uint32_t sbo) {
    const uint32_t lo = ((saddr >> 4) & 0x3FFFu) | (1u << 16);                 // leading byte offset: unused with a swizzle
    const uint32_t hi = ((sbo >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);      // version 1 (sm_100), SWIZZLE_128B
    return ((uint64_t)hi << 32) | lo;
}
// Instruction descriptor: int32 accumulate, A unsigned or signed 8-bit, B signed 8-bit, both K-major.
__host__ __device__ constexpr uint32_t umma_idesc_i8(int a_signed, int M, int N) {
    return (2u << 4) | ((uint32_t)a_signed << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
// 16 consecutive 32-bit columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, int (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void sts128(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

// ---- activation side ---------------------------------------------------------------------------------
// One warp per (token slot, 256-value block): Q8_K codes (bit-equal to the row quantiser) into the tile
// layout of dc_gemm_tc.h, block scale into the tile's tail.  slot_token (optional) maps a slot to its source
// row, < 0 or beyond n_rows: the slot holds zeros.
__global__ void __launch_bounds__(256) k_quantize_q8k_tiled(const float* __restrict__ x, int ldx, int n_rows, int K,
                                                            uint8_t* __restrict__ act, int n_tt,
                                                            const int* __restrict__ slot_token) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = K / DC_QK_K;
    const long long total = (long long)n_tt * TC_NTOK * nb;
    for (long long item = (long long)blockIdx.x * 8 + warp; item < total; item += (long long)gridDim.x * 8) {
        const int b = (int)(item % nb);
        const int slot = (int)(item / nb);
        int row = slot_token ? slot_token[slot] : slot;
        if (row >= n_rows) row = -1;
        uint8_t* tile = act + ((size_t)b * n_tt + slot / TC_NTOK) * TC_ACT_TILE;
        uint32_t w0 = 0, w1 = 0, bw = 0;
        float d = 0.0f;
        if (row >= 0) {
            const float4* src = reinterpret_cast<const float4*>(x + (size_t)row * ldx + (size_t)b * DC_QK_K + 8 * lane);
            const float4 a = src[0], c = src[1];
            const float v[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
            q8k_block_core(v, lane, w0, w1, bw, d);
        }
        *reinterpret_cast<uint2*>(tile + tc_act_code_offset(slot % TC_NTOK, lane)) = make_uint2(w0, w1);
        if (lane == 0) reinterpret_cast<float*>(tile + TC_B_Q)[slot % TC_NTOK] = d;
    }
}

// ---- weight side ---------------------------------------------------------------------------------------
template <int TYPE>
struct TcTraits;
template <>
struct TcTraits<DC_TYPE_Q4_K> {
    static constexpr int NP = 3, BB = DC_Q4K_BYTES, A_SIGNED = 0;
};
template <>
struct TcTraits<DC_TYPE_Q6_K> {
    static constexpr int NP = 4, BB = DC_Q6K_BYTES, A_SIGNED = 1;
};

__device__ __forceinline__ void q4k_scale_min(uint32_t s0, uint32_t s1, uint32_t s2, int j, uint32_t& sc, uint32_t& m) {
    // 12 packed bytes -> the 6-bit scale and minimum of sub-block j (get_scale_min_k4 of ggml's K-quants)
    const uint64_t lo = ((uint64_t)s1 << 32) | s0;
    auto byte = [&](int i) -> uint32_t { return i < 8 ? (uint32_t)(lo >> (8 * i)) & 0xFFu : (s2 >> (8 * (i - 8))) & 0xFFu; };
    if (j < 4) {
        sc = byte(j) & 63u;
        m = byte(j + 4) & 63u;
    } else {
        sc = (byte(j + 4) & 0xFu) | ((byte(j - 4) >> 6) << 4);
        m = (byte(j + 4) >> 4) | ((byte(j) >> 6) << 4);
    }
}

// ---- the kernel: the three jobs of a block (expanding operand planes, issuing UMMAs, reading
// the accumulators out) run on different warps of one CTA per SM and overlap; a CTA owns 128 rows x two
// 64-token tiles, so that a block's planes are expanded once for 128 tokens and every UMMA is 128 tokens wide
// (the instruction takes about as long at N = 64 as at N = 128: measured 144 cycles each at N = 64).
//   warps 0-3   expanders: thread r turns its row's half block into the planes of stage h (two stages)
//   warp 4      one thread issues the UMMAs (stage h x 128 tokens -> accumulators in TMEM), commits
//               "stage free", "token codes free" and "accumulators full"
//   warp 5      one thread loads the token tiles (codes double-buffered, interleaved so that the two tiles
//               form one 128-row operand; block scales in a ring of four)
//   warps 6-13  read-out: warp w owns TMEM lane quarter w % 4 and tokens 64 ((w - 6) / 4) .. + 63: adds the
//               block's float terms for its row, then frees the accumulators
// The accumulators are single-buffered (3 or 4 planes x 128 columns of the 512): the UMMAs of the next block
// wait for the read-out, the expansion does not.  Every wait is bounded and watches a CTA-wide give-up flag.
constexpr int TC_THREADS = 448;
constexpr int TC_EXPAND = 128;
constexpr int TC_N = 128;                  // tokens per CTA

struct TcBars {       // shared addresses of the mbarriers
    uint32_t a_full[2], a_free[2], b_full[2], b_free[2], s_full[4], d_full[4], acc_full, acc_free;
};

__device__ __forceinline__ bool tc_wait_raw(uint32_t bar, uint32_t parity, volatile int* give_up, int* err) {
    for (uint32_t i = 0; i < DC_WAIT_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 63u && *give_up) return false;
    }
    *give_up = 1;
    if (err) atomicExch(err, DC_ERR_MBAR_TIMEOUT);
    return false;
}
#ifdef DC_TC_TIMING
// instrumented build: cycles one thread of every role spends in each kind of wait, summed over CTAs
// 0 a_free (expander)  1 b_full  2 a_full  3 acc_free (issuer)  4 b_free (loader)  5 d/s_full  6 acc_full (read-out)
// 7 whole kernel (thread 0)
__device__ unsigned long long g_tc_wait[8];
__device__ __forceinline__ bool tc_wait_k(int kind, uint32_t bar, uint32_t parity, volatile int* give_up, int* err) {
    const long long t0 = clock64();
    const bool ok = tc_wait_raw(bar, parity, give_up, err);
    if ((threadIdx.x & 31) == 0) atomicAdd(&g_tc_wait[kind], (unsigned long long)(clock64() - t0));
    return ok;
}
#else
#define tc_wait_k(kind, bar, parity, give_up, err) tc_wait_raw(bar, parity, give_up, err)
#endif
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

template <int TYPE>
constexpr size_t tc_smem_bytes() {
    using T = TcTraits<TYPE>;
    // planes: 2 stages; token codes: 2 buffers x 2 tiles; block scales: 4 x 128 floats; row scales: 4 x 128 x 2 floats;
    // 1024 bytes of slack to start the swizzled tiles on a 1024-byte boundary
    return (size_t)2 * T::NP * TC_PLANE + (size_t)4 * TC_B_Q + 4 * 128 * 4 + 4 * 128 * 8 + 256 + 1024;
}

template <int TYPE>
__global__ void __launch_bounds__(TC_THREADS, 1) k_gemm_tc(GemmTcParams p) {
    using T = TcTraits<TYPE>;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ int s_give_up;
    const uint32_t sA = (smem_u32(smem_raw) + 1023u) & ~1023u;   // [2 stages][NP planes][16 KB], swizzle-aligned
    const uint32_t sBq = sA + 2 * T::NP * TC_PLANE;              // [2 buffers][2 sets][16 KB]
    const uint32_t sS = sBq + 4 * TC_B_Q;                        // [4][128] block scales of the tokens
    const uint32_t sD = sS + 4 * 128 * 4;                        // [4][128][2] d, dmin of the rows
    const uint32_t sBar = sD + 4 * 128 * 8;
    TcBars B;
    {
        uint32_t a = sBar;
        for (int i = 0; i < 2; ++i) B.a_full[i] = a, a += 8;
        for (int i = 0; i < 2; ++i) B.a_free[i] = a, a += 8;
        for (int i = 0; i < 2; ++i) B.b_full[i] = a, a += 8;
        for (int i = 0; i < 2; ++i) B.b_free[i] = a, a += 8;
        for (int i = 0; i < 4; ++i) B.s_full[i] = a, a += 8;
        for (int i = 0; i < 4; ++i) B.d_full[i] = a, a += 8;
        B.acc_full = a, a += 8;
        B.acc_free = a, a += 8;
    }
    const uint32_t tmem_slot = sBar + 22 * 8;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // work item: a pair of neighbouring 64-token tiles of one expert
    int tt0, nset;
    if (p.pair_tile0) {
        tt0 = p.pair_tile0[blockIdx.x];
        if (tt0 < 0) return;
        nset = p.pair_nset[blockIdx.x];
    } else {
        tt0 = 2 * blockIdx.x;
        nset = min(2, p.n_tt - tt0);
    }
    const int expert = p.tile_expert ? p.tile_expert[tt0] : 0;
    if (expert < 0) return;
    int seg = 0, rt = blockIdx.y;
    while (seg + 1 < p.nseg && rt >= (p.seg[seg].N + TC_ROWS - 1) / TC_ROWS) {
        rt -= (p.seg[seg].N + TC_ROWS - 1) / TC_ROWS;
        ++seg;
    }
    const int N = p.seg[seg].N, row0 = rt * TC_ROWS;
    const uint8_t* wbase = p.seg[seg].w + (size_t)expert * p.estride;
    const int nb = p.K / DC_QK_K;
    constexpr uint32_t NCOLS = 512;

    if (warp == 4) {
        tmem_alloc(tmem_slot, NCOLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        s_give_up = 0;
        for (int i = 0; i < 2; ++i) {
            mbar_init(B.a_full[i], TC_EXPAND);
            mbar_init(B.a_free[i], 1);
            mbar_init(B.b_full[i], 1);
            mbar_init(B.b_free[i], 1);
        }
        mbar_init(B.acc_full, 1);
        mbar_init(B.acc_free, 128 * nset);
        for (int i = 0; i < 4; ++i) {
            mbar_init(B.s_full[i], 1);
            mbar_init(B.d_full[i], TC_EXPAND);
        }
        mbar_fence_init();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = lds32(tmem_slot);
    volatile int* give_up = &s_give_up;
#ifdef DC_TC_TIMING
    const long long t_kernel0 = clock64();
#endif

    if (warp < 4) {
        // ------------------------------------------------------------------ expanders
        const int r = tid;
        const int grow = min(row0 + r, N - 1);
        const uint8_t* rp = wbase + (size_t)grow * p.row_bytes;
        if (TYPE == DC_TYPE_Q4_K) {
            uint4 hdr = make_uint4(0, 0, 0, 0), q[4];
            auto fetch = [&](int kb, int h) {
                const uint4* b = reinterpret_cast<const uint4*>(rp + (size_t)kb * T::BB);
                hdr = __ldg(b);
#pragma unroll
                for (int i = 0; i < 4; ++i) q[i] = __ldg(b + 1 + 4 * h + i);
            };
            fetch(0, 0);
            for (int kb = 0; kb < nb; ++kb) {
#pragma unroll 1
                for (int h = 0; h < 2; ++h) {
                    const uint4 H = hdr;
                    uint4 Q[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) Q[i] = q[i];
                    if (h == 0) fetch(kb, 1);
                    else if (kb + 1 < nb) fetch(kb + 1, 0);
                    if (kb > 0 && !tc_wait_k(0, B.a_free[h], (kb - 1) & 1, give_up, p.err)) goto done;
                    if (h == 0) {
                        // this row's scales for the read-out warps
                        const uint32_t da = sD + ((kb & 3) * 128 + r) * 8;
                        asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(da), "f"(fp16_bits_to_float((uint16_t)(H.x & 0xFFFF))),
                                     "f"(fp16_bits_to_float((uint16_t)(H.x >> 16)))
                                     : "memory");
                        mbar_arrive(B.d_full[kb & 3]);
                    }
                    // row r of the stage's planes; chunk c of the row goes to chunk position c ^ (r % 8)
                    const uint32_t stage = sA + h * (T::NP * TC_PLANE) + (r >> 3) * 1024 + (r & 7) * 128;
                    const uint32_t rx = (uint32_t)(r & 7);
#pragma unroll
                    for (int gl = 0; gl < 2; ++gl) {          // sub-block pairs 2h + gl of the block
                        const int g = 2 * h + gl;
                        uint32_t sc0, m0, sc1, m1;
                        q4k_scale_min(H.y, H.z, H.w, 2 * g, sc0, m0);
                        q4k_scale_min(H.y, H.z, H.w, 2 * g + 1, sc1, m1);
                        const uint32_t mm0 = m0 * 0x01010101u, mm1 = m1 * 0x01010101u;
                        const uint32_t a0 = sc0 >> 3, a1 = sc0 & 7u, b0 = sc1 >> 3, b1 = sc1 & 7u;
#pragma unroll
                        for (int hf = 0; hf < 2; ++hf) {
                            const uint4 qv = Q[2 * gl + hf];
                            const uint32_t in[4] = {qv.x, qv.y, qv.z, qv.w};
                            uint32_t lo[4], hi[4];
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                lo[k] = in[k] & 0x0F0F0F0Fu;
                                hi[k] = (in[k] >> 4) & 0x0F0F0F0Fu;
                            }
                            const uint32_t c_lo = stage + (((uint32_t)(4 * gl + hf) ^ rx) << 4);
                            const uint32_t c_hi = stage + (((uint32_t)(4 * gl + hf + 2) ^ rx) << 4);
                            sts128(c_lo, lo[0] * a0, lo[1] * a0, lo[2] * a0, lo[3] * a0);
                            sts128(c_lo + TC_PLANE, lo[0] * a1, lo[1] * a1, lo[2] * a1, lo[3] * a1);
                            sts128(c_lo + 2 * TC_PLANE, mm0, mm0, mm0, mm0);
                            sts128(c_hi, hi[0] * b0, hi[1] * b0, hi[2] * b0, hi[3] * b0);
                            sts128(c_hi + TC_PLANE, hi[0] * b1, hi[1] * b1, hi[2] * b1, hi[3] * b1);
                            sts128(c_hi + 2 * TC_PLANE, mm1, mm1, mm1, mm1);
                        }
                    }
                    fence_async_smem();
                    mbar_arrive(B.a_full[h]);
                }
            }
        } else {
            // Q6_K: 210-byte blocks at 2-byte aligned addresses: aligned 32-bit loads and a funnel shift
            uint32_t wl[17], wh[9], ws[3], wd = 0;
            auto fetch = [&](int kb, int h) {
                const uintptr_t a = (uintptr_t)(rp + (size_t)kb * T::BB);
                const uint32_t* bl = reinterpret_cast<const uint32_t*>((a + 64 * h) & ~(uintptr_t)3);
                const uint32_t* bh = reinterpret_cast<const uint32_t*>((a + 128 + 32 * h) & ~(uintptr_t)3);
                const uint32_t* bs = reinterpret_cast<const uint32_t*>((a + 192 + 8 * h) & ~(uintptr_t)3);
#pragma unroll
                for (int i = 0; i < 17; ++i) wl[i] = __ldg(bl + i);
#pragma unroll
                for (int i = 0; i < 9; ++i) wh[i] = __ldg(bh + i);
#pragma unroll
                for (int i = 0; i < 3; ++i) ws[i] = __ldg(bs + i);
                wd = __ldg(reinterpret_cast<const uint32_t*>((a + 208) & ~(uintptr_t)3));
            };
            fetch(0, 0);
            for (int kb = 0; kb < nb; ++kb) {
#pragma unroll 1
                for (int h = 0; h < 2; ++h) {
                    const uintptr_t a = (uintptr_t)(rp + (size_t)kb * T::BB);
                    const uint32_t sh = (uint32_t)(a & 2u) * 8u;       // every field of the block shares the 2-byte phase
                    uint32_t ql[16], qh[8], scw[2];
#pragma unroll
                    for (int i = 0; i < 16; ++i) ql[i] = __funnelshift_r(wl[i], wl[i + 1], sh);
#pragma unroll
                    for (int i = 0; i < 8; ++i) qh[i] = __funnelshift_r(wh[i], wh[i + 1], sh);
#pragma unroll
                    for (int i = 0; i < 2; ++i) scw[i] = __funnelshift_r(ws[i], ws[i + 1], sh);
                    const float d = fp16_bits_to_float((uint16_t)((wd >> sh) & 0xFFFFu));
                    if (h == 0) fetch(kb, 1);
                    else if (kb + 1 < nb) fetch(kb + 1, 0);
                    if (kb > 0 && !tc_wait_k(0, B.a_free[h], (kb - 1) & 1, give_up, p.err)) goto done;
                    if (h == 0) {
                        const uint32_t da = sD + ((kb & 3) * 128 + r) * 8;
                        asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(da), "f"(d), "f"(0.0f) : "memory");
                        mbar_arrive(B.d_full[kb & 3]);
                    }
                    const uint32_t stage = sA + h * (T::NP * TC_PLANE) + (r >> 3) * 1024 + (r & 7) * 128;
                    const uint32_t rx = (uint32_t)(r & 7);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {                       // chunk i of the half: quadrant i / 2, words 4 (i & 1)..
                        const int qd = i >> 1, w0 = 4 * (i & 1);
                        const int sc = (int)(int8_t)((scw[i >> 2] >> (8 * (i & 3))) & 0xFFu);
                        const uint32_t mag = (uint32_t)(sc < 0 ? -sc : sc);
                        uint32_t u[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            u[k] = ((ql[8 * (qd & 1) + w0 + k] >> (4 * (qd >> 1))) & 0x0F0F0F0Fu) |
                                   (((qh[w0 + k] >> (2 * qd)) & 0x03030303u) << 4);
#pragma unroll
                        for (int di = 0; di < 4; ++di) {
                            // signed digit m in -3..3; per byte m * (u - 32) + 128 = m * u + (128 - 32 m) lies in 32..224, so
                            // one 32-bit multiply-add does the four bytes without carries between them, and flipping
                            // each byte's top bit turns the biased value into the two's-complement byte m * (u - 32)
                            const int dg = (int)((mag >> (2 * di)) & 3u);
                            const int m = sc < 0 ? -dg : dg;
                            const uint32_t K = (uint32_t)(128 - 32 * m) * 0x01010101u;
                            sts128(stage + (((uint32_t)i ^ rx) << 4) + di * TC_PLANE, (u[0] * (uint32_t)m + K) ^ 0x80808080u,
                                   (u[1] * (uint32_t)m + K) ^ 0x80808080u, (u[2] * (uint32_t)m + K) ^ 0x80808080u,
                                   (u[3] * (uint32_t)m + K) ^ 0x80808080u);
                        }
                    }
                    fence_async_smem();
                    mbar_arrive(B.a_full[h]);
                }
            }
        }
    } else if (warp == 4) {
        // ------------------------------------------------------------------ UMMA issue
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_i8(T::A_SIGNED, TC_ROWS, TC_NTOK * nset);
            for (int kb = 0; kb < nb; ++kb) {
                if (!tc_wait_k(1, B.b_full[kb & 1], (kb >> 1) & 1, give_up, p.err)) break;
                const uint32_t sBcur = sBq + (kb & 1) * (2 * TC_B_Q);
                bool ok = true;
                for (int h = 0; h < 2 && ok; ++h) {
                    if (!tc_wait_k(2, B.a_full[h], kb & 1, give_up, p.err)) { ok = false; break; }
                    // the read-out of the previous block must have drained the accumulators
                    if (h == 0 && kb > 0 && !tc_wait_k(3, B.acc_free, (kb - 1) & 1, give_up, p.err)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int pl = 0; pl < T::NP; ++pl)
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk)
                            umma_i8(tmem + pl * TC_N, umma_desc_sw128(sA + h * (T::NP * TC_PLANE) + pl * TC_PLANE + 32 * kk, 1024),
                                    umma_desc_sw128(sBcur + h * (2 * TC_B_HALF) + 32 * kk, 1024), idesc, (h | kk) ? 1u : 0u);
                    if (h == 1) umma_commit(B.acc_full);
                    umma_commit(B.a_free[h]);
                }
                if (!ok) break;
                umma_commit(B.b_free[kb & 1]);
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------------ token tiles
        if (lane == 0) {
            for (int kb = 0; kb < nb; ++kb) {
                if (kb >= 2 && !tc_wait_k(4, B.b_free[kb & 1], ((kb - 2) >> 1) & 1, give_up, p.err)) break;
                const uint8_t* src = p.act + ((size_t)kb * p.n_tt + tt0) * TC_ACT_TILE;
                mbar_expect_tx(B.b_full[kb & 1], (uint32_t)nset * TC_B_Q);
                mbar_expect_tx(B.s_full[kb & 3], (uint32_t)nset * TC_NTOK * 4);
                // operand rows 0..63 come from the first tile, 64..127 from the second: per half block, the two tiles'
                // 8 KB of swizzled rows back to back
                const uint32_t dst = sBq + (kb & 1) * (2 * TC_B_Q);
                for (int th = 0; th < nset; ++th) {
                    for (int hh = 0; hh < 2; ++hh)
                        bulk_g2s(dst + hh * (2 * TC_B_HALF) + th * TC_B_HALF, src + (size_t)th * TC_ACT_TILE + hh * TC_B_HALF, TC_B_HALF,
                                 B.b_full[kb & 1]);
                    bulk_g2s(sS + ((kb & 3) * 128 + th * TC_NTOK) * 4, src + (size_t)th * TC_ACT_TILE + TC_B_Q, TC_NTOK * 4, B.s_full[kb & 3]);
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ read-out
        // a warp reaches the TMEM lanes 32 (warp index % 4) .. + 31: warps 6..9 read set 0, warps 10..13 set 1
        const int q = warp & 3, th = (warp - 6) >> 2;
        if (th < nset) {
            float sumf[TC_NTOK];
#pragma unroll
            for (int i = 0; i < TC_NTOK; ++i) sumf[i] = 0.0f;
            const uint32_t t_lane = tmem + ((uint32_t)(32 * q) << 16) + th * TC_NTOK;
            const int r = 32 * q + lane;
            bool ok = true;
            for (int kb = 0; kb < nb && ok; ++kb) {
                if (!tc_wait_k(5, B.d_full[kb & 3], (kb >> 2) & 1, give_up, p.err) ||
                    !tc_wait_k(5, B.s_full[kb & 3], (kb >> 2) & 1, give_up, p.err) ||
                    !tc_wait_k(6, B.acc_full, kb & 1, give_up, p.err)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint2 dd = lds64(sD + ((kb & 3) * 128 + r) * 8);
                const float d = __uint_as_float(dd.x), dmin = __uint_as_float(dd.y);
                const uint32_t yd_base = sS + ((kb & 3) * 128 + th * TC_NTOK) * 4;
#pragma unroll
                for (int piece = 0; piece < TC_NTOK / 16; ++piece) {
                    int a0[16], a1[16], a2[16], a3[16];
                    tmem_ld16(t_lane + 16 * piece, a0);
                    tmem_ld16(t_lane + TC_N + 16 * piece, a1);
                    tmem_ld16(t_lane + 2 * TC_N + 16 * piece, a2);
                    if (T::NP == 4) tmem_ld16(t_lane + 3 * TC_N + 16 * piece, a3);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float yd = __uint_as_float(lds32(yd_base + 4 * (16 * piece + i)));
                        float& s = sumf[16 * piece + i];
                        if (TYPE == DC_TYPE_Q4_K) {
                            const int I = 8 * a0[i] + a1[i];
                            const float tI = __fmul_rn(__fmul_rn(d, yd), (float)I);
                            const float tM = __fmul_rn(__fmul_rn(dmin, yd), (float)a2[i]);
                            s = __fsub_rn(__fadd_rn(s, tI), tM);
                        } else {
                            const int I = a0[i] + 4 * a1[i] + 16 * a2[i] + 64 * a3[i];
                            s = __fadd_rn(s, __fmul_rn(__fmul_rn(d, yd), (float)I));
                        }
                    }
                }
                tc_fence_before();
                mbar_arrive(B.acc_free);
            }
            if (ok) {
                const int row = row0 + r;
                if (row < N) {
                    float* out = p.out + p.seg[seg].out_off;
#pragma unroll
                    for (int i = 0; i < TC_NTOK; ++i) {
                        const int slot = (tt0 + th) * TC_NTOK + i;
                        if (slot >= p.n_slots) continue;
                        const int orow = p.slot_row ? p.slot_row[slot] : slot;
                        if (orow < 0) continue;
                        float* o = out + (size_t)orow * p.ldo + row;
                        *o = p.accumulate ? __fadd_rn(*o, sumf[i]) : sumf[i];
                    }
                }
            }
        }
    }
done:
    tc_fence_before();
    __syncthreads();
#ifdef DC_TC_TIMING
    if (tid == 0) atomicAdd(&g_tc_wait[7], (unsigned long long)(clock64() - t_kernel0));
#endif
    if (warp == 4) tmem_dealloc(tmem, NCOLS);
}

}  // namespace dc

using namespace dc;

size_t dc_gemm_tc_act_bytes(int n_slots, int K) {
    const int n_tt = (n_slots + TC_NTOK - 1) / TC_NTOK;
    return (size_t)(K / DC_QK_K) * n_tt * TC_ACT_TILE;
}

int dc_gemm_tc_tiles(int n_slots) { return (n_slots + TC_NTOK - 1) / TC_NTOK; }

// x [n_rows, K] f32 (row stride ldx) -> tiled Q8_K activations for n_tt token tiles; slot_token: optional
// device array [n_tt * 64] mapping slots to rows of x.
int dc_launch_quantize_q8k_tiled(dc_ctx* ctx, const float* x, int ldx, int n_rows, int K, uint8_t* act, int n_tt,
                                 const int* slot_token) {
    if (K % DC_QK_K || ldx % 4 || ((uintptr_t)x & 15)) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "quantize_q8k_tiled: K=%d ldx=%d", K, ldx);
    const long long items = (long long)n_tt * TC_NTOK * (K / DC_QK_K);
    long long blocks = (items + 7) / 8;
    if (blocks > 148 * 16) blocks = 148 * 16;
    k_quantize_q8k_tiled<<<(unsigned)blocks, 256, 0, ctx->stream>>>(x, ldx, n_rows, K, act, n_tt, slot_token);
    return dc_check_cuda(ctx, cudaGetLastError(), "k_quantize_q8k_tiled");
}

bool dc_gemm_tc_supports(const dc_weight* w) {
    if (w->type == DC_TYPE_Q4_K) return ((uintptr_t)w->dev & 15) == 0 && w->row_bytes % 16 == 0;
    return w->type == DC_TYPE_Q6_K && ((uintptr_t)w->dev & 1) == 0;
}

// out[slot * ldo + row] = sum over K of w[row] . act[slot] for rows [0, N) and slots [0, n_slots); with tile_expert,
// token tile t uses the matrix of expert tile_expert[t] (skipped when negative).
// Up to three matrices of one shape family (same type, K and row bytes: Q | K | V, or gate | up) in one launch;
// matrix i writes its rows to columns out_off[i].. of out.
int dc_launch_gemm_tc_multi(dc_ctx* ctx, const dc_weight* const* ws, const int* out_off, int nseg, const uint8_t* act,
                            int n_slots, float* out, int ldo, const int* tile_expert, const int* slot_row, bool accumulate,
                            const int* pair_tile0, const int* pair_nset, int n_pairs) {
    if (nseg < 1 || nseg > 3) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "gemm_tc: %d matrices", nseg);
    const dc_weight* w = ws[0];
    GemmTcParams p = {};
    int row_tiles = 0;
    for (int i = 0; i < nseg; ++i) {
        if (!dc_gemm_tc_supports(ws[i])) return dc_fail(ctx, DC_B200_UNSUPPORTED, "gemm_tc: weight type %d or alignment", ws[i]->type);
        if (ws[i]->type != w->type || ws[i]->K != w->K || ws[i]->row_bytes != w->row_bytes || (tile_expert && ws[i]->N != w->N))
            return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "gemm_tc: matrices of one launch must share type, K and row bytes");
        p.seg[i] = {ws[i]->dev, (int)ws[i]->N, out_off ? out_off[i] : 0};
        row_tiles += ((int)ws[i]->N + TC_ROWS - 1) / TC_ROWS;
    }
    p.nseg = nseg;
    p.row_bytes = (int)w->row_bytes;
    p.K = (int)w->K;
    p.act = act;
    p.n_tt = dc_gemm_tc_tiles(n_slots);
    p.n_slots = n_slots;
    p.out = out;
    p.ldo = ldo;
    p.tile_expert = tile_expert;
    p.slot_row = slot_row;
    p.accumulate = accumulate ? 1 : 0;
    p.estride = (size_t)w->N * w->row_bytes;
    p.err = ctx->d_err;
#ifdef DC_TC_TIMING
    {
        if (getenv("DC_TC_TIMING_DUMP")) {
            unsigned long long w2[8];
            cudaMemcpyFromSymbol(w2, g_tc_wait, sizeof(w2));
            fprintf(stderr, "gemm_tc wait cycles so far: a_free %llu b_full %llu a_full %llu acc_free %llu b_free %llu d/s_full %llu acc_full %llu kernel %llu\n",
                    w2[0], w2[1], w2[2], w2[3], w2[4], w2[5], w2[6], w2[7]);
        }
    }
#endif
    if (tile_expert && !pair_tile0) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "gemm_tc: grouped matmul without its tile pairs");
    p.pair_tile0 = pair_tile0;
    p.pair_nset = pair_nset;
    const dim3 grid(pair_tile0 ? n_pairs : (p.n_tt + 1) / 2, row_tiles);
    if (w->type == DC_TYPE_Q4_K) {
        constexpr size_t smem = tc_smem_bytes<DC_TYPE_Q4_K>();
        DC_TRY(dc_kernel_setup(ctx, (const void*)k_gemm_tc<DC_TYPE_Q4_K>, smem, "k_gemm_tc<Q4_K>"));
        k_gemm_tc<DC_TYPE_Q4_K><<<grid, TC_THREADS, smem, ctx->stream>>>(p);
    } else {
        constexpr size_t smem = tc_smem_bytes<DC_TYPE_Q6_K>();
        DC_TRY(dc_kernel_setup(ctx, (const void*)k_gemm_tc<DC_TYPE_Q6_K>, smem, "k_gemm_tc<Q6_K>"));
        k_gemm_tc<DC_TYPE_Q6_K><<<grid, TC_THREADS, smem, ctx->stream>>>(p);
    }
    return dc_check_cuda(ctx, cudaGetLastError(), "k_gemm_tc");
}

int dc_launch_gemm_tc(dc_ctx* ctx, const dc_weight* w, const uint8_t* act, int n_slots, float* out, int ldo,
                      const int* tile_expert, const int* slot_row, bool accumulate, const int* pair_tile0, const int* pair_nset,
                      int n_pairs) {
    if (pair_tile0)
        return dc_launch_gemm_tc_multi(ctx, &w, nullptr, 1, act, n_slots, out, ldo, tile_expert, slot_row, accumulate, pair_tile0,
                                       pair_nset, n_pairs);
    return dc_launch_gemm_tc_multi(ctx, &w, nullptr, 1, act, n_slots, out, ldo, tile_expert, slot_row, accumulate, nullptr, nullptr, 0);
}
