// Batched MUL_MAT for prompt chunks (M >= 32 token rows): K-quant weights x Q8_K activations on the
// 5th-generation tensor cores (tcgen05.mma kind::i8, accumulators in tensor memory), with the block sums
// kept as exact integers so that the float steps per 256-value block are the CPU kernels' own
// (core/src/llm/matmul/batched_exec.cpp:1040-1240 serves these shapes on the CPU; per block
// sumf += (d*yd)*float(I); sumf -= (dmin*yd)*float(M), core/src/kernels/hwy/hwy_moe_quant.cc:248-253).
//
// One CTA per SM walks work items of 128 weight rows x two 64-token tiles over the whole reduction length; its
// warps split the three jobs of a 256-value block and overlap them, across items too (see k_gemm_tc below):
//   1. expanders turn the raw quants of the 128 rows into 8-bit operand planes in shared memory, K-major rows
//      of 128 bytes with the 128-byte swizzle the tensor core reads at full rate (a half block is exactly one
//      such row):
//        Q4_K: q4 * (sc >> 3) and q4 * (sc & 7) (2 planes, unsigned), so that I = 8 * acc0 + acc1 =
//              sum sc_j * sum q4*q8; the minimum term M = sum m_j * (sum of the token's codes in sub-block j)
//              needs no contraction over the values: the read-out warps form it from the eight sub-block sums
//              that the activation tile carries per token (four two-way 16 x 8-bit dot instructions);
//        Q6_K: sign(sc) * digit_i(|sc|) * (q6 - 32) for the four base-4 digits of |sc| (4 planes, signed),
//              so that I = acc0 + 4 acc1 + 16 acc2 + 64 acc3;
//      every plane entry fits 8 bits and the 32-bit accumulators are exact;
//   2. one thread issues the UMMAs (128 rows x 128 tokens x 32 values each), two halves of 128 values per block;
//   3. read-out warps fetch the accumulators (tcgen05.ld) and add the block's float terms in block order.
// Q4_K's two planes x 128 token columns fit the 512 columns of tensor memory twice, so its accumulators are
// double-buffered and the UMMAs of a block run while the block before is read out; Q6_K's four planes fit once.
// The token side is prepared once per activation matrix by k_quantize_q8k_tiled: the Q8_K codes of every
// (block, 64-token tile) stored as the B operand (two halves of 64 swizzled 128-byte rows), followed by the
// 64 block scales and the tokens' sub-block sums, so that a tile half is one contiguous bulk copy.  No multicast
// load anywhere.
//
// Q4_K results are bit-equal to the GEMV path and the CPU oracle.  Q6_K adds one float term per block
// instead of the CPU small-batch kernel's eight lane partials (q6_small_batch.h:62-103): equal integers,
// a different float order, relative difference ~1e-7.
#include <algorithm>
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
    int tiles_x, tiles_y;     // work items: token-tile pairs x row tiles (of all matrices of the launch)
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
// Packed single precision (two lanes per instruction), each lane rounded to nearest like the scalar
// instruction, never contracted with a neighbouring operation.
__device__ __forceinline__ float2 mul2_rn(float2 a, float2 b) {
    float2 r;
    asm("{\n .reg .b64 ra, rb, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %5};\n mul.rn.f32x2 rd, ra, rb;\n mov.b64 {%0, %1}, rd;\n}"
        : "=f"(r.x), "=f"(r.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return r;
}
__device__ __forceinline__ float2 add2_rn(float2 a, float2 b) {
    float2 r;
    asm("{\n .reg .b64 ra, rb, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %5};\n add.rn.f32x2 rd, ra, rb;\n mov.b64 {%0, %1}, rd;\n}"
        : "=f"(r.x), "=f"(r.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return r;
}
__device__ __forceinline__ float2 fma2_rn(float2 a, float2 b, float2 c) {
    float2 r;
    asm("{\n .reg .b64 ra, rb, rc, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %5};\n mov.b64 rc, {%6, %7};\n"
        " fma.rn.f32x2 rd, ra, rb, rc;\n mov.b64 {%0, %1}, rd;\n}"
        : "=f"(r.x), "=f"(r.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return r;
}
// 8 consecutive 32-bit columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, int (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
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
        tc_act_store(tile, slot % TC_NTOK, lane, w0, w1, bw, d);
    }
}

// ---- weight side ---------------------------------------------------------------------------------------
template <int TYPE>
struct TcTraits;
template <>
struct TcTraits<DC_TYPE_Q4_K> {
    // two operand planes and two sets of accumulators (the minimum term comes from the tokens' sub-block sums)
    static constexpr int NP = 2, NSET = 2, BB = DC_Q4K_BYTES, A_SIGNED = 0, TAIL_COPY = TC_ACT_TAIL;
    static constexpr int RO_TOK = 32;         // tokens per read-out warp: 16 read-out warps, four per scheduler
    static constexpr int A_STAGES = 2;        // half blocks of operand planes in shared memory
};
template <>
struct TcTraits<DC_TYPE_Q6_K> {
    static constexpr int NP = 4, NSET = 1, BB = DC_Q6K_BYTES, A_SIGNED = 1, TAIL_COPY = TC_ACT_SCALES;
    static constexpr int RO_TOK = 32;
    static constexpr int A_STAGES = 2;
};

// ---- the kernel: the three jobs of a block (expanding operand planes, issuing UMMAs, reading the accumulators
// out) run on different warps of one CTA per SM and overlap.  A work item is 128 rows x two 64-token tiles, so
// that a block's planes are expanded once for 128 tokens and every UMMA is 128 tokens wide (a stand-alone loop
// runs the instruction in 49 cycles at N = 64 and 65 at N = 128); the CTA walks its items round robin.
//   warps 0-3   expanders: thread r turns its row's half block into the planes of a stage (two stages)
//   warp 4      one thread issues the UMMAs (stage x 128 tokens -> accumulators in TMEM), commits
//               "stage free", "token codes free" and "accumulators full"
//   warp 5      one thread loads the token tiles (codes double-buffered, interleaved so that the two tiles
//               form one 128-row operand; block scales and sub-block sums in a ring of four)
//   warps 6-21  read-out: warp w owns TMEM lane quarter w % 4 and tokens 32 ((w - 6) / 4) .. + 31: adds the
//               block's float terms for its row, then frees the accumulators
// Q4_K: two sets of accumulators (2 planes x 128 columns each) alternate by block.  Q6_K: one set (4 planes x 128
// columns of the 512): the UMMAs of the next block wait for the read-out, the expansion does not.  Every wait is
// bounded and watches a CTA-wide give-up flag.
template <int TYPE>
constexpr int tc_threads() {
    return (6 + 4 * (128 / TcTraits<TYPE>::RO_TOK)) * 32;
}
constexpr int TC_EXPAND = 128;
constexpr int TC_N = 128;                  // tokens per CTA

// mbarriers of the kernel, as word offsets from the first one (addresses are computed, not looked up: several are
// indexed with run-time values)
enum TcBar { A_FULL = 0, A_FREE = 4, B_FULL = 8, B_FREE = 10, S_FULL = 12, D_FULL = 16, ACC_FULL = 20, ACC_FREE = 22, TC_NBARS = 24 };

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
    // planes: 2 stages; token codes: 2 buffers x 2 tiles; tile tails (block scales, sub-block sums): 4 x 2 tiles;
    // row constants: 4 x 128 x 16 bytes; 1024 bytes of slack to start the swizzled tiles on a 1024-byte boundary
    return (size_t)T::A_STAGES * T::NP * TC_PLANE + (size_t)4 * TC_B_Q + 4 * 2 * TC_ACT_TAIL + 4 * 128 * 16 + 384 + 1024;
}

struct TcTile {       // one work item: 128 rows of one matrix x a pair of neighbouring 64-token tiles of one expert
    bool live;
    int tt0, nset, seg, N, row0;
    const uint8_t* wbase;
};
__device__ __forceinline__ TcTile tc_tile_at(const GemmTcParams& p, int t) {
    TcTile ti;
    ti.live = false;
    const int px = t % p.tiles_x, py = t / p.tiles_x;
    if (p.pair_tile0) {
        ti.tt0 = p.pair_tile0[px];
        if (ti.tt0 < 0) return ti;
        ti.nset = p.pair_nset[px];
    } else {
        ti.tt0 = 2 * px;
        ti.nset = min(2, p.n_tt - ti.tt0);
    }
    const int expert = p.tile_expert ? p.tile_expert[ti.tt0] : 0;
    if (expert < 0) return ti;
    int seg = 0, rt = py;
    while (seg + 1 < p.nseg && rt >= (p.seg[seg].N + TC_ROWS - 1) / TC_ROWS) {
        rt -= (p.seg[seg].N + TC_ROWS - 1) / TC_ROWS;
        ++seg;
    }
    ti.seg = seg;
    ti.N = p.seg[seg].N;
    ti.row0 = rt * TC_ROWS;
    ti.wbase = p.seg[seg].w + (size_t)expert * p.estride;
    ti.live = true;
    return ti;
}

template <int TYPE>
__global__ void __launch_bounds__(tc_threads<TYPE>(), 1) k_gemm_tc(GemmTcParams p) {
    using T = TcTraits<TYPE>;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ int s_give_up;
    const uint32_t sA = (smem_u32(smem_raw) + 1023u) & ~1023u;   // [A_STAGES][NP planes][16 KB], swizzle-aligned
    const uint32_t sBq = sA + T::A_STAGES * T::NP * TC_PLANE;    // [2 buffers][2 halves][2 tiles][8 KB]
    const uint32_t sS = sBq + 4 * TC_B_Q;                        // [4][2 tiles] tails: 64 block scales, 64 x 8 sub-block sums
    const uint32_t sD = sS + 4 * 2 * TC_ACT_TAIL;                // [4][128] d, dmin, the eight sub-block minima of the rows
    const uint32_t sBar = sD + 4 * 128 * 16;
    auto bar = [sBar](int which, int i) -> uint32_t { return sBar + 8u * (uint32_t)(which + i); };
    const uint32_t tmem_slot = sBar + TC_NBARS * 8;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nb = p.K / DC_QK_K, total = p.tiles_x * p.tiles_y;
    constexpr uint32_t NCOLS = 512;
    constexpr int RO_THREADS = 4 * (128 / T::RO_TOK) * 32;

    if (warp == 4) {
        tmem_alloc(tmem_slot, NCOLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        s_give_up = 0;
        for (int i = 0; i < 4; ++i) {
            mbar_init(bar(A_FULL, i), TC_EXPAND);
            mbar_init(bar(A_FREE, i), 1);
            mbar_init(bar(S_FULL, i), 1);
            mbar_init(bar(D_FULL, i), TC_EXPAND);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar(B_FULL, i), 1);
            mbar_init(bar(B_FREE, i), 1);
            mbar_init(bar(ACC_FULL, i), 1);
            mbar_init(bar(ACC_FREE, i), RO_THREADS);   // every read-out thread arrives, with or without tokens of its own
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
    // Every role walks the same list of tiles (this CTA's share, round robin) and counts 256-value blocks across
    // tiles: g = blocks before this tile + block index picks ring slots, accumulator sets and barrier phases, so
    // the expansion of a tile's first blocks overlaps the read-out and the stores of the tile before.

    if (warp < 4) {
        // ------------------------------------------------------------------ expanders
        const int r = tid;
        int g0 = 0;
        for (int t = blockIdx.x; t < total; t += gridDim.x) {
            const TcTile ti = tc_tile_at(p, t);
            if (!ti.live) continue;
            const uint8_t* rp = ti.wbase + (size_t)min(ti.row0 + r, ti.N - 1) * p.row_bytes;
            if (TYPE == DC_TYPE_Q4_K) {
                // the raw quants of a half block (header + 64 bytes) are requested two halves ahead of their expansion:
                // one half of expansion work is shorter than a round trip to memory
                struct HalfRaw { uint4 hdr, q[4]; };
                HalfRaw n1, n2;
                auto fetch = [&](HalfRaw& f, int idx) {
                    const uint4* b = reinterpret_cast<const uint4*>(rp + (size_t)(idx >> 1) * T::BB);
                    f.hdr = __ldg(b);
#pragma unroll
                    for (int i = 0; i < 4; ++i) f.q[i] = __ldg(b + 1 + 4 * (idx & 1) + i);
                };
                fetch(n1, 0);
                fetch(n2, 1);
                for (int kb = 0; kb < nb; ++kb) {
                    const int g = g0 + kb;
#pragma unroll 1
                    for (int h = 0; h < 2; ++h) {
                        const uint4 H = n1.hdr;
                        uint4 Q[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) Q[i] = n1.q[i];
                        n1 = n2;
                        if (2 * kb + h + 2 < 2 * nb) fetch(n2, 2 * kb + h + 2);
                        const int hg = 2 * g + h, stg = hg % T::A_STAGES, use = hg / T::A_STAGES;   // stage of this half, its use count
                        if (use > 0 && !tc_wait_k(0, bar(A_FREE, stg), (use - 1) & 1, give_up, p.err)) goto done;
                        // the 6-bit scales and minima of the eight sub-blocks, four to a word (get_scale_min_k4 of ggml's
                        // K-quants on packed bytes)
                        const uint32_t scw = h ? ((H.w & 0x0F0F0F0Fu) | (((H.y >> 6) & 0x03030303u) << 4)) : (H.y & 0x3F3F3F3Fu);
                        if (h == 0) {
                            // this row's scales and minima for the read-out warps (the minima negated: the read-out
                            // subtracts their term)
                            const uint32_t mA = __vneg4(H.z & 0x3F3F3F3Fu),
                                           mB = __vneg4(((H.w >> 4) & 0x0F0F0F0Fu) | (((H.z >> 6) & 0x03030303u) << 4));
                            sts128(sD + ((g & 3) * 128 + r) * 16, __float_as_uint(fp16_bits_to_float((uint16_t)(H.x & 0xFFFF))),
                                   __float_as_uint(fp16_bits_to_float((uint16_t)(H.x >> 16))), mA, mB);
                            mbar_arrive(bar(D_FULL, g & 3));
                        }
                        // row r of the stage's planes; chunk c of the row goes to chunk position c ^ (r % 8)
                        const uint32_t stage = sA + stg * (T::NP * TC_PLANE) + (r >> 3) * 1024 + (r & 7) * 128;
                        const uint32_t rx = (uint32_t)(r & 7);
#pragma unroll
                        for (int gl = 0; gl < 2; ++gl) {          // sub-blocks 4h + 2gl (low nibbles) and 4h + 2gl + 1 (high nibbles)
                            const uint32_t sc0 = (scw >> (16 * gl)) & 0xFFu, sc1 = (scw >> (16 * gl + 8)) & 0xFFu;
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
                                sts128(c_hi, hi[0] * b0, hi[1] * b0, hi[2] * b0, hi[3] * b0);
                                sts128(c_hi + TC_PLANE, hi[0] * b1, hi[1] * b1, hi[2] * b1, hi[3] * b1);
                            }
                        }
                        fence_async_smem();
                        mbar_arrive(bar(A_FULL, stg));
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
                    const int g = g0 + kb;
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
                        const int hg = 2 * g + h, stg = hg % T::A_STAGES, use = hg / T::A_STAGES;
                        if (use > 0 && !tc_wait_k(0, bar(A_FREE, stg), (use - 1) & 1, give_up, p.err)) goto done;
                        if (h == 0) {
                            sts128(sD + ((g & 3) * 128 + r) * 16, __float_as_uint(d), 0u, 0u, 0u);
                            mbar_arrive(bar(D_FULL, g & 3));
                        }
                        const uint32_t stage = sA + stg * (T::NP * TC_PLANE) + (r >> 3) * 1024 + (r & 7) * 128;
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
                        mbar_arrive(bar(A_FULL, stg));
                    }
                }
            }
            g0 += nb;
        }
    } else if (warp == 4) {
        // ------------------------------------------------------------------ UMMA issue
        if (lane == 0) {
            int g0 = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                const TcTile ti = tc_tile_at(p, t);
                if (!ti.live) continue;
                const uint32_t idesc = umma_idesc_i8(T::A_SIGNED, TC_ROWS, TC_NTOK * ti.nset);
                for (int kb = 0; kb < nb && ok; ++kb) {
                    const int g = g0 + kb;
                    if (!tc_wait_k(1, bar(B_FULL, g & 1), (g >> 1) & 1, give_up, p.err)) { ok = false; break; }
                    const uint32_t sBcur = sBq + (g & 1) * (2 * TC_B_Q);
                    const int set = g % T::NSET;
                    const uint32_t tmem_set = tmem + set * (T::NP * TC_N);
                    for (int h = 0; h < 2 && ok; ++h) {
                        const int hg = 2 * g + h, stg = hg % T::A_STAGES, use = hg / T::A_STAGES;
                        if (!tc_wait_k(2, bar(A_FULL, stg), use & 1, give_up, p.err)) { ok = false; break; }
                        // the read-out of the block that used this set of accumulators last must have drained them
                        if (h == 0 && g >= T::NSET && !tc_wait_k(3, bar(ACC_FREE, set), (g / T::NSET - 1) & 1, give_up, p.err)) { ok = false; break; }
                        tc_fence_after();
#pragma unroll
                        for (int pl = 0; pl < T::NP; ++pl)
#pragma unroll
                            for (int kk = 0; kk < 4; ++kk)
                                umma_i8(tmem_set + pl * TC_N, umma_desc_sw128(sA + stg * (T::NP * TC_PLANE) + pl * TC_PLANE + 32 * kk, 1024),
                                        umma_desc_sw128(sBcur + h * (2 * TC_B_HALF) + 32 * kk, 1024), idesc, (h | kk) ? 1u : 0u);
                        if (h == 1) umma_commit(bar(ACC_FULL, set));
                        umma_commit(bar(A_FREE, stg));
                    }
                    if (!ok) break;
                    umma_commit(bar(B_FREE, g & 1));
                }
                g0 += nb;
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------------ token tiles
        if (lane == 0) {
            int g0 = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                const TcTile ti = tc_tile_at(p, t);
                if (!ti.live) continue;
                for (int kb = 0; kb < nb; ++kb) {
                    const int g = g0 + kb;
                    if (g >= 2 && !tc_wait_k(4, bar(B_FREE, g & 1), ((g - 2) >> 1) & 1, give_up, p.err)) { ok = false; break; }
                    const uint8_t* src = p.act + ((size_t)kb * p.n_tt + ti.tt0) * TC_ACT_TILE;
                    mbar_expect_tx(bar(B_FULL, g & 1), (uint32_t)ti.nset * TC_B_Q);
                    mbar_expect_tx(bar(S_FULL, g & 3), (uint32_t)ti.nset * T::TAIL_COPY);
                    // operand rows 0..63 come from the first tile, 64..127 from the second: per half block, the two tiles'
                    // 8 KB of swizzled rows back to back
                    const uint32_t dst = sBq + (g & 1) * (2 * TC_B_Q);
                    for (int th = 0; th < ti.nset; ++th) {
                        for (int hh = 0; hh < 2; ++hh)
                            bulk_g2s(dst + hh * (2 * TC_B_HALF) + th * TC_B_HALF, src + (size_t)th * TC_ACT_TILE + hh * TC_B_HALF, TC_B_HALF,
                                     bar(B_FULL, g & 1));
                        bulk_g2s(sS + ((g & 3) * 2 + th) * TC_ACT_TAIL, src + (size_t)th * TC_ACT_TILE + TC_B_Q, T::TAIL_COPY, bar(S_FULL, g & 3));
                    }
                }
                g0 += nb;
            }
        }
    } else {
        // ------------------------------------------------------------------ read-out
        // a warp reaches the TMEM lanes 32 (warp index % 4) .. + 31: warps 6..9 read the first token tile, 10..13 the second
        constexpr int RO_TOK = T::RO_TOK;
        const int q = warp & 3, tok0 = ((warp - 6) >> 2) * RO_TOK, th = tok0 / TC_NTOK, tin = tok0 % TC_NTOK;
        const uint32_t t_lane0 = tmem + ((uint32_t)(32 * q) << 16) + tok0;
        const int r = 32 * q + lane;
        int g0 = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
            const TcTile ti = tc_tile_at(p, t);
            if (!ti.live) continue;
            const bool mine = th < ti.nset;      // (a lone tile: the second tile's warps only keep the barrier counts)
            float2 sumf[RO_TOK / 2];
#pragma unroll
            for (int i = 0; i < RO_TOK / 2; ++i) sumf[i] = make_float2(0.0f, 0.0f);
            for (int kb = 0; kb < nb && ok; ++kb) {
                const int g = g0 + kb;
                if ((mine && (!tc_wait_k(5, bar(D_FULL, g & 3), (g >> 2) & 1, give_up, p.err) ||
                              !tc_wait_k(5, bar(S_FULL, g & 3), (g >> 2) & 1, give_up, p.err))) ||
                    !tc_wait_k(6, bar(ACC_FULL, g % T::NSET), (g / T::NSET) & 1, give_up, p.err)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                if (mine) {
                    const uint4 dd = lds128(sD + ((g & 3) * 128 + r) * 16);
                    const float d = __uint_as_float(dd.x), dmin = __uint_as_float(dd.y);
                    const uint32_t tail = sS + ((g & 3) * 2 + th) * TC_ACT_TAIL;
                    const uint32_t yd_base = tail + 4 * tin, ys_base = tail + TC_ACT_SCALES + 16 * tin;
                    const uint32_t t_lane = t_lane0 + (g % T::NSET) * (T::NP * TC_N);
                    // eight tokens at a time: few enough live registers beside the 64 running sums for the compiler to
                    // keep several token pairs in flight (the read-out is a chain of dependent short operations)
                    const float2 d2 = make_float2(d, d), dm2 = make_float2(dmin, dmin);
#pragma unroll
                    for (int piece = 0; piece < RO_TOK / 8; ++piece) {
                        int a0[8], a1[8], a2[8], a3[8];
                        tmem_ld8(t_lane + 8 * piece, a0);
                        tmem_ld8(t_lane + TC_N + 8 * piece, a1);
                        if (T::NP == 4) {
                            tmem_ld8(t_lane + 2 * TC_N + 8 * piece, a2);
                            tmem_ld8(t_lane + 3 * TC_N + 8 * piece, a3);
                        }
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 8; i += 2) {
                            const uint2 yw = lds64(yd_base + 4 * (8 * piece + i));
                            const float2 yd = make_float2(__uint_as_float(yw.x), __uint_as_float(yw.y));
                            float2& s = sumf[4 * piece + (i >> 1)];
                            if (TYPE == DC_TYPE_Q4_K) {
                                // |acc0|, |acc1| <= 7 * 15 * 127 * 256 and |M| <= 63 * 127 * 256 stay below 2^22: adding the
                                // integer to the bits of 1.5 * 2^23 and subtracting that constant converts it exactly without
                                // the conversion unit; 8 * acc0 + acc1 then rounds once, in the fused multiply-add: float(I).
                                // -M = sum over sub-blocks of (-minimum) x (sum of the token's codes there), accumulated on
                                // top of the constant's bits.
                                const uint4 ya = lds128(ys_base + 16 * (8 * piece + i)), yb = lds128(ys_base + 16 * (8 * piece + i + 1));
                                int Ma = __dp2a_lo((int)ya.x, (int)dd.z, 0x4B400000);
                                int Mb = __dp2a_lo((int)yb.x, (int)dd.z, 0x4B400000);
                                Ma = __dp2a_hi((int)ya.y, (int)dd.z, Ma);
                                Mb = __dp2a_hi((int)yb.y, (int)dd.z, Mb);
                                Ma = __dp2a_lo((int)ya.z, (int)dd.w, Ma);
                                Mb = __dp2a_lo((int)yb.z, (int)dd.w, Mb);
                                Ma = __dp2a_hi((int)ya.w, (int)dd.w, Ma);
                                Mb = __dp2a_hi((int)yb.w, (int)dd.w, Mb);
                                const float2 kc = make_float2(-12582912.0f, -12582912.0f);
                                const float2 f0 = add2_rn(make_float2(__int_as_float(0x4B400000 + a0[i]), __int_as_float(0x4B400000 + a0[i + 1])), kc);
                                const float2 f1 = add2_rn(make_float2(__int_as_float(0x4B400000 + a1[i]), __int_as_float(0x4B400000 + a1[i + 1])), kc);
                                const float2 fMn = add2_rn(make_float2(__int_as_float(Ma), __int_as_float(Mb)), kc);
                                const float2 fI = fma2_rn(f0, make_float2(8.0f, 8.0f), f1);
                                const float2 tI = mul2_rn(mul2_rn(d2, yd), fI);
                                const float2 tMn = mul2_rn(mul2_rn(dm2, yd), fMn);     // -(dmin * yd) * float(M), exactly
                                // (the two additions stay scalar: behind a packed multiply, a packed add or 1 * x + y was seen
                                // to round once instead of twice, as if fused with the multiply)
                                s.x = __fadd_rn(__fadd_rn(s.x, tI.x), tMn.x);
                                s.y = __fadd_rn(__fadd_rn(s.y, tI.y), tMn.y);
                            } else {
                                const int Ia = a0[i] + 4 * a1[i] + 16 * a2[i] + 64 * a3[i];
                                const int Ib = a0[i + 1] + 4 * a1[i + 1] + 16 * a2[i + 1] + 64 * a3[i + 1];
                                const float2 tt = mul2_rn(mul2_rn(d2, yd), make_float2((float)Ia, (float)Ib));
                                s.x = __fadd_rn(s.x, tt.x);
                                s.y = __fadd_rn(s.y, tt.y);
                            }
                        }
                    }
                }
                tc_fence_before();
                mbar_arrive(bar(ACC_FREE, g % T::NSET));
            }
            if (ok && mine) {
                const int row = ti.row0 + r;
                if (row < ti.N) {
                    float* out = p.out + p.seg[ti.seg].out_off;
#pragma unroll
                    for (int i = 0; i < RO_TOK; ++i) {
                        const int slot = ti.tt0 * TC_NTOK + tok0 + i;
                        if (slot >= p.n_slots) continue;
                        const int orow = p.slot_row ? p.slot_row[slot] : slot;
                        if (orow < 0) continue;
                        float* o = out + (size_t)orow * p.ldo + row;
                        const float v = (i & 1) ? sumf[i >> 1].y : sumf[i >> 1].x;
                        *o = p.accumulate ? __fadd_rn(*o, v) : v;
                    }
                }
            }
            g0 += nb;
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
    p.tiles_x = pair_tile0 ? n_pairs : (p.n_tt + 1) / 2;
    p.tiles_y = row_tiles;
    // one CTA per SM walks its share of the tiles
    const dim3 grid((unsigned)std::min(p.tiles_x * p.tiles_y, ctx->num_sms));
    if (w->type == DC_TYPE_Q4_K) {
        constexpr size_t smem = tc_smem_bytes<DC_TYPE_Q4_K>();
        DC_TRY(dc_kernel_setup(ctx, (const void*)k_gemm_tc<DC_TYPE_Q4_K>, smem, "k_gemm_tc<Q4_K>"));
        k_gemm_tc<DC_TYPE_Q4_K><<<grid, tc_threads<DC_TYPE_Q4_K>(), smem, ctx->stream>>>(p);
    } else {
        constexpr size_t smem = tc_smem_bytes<DC_TYPE_Q6_K>();
        DC_TRY(dc_kernel_setup(ctx, (const void*)k_gemm_tc<DC_TYPE_Q6_K>, smem, "k_gemm_tc<Q6_K>"));
        k_gemm_tc<DC_TYPE_Q6_K><<<grid, tc_threads<DC_TYPE_Q6_K>(), smem, ctx->stream>>>(p);
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
