// Causal attention of a prompt chunk over the paged fp16 cache: one CTA per (64 query tokens, head), K and V
// tiles of 64 keys staged in shared memory by asynchronous copies, scores and P.V on the tensor cores
// (fp16 operands, the query as a sum of two fp16 terms, fp32 accumulation), online softmax in fp32.  What the CPU does for prompt chunks is
// ggml_flash_attn_ext over fp16 K/V with the query converted to fp16 (core/src/llm/attention/exec.cpp:255-275);
// the decode kernels' exact running-max chain (attn.cu) stays available for chunks through the model option
// "prefill_attention" = 0.
//
// The chunk's own K/V rows are in the cache already (written by the RoPE kernel before this one), so the keys
// of query i are simply positions 0 .. pos0 + i of the sequence's block table.
#include <cuda_fp16.h>

#include "dc_common.cuh"
#include "dc_internal.h"

using dc::smem_u32;

namespace {

constexpr int PA_Q = 64;          // queries per CTA (16 per warp)
constexpr int PA_K = 64;          // keys per tile
constexpr int PA_LD = 136;        // halves per shared row: 128 + 8 padding (272 bytes, conflict-free for ldmatrix)

struct PfAttnParams {
    const float* q;               // [n][n_head][128] f32 (after per-head norm and RoPE)
    const __half* k_arena;        // one layer
    const __half* v_arena;
    const int32_t* table;         // the sequence's block table
    int pos0, n, n_head, n_kv;
    float scale;
    float* out;                   // [n][n_head][128]
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;   // 0: the 16 bytes are zero-filled, the address is not read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

__global__ void __launch_bounds__(128, 2) k_attn_prefill(const PfAttnParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    __half* sQ = reinterpret_cast<__half*>(smem);                 // [2][64][PA_LD]: fp16 head and remainder of the f32 query
    __half* sK = sQ + 2 * PA_Q * PA_LD;                           // [2][64][PA_LD]
    __half* sV = sK + 2 * PA_K * PA_LD;                           // [2][64][PA_LD]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int q0 = blockIdx.x * PA_Q, head = blockIdx.y, kvh = head / (p.n_head / p.n_kv);
    const int last_pos = p.pos0 + min(q0 + PA_Q, p.n) - 1;        // newest key any query of this tile may see
    const int n_tiles = last_pos / PA_K + 1;

    auto load_kv = [&](int tile, int buf) {
        const int k0 = tile * PA_K;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = tid + i * 128, key = c >> 4, part = c & 15;   // 16 chunks of 16 bytes per key row
            const int pos = k0 + key;
            const bool valid = pos <= last_pos;
            const int pp = valid ? pos : 0;
            const size_t off = (((size_t)p.table[pp / DC_KV_BLOCK] * DC_KV_BLOCK + pp % DC_KV_BLOCK) * p.n_kv + kvh) * 128 + part * 8;
            cp_async16(smem_u32(sK + (buf * PA_K + key) * PA_LD + part * 8), p.k_arena + off, valid);
            cp_async16(smem_u32(sV + (buf * PA_K + key) * PA_LD + part * 8), p.v_arena + off, valid);
        }
        cp_async_commit();
    };
    load_kv(0, 0);
    // queries: every f32 value as two fp16 terms, q = hi + lo (lo = fp16(q - hi)), so that the scores keep
    // 22 bits of the query instead of 11; the keys are fp16 in the cache already.  Rows beyond the chunk are zero.
    for (int i = tid; i < PA_Q * 32; i += 128) {
        const int row = i >> 5, c4 = i & 31;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (q0 + row < p.n) v = *reinterpret_cast<const float4*>(p.q + ((size_t)(q0 + row) * p.n_head + head) * 128 + c4 * 4);
        const float in[4] = {v.x, v.y, v.z, v.w};
        float lo[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) lo[k] = in[k] - __half2float(__float2half_rn(in[k]));
        uint2 h, l;
        h.x = pack_half2(in[0], in[1]);
        h.y = pack_half2(in[2], in[3]);
        l.x = pack_half2(lo[0], lo[1]);
        l.y = pack_half2(lo[2], lo[3]);
        *reinterpret_cast<uint2*>(sQ + row * PA_LD + c4 * 4) = h;
        *reinterpret_cast<uint2*>(sQ + (PA_Q + row) * PA_LD + c4 * 4) = l;
    }
    __syncthreads();
    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_run[2] = {-1e30f, -1e30f}, l_run[2] = {0.0f, 0.0f};
    const float sl2 = p.scale * 1.4426950408889634f;
    const int g = lane >> 2, t4 = lane & 3;
    const int qpos0 = p.pos0 + q0 + 16 * warp + g;               // rows g and g + 8 of this warp's 16

    for (int tile = 0; tile < n_tiles; ++tile) {
        const int buf = tile & 1;
        if (tile + 1 < n_tiles) {
            load_kv(tile + 1, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int k0 = tile * PA_K;
        // ---- S = Q K^T for this warp's 16 rows x 64 keys
        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
        {
            const int mi = lane >> 3, r = lane & 7;
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                uint32_t qh[4], ql[4];
                ldsm_x4(smem_u32(sQ + (16 * warp + (mi & 1) * 8 + r) * PA_LD + 16 * kk + (mi >> 1) * 8), qh);
                ldsm_x4(smem_u32(sQ + (PA_Q + 16 * warp + (mi & 1) * 8 + r) * PA_LD + 16 * kk + (mi >> 1) * 8), ql);
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    uint32_t b[4];
                    ldsm_x4(smem_u32(sK + (buf * PA_K + 16 * np + (mi >> 1) * 8 + r) * PA_LD + 16 * kk + (mi & 1) * 8), b);
                    mma16816(s[2 * np], ql, b[0], b[1]);
                    mma16816(s[2 * np + 1], ql, b[2], b[3]);
                    mma16816(s[2 * np], qh, b[0], b[1]);
                    mma16816(s[2 * np + 1], qh, b[2], b[3]);
                }
            }
        }
        // ---- scale, causal mask, online softmax (rows g and g + 8)
        float mx[2] = {-1e30f, -1e30f};
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int kp = k0 + 8 * nt + 2 * t4 + (j & 1), qp = qpos0 + (j >> 1) * 8;
                const float v = kp <= qp ? s[nt][j] * sl2 : -INFINITY;
                s[nt][j] = v;
                mx[j >> 1] = fmaxf(mx[j >> 1], v);
            }
        }
        float corr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m_run[h], mx[h]);
            corr[h] = exp2f(m_run[h] - m_new);
            m_run[h] = m_new;
            l_run[h] *= corr[h];
        }
        float rs[2] = {0.0f, 0.0f};
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float e = exp2f(s[nt][j] - m_run[j >> 1]);
                s[nt][j] = e;
                rs[j >> 1] += e;
            }
        }
        l_run[0] += rs[0];
        l_run[1] += rs[1];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            o[i][0] *= corr[0];
            o[i][1] *= corr[0];
            o[i][2] *= corr[1];
            o[i][3] *= corr[1];
        }
        // ---- O += P V
        {
            const int mi = lane >> 3, r = lane & 7;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                uint32_t a[4];
                a[0] = pack_half2(s[2 * ks][0], s[2 * ks][1]);
                a[1] = pack_half2(s[2 * ks][2], s[2 * ks][3]);
                a[2] = pack_half2(s[2 * ks + 1][0], s[2 * ks + 1][1]);
                a[3] = pack_half2(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
                for (int dp = 0; dp < 8; ++dp) {
                    uint32_t b[4];
                    ldsm_x4_t(smem_u32(sV + (buf * PA_K + 16 * ks + (mi & 1) * 8 + r) * PA_LD + 16 * dp + (mi >> 1) * 8), b);
                    mma16816(o[2 * dp], a, b[0], b[1]);
                    mma16816(o[2 * dp + 1], a, b[2], b[3]);
                }
            }
        }
        __syncthreads();     // every warp is done with this buffer before the next load overwrites it
    }
    // ---- normalise and store
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = q0 + 16 * warp + g + 8 * h;
        if (row >= p.n) continue;
        const float inv = 1.0f / l_run[h];
        float* dst = p.out + ((size_t)row * p.n_head + head) * 128;
#pragma unroll
        for (int nt = 0; nt < 16; ++nt)
            *reinterpret_cast<float2*>(dst + 8 * nt + 2 * t4) = make_float2(o[nt][2 * h] * inv, o[nt][2 * h + 1] * inv);
    }
}

}  // namespace

// Attention of chunk tokens 0..n-1 at positions pos0.. of one sequence (table: its block table on the device).
int dc_launch_attention_prefill(dc_ctx* ctx, const float* q, const void* k_arena, const void* v_arena, const int32_t* table,
                                int pos0, int n, int n_head, int n_kv, float scale, float* out) {
    if (n < 1 || n_kv < 1 || n_head % n_kv) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "attention_prefill: bad shape");
    PfAttnParams p = {q, (const __half*)k_arena, (const __half*)v_arena, table, pos0, n, n_head, n_kv, scale, out};
    const size_t smem = (size_t)(2 * PA_Q + 4 * PA_K) * PA_LD * sizeof(__half);
    int st = dc_kernel_setup(ctx, (const void*)k_attn_prefill, (int)smem, "k_attn_prefill");
    if (st != DC_B200_OK) return st;
    k_attn_prefill<<<dim3((n + PA_Q - 1) / PA_Q, n_head), 128, smem, ctx->stream>>>(p);
    return dc_check_cuda(ctx, cudaGetLastError(), "k_attn_prefill");
}
