// Seeded synthetic weights generated and quantised on the device: a
// counter-based generator (Philox4x32-10) feeds this library's own Q4_K / Q6_K
// block quantisers.  ggml's K-quant weight quantiser is not part of the
// DenseCore tree (its tool calls ggml_quantize_chunk, core/src/tools/quantize.cpp:98);
// any valid block encoding is a legal input to the dot kernels.  Every float
// step is a single correctly rounded operation so the CPU restatement used by
// the tests produces the same bytes.
#include "dc_common.cuh"
#include "dc_internal.h"
#include "dc_model.h"

using namespace dc;

__device__ __forceinline__ void philox(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1,
                                       uint32_t o[4]) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t h0 = __umulhi(0xD2511F53u, c0), l0 = 0xD2511F53u * c0;
        const uint32_t h1 = __umulhi(0xCD9E8D57u, c2), l1 = 0xCD9E8D57u * c2;
        const uint32_t n0 = h1 ^ c1 ^ k0, n2 = h0 ^ c3 ^ k1;
        c0 = n0; c1 = l1; c2 = n2; c3 = l0;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    o[0] = c0; o[1] = c1; o[2] = c2; o[3] = c3;
}

// Sum of the eight 16-bit halves of one Philox block (Irwin-Hall, n = 8),
// centred and scaled to unit variance, times sigma, rounded through fp16.
__device__ __forceinline__ float synth_normal(uint64_t seed, uint64_t index, float sigma) {
    uint32_t o[4];
    philox((uint32_t)index, (uint32_t)(index >> 32), 0x5eedu, 0u, (uint32_t)seed, (uint32_t)(seed >> 32), o);
    int s = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) s += (int)(o[j] & 0xFFFFu) + (int)(o[j] >> 16);
    const float z = __fmul_rn((float)(s - 262140), 1.0f / 53509.9f);
    return __half2float(__float2half_rn(__fmul_rn(z, sigma)));
}

__device__ __forceinline__ int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

// One thread per super-block.
__global__ void __launch_bounds__(128) k_synth_quantized(int type, uint64_t seed, int64_t first_block, int64_t n_blocks,
                                                         float sigma, uint8_t* __restrict__ out) {
    const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    float x[256];
    // element index within the whole tensor, so a shard holds the same values as the full tensor's slice
    for (int i = 0; i < 256; ++i) x[i] = synth_normal(seed, (uint64_t)((first_block + b) * 256 + i), sigma);
    if (type == DC_TYPE_Q4_K) {
        uint8_t* blk = out + b * DC_Q4K_BYTES;
        float sc[8], mn[8], max_sc = 0.0f, max_mn = 0.0f;
        for (int s = 0; s < 8; ++s) {
            float lo = 0.0f, hi = 0.0f;
            for (int l = 0; l < 32; ++l) {
                const float v = x[32 * s + l];
                lo = v < lo ? v : lo;
                hi = v > hi ? v : hi;
            }
            sc[s] = __fdiv_rn(__fsub_rn(hi, lo), 15.0f);
            mn[s] = -lo;
            max_sc = sc[s] > max_sc ? sc[s] : max_sc;
            max_mn = mn[s] > max_mn ? mn[s] : max_mn;
        }
        const __half dh = __float2half_rn(__fdiv_rn(max_sc, 63.0f)), mh = __float2half_rn(__fdiv_rn(max_mn, 63.0f));
        const float d = __half2float(dh), dmin = __half2float(mh);
        int ls[8], lm[8];
        for (int s = 0; s < 8; ++s) {
            ls[s] = d > 0.0f ? clampi((int)rintf(__fdiv_rn(sc[s], d)), 0, 63) : 0;
            lm[s] = dmin > 0.0f ? clampi((int)rintf(__fdiv_rn(mn[s], dmin)), 0, 63) : 0;
        }
        *reinterpret_cast<uint16_t*>(blk) = __half_as_ushort(dh);
        *reinterpret_cast<uint16_t*>(blk + 2) = __half_as_ushort(mh);
        for (int j = 0; j < 4; ++j) {
            blk[4 + j] = (uint8_t)((ls[j] & 63) | ((ls[j + 4] >> 4) << 6));
            blk[8 + j] = (uint8_t)((lm[j] & 63) | ((lm[j + 4] >> 4) << 6));
            blk[12 + j] = (uint8_t)((ls[j + 4] & 0xF) | ((lm[j + 4] & 0xF) << 4));
        }
        for (int c = 0; c < 4; ++c) {
            const float d1 = __fmul_rn(d, (float)ls[2 * c]), m1 = __fmul_rn(dmin, (float)lm[2 * c]);
            const float d2 = __fmul_rn(d, (float)ls[2 * c + 1]), m2 = __fmul_rn(dmin, (float)lm[2 * c + 1]);
            for (int l = 0; l < 32; ++l) {
                const float a = __fadd_rn(x[64 * c + l], m1), bb = __fadd_rn(x[64 * c + 32 + l], m2);
                const int q1 = d1 > 0.0f ? clampi((int)rintf(__fdiv_rn(a, d1)), 0, 15) : 0;
                const int q2 = d2 > 0.0f ? clampi((int)rintf(__fdiv_rn(bb, d2)), 0, 15) : 0;
                blk[16 + 32 * c + l] = (uint8_t)(q1 | (q2 << 4));
            }
        }
    } else {
        uint8_t* blk = out + b * DC_Q6K_BYTES;
        float sc[16], max_sc = 0.0f;
        for (int g = 0; g < 16; ++g) {
            float am = 0.0f;
            for (int l = 0; l < 16; ++l) {
                const float a = fabsf(x[16 * g + l]);
                am = a > am ? a : am;
            }
            sc[g] = __fdiv_rn(am, 31.0f);
            max_sc = sc[g] > max_sc ? sc[g] : max_sc;
        }
        const __half dh = __float2half_rn(__fdiv_rn(max_sc, 127.0f));
        const float d = __half2float(dh);
        for (int i = 0; i < 192; ++i) blk[i] = 0;
        for (int g = 0; g < 16; ++g) {
            const int s = d > 0.0f ? clampi((int)rintf(__fdiv_rn(sc[g], d)), 0, 127) : 0;
            blk[192 + g] = (uint8_t)(int8_t)s;
            const float ds = __fmul_rn(d, (float)s);
            for (int l = 0; l < 16; ++l) {
                const int e = 16 * g + l;
                const int q = ds > 0.0f ? clampi((int)rintf(__fdiv_rn(x[e], ds)), -32, 31) : 0;
                const int u = q + 32;
                const int j = e >> 7, qd = (e >> 5) & 3, ll = e & 31;
                const int qli = 64 * j + 32 * (qd & 1) + ll;
                blk[qli] |= (uint8_t)((u & 15) << ((qd & 2) ? 4 : 0));
                blk[128 + 32 * j + ll] |= (uint8_t)((u >> 4) << (2 * qd));
            }
        }
        blk[208] = (uint8_t)(__half_as_ushort(dh) & 0xFF);
        blk[209] = (uint8_t)(__half_as_ushort(dh) >> 8);
    }
}

__global__ void k_synth_f32(uint64_t seed, int64_t n, float sigma, float offset, float* __restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __fadd_rn(offset, synth_normal(seed, (uint64_t)i, sigma));
}

int dc_launch_synth_quantized(dc_ctx* ctx, int type, uint64_t seed, int64_t first_row, int64_t rows, int64_t K, float sigma,
                              uint8_t* out) {
    const int64_t nb = rows * (K / DC_QK_K), first_block = first_row * (K / DC_QK_K);
    const int64_t grid = (nb + 127) / 128;
    k_synth_quantized<<<(unsigned)grid, 128, 0, ctx->stream>>>(type, seed, first_block, nb, sigma, out);
    return dc_check_cuda(ctx, cudaGetLastError(), "k_synth_quantized");
}

int dc_launch_synth_f32(dc_ctx* ctx, uint64_t seed, int64_t n, float sigma, float offset, float* out) {
    k_synth_f32<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(seed, n, sigma, offset, out);
    return dc_check_cuda(ctx, cudaGetLastError(), "k_synth_f32");
}
