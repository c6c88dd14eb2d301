// Layout of the quantised activations that the tensor-core MUL_MAT reads (gemm_tc.cu), shared with the kernels
// that produce them (prefill.cu).
//
// Per (256-value block, 64-token tile): TC_ACT_TILE bytes = the Q8_K codes as the UMMA's B operand, then the
// tile's 64 block scales (f32), then per token the eight sums of its codes over 32-value sub-blocks (int16; the
// Q4_K minimum term sum_j m_j * sum_{k in j} q8_k needs only these).  The codes are two halves of 128 values; a
// half is 64 token rows of 128 bytes, K-major, in 8-row groups of 1024 bytes with the 128-byte swizzle: the
// 16-byte chunk c of row t sits at chunk position c ^ (t % 8) of its row.
#pragma once
#include <stdint.h>

namespace dc {

constexpr int TC_NTOK = 64;                               // tokens per activation tile
constexpr int TC_B_HALF = TC_NTOK * 128;                  // codes of one half block of a tile
constexpr int TC_B_Q = 2 * TC_B_HALF;                     // codes of one (block, tile)
constexpr int TC_ACT_SCALES = TC_NTOK * 4;                // the tile's 64 block scales
constexpr int TC_ACT_SUMS = TC_NTOK * 16;                 // per token 8 int16 sums of 32 codes
constexpr int TC_ACT_TAIL = TC_ACT_SCALES + TC_ACT_SUMS;
constexpr int TC_ACT_TILE = TC_B_Q + TC_ACT_TAIL;

// Byte offset, inside a tile's codes, of the 8 codes that lane `lane` of a quantising warp holds (values
// 8 lane .. 8 lane + 7 of the block) for token t of the tile.
__host__ __device__ inline uint32_t tc_act_code_offset(int t, int lane) {
    const int half = lane >> 4, chunk = (lane & 15) >> 1;
    return (uint32_t)(half * TC_B_HALF + (t >> 3) * 1024 + (t & 7) * 128 + ((chunk ^ (t & 7)) << 4) + 8 * (lane & 1));
}

#ifdef __CUDACC__
// A quantising warp stores token t's block into a tile: lane's 8 codes (w0, w1), the block scale d, and from
// bsum_word (q8k_block_core: the sums of the 16-value group of lanes 2g, 2g+1 and of its neighbour, on every
// lane) the 32-value sums.
__device__ __forceinline__ void tc_act_store(uint8_t* tile, int t, int lane, uint32_t w0, uint32_t w1, uint32_t bsum_word,
                                             float d) {
    *reinterpret_cast<uint2*>(tile + tc_act_code_offset(t, lane)) = make_uint2(w0, w1);
    if (lane == 0) reinterpret_cast<float*>(tile + TC_B_Q)[t] = d;
    if ((lane & 3) == 0) {
        const int s32 = (int)(int16_t)(bsum_word & 0xFFFFu) + (int)(int16_t)(bsum_word >> 16);
        reinterpret_cast<int16_t*>(tile + TC_B_Q + TC_ACT_SCALES)[t * 8 + (lane >> 2)] = (int16_t)s32;
    }
}
#endif

}  // namespace dc
