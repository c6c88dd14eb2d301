// Layout of the quantised activations that the tensor-core MUL_MAT reads (gemm_tc.cu), shared with the kernels
// that produce them (prefill.cu).
//
// Per (256-value block, 64-token tile): TC_ACT_TILE bytes = the Q8_K codes as the UMMA's B operand, then the
// tile's 64 block scales (f32).  The codes are two halves of 128 values; a half is 64 token rows of 128 bytes,
// K-major, in 8-row groups of 1024 bytes with the 128-byte swizzle: the 16-byte chunk c of row t sits at chunk
// position c ^ (t % 8) of its row.
#pragma once
#include <stdint.h>

namespace dc {

constexpr int TC_NTOK = 64;                               // tokens per activation tile
constexpr int TC_B_HALF = TC_NTOK * 128;                  // codes of one half block of a tile
constexpr int TC_B_Q = 2 * TC_B_HALF;                     // codes of one (block, tile)
constexpr int TC_ACT_TILE = TC_B_Q + TC_NTOK * 4;         // + the tile's 64 block scales

// Byte offset, inside a tile's codes, of the 8 codes that lane `lane` of a quantising warp holds (values
// 8 lane .. 8 lane + 7 of the block) for token t of the tile.
__host__ __device__ inline uint32_t tc_act_code_offset(int t, int lane) {
    const int half = lane >> 4, chunk = (lane & 15) >> 1;
    return (uint32_t)(half * TC_B_HALF + (t >> 3) * 1024 + (t & 7) * 128 + ((chunk ^ (t & 7)) << 4) + 8 * (lane & 1));
}

}  // namespace dc
