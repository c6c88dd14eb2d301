/*
 * Stand-in for the two declarations of ggml.h that DenseCore's
 * core/src/llm/matmul/q6_small_batch.h uses: the fp16 storage type and its
 * widening conversion.  TEST INFRASTRUCTURE: lets that header compile without
 * the ggml submodule so that its Q6_K x Q8_K kernel can be run as a reference.
 * The conversion is the exact IEEE half -> single widening (every half value
 * is representable), so any correct implementation gives the same bits.
 */
#pragma once
#include <stdint.h>
#include <string.h>

typedef uint16_t ggml_fp16_t;

static inline float ggml_fp16_to_fp32(ggml_fp16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {  /* subnormal: renormalise */
            int e = -1;
            do {
                ++e;
                man <<= 1;
            } while ((man & 0x400u) == 0);
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}
