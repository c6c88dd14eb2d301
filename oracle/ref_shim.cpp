// C entry points over two pieces of DenseCore that compile from their own sources without the
// ggml submodule: the sampler (core/src/sampler/sampler.cpp) and the Q6_K x Q8_K small-batch
// kernel (core/src/llm/matmul/q6_small_batch.h).  TEST INFRASTRUCTURE: the resulting library is the
// reference itself for these functions; the oracle and the golden vectors are checked against it.
// Nothing of DenseCore is copied: both files are included from where the DenseCore tree lies
// (include path given by the build recipe, oracle/Makefile target _ref).
#include <cstdint>
#include <vector>

#include "core/src/sampler/sampler.cpp"          // ArgmaxScalar :42-57, SampleTopP :235-262
#include "core/src/llm/matmul/q6_small_batch.h"  // ComputeQ6KQ8KM4Native :36-103

extern "C" {

__attribute__((visibility("default"))) int dcref_argmax(const float* v, int n) {
    return densecore::sampler::ArgmaxScalar(v, n, 1);
}

// Probabilities SampleTopP forms before it samples: v * (1/T), minus the maximum, std::exp, times 1/sum.
// Returns the token it then draws (top_p = 1, the given seed).
__attribute__((visibility("default"))) int dcref_softmax_temperature(const float* logits, int n, float temperature,
                                                                    uint64_t seed, float* probs_out) {
    densecore::sampler::SamplingParams prm;
    prm.top_k = 0;
    prm.top_p = 1.0f;
    prm.temperature = temperature;
    prm.seed = seed;
    std::vector<float> probs;
    std::vector<int> idx;
    const int tok = densecore::sampler::SampleTopP(logits, n, 1, prm, probs, idx);
    for (int i = 0; i < n && i < (int)probs.size(); ++i) probs_out[i] = probs[(size_t)i];
    return tok;
}

// One Q6_K weight row against four Q8_K activation rows (row stride q8_stride bytes), K values per row.
// Returns 1 when the AVX2 kernel ran.
__attribute__((visibility("default"))) int dcref_q6k_q8k_m4(const void* w_row, const void* q8_rows, uint64_t q8_stride,
                                                           int K, float* sums4) {
    return ComputeQ6KQ8KM4Native(w_row, static_cast<const uint8_t*>(q8_rows), (size_t)q8_stride, 4, K, sums4) ? 1 : 0;
}

}  // extern "C"
