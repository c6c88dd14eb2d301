// MUL_MAT for callers that must not allocate.
//
// dc_b200_mul_mat_dev quantises the activation rows to Q8_K into scratch memory
// that the context grows with cudaMalloc on demand.  Some callers cannot
// tolerate that: a ggml custom-op callback that runs while the graph executor
// holds its buffers fixed, a serving loop that has promised its host it will
// not touch the CUDA allocator after warm-up (cudaMalloc takes a driver lock
// and synchronises the device), or code running between cudaStreamBeginCapture
// and cudaStreamEndCapture, where allocation calls are illegal.  This entry
// point does the same arithmetic with its Q8_K scratch in a fixed array that
// is part of the library image, so the call performs no allocation of any
// kind; the caller supplies the device input and output buffers.
#include <mutex>

#include "dc_common.cuh"
#include "dc_internal.h"

// Q8_K rows of one call: up to 16 activation rows of up to 16384 values
// (64 blocks of 292 bytes each).  Every GPU that loads the library holds these
// 299,008 bytes until the process exits.
#define NA_MAX_ROWS 16
#define NA_MAX_K 16384
#define NA_BYTES (NA_MAX_ROWS * (NA_MAX_K / DC_QK_K) * DC_Q8K_BYTES)
static __device__ __align__(256) uint8_t g_noalloc_q8[NA_BYTES];

// In host code the array's name is only a handle; the device address of each
// GPU's copy has to be asked for with that GPU current.
#define NA_MAX_DEVICES 64
static uint8_t* g_noalloc_ptr[NA_MAX_DEVICES];
static std::mutex g_noalloc_mu;

static int noalloc_scratch(dc_ctx* ctx, uint8_t** out) {
    if (ctx->device < 0 || ctx->device >= NA_MAX_DEVICES)
        return dc_fail(ctx, DC_B200_UNSUPPORTED, "mul_mat_noalloc: device index %d out of range", ctx->device);
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (!g_noalloc_ptr[ctx->device]) {
        cudaError_t e = cudaSetDevice(ctx->device);
        void* p = nullptr;
        if (e == cudaSuccess) e = cudaGetSymbolAddress(&p, g_noalloc_q8);
        if (e != cudaSuccess) return dc_check_cuda(ctx, e, "mul_mat_noalloc: cudaGetSymbolAddress");
        g_noalloc_ptr[ctx->device] = (uint8_t*)p;
    }
    *out = g_noalloc_ptr[ctx->device];
    return DC_B200_OK;
}

extern "C" int dc_b200_mul_mat_dev_noalloc(dc_ctx* ctx, const dc_weight* w, const float* x_dev, int M, float* y_dev) {
    if (!ctx) return DC_B200_INVALID_ARGUMENT;
    if (!w || !x_dev || !y_dev || M <= 0) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "mul_mat_noalloc: null argument or M=%d", M);
    if (w->type != DC_TYPE_Q4_K && w->type != DC_TYPE_Q6_K)
        return dc_fail(ctx, DC_B200_UNSUPPORTED, "mul_mat_noalloc: weight type %d is not Q4_K/Q6_K", w->type);
    if (w->E != 1) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "mul_mat_noalloc: expert tensor passed to a dense op");
    if (M > NA_MAX_ROWS || w->K > NA_MAX_K)
        return dc_fail(ctx, DC_B200_UNSUPPORTED,
                       "mul_mat_noalloc: M=%d rows of K=%lld exceed the built-in scratch (at most %d rows of %d values); "
                       "use dc_b200_mul_mat_dev",
                       M, (long long)w->K, NA_MAX_ROWS, NA_MAX_K);
    uint8_t* q8 = nullptr;
    int st = noalloc_scratch(ctx, &q8);
    if (st != DC_B200_OK) return st;
    cudaSetDevice(ctx->device);
    // the activations are fully rewritten by every call, so nothing has to be cleared first
    st = dc_launch_quantize_q8k(ctx, x_dev, M, (int)w->K, q8);
    if (st != DC_B200_OK) return st;
    dc_gemv_seg seg = {w->dev, w->type, (int)w->N, (int)w->row_bytes, y_dev, (int)w->N};
    return dc_launch_gemv(ctx, &seg, 1, DC_EPI_STORE, q8, M, (int)w->K, nullptr);
}
