// C-ABI layer: context, weight upload, and the op-level entry points.  Thin
// host code; all arithmetic is in the kernels.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>
#include <cuda_profiler_api.h>

#include <map>
#include <tuple>

#include "dc_common.cuh"
#include "dc_internal.h"

int dc_fail(dc_ctx* ctx, int status, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    if (ctx) ctx->last_error = buf;
    // one CRITICAL line, the convention of core/src/llm/matmul/gemv_exec.cpp:119,138
    fprintf(stderr, "[dc_b200] CRITICAL: %s\n", buf);
    return status;
}

int dc_check_cuda(dc_ctx* ctx, cudaError_t e, const char* what) {
    if (e == cudaSuccess) return DC_B200_OK;
    return dc_fail(ctx, e == cudaErrorMemoryAllocation ? DC_B200_OUT_OF_MEMORY : DC_B200_BACKEND_ERROR, "%s: %s", what,
                   cudaGetErrorString(e));
}

// Kernel attributes and occupancy answers belong to a device, not to the process: a second context on
// another GPU must opt its own kernels into large dynamic shared memory.  Both tables are keyed by
// (device, kernel) and guarded by one mutex, so contexts on several GPUs and several host threads can
// launch at once.
static std::mutex g_kernel_mu;
static std::map<std::pair<int, const void*>, int> g_kernel_smem;                    // opted-in bytes
static std::map<std::tuple<int, const void*, int, size_t>, int> g_kernel_occupancy;

int dc_kernel_setup(dc_ctx* ctx, const void* func, int max_dyn_smem, const char* name) {
    std::lock_guard<std::mutex> lk(g_kernel_mu);
    auto key = std::make_pair(ctx->device, func);
    auto it = g_kernel_smem.find(key);
    if (it != g_kernel_smem.end() && it->second >= max_dyn_smem) return DC_B200_OK;
    cudaError_t e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, max_dyn_smem);
    if (e != cudaSuccess) return dc_check_cuda(ctx, e, name);
    g_kernel_smem[key] = max_dyn_smem;
    return DC_B200_OK;
}

int dc_kernel_occupancy(dc_ctx* ctx, const void* func, int threads, size_t dyn_smem) {
    std::lock_guard<std::mutex> lk(g_kernel_mu);
    auto key = std::make_tuple(ctx->device, func, threads, dyn_smem);
    auto it = g_kernel_occupancy.find(key);
    if (it != g_kernel_occupancy.end()) return it->second;
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, func, threads, dyn_smem) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
    }
    g_kernel_occupancy[key] = n;
    return n;
}

uint8_t* dc_scratch(dc_ctx* ctx, size_t bytes) {
    if (bytes <= ctx->scratch_bytes) return ctx->scratch;
    // growing: wait for work that may still use the old buffer
    cudaStreamSynchronize(ctx->stream);
    if (ctx->scratch) cudaFree(ctx->scratch);
    ctx->scratch = nullptr;
    ctx->scratch_bytes = 0;
    size_t want = bytes + (bytes >> 2) + 4096;
    if (dc_check_cuda(ctx, cudaMalloc(&ctx->scratch, want), "cudaMalloc(scratch)") != DC_B200_OK) return nullptr;
    ctx->scratch_bytes = want;
    return ctx->scratch;
}

void* dc_pinned(dc_ctx* ctx, size_t bytes) {
    if (bytes <= ctx->pinned_bytes) return ctx->pinned;
    cudaStreamSynchronize(ctx->stream);
    if (ctx->pinned) cudaFreeHost(ctx->pinned);
    ctx->pinned = nullptr;
    ctx->pinned_bytes = 0;
    size_t want = bytes + 4096;
    if (dc_check_cuda(ctx, cudaMallocHost(&ctx->pinned, want), "cudaMallocHost") != DC_B200_OK) return nullptr;
    ctx->pinned_bytes = want;
    return ctx->pinned;
}

int dc_check_device_error(dc_ctx* ctx) {
    int err = 0;
    cudaError_t e = cudaMemcpyAsync(&err, ctx->d_err, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) return dc_check_cuda(ctx, e, "reading device error word");
    if (err != 0) {
        cudaMemsetAsync(ctx->d_err, 0, sizeof(int), ctx->stream);
        return dc_fail(ctx, DC_B200_BACKEND_ERROR, "a kernel gave up a bounded wait (code %d)", err);
    }
    return DC_B200_OK;
}

#define DC_TRY(expr)                     \
    do {                                 \
        int _st = (expr);                \
        if (_st != DC_B200_OK) return _st; \
    } while (0)

extern "C" {

int dc_b200_init(int device, dc_ctx** out_ctx) {
    if (!out_ctx) return DC_B200_INVALID_ARGUMENT;
    *out_ctx = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0)
        return dc_fail(nullptr, DC_B200_BACKEND_ERROR, "no CUDA device: %s (this library has no CPU path)",
                       e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    if (device < 0 || device >= n) return dc_fail(nullptr, DC_B200_INVALID_ARGUMENT, "device %d out of range", device);
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return dc_check_cuda(nullptr, e, "cudaGetDeviceProperties");
    if (prop.major != 10)
        return dc_fail(nullptr, DC_B200_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only",
                       device, prop.major, prop.minor);
    dc_ctx* ctx = new dc_ctx();
    ctx->device = device;
    ctx->num_sms = prop.multiProcessorCount;
    if ((e = cudaSetDevice(device)) != cudaSuccess || (e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking)) != cudaSuccess ||
        (e = cudaMalloc(&ctx->d_err, 256)) != cudaSuccess || (e = cudaMemset(ctx->d_err, 0, 256)) != cudaSuccess) {
        int st = dc_check_cuda(nullptr, e, "context set-up");
        delete ctx;
        return st;
    }
    *out_ctx = ctx;
    return DC_B200_OK;
}

void dc_b200_destroy(dc_ctx* ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (dc_weight* w : ctx->weights) {
        if (w) {
            cudaFree(w->dev);
            delete w;
        }
    }
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->pinned) cudaFreeHost(ctx->pinned);
    cudaFree(ctx->d_err);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
}

const char* dc_b200_last_error(dc_ctx* ctx) { return ctx ? ctx->last_error.c_str() : "null context"; }
void* dc_b200_stream(dc_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

int dc_b200_synchronize(dc_ctx* ctx) {
    if (!ctx) return DC_B200_INVALID_ARGUMENT;
    cudaSetDevice(ctx->device);
    DC_TRY(dc_check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize"));
    return dc_check_device_error(ctx);
}

int dc_b200_profiler_range(int start) {
    return (start ? cudaProfilerStart() : cudaProfilerStop()) == cudaSuccess ? DC_B200_OK : DC_B200_BACKEND_ERROR;
}

int dc_b200_set_option(dc_ctx* ctx, const char* name, int value) {
    if (!ctx || !name) return DC_B200_INVALID_ARGUMENT;
    if (!strcmp(name, "pdl")) {
        ctx->use_pdl = value ? 1 : 0;
        return DC_B200_OK;
    }
    if (!strcmp(name, "route_mode")) {
        if (value != DC_ROUTE_STABLE && value != DC_ROUTE_SOFTMAX) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "route_mode must be 0 or 1");
        ctx->route_mode = value;
        return DC_B200_OK;
    }
    if (!strcmp(name, "gemm_tc_min_rows")) {   // 0 or less: never (every MUL_MAT runs the row-streaming kernels)
        ctx->gemm_tc_min_rows = value > 0 ? value : 0x7fffffff;
        return DC_B200_OK;
    }
    return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "unknown option '%s'", name);
}

static size_t type_row_bytes(int type, int64_t K) {
    switch (type) {
    case DC_TYPE_F32: return (size_t)K * 4;
    case DC_TYPE_F16: return (size_t)K * 2;
    case DC_TYPE_Q4_K: return (size_t)(K / DC_QK_K) * DC_Q4K_BYTES;
    case DC_TYPE_Q6_K: return (size_t)(K / DC_QK_K) * DC_Q6K_BYTES;
    }
    return 0;
}

int dc_b200_upload_weight(dc_ctx* ctx, int ggml_type, const int64_t ne[4], const void* data_host,
                          dc_weight** out_weight) {
    if (!ctx || !ne || !data_host || !out_weight) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "upload_weight: null argument");
    *out_weight = nullptr;
    const int64_t K = ne[0], N = ne[1], E = ne[2] > 0 ? ne[2] : 1;
    if (K <= 0 || N <= 0 || (ne[3] != 0 && ne[3] != 1))
        return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "upload_weight: bad shape");
    const bool kq = ggml_type == DC_TYPE_Q4_K || ggml_type == DC_TYPE_Q6_K;
    if (!kq && ggml_type != DC_TYPE_F32 && ggml_type != DC_TYPE_F16)
        return dc_fail(ctx, DC_B200_UNSUPPORTED, "upload_weight: ggml type %d is not supported", ggml_type);
    if (kq && (K % DC_QK_K))
        return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "upload_weight: K=%lld is not a multiple of 256", (long long)K);
    cudaSetDevice(ctx->device);
    dc_weight* w = new dc_weight();
    w->type = ggml_type;
    w->K = K;
    w->N = N;
    w->E = E;
    w->row_bytes = type_row_bytes(ggml_type, K);
    w->bytes = w->row_bytes * (size_t)N * (size_t)E;
    // 64 bytes of slack: bulk copies round row ranges out to 16-byte boundaries
    cudaError_t e = cudaMalloc(&w->dev, w->bytes + 64);
    if (e == cudaSuccess) e = cudaMemsetAsync(w->dev + w->bytes, 0, 64, ctx->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(w->dev, data_host, w->bytes, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        if (w->dev) cudaFree(w->dev);
        delete w;
        return dc_check_cuda(ctx, e, "upload_weight");
    }
    std::lock_guard<std::mutex> lk(ctx->mu);
    ctx->weights.push_back(w);
    *out_weight = w;
    return DC_B200_OK;
}

int dc_b200_free_weight(dc_ctx* ctx, dc_weight* w) {
    if (!ctx || !w) return DC_B200_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lk(ctx->mu);
    for (auto& p : ctx->weights) {
        if (p == w) {
            cudaStreamSynchronize(ctx->stream);
            cudaFree(w->dev);
            delete w;
            p = nullptr;
            return DC_B200_OK;
        }
    }
    return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "free_weight: unknown handle");
}

void* dc_b200_weight_data(const dc_weight* w, size_t* bytes) {
    if (!w) return nullptr;
    if (bytes) *bytes = w->bytes;
    return w->dev;
}

int dc_b200_quantize_q8k_dev(dc_ctx* ctx, const float* x_dev, int rows, int K, void* q8_dev) {
    if (!ctx || !x_dev || !q8_dev || rows <= 0 || K <= 0 || (K % DC_QK_K))
        return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "quantize_q8k: bad argument (rows=%d K=%d)", rows, K);
    cudaSetDevice(ctx->device);
    return dc_launch_quantize_q8k(ctx, x_dev, rows, K, (uint8_t*)q8_dev);
}

int dc_b200_quantize_q8k(dc_ctx* ctx, const float* x_host, int rows, int K, void* q8_host) {
    if (!ctx || !x_host || !q8_host || rows <= 0 || K <= 0 || (K % DC_QK_K))
        return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "quantize_q8k: bad argument (rows=%d K=%d)", rows, K);
    cudaSetDevice(ctx->device);
    const size_t xb = (size_t)rows * K * 4, qb = (size_t)rows * (K / DC_QK_K) * DC_Q8K_BYTES;
    uint8_t* s = dc_scratch(ctx, xb + qb + 256);
    if (!s) return DC_B200_OUT_OF_MEMORY;
    uint8_t* q = s + ((xb + 255) & ~(size_t)255);
    DC_TRY(dc_check_cuda(ctx, cudaMemcpyAsync(s, x_host, xb, cudaMemcpyHostToDevice, ctx->stream), "H2D x"));
    DC_TRY(dc_launch_quantize_q8k(ctx, (const float*)s, rows, K, q));
    DC_TRY(dc_check_cuda(ctx, cudaMemcpyAsync(q8_host, q, qb, cudaMemcpyDeviceToHost, ctx->stream), "D2H q8"));
    return dc_b200_synchronize(ctx);
}

// Scratch layout for a chunk of <= 16 rows: [Q8_K rows]
static int mul_mat_chunks(dc_ctx* ctx, const dc_weight* w, const float* x_dev, int M, float* y_dev, uint8_t* q8) {
    const int K = (int)w->K, N = (int)w->N;
    for (int m0 = 0; m0 < M; m0 += DC_MAX_T) {
        const int T = M - m0 < DC_MAX_T ? M - m0 : DC_MAX_T;
        DC_TRY(dc_launch_quantize_q8k(ctx, x_dev + (size_t)m0 * K, T, K, q8));
        dc_gemv_seg seg = {w->dev, w->type, N, (int)w->row_bytes, y_dev + (size_t)m0 * N, N};
        DC_TRY(dc_launch_gemv(ctx, &seg, 1, DC_EPI_STORE, q8, T, K, nullptr));
    }
    return DC_B200_OK;
}

static int check_mul_mat_args(dc_ctx* ctx, const dc_weight* w, const void* x, int M, const void* y) {
    if (!ctx) return DC_B200_INVALID_ARGUMENT;
    if (!w || !x || !y || M <= 0) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "mul_mat: null argument or M=%d", M);
    if (w->type != DC_TYPE_Q4_K && w->type != DC_TYPE_Q6_K)
        return dc_fail(ctx, DC_B200_UNSUPPORTED, "mul_mat: weight type %d is not Q4_K/Q6_K", w->type);
    if (w->E != 1) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "mul_mat: expert tensor passed to a dense op");
    return DC_B200_OK;
}

// Bytes of the quantised-activation scratch of one MUL_MAT with M token rows.
static size_t mul_mat_act_bytes(dc_ctx* ctx, const dc_weight* w, int M) {
    if (M >= ctx->gemm_tc_min_rows && dc_gemm_tc_supports(w)) return dc_gemm_tc_act_bytes(M, (int)w->K);
    return (size_t)DC_MAX_T * (w->K / DC_QK_K) * DC_Q8K_BYTES;
}

// Prompt-sized inputs take the tensor-core kernel (cb_gemv_batched_custom serves M up to 4096 on the CPU,
// core/src/llm/matmul/dispatch.cpp:622,985-989); decode-sized ones the row-streaming kernels, 16 rows a pass.
static int mul_mat_any(dc_ctx* ctx, const dc_weight* w, const float* x_dev, int M, float* y_dev, uint8_t* act) {
    if (M >= ctx->gemm_tc_min_rows && dc_gemm_tc_supports(w) && ((uintptr_t)x_dev & 15) == 0) {
        DC_TRY(dc_launch_quantize_q8k_tiled(ctx, x_dev, (int)w->K, M, (int)w->K, act, dc_gemm_tc_tiles(M), nullptr));
        return dc_launch_gemm_tc(ctx, w, act, M, y_dev, (int)w->N);
    }
    return mul_mat_chunks(ctx, w, x_dev, M, y_dev, act);
}

int dc_b200_mul_mat_dev(dc_ctx* ctx, const dc_weight* w, const float* x_dev, int M, float* y_dev) {
    DC_TRY(check_mul_mat_args(ctx, w, x_dev, M, y_dev));
    cudaSetDevice(ctx->device);
    uint8_t* s = dc_scratch(ctx, mul_mat_act_bytes(ctx, w, M));
    if (!s) return DC_B200_OUT_OF_MEMORY;
    return mul_mat_any(ctx, w, x_dev, M, y_dev, s);
}

int dc_b200_mul_mat(dc_ctx* ctx, const dc_weight* w, const float* x_host, int M, float* y_host) {
    int st = check_mul_mat_args(ctx, w, x_host, M, y_host);
    if (st != DC_B200_OK) {
        if (y_host && w && M > 0) memset(y_host, 0, (size_t)M * w->N * sizeof(float));  // fail closed
        return st;
    }
    cudaSetDevice(ctx->device);
    const size_t xb = ((size_t)M * w->K * 4 + 255) & ~(size_t)255, yb = ((size_t)M * w->N * 4 + 255) & ~(size_t)255;
    const size_t qb = mul_mat_act_bytes(ctx, w, M);
    uint8_t* s = dc_scratch(ctx, xb + yb + qb);
    if (!s) return DC_B200_OUT_OF_MEMORY;
    float* xd = (float*)s;
    float* yd = (float*)(s + xb);
    st = dc_check_cuda(ctx, cudaMemcpyAsync(xd, x_host, (size_t)M * w->K * 4, cudaMemcpyHostToDevice, ctx->stream), "H2D x");
    if (st == DC_B200_OK) st = mul_mat_any(ctx, w, xd, M, yd, s + xb + yb);
    if (st == DC_B200_OK)
        st = dc_check_cuda(ctx, cudaMemcpyAsync(y_host, yd, (size_t)M * w->N * 4, cudaMemcpyDeviceToHost, ctx->stream), "D2H y");
    if (st == DC_B200_OK) st = dc_b200_synchronize(ctx);
    if (st != DC_B200_OK) memset(y_host, 0, (size_t)M * w->N * sizeof(float));
    return st;
}

int dc_b200_mul_mat_block_sums(dc_ctx* ctx, const dc_weight* w, const float* x_host, int M, int32_t* I_host,
                               int32_t* Mn_host) {
    DC_TRY(check_mul_mat_args(ctx, w, x_host, M, I_host));
    if (M > DC_MAX_T) return dc_fail(ctx, DC_B200_INVALID_ARGUMENT, "block_sums: M=%d > %d", M, DC_MAX_T);
    cudaSetDevice(ctx->device);
    const int K = (int)w->K, nb = K / DC_QK_K;
    const size_t xb = ((size_t)M * K * 4 + 255) & ~(size_t)255;
    const size_t qb = ((size_t)M * nb * DC_Q8K_BYTES + 255) & ~(size_t)255;
    const size_t ib = ((size_t)M * w->N * nb * 4 + 255) & ~(size_t)255;
    const size_t yb = ((size_t)M * w->N * 4 + 255) & ~(size_t)255;
    uint8_t* s = dc_scratch(ctx, xb + qb + 2 * ib + yb);
    if (!s) return DC_B200_OUT_OF_MEMORY;
    int32_t* Id = (int32_t*)(s + xb + qb);
    int32_t* Md = (int32_t*)(s + xb + qb + ib);
    float* yd = (float*)(s + xb + qb + 2 * ib);
    DC_TRY(dc_check_cuda(ctx, cudaMemcpyAsync(s, x_host, (size_t)M * K * 4, cudaMemcpyHostToDevice, ctx->stream), "H2D x"));
    DC_TRY(dc_launch_quantize_q8k(ctx, (const float*)s, M, K, s + xb));
    // the production GEMV kernel itself, asked to store the integer sums it forms on the way
    dc_gemv_seg seg = {w->dev, w->type, (int)w->N, (int)w->row_bytes, yd, (int)w->N};
    DC_TRY(dc_launch_gemv(ctx, &seg, 1, DC_EPI_STORE, s + xb, M, K, nullptr, Id, w->type == DC_TYPE_Q4_K ? Md : nullptr));
    DC_TRY(dc_check_cuda(ctx, cudaMemcpyAsync(I_host, Id, (size_t)M * w->N * nb * 4, cudaMemcpyDeviceToHost, ctx->stream), "D2H I"));
    if (Mn_host && w->type == DC_TYPE_Q4_K)
        DC_TRY(dc_check_cuda(ctx, cudaMemcpyAsync(Mn_host, Md, (size_t)M * w->N * nb * 4, cudaMemcpyDeviceToHost, ctx->stream), "D2H M"));
    return dc_b200_synchronize(ctx);
}

}  // extern "C"
