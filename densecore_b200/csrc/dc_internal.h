// Host-side structures shared by the translation units of libdc_b200.so.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <string>
#include <vector>

#include "../../include/dc_b200.h"

#define DC_NSTAGE 4
#define DC_WARPS 8
#define DC_STAGE_TARGET 2304  // bytes of weight rows one pipeline stage aims to hold

struct dc_weight {
    int type;        // ggml type id
    int64_t K;       // ne[0]: reduction length
    int64_t N;       // ne[1]: rows (outputs) per expert slab
    int64_t E;       // ne[2]: experts (1 for dense tensors)
    size_t row_bytes;
    size_t bytes;
    uint8_t* dev;
};

struct dc_ctx {
    int device = 0;
    int num_sms = 148;
    cudaStream_t stream = nullptr;
    int* d_err = nullptr;          // device error word (bounded waits report here)
    std::string last_error;
    std::mutex mu;
    std::vector<dc_weight*> weights;
    // op-level scratch (grown on demand, never shrunk)
    uint8_t* scratch = nullptr;
    size_t scratch_bytes = 0;
    void* pinned = nullptr;        // small pinned staging area for host<->device results
    size_t pinned_bytes = 0;
    int use_pdl = 1;
};

int dc_fail(dc_ctx* ctx, int status, const char* fmt, ...);
int dc_check_cuda(dc_ctx* ctx, cudaError_t e, const char* what);
uint8_t* dc_scratch(dc_ctx* ctx, size_t bytes);   // returns nullptr on failure (error recorded)
void* dc_pinned(dc_ctx* ctx, size_t bytes);
int dc_check_device_error(dc_ctx* ctx);            // reads d_err after a sync

// ---- launch helpers implemented in the kernel translation units ----
struct dc_gemv_seg {
    const uint8_t* w;  // first row
    int type;
    int n_rows;
    int row_bytes;
    float* out;        // out[t * ldo + row]
    int ldo;
};
enum { DC_EPI_STORE = 0, DC_EPI_ACC = 1, DC_EPI_SWIGLU = 2 };

// y = W x for T <= 16 tokens whose Q8_K activations are at act_q8 (row stride K/256*292).
// n_seg 1..3 segments share the activations.  DC_EPI_SWIGLU: seg[0]=gate, seg[1]=up,
// result silu(gate.x)*(up.x) stored to seg[0].out.  argmax (optional, [T] u64 keys,
// zeroed by the caller) receives the packed (value,row) maximum of the stored rows.
int dc_launch_gemv(dc_ctx* ctx, const dc_gemv_seg* segs, int n_seg, int epi, const uint8_t* act_q8, int T, int K,
                   unsigned long long* argmax);
// rows x K f32 -> native Q8_K blocks (row stride K/256*292)
int dc_launch_quantize_q8k(dc_ctx* ctx, const float* x, int rows, int K, uint8_t* out);
// per-block integer sums of W x (debug/parity): I[T][N][nb], M[T][N][nb] (M only for Q4_K)
int dc_launch_block_sums(dc_ctx* ctx, const dc_weight* w, const uint8_t* act_q8, int T, int32_t* I, int32_t* M);
