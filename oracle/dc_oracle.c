/*
 * dc_oracle.c -- CPU restatement of DenseCore's quantized decode hot path.
 *
 * THIS FILE IS TEST INFRASTRUCTURE.  It is the checker the CUDA library is
 * compared against and the timed CPU baseline of the benchmark.  Nothing in
 * the product library links, loads or calls it.
 *
 * Every function cites the DenseCore source (path within the DenseCore tree,
 * file:line) whose arithmetic it follows.  DenseCore delegates the K-quant
 * inner loops to a ggml fork (github.com/DenseAI/ggml, git submodule at
 * core/third_party/ggml, pinned commit not recoverable from the tree), so the
 * text followed here is DenseCore's own in-tree restatements of that math.
 *
 * Parity status:
 *   pinned by in-tree source (exact integer / comparison semantics):
 *     Q8_K quantiser, Q4_K and Q6_K integer block sums, router expert ids,
 *     assignment bucketing, greedy argmax.
 *   parity unpinned (no source and no golden vectors in the DenseCore tree):
 *     float accumulation order of ggml's own vec_dot kernels, ggml's weight
 *     quantiser, ggml_flash_attn_ext rounding, and the speculative
 *     verify/accept rule (DenseCore has no implementation of it).
 *
 * Build: see oracle/Makefile (gcc -O3 -mavx2 -mfma -ffp-contract=off -pthread).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>
#if defined(__F16C__)
#include <immintrin.h>
#endif
#include <stdatomic.h>
#include <unistd.h>

#define DCO_API __attribute__((visibility("default")))
#define QK_K 256
#define KV_BLOCK 16 /* core/include/densecore/memory/kv_cache.h:50 */

enum { DCO_TYPE_F32 = 0, DCO_TYPE_F16 = 1, DCO_TYPE_Q4_K = 12, DCO_TYPE_Q6_K = 14 };

/* core/src/kernels/hwy/hwy_moe_quant.cc:28-35 */
typedef struct {
    uint16_t d, dmin;
    uint8_t scales[12];
    uint8_t qs[128];
} blk_q4k; /* 144 B */
/* core/src/llm/matmul/q6_small_batch.h:13-18 */
typedef struct {
    uint8_t ql[128];
    uint8_t qh[64];
    int8_t scales[16];
    uint16_t d;
} blk_q6k; /* 210 B */
/* core/src/kernels/hwy/hwy_moe_quant.cc:47-51 */
typedef struct {
    float d;
    int8_t qs[256];
    int16_t bsums[16];
} blk_q8k; /* 292 B */

_Static_assert(sizeof(blk_q4k) == 144, "Q4_K");
_Static_assert(sizeof(blk_q6k) == 210, "Q6_K");
_Static_assert(sizeof(blk_q8k) == 292, "Q8_K");

/* ---------------------------------------------------------- thread pool */
/* Output rows are split across a fixed pool, thread i taking the contiguous
 * range [i*ceil(n/nth), ...) as core/src/llm/matmul/gemv_exec.cpp:376-380 does;
 * workers spin briefly on a generation counter before sleeping, like the
 * bounded spin of gemv_exec.cpp:327-337. */
typedef void (*dco_range_fn)(int64_t lo, int64_t hi, void* ctx);
#define DCO_MAX_THREADS 256
static int g_threads = 1;
static pthread_t g_workers[DCO_MAX_THREADS];
static int g_started = 0;
static atomic_uint g_gen;
static atomic_int g_pending;
static atomic_int g_quit;
static pthread_mutex_t g_mu = PTHREAD_MUTEX_INITIALIZER;
static pthread_cond_t g_cv = PTHREAD_COND_INITIALIZER;
static dco_range_fn g_fn;
static void* g_ctx;
static int64_t g_n;
static int g_nth;
static unsigned g_start_gen; /* generation counter at the time the current workers were created */

static void run_slice(int ith) {
    const int64_t per = (g_n + g_nth - 1) / g_nth;
    int64_t lo = per * ith, hi = lo + per;
    if (hi > g_n) hi = g_n;
    if (lo < hi) g_fn(lo, hi, g_ctx);
}
static void* worker_main(void* arg) {
    const int ith = (int)(intptr_t)arg;
    /* a worker created after earlier generations have passed must not take them for new work */
    unsigned seen = g_start_gen;
    for (;;) {
        int spins = 0;
        while (atomic_load_explicit(&g_gen, memory_order_acquire) == seen) {
            if (atomic_load(&g_quit)) return NULL;
            if (++spins < 20000) {
                __builtin_ia32_pause();
            } else {
                pthread_mutex_lock(&g_mu);
                while (atomic_load(&g_gen) == seen && !atomic_load(&g_quit)) pthread_cond_wait(&g_cv, &g_mu);
                pthread_mutex_unlock(&g_mu);
            }
        }
        seen = atomic_load(&g_gen);
        if (ith < g_nth) run_slice(ith);
        atomic_fetch_sub_explicit(&g_pending, 1, memory_order_release);
    }
}
static void stop_pool(void) {
    if (g_started <= 1) {
        g_started = 0;
        return;
    }
    atomic_store(&g_quit, 1);
    pthread_mutex_lock(&g_mu);
    pthread_cond_broadcast(&g_cv);
    pthread_mutex_unlock(&g_mu);
    for (int i = 1; i < g_started; ++i) pthread_join(g_workers[i], NULL);
    atomic_store(&g_quit, 0);
    g_started = 0;
}
static void parallel_for(int64_t n, dco_range_fn fn, void* ctx) {
    if (g_threads <= 1 || n <= 1) {
        fn(0, n, ctx);
        return;
    }
    if (g_started != g_threads) {
        stop_pool();
        g_start_gen = atomic_load(&g_gen);
        for (int i = 1; i < g_threads; ++i) pthread_create(&g_workers[i], NULL, worker_main, (void*)(intptr_t)i);
        g_started = g_threads;
    }
    g_fn = fn;
    g_ctx = ctx;
    g_n = n;
    g_nth = g_threads;
    atomic_store(&g_pending, g_threads - 1);
    pthread_mutex_lock(&g_mu);
    atomic_fetch_add_explicit(&g_gen, 1, memory_order_release);
    pthread_cond_broadcast(&g_cv);
    pthread_mutex_unlock(&g_mu);
    run_slice(0);
    while (atomic_load_explicit(&g_pending, memory_order_acquire) > 0) __builtin_ia32_pause();
}
DCO_API void dco_set_threads(int n) {
    if (n < 1) n = 1;
    if (n > DCO_MAX_THREADS) n = DCO_MAX_THREADS;
    if (n != g_threads) stop_pool();
    g_threads = n;
}
DCO_API int dco_get_threads(void) { return g_threads; }
DCO_API int dco_max_threads(void) {
    const long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}

/* ------------------------------------------------------------------ fp16 */
/* core/src/kernels/hwy/hwy_moe_quant.cc:55-81 (exact half -> single). */
DCO_API float dco_fp16_to_fp32(uint16_t h) {
#if defined(__F16C__)
    return _cvtsh_ss(h); /* the hardware conversion is exact, identical to the bit manipulation below */
#endif
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1Fu;
    const uint32_t mant = h & 0x03FFu;
    uint32_t bits;
    if (exp == 0) {
        if (mant == 0) {
            bits = sign;
        } else {
            uint32_t m = mant, e = 113u;
            while ((m & 0x0400u) == 0) {
                m <<= 1;
                --e;
            }
            m &= 0x03FFu;
            bits = sign | (e << 23) | (m << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (mant << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (mant << 13);
    }
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

/* IEEE single -> half, round to nearest even (what the F16 KV-cache store does,
 * core/src/runtime/memory/kv_cache_storage.cpp:436). */
DCO_API uint16_t dco_fp32_to_fp16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7FFFFFFFu;
    if (x >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | ((x > 0x7F800000u) ? 0x0200u : 0));
    if (x >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u); /* rounds to inf */
    if (x < 0x33000001u) return (uint16_t)sign;               /* rounds to zero */
    int e = (int)(x >> 23) - 127;
    uint32_t m = (x & 0x7FFFFFu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) {
        shift = 13 + (-14 - e);
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(e + 15) << 10;
        m &= 0x7FFFFFu;
    }
    uint32_t q = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q++;
    return (uint16_t)(sign | (base + q));
}

/* ------------------------------------------------------------- fast exp */
/* core/src/backend/cpu_backend_internal.h:99-114; copy at
 * core/src/llm/moe/native.cpp:287-301.  Plain multiply-add Horner form. */
DCO_API float dco_fast_exp(float x) {
    if (x < -50.0f) x = -50.0f;
    if (x > 50.0f) x = 50.0f;
    const float y = x * 1.4426950408889634f;
    const int32_t i = (int32_t)floorf(y);
    const float f = y - (float)i;
    const float p = 1.0f + f * (0.6960656421638072f + f * (0.224494337302845f + f * 0.07944023841053369f));
    const int32_t bits = (i + 127) << 23;
    float two_i;
    memcpy(&two_i, &bits, 4);
    return two_i * p;
}
/* core/src/kernels/hwy/hwy_fastexp.h:50-84.  The vector form uses MulAdd,
 * i.e. fused multiply-add on FMA targets; fmaf reproduces that. */
DCO_API float dco_fast_exp_fma(float x) {
    x = fmaxf(fminf(x, 50.0f), -50.0f);
    const float y = x * 1.4426950408889634f;
    const float i_f = floorf(y);
    const float f = y - i_f;
    float p = fmaf(0.07944023841053369f, f, 0.224494337302845f);
    p = fmaf(p, f, 0.6960656421638072f);
    p = fmaf(p, f, 1.0f);
    const int32_t bits = ((int32_t)i_f + 127) << 23;
    float two_i;
    memcpy(&two_i, &bits, 4);
    return p * two_i;
}

/* ------------------------------------------------------- Q8_K quantiser */
/* core/src/kernels/hwy/hwy_moe_quant.cc:83-88 */
static inline int nearest_int_q8k(float v) {
    float biased = v + 12582912.0f;
    int bits;
    memcpy(&bits, &biased, 4);
    return (bits & 0x007fffff) - 0x00400000;
}
/* core/src/kernels/hwy/hwy_moe_quant.cc:103-144 */
DCO_API int dco_quantize_row_q8k(const float* input, void* out, int64_t cols) {
    if (!input || !out || cols <= 0 || (cols % QK_K) != 0) return 0;
    blk_q8k* blocks = (blk_q8k*)out;
    const int64_t nb = cols / QK_K;
    for (int64_t bi = 0; bi < nb; ++bi) {
        const float* x = input + bi * QK_K;
        blk_q8k* y = &blocks[bi];
        float max = 0.0f, amax = 0.0f;
        for (int j = 0; j < QK_K; ++j) {
            const float ax = fabsf(x[j]);
            if (ax > amax) {
                amax = ax;
                max = x[j];
            }
        }
        if (amax == 0.0f) {
            memset(y, 0, sizeof(*y));
            continue;
        }
        const float iscale = -127.0f / max;
        for (int j = 0; j < QK_K; ++j) {
            const float prod = iscale * x[j];
            int v = nearest_int_q8k(prod);
            y->qs[j] = (int8_t)(v < 127 ? v : 127);
        }
        for (int j = 0; j < QK_K / 16; ++j) {
            int sum = 0;
            for (int ii = 0; ii < 16; ++ii) sum += y->qs[j * 16 + ii];
            y->bsums[j] = (int16_t)sum;
        }
        y->d = 1.0f / iscale;
    }
    return 1;
}

/* ------------------------------------------------------------ Q4_K dot */
/* core/src/kernels/hwy/hwy_moe_quant.cc:90-101.  out[0..7] = sub-block scales,
 * out[8..15] = sub-block mins. */
DCO_API void dco_q4k_decode_scales(const uint8_t packed[12], uint8_t out[16]) {
    const uint32_t k1 = 0x3f3f3f3f, k2 = 0x0f0f0f0f, k3 = 0x03030303;
    uint32_t u[4];
    memcpy(u, packed, 12);
    u[3] = ((u[2] >> 4) & k2) | (((u[1] >> 6) & k3) << 4);
    const uint32_t uaux = u[1] & k1;
    u[1] = (u[2] & k2) | (((u[0] >> 6) & k3) << 4);
    u[2] = uaux;
    u[0] &= k1;
    memcpy(out, u, 16);
}

/* Integer parts of one Q4_K x Q8_K super-block:
 *   I = sum_{s<8} scale_s * sum_{32} q*y ; M = sum_{g<16} bsums_g * min_{g/2}
 * core/src/kernels/hwy/hwy_moe_quant.cc:202-246,
 * core/src/llm/matmul/kquant_batched_kernels.h:64-106. */
static inline void q4k_block_ints(const blk_q4k* xb, const blk_q8k* yb, int32_t* I, int32_t* M) {
    uint8_t sm[16];
    dco_q4k_decode_scales(xb->scales, sm);
    int32_t mn = 0;
    for (int j = 0; j < 16; ++j) mn += (int32_t)yb->bsums[j] * (int32_t)sm[8 + j / 2];
    int32_t acc = 0;
    for (int c = 0; c < 4; ++c) {
        const uint8_t* q = xb->qs + 32 * c;
        const int8_t* ylo = yb->qs + 64 * c;
        const int8_t* yhi = ylo + 32;
        int32_t lo = 0, hi = 0;
        for (int l = 0; l < 32; ++l) {
            lo += (int32_t)(q[l] & 0xF) * ylo[l];
            hi += (int32_t)(q[l] >> 4) * yhi[l];
        }
        acc += (int32_t)sm[2 * c] * lo + (int32_t)sm[2 * c + 1] * hi;
    }
    *I = acc;
    *M = mn;
}

DCO_API void dco_q4k_q8k_block_sums(const void* w_row, const void* y_row, int64_t cols, int32_t* I, int32_t* M) {
    const blk_q4k* x = (const blk_q4k*)w_row;
    const blk_q8k* y = (const blk_q8k*)y_row;
    for (int64_t b = 0; b < cols / QK_K; ++b) q4k_block_ints(&x[b], &y[b], &I[b], &M[b]);
}

/* Row dot, float order of core/src/kernels/hwy/hwy_moe_quant.cc:248-253:
 * per block, sumf += (d*yd)*float(I); sumf -= (dmin*yd)*float(M). */
DCO_API float dco_vec_dot_q4k_q8k(const void* w_row, const void* y_row, int64_t cols) {
    const blk_q4k* x = (const blk_q4k*)w_row;
    const blk_q8k* y = (const blk_q8k*)y_row;
    float sumf = 0.0f;
    for (int64_t b = 0; b < cols / QK_K; ++b) {
        int32_t I, M;
        q4k_block_ints(&x[b], &y[b], &I, &M);
        const float d = dco_fp16_to_fp32(x[b].d) * y[b].d;
        const float dmin = dco_fp16_to_fp32(x[b].dmin) * y[b].d;
        sumf += d * (float)I;
        sumf -= dmin * (float)M;
    }
    return sumf;
}

/* ------------------------------------------------------------ Q6_K dot */
/* Element order core/src/llm/matmul/q6_small_batch.h:52-74. */
static inline void q6k_unpack(const blk_q6k* xb, int8_t q[256]) {
    for (int j = 0; j < 2; ++j) {
        const uint8_t* ql = xb->ql + 64 * j;
        const uint8_t* qh = xb->qh + 32 * j;
        int8_t* o = q + 128 * j;
        for (int l = 0; l < 32; ++l) {
            o[l] = (int8_t)((ql[l] & 15) | ((qh[l] & 3) << 4)) - 32;
            o[32 + l] = (int8_t)((ql[32 + l] & 15) | (((qh[l] >> 2) & 3) << 4)) - 32;
            o[64 + l] = (int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
            o[96 + l] = (int8_t)((ql[32 + l] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
        }
    }
}
/* The eight int32 partials are the AVX2 lanes of q6_small_batch.h:62-83: lane L
 * collects bytes 4L..4L+3 of every 32-element quadrant, scaled by scales[e/16]. */
static inline void q6k_block_lanes(const blk_q6k* xb, const blk_q8k* yb, int32_t lane[8]) {
    int8_t q[256];
    q6k_unpack(xb, q);
    for (int L = 0; L < 8; ++L) lane[L] = 0;
    for (int e = 0; e < 256; ++e) {
        const int L = (e % 32) / 4;
        lane[L] += (int32_t)xb->scales[e / 16] * ((int32_t)q[e] * (int32_t)yb->qs[e]);
    }
}
DCO_API void dco_q6k_q8k_block_sums(const void* w_row, const void* y_row, int64_t cols, int32_t* I) {
    const blk_q6k* x = (const blk_q6k*)w_row;
    const blk_q8k* y = (const blk_q8k*)y_row;
    for (int64_t b = 0; b < cols / QK_K; ++b) {
        int32_t lane[8];
        q6k_block_lanes(&x[b], &y[b], lane);
        int32_t s = 0;
        for (int L = 0; L < 8; ++L) s += lane[L];
        I[b] = s;
    }
}
/* Row dot, float order of q6_small_batch.h:84-92: acc[L] = fma(yd*xd, float(lane L), acc[L])
 * per block, then ((a0+a4)+(a2+a6)) + ((a1+a5)+(a3+a7)). */
DCO_API float dco_vec_dot_q6k_q8k(const void* w_row, const void* y_row, int64_t cols) {
    const blk_q6k* x = (const blk_q6k*)w_row;
    const blk_q8k* y = (const blk_q8k*)y_row;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int64_t b = 0; b < cols / QK_K; ++b) {
        int32_t lane[8];
        q6k_block_lanes(&x[b], &y[b], lane);
        const float s = y[b].d * dco_fp16_to_fp32(x[b].d);
        for (int L = 0; L < 8; ++L) acc[L] = fmaf(s, (float)lane[L], acc[L]);
    }
    const float r0 = acc[0] + acc[4], r1 = acc[1] + acc[5], r2 = acc[2] + acc[6], r3 = acc[3] + acc[7];
    return (r0 + r2) + (r1 + r3);
}

/* ---------------------------------------------------------- dequantise */
/* w = d*sc*q - dmin*m (core/src/llm/moe/q4_rowpair.h:61-62, hwy_moe_quant.cc:202-211). */
DCO_API void dco_dequantize_row_q4k(const void* row, float* out, int64_t cols) {
    const blk_q4k* x = (const blk_q4k*)row;
    for (int64_t b = 0; b < cols / QK_K; ++b) {
        uint8_t sm[16];
        dco_q4k_decode_scales(x[b].scales, sm);
        const float d = dco_fp16_to_fp32(x[b].d), dmin = dco_fp16_to_fp32(x[b].dmin);
        float* o = out + b * QK_K;
        for (int c = 0; c < 4; ++c) {
            const float d1 = d * sm[2 * c], m1 = dmin * sm[8 + 2 * c];
            const float d2 = d * sm[2 * c + 1], m2 = dmin * sm[8 + 2 * c + 1];
            for (int l = 0; l < 32; ++l) {
                o[64 * c + l] = d1 * (float)(x[b].qs[32 * c + l] & 0xF) - m1;
                o[64 * c + 32 + l] = d2 * (float)(x[b].qs[32 * c + l] >> 4) - m2;
            }
        }
    }
}
DCO_API void dco_dequantize_row_q6k(const void* row, float* out, int64_t cols) {
    const blk_q6k* x = (const blk_q6k*)row;
    for (int64_t b = 0; b < cols / QK_K; ++b) {
        int8_t q[256];
        q6k_unpack(&x[b], q);
        const float d = dco_fp16_to_fp32(x[b].d);
        for (int e = 0; e < 256; ++e) out[b * QK_K + e] = d * (float)x[b].scales[e / 16] * (float)q[e];
    }
}

static inline int64_t row_bytes_of(int type, int64_t K) {
    switch (type) {
    case DCO_TYPE_Q4_K: return K / QK_K * 144;
    case DCO_TYPE_Q6_K: return K / QK_K * 210;
    case DCO_TYPE_F32: return K * 4;
    case DCO_TYPE_F16: return K * 2;
    }
    return 0;
}
DCO_API int64_t dco_row_bytes(int type, int64_t K) { return row_bytes_of(type, K); }

static inline float vec_dot_typed(int type, const void* w_row, const void* y_row, int64_t K) {
    return type == DCO_TYPE_Q4_K ? dco_vec_dot_q4k_q8k(w_row, y_row, K) : dco_vec_dot_q6k_q8k(w_row, y_row, K);
}

/* ------------------------------------------------------------- MUL_MAT */
/* y[m, n] = W[n, :] . x[m, :].  Activation rows -> Q8_K once, output rows split
 * across threads (core/src/llm/matmul/gemv_exec.cpp:283-346, :376-380, :958-986;
 * batched form core/src/llm/matmul/batched_exec.cpp:55).  F32 weights take a
 * plain float dot (router, core/src/llm/graph/decoder.cpp:2265).
 * q8_scratch: M * K/256 * 292 bytes, or NULL to allocate. */
typedef struct {
    int type;
    const void* W;
    int64_t N, K, M, rb, q8_row;
    const float* x;
    const char* q8;
    float* y;
} mm_ctx;
static void mm_rows(int64_t lo, int64_t hi, void* p) {
    const mm_ctx* c = (const mm_ctx*)p;
    for (int64_t n = lo; n < hi; ++n) {
        if (c->type == DCO_TYPE_F32) {
            const float* w = (const float*)c->W + n * c->K;
            for (int64_t m = 0; m < c->M; ++m) {
                float s = 0.0f;
                for (int64_t k = 0; k < c->K; ++k) s += w[k] * c->x[m * c->K + k];
                c->y[m * c->N + n] = s;
            }
        } else {
            const char* w_row = (const char*)c->W + n * c->rb;
            for (int64_t m = 0; m < c->M; ++m)
                c->y[m * c->N + n] = vec_dot_typed(c->type, w_row, c->q8 + m * c->q8_row, c->K);
        }
    }
}
DCO_API int dco_mul_mat(int type, const void* W, int64_t N, int64_t K, const float* x, int64_t M, float* y,
                        void* q8_scratch) {
    if (!W || !x || !y || N <= 0 || K <= 0 || M <= 0) return 0;
    mm_ctx c = {type, W, N, K, M, row_bytes_of(type, K), K / QK_K * 292, x, NULL, y};
    if (type == DCO_TYPE_F32) {
        parallel_for(N, mm_rows, &c);
        return 1;
    }
    if ((type != DCO_TYPE_Q4_K && type != DCO_TYPE_Q6_K) || (K % QK_K) != 0) return 0;
    void* own = NULL;
    if (!q8_scratch) q8_scratch = own = malloc((size_t)(M * c.q8_row));
    for (int64_t m = 0; m < M; ++m) dco_quantize_row_q8k(x + m * K, (char*)q8_scratch + m * c.q8_row, K);
    c.q8 = (const char*)q8_scratch;
    parallel_for(N, mm_rows, &c);
    free(own);
    return 1;
}

/* -------------------------------------------------------------- router */
/* Generic route: softmax over all experts (expf(x-max), * 1/sum:
 * core/include/densecore/simd/simd_ops.h:1171-1195), top-k by descending
 * insertion with strict '>' (core/src/moe/moe_routing.cpp:61-88), renormalise
 * (:90-101), then * routed scaling factor (core/src/llm/moe/exec.cpp:764-768). */
DCO_API void dco_route_softmax_topk(const float* logits, int T, int n_experts, int top_k, int normalize, float scale,
                                    int32_t* ids, float* weights) {
    float* probs = (float*)malloc(sizeof(float) * (size_t)n_experts);
    for (int t = 0; t < T; ++t) {
        const float* l = logits + (size_t)t * n_experts;
        float mx = l[0];
        for (int e = 1; e < n_experts; ++e) mx = l[e] > mx ? l[e] : mx;
        float sum = 0.0f;
        for (int e = 0; e < n_experts; ++e) {
            probs[e] = expf(l[e] - mx);
            sum += probs[e];
        }
        const float inv = 1.0f / sum;
        for (int e = 0; e < n_experts; ++e) probs[e] *= inv;
        int32_t* oi = ids + (size_t)t * top_k;
        float* ow = weights + (size_t)t * top_k;
        for (int i = 0; i < top_k; ++i) {
            ow[i] = -INFINITY;
            oi[i] = -1;
        }
        for (int e = 0; e < n_experts; ++e) {
            const float v = probs[e];
            if (v <= ow[top_k - 1]) continue;
            int j = top_k - 1;
            while (j > 0 && v > ow[j - 1]) {
                ow[j] = ow[j - 1];
                oi[j] = oi[j - 1];
                --j;
            }
            ow[j] = v;
            oi[j] = e;
        }
        if (normalize) {
            float s = 0.0f;
            for (int i = 0; i < top_k; ++i) s += ow[i];
            if (s > 0.0f) {
                const float is = 1.0f / s;
                for (int i = 0; i < top_k; ++i) ow[i] *= is;
            }
        }
        for (int i = 0; i < top_k; ++i) ow[i] *= scale;
    }
    free(probs);
}

/* Stable route on raw logits: "larger logit first, then lower id, NaN last",
 * weights = exp(l - max_sel) / sum over the selected k only; degenerate
 * denominator -> uniform (core/src/llm/moe/native.cpp:610-676). */
static int precedes(float a, int32_t ai, float b, int32_t bi) {
    const int an = isnan(a), bn = isnan(b);
    if (an != bn) return !an;
    if (a > b) return 1;
    if (a < b) return 0;
    return ai < bi;
}
DCO_API int dco_route_stable_topk(const float* logits, int T, int n_experts, int top_k, float scale, int32_t* ids,
                                  float* weights) {
    if (top_k <= 0 || top_k > n_experts) return 0;
    for (int t = 0; t < T; ++t) {
        const float* l = logits + (size_t)t * n_experts;
        int32_t* sel = ids + (size_t)t * top_k;
        float* w = weights + (size_t)t * top_k;
        int count = 0;
        for (int32_t e = 0; e < n_experts; ++e) {
            int at = count;
            while (at > 0 && precedes(l[e], e, l[sel[at - 1]], sel[at - 1])) --at;
            if (at >= top_k) continue;
            const int move_end = count < top_k - 1 ? count : top_k - 1;
            for (int p = move_end; p > at; --p) sel[p] = sel[p - 1];
            sel[at] = e;
            count = count + 1 < top_k ? count + 1 : top_k;
        }
        float mx = -INFINITY;
        int finite = 1;
        for (int k = 0; k < top_k; ++k) {
            const float v = l[sel[k]];
            finite = finite && isfinite(v);
            if (isfinite(v) && v > mx) mx = v;
        }
        float den = 0.0f;
        if (finite && isfinite(mx)) {
            for (int k = 0; k < top_k; ++k) {
                w[k] = expf(l[sel[k]] - mx);
                den += w[k];
            }
        }
        if (!(den > 0.0f) || !isfinite(den)) {
            for (int k = 0; k < top_k; ++k) w[k] = 1.0f / (float)top_k;
        } else {
            for (int k = 0; k < top_k; ++k) w[k] /= den;
        }
        for (int k = 0; k < top_k; ++k) w[k] *= scale;
    }
    return 1;
}

/* Expert-grouped reorder map: counts, prefix sums, stable scatter in routing
 * order (core/src/moe/moe_routing.cpp:534-603).  offsets has n_experts+1
 * entries; tokens/slot_of have T*top_k entries (slot_of[pos] = routing index). */
DCO_API void dco_build_reorder_map(const int32_t* ids, int T, int top_k, int n_experts, int32_t* offsets,
                                   int32_t* tokens, int32_t* slot_of) {
    const int total = T * top_k;
    int32_t* cursor = (int32_t*)calloc((size_t)n_experts + 1, sizeof(int32_t));
    memset(offsets, 0, sizeof(int32_t) * ((size_t)n_experts + 1));
    for (int i = 0; i < total; ++i)
        if (ids[i] >= 0 && ids[i] < n_experts) offsets[ids[i] + 1]++;
    for (int e = 0; e < n_experts; ++e) offsets[e + 1] += offsets[e];
    memcpy(cursor, offsets, sizeof(int32_t) * (size_t)n_experts);
    for (int i = 0; i < total; ++i) {
        if (ids[i] < 0 || ids[i] >= n_experts) continue;
        const int pos = cursor[ids[i]]++;
        tokens[pos] = i / top_k;
        slot_of[pos] = i;
    }
    free(cursor);
}

/* ----------------------------------------------------------- MoE layer */
/* Quantised production path.  Per (token, selected expert): x -> Q8_K once per
 * token (core/src/llm/moe/native.cpp:1577-1630); h[r] = silu(gate_r.x)*(up_r.x)
 * with silu(g) = g/(1+exp(-g)) (native.cpp:3929-4345; fast-exp polynomial when
 * fast_exp != 0, std exp otherwise); h -> Q8_K (native.cpp:3075); down dot;
 * out[t] += w * down (dst += w*src).  Combine order: routing order when T <= 4
 * and T*top_k <= 32 (core/src/backend/cpu_backend_moe_ops.cpp:66,1247-1248,
 * :1578-1597), else ascending expert id with tokens in routing order inside an
 * expert (core/src/moe/moe_routing.cpp:647-676). */
typedef struct {
    int gate_type, up_type, down_type, n_experts, hidden, inter, top_k, fast_exp;
    const void *gate_w, *up_w, *down_w;
    const int32_t* ids;
    const char *xq, *hq;
    int64_t g_rb, u_rb, d_rb, xq_row, hq_row;
    float *h, *dn;
} moe_ctx;
static void moe_gate_up(int64_t lo, int64_t hi, void* p) {
    const moe_ctx* c = (const moe_ctx*)p;
    for (int64_t idx = lo; idx < hi; ++idx) {
        const int i = (int)(idx / c->inter), r = (int)(idx % c->inter), e = c->ids[i];
        if (e < 0 || e >= c->n_experts) {
            c->h[idx] = 0.0f;
            continue;
        }
        const char* gw = (const char*)c->gate_w + ((int64_t)e * c->inter + r) * c->g_rb;
        const char* uw = (const char*)c->up_w + ((int64_t)e * c->inter + r) * c->u_rb;
        const char* xr = c->xq + (i / c->top_k) * c->xq_row;
        const float g = vec_dot_typed(c->gate_type, gw, xr, c->hidden);
        const float u = vec_dot_typed(c->up_type, uw, xr, c->hidden);
        const float ex = c->fast_exp ? dco_fast_exp(-g) : expf(-g);
        c->h[idx] = (g / (1.0f + ex)) * u;
    }
}
static void moe_down(int64_t lo, int64_t hi, void* p) {
    const moe_ctx* c = (const moe_ctx*)p;
    for (int64_t idx = lo; idx < hi; ++idx) {
        const int i = (int)(idx / c->hidden), r = (int)(idx % c->hidden), e = c->ids[i];
        if (e < 0 || e >= c->n_experts) {
            c->dn[idx] = 0.0f;
            continue;
        }
        const char* dw = (const char*)c->down_w + ((int64_t)e * c->hidden + r) * c->d_rb;
        c->dn[idx] = vec_dot_typed(c->down_type, dw, c->hq + i * c->hq_row, c->inter);
    }
}
DCO_API int dco_moe_forward(int gate_type, int up_type, int down_type, const void* gate_w, const void* up_w,
                            const void* down_w, int n_experts, int hidden, int inter, const float* x, int T,
                            int top_k, const int32_t* ids, const float* weights, int fast_exp, float* out,
                            float* h_out /* optional [T*top_k*inter] */) {
    if ((hidden % QK_K) || (inter % QK_K)) return 0;
    const int64_t xq_row = hidden / QK_K * 292, hq_row = inter / QK_K * 292;
    const int total = T * top_k;
    char* xq = (char*)malloc((size_t)(T * xq_row));
    char* hq = (char*)malloc((size_t)(total * hq_row));
    float* h = (float*)malloc(sizeof(float) * (size_t)total * inter);
    float* dn = (float*)malloc(sizeof(float) * (size_t)total * hidden);
    for (int t = 0; t < T; ++t) dco_quantize_row_q8k(x + (size_t)t * hidden, xq + t * xq_row, hidden);
    moe_ctx c = {gate_type, up_type, down_type, n_experts, hidden, inter, top_k, fast_exp, gate_w, up_w, down_w, ids,
                 xq, hq, row_bytes_of(gate_type, hidden), row_bytes_of(up_type, hidden), row_bytes_of(down_type, inter),
                 xq_row, hq_row, h, dn};
    parallel_for((int64_t)total * inter, moe_gate_up, &c);
    for (int i = 0; i < total; ++i) dco_quantize_row_q8k(h + (size_t)i * inter, hq + i * hq_row, inter);
    parallel_for((int64_t)total * hidden, moe_down, &c);
    memset(out, 0, sizeof(float) * (size_t)T * hidden);
    if (T <= 4 && total <= 32) {
        for (int i = 0; i < total; ++i) {
            if (ids[i] < 0 || ids[i] >= n_experts || weights[i] == 0.0f) continue;
            float* dst = out + (size_t)(i / top_k) * hidden;
            const float* src = dn + (size_t)i * hidden;
            for (int d = 0; d < hidden; ++d) dst[d] += weights[i] * src[d];
        }
    } else {
        int32_t* offsets = (int32_t*)malloc(sizeof(int32_t) * ((size_t)n_experts + 1));
        int32_t* tokens = (int32_t*)malloc(sizeof(int32_t) * (size_t)total);
        int32_t* slot_of = (int32_t*)malloc(sizeof(int32_t) * (size_t)total);
        dco_build_reorder_map(ids, T, top_k, n_experts, offsets, tokens, slot_of);
        for (int p = 0; p < offsets[n_experts]; ++p) {
            const int i = slot_of[p];
            float* dst = out + (size_t)tokens[p] * hidden;
            const float* src = dn + (size_t)i * hidden;
            for (int d = 0; d < hidden; ++d) dst[d] += weights[i] * src[d];
        }
        free(offsets);
        free(tokens);
        free(slot_of);
    }
    if (h_out) memcpy(h_out, h, sizeof(float) * (size_t)total * inter);
    free(xq);
    free(hq);
    free(h);
    free(dn);
    return 1;
}

static void dequant_row_typed(int type, const void* row, float* out, int64_t K) {
    if (type == DCO_TYPE_Q4_K) dco_dequantize_row_q4k(row, out, K);
    else if (type == DCO_TYPE_Q6_K) dco_dequantize_row_q6k(row, out, K);
    else if (type == DCO_TYPE_F32) memcpy(out, row, (size_t)K * 4);
}
DCO_API void dco_dequantize_row(int type, const void* row, float* out, int64_t K) {
    dequant_row_typed(type, row, out, K);
}

/* DenseCore's own f32 oracle for the MoE layer: dequantise the selected
 * experts, float dots, std::exp SiLU, weighted sum in assignment order
 * (core/src/backend/cpu_backend_moe_reference.inl:774-846). */
DCO_API int dco_moe_forward_f32ref(int gate_type, int up_type, int down_type, const void* gate_w, const void* up_w,
                                   const void* down_w, int n_experts, int hidden, int inter, const float* x, int T,
                                   int top_k, const int32_t* ids, const float* weights, float* out) {
    const int64_t g_rb = row_bytes_of(gate_type, hidden), u_rb = row_bytes_of(up_type, hidden);
    const int64_t d_rb = row_bytes_of(down_type, inter);
    float* wrow = (float*)malloc(sizeof(float) * (size_t)(hidden > inter ? hidden : inter));
    float* hbuf = (float*)malloc(sizeof(float) * (size_t)inter);
    memset(out, 0, sizeof(float) * (size_t)T * hidden);
    for (int i = 0; i < T * top_k; ++i) {
        const int e = ids[i];
        if (e < 0 || e >= n_experts || weights[i] == 0.0f) continue;
        const float* xin = x + (size_t)(i / top_k) * hidden;
        for (int r = 0; r < inter; ++r) {
            dequant_row_typed(gate_type, (const char*)gate_w + ((int64_t)e * inter + r) * g_rb, wrow, hidden);
            float g = 0.0f;
            for (int k = 0; k < hidden; ++k) g += xin[k] * wrow[k];
            dequant_row_typed(up_type, (const char*)up_w + ((int64_t)e * inter + r) * u_rb, wrow, hidden);
            float u = 0.0f;
            for (int k = 0; k < hidden; ++k) u += xin[k] * wrow[k];
            hbuf[r] = (g / (1.0f + expf(-g))) * u;
        }
        float* dst = out + (size_t)(i / top_k) * hidden;
        for (int r = 0; r < hidden; ++r) {
            dequant_row_typed(down_type, (const char*)down_w + ((int64_t)e * hidden + r) * d_rb, wrow, inter);
            float s = 0.0f;
            for (int k = 0; k < inter; ++k) s += hbuf[k] * wrow[k];
            dst[r] += weights[i] * s;
        }
    }
    free(wrow);
    free(hbuf);
    return 1;
}

/* ------------------------------------------------------ paged KV cache */
/* Arena [layer][block][16 slots][kv_head][head_dim] fp16, separate K and V
 * (core/src/runtime/memory/kv_cache_storage.cpp:146-200).  These helpers work
 * on ONE layer's arena: base + block*16*n_kv*hd. */
DCO_API void dco_kv_write(uint16_t* k_arena, uint16_t* v_arena, const int32_t* block_table, int pos, int n_kv,
                          int head_dim, const float* k, const float* v) {
    const int blk = block_table[pos / KV_BLOCK], slot = pos % KV_BLOCK;
    const size_t off = ((size_t)blk * KV_BLOCK + slot) * n_kv * head_dim;
    for (int i = 0; i < n_kv * head_dim; ++i) {
        k_arena[off + i] = dco_fp32_to_fp16(k[i]);
        v_arena[off + i] = dco_fp32_to_fp16(v[i]);
    }
}

/* Scalar two-pass reference: std::exp, divide by the plain denominator
 * (core/src/llm/attention/paged_exec.cpp:37-223; no window, no soft-cap).
 * One query token at position query_pos attends keys 0..query_pos. */
typedef struct {
    const float* q;
    const uint16_t *k_arena, *v_arena;
    const int32_t* block_table;
    int query_pos, n_head, n_kv, head_dim;
    float scale;
    float* out;
} attn_ctx;
static void attn_scalar_heads(int64_t h_lo, int64_t h_hi, void* p) {
    const attn_ctx* a = (const attn_ctx*)p;
    const float* q = a->q;
    const uint16_t *k_arena = a->k_arena, *v_arena = a->v_arena;
    const int32_t* block_table = a->block_table;
    const int n_head = a->n_head, n_kv = a->n_kv, head_dim = a->head_dim;
    const float scale = a->scale;
    float* out = a->out;
    const int group = n_head / n_kv, ctx = a->query_pos + 1;
    float* scores = (float*)malloc(sizeof(float) * (size_t)ctx);
    for (int h = (int)h_lo; h < (int)h_hi; ++h) {
        const float* qh = q + (size_t)h * head_dim;
        float* oh = out + (size_t)h * head_dim;
        const int kvh = h / group;
        memset(oh, 0, sizeof(float) * (size_t)head_dim);
        float mx = -INFINITY;
        for (int t = 0; t < ctx; ++t) {
            const size_t off = (((size_t)block_table[t / KV_BLOCK] * KV_BLOCK + t % KV_BLOCK) * n_kv + kvh) * head_dim;
            float dot = 0.0f;
            for (int d = 0; d < head_dim; ++d) dot += qh[d] * dco_fp16_to_fp32(k_arena[off + d]);
            scores[t] = dot * scale;
            if (isfinite(scores[t]) && scores[t] > mx) mx = scores[t];
        }
        if (!isfinite(mx)) continue;
        float den = 0.0f;
        for (int t = 0; t < ctx; ++t) {
            if (!isfinite(scores[t])) continue;
            const float w = expf(scores[t] - mx);
            if (!(w > 0.0f) || !isfinite(w)) continue;
            const size_t off = (((size_t)block_table[t / KV_BLOCK] * KV_BLOCK + t % KV_BLOCK) * n_kv + kvh) * head_dim;
            for (int d = 0; d < head_dim; ++d) oh[d] += w * dco_fp16_to_fp32(v_arena[off + d]);
            den += w;
        }
        if (!(den > 0.0f) || !isfinite(den)) {
            memset(oh, 0, sizeof(float) * (size_t)head_dim);
            continue;
        }
        const float inv = 1.0f / den;
        for (int d = 0; d < head_dim; ++d) oh[d] *= inv;
    }
    free(scores);
}
/* Heads are split across threads as the reference splits head tiles
 * (core/src/llm/attention/paged_exec.cpp:552-573). */
DCO_API void dco_paged_attention_scalar(const float* q, const uint16_t* k_arena, const uint16_t* v_arena,
                                        const int32_t* block_table, int query_pos, int n_head, int n_kv,
                                        int head_dim, float scale, float* out) {
    attn_ctx a = {q, k_arena, v_arena, block_table, query_pos, n_head, n_kv, head_dim, scale, out};
    parallel_for(n_head, attn_scalar_heads, &a);
}

/* Production kernel: per 16-token block online softmax with the fast-exp
 * polynomial, final acc * 1/(d + 1e-6)
 * (core/src/kernels/hwy/hwy_paged_attention.cc:428-629). */
static void attn_blockwise_heads(int64_t h_lo, int64_t h_hi, void* p) {
    const attn_ctx* a = (const attn_ctx*)p;
    const float* q = a->q;
    const uint16_t *k_arena = a->k_arena, *v_arena = a->v_arena;
    const int32_t* block_table = a->block_table;
    const int n_head = a->n_head, n_kv = a->n_kv, head_dim = a->head_dim;
    const float scale = a->scale;
    float* out = a->out;
    const int group = n_head / n_kv, ctx = a->query_pos + 1;
    for (int h = (int)h_lo; h < (int)h_hi; ++h) {
        const float* qh = q + (size_t)h * head_dim;
        float* oh = out + (size_t)h * head_dim;
        const int kvh = h / group;
        memset(oh, 0, sizeof(float) * (size_t)head_dim);
        float m_prev = -1e30f, d_prev = 0.0f;
        for (int b0 = 0; b0 < ctx; b0 += KV_BLOCK) {
            const int nt = ctx - b0 < KV_BLOCK ? ctx - b0 : KV_BLOCK;
            float s[KV_BLOCK], m_block = -1e30f;
            const size_t base = (size_t)block_table[b0 / KV_BLOCK] * KV_BLOCK;
            for (int t = 0; t < nt; ++t) {
                const size_t off = ((base + t) * n_kv + kvh) * head_dim;
                float dot = 0.0f;
                for (int d = 0; d < head_dim; ++d) dot += qh[d] * dco_fp16_to_fp32(k_arena[off + d]);
                s[t] = dot * scale;
                if (s[t] > m_block) m_block = s[t];
            }
            const float m_new = m_prev > m_block ? m_prev : m_block;
            const float alpha = dco_fast_exp_fma(m_prev - m_new);
            if (alpha != 1.0f)
                for (int d = 0; d < head_dim; ++d) oh[d] *= alpha;
            float d_block = 0.0f;
            for (int t = 0; t < nt; ++t) {
                s[t] = dco_fast_exp_fma(s[t] - m_new);
                d_block += s[t];
            }
            for (int t = 0; t < nt; ++t) {
                const size_t off = ((base + t) * n_kv + kvh) * head_dim;
                for (int d = 0; d < head_dim; ++d) oh[d] += s[t] * dco_fp16_to_fp32(v_arena[off + d]);
            }
            d_prev = d_prev * alpha + d_block;
            m_prev = m_new;
        }
        if (!(d_prev > 0.0f) || !isfinite(d_prev)) {
            memset(oh, 0, sizeof(float) * (size_t)head_dim);
            continue;
        }
        const float inv = 1.0f / (d_prev + 1e-6f);
        for (int d = 0; d < head_dim; ++d) oh[d] *= inv;
    }
}
DCO_API void dco_paged_attention_blockwise(const float* q, const uint16_t* k_arena, const uint16_t* v_arena,
                                           const int32_t* block_table, int query_pos, int n_head, int n_kv,
                                           int head_dim, float scale, float* out) {
    attn_ctx a = {q, k_arena, v_arena, block_table, query_pos, n_head, n_kv, head_dim, scale, out};
    parallel_for(n_head, attn_blockwise_heads, &a);
}

/* ------------------------------------------------- norm, RoPE, sampling */
/* RMSNorm: y = x / sqrt(mean(x^2) + eps) * w (core/src/llm/graph/decoder.cpp:268;
 * ggml_rms_norm sums squares in double).  w may be NULL. */
DCO_API void dco_rms_norm(const float* x, const float* w, int n, float eps, float* out) {
    double ss = 0.0;
    for (int i = 0; i < n; ++i) ss += (double)x[i] * (double)x[i];
    const float mean = (float)(ss / n);
    const float sc = 1.0f / sqrtf(mean + eps);
    for (int i = 0; i < n; ++i) out[i] = w ? (x[i] * sc) * w[i] : x[i] * sc;
}
/* RoPE on interleaved pairs (x[2i], x[2i+1]) with a cos/sin table
 * (core/src/kernels/hwy/hwy_rope.cc:96-104).  Table entry for (pos, i):
 * cos/sin(pos * theta^(-2i/head_dim)); computed here in double, rounded to f32,
 * the same table is handed to the GPU. */
DCO_API void dco_rope_table(int max_pos, int head_dim, double theta, float* cos_sin /* [max_pos][head_dim] */) {
    for (int p = 0; p < max_pos; ++p)
        for (int i = 0; i < head_dim / 2; ++i) {
            const double a = (double)p * pow(theta, -2.0 * i / head_dim);
            cos_sin[(size_t)p * head_dim + 2 * i] = (float)cos(a);
            cos_sin[(size_t)p * head_dim + 2 * i + 1] = (float)sin(a);
        }
}
DCO_API void dco_rope(float* x, const float* cos_sin_row, int head_dim) {
    for (int d = 0; d + 1 < head_dim; d += 2) {
        const float x0 = x[d], x1 = x[d + 1], c = cos_sin_row[d], s = cos_sin_row[d + 1];
        x[d] = x0 * c - x1 * s;
        x[d + 1] = x0 * s + x1 * c;
    }
}
/* First maximum wins (core/src/sampler/sampler.cpp:42-57). */
DCO_API int dco_argmax(const float* v, int n) {
    if (n <= 0) return -1;
    float best = v[0];
    int bi = 0;
    for (int i = 1; i < n; ++i)
        if (v[i] > best) {
            best = v[i];
            bi = i;
        }
    return bi;
}

/* -------------------------------------------------------- Philox4x32-10 */
/* Counter-based generator of Salmon et al., "Parallel random numbers: as easy
 * as 1, 2, 3" (SC'11); constants from that paper. */
DCO_API void dco_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]) {
    uint32_t c0 = ctr[0], c1 = ctr[1], c2 = ctr[2], c3 = ctr[3], k0 = key[0], k1 = key[1];
    for (int r = 0; r < 10; ++r) {
        const uint64_t p0 = (uint64_t)0xD2511F53u * c0, p1 = (uint64_t)0xCD9E8D57u * c2;
        const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0, n1 = (uint32_t)p1;
        const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1, n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}
/* Uniform in [0,1) with 24 bits: (r >> 8) * 2^-24. */
static inline float u01(uint32_t r) { return (float)(r >> 8) * (1.0f / 16777216.0f); }
/* Uniforms of one verify step: counter = (step, 0, 0, 0), key = seed lo/hi;
 * word j of block i -> uniform 4i+j.  n <= 8. */
DCO_API void dco_verify_uniforms(uint64_t seed, uint32_t step, int n, float* u) {
    const uint32_t key[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
    for (int i = 0; i < n; i += 4) {
        const uint32_t ctr[4] = {step, (uint32_t)(i / 4), 0, 0};
        uint32_t o[4];
        dco_philox4x32_10(ctr, key, o);
        for (int j = 0; j < 4 && i + j < n; ++j) u[i + j] = u01(o[j]);
    }
}

/* ------------------------------------------- deterministic exp / softmax */
/* A fully specified exp used by the verify step so that CPU and GPU produce
 * bit-identical probabilities: for x <= 0, y = x*log2e, i = rint(y),
 * f = y - i in [-0.5, 0.5], result 2^i * P(f) with P the degree-6 Taylor
 * polynomial of 2^f in Horner form with fmaf (relative error ~2e-7).  Only
 * *, fma, rint are used, so it rounds identically on any IEEE-754 machine. */
DCO_API float dco_det_exp(float x) {
    if (x < -87.0f) return 0.0f;
    if (x > 0.0f) x = 0.0f;
    const float y = x * 1.4426950408889634f;
    const float r = rintf(y);
    const float f = y - r;
    float p = 1.5403530e-4f;
    p = fmaf(p, f, 1.3333558e-3f);
    p = fmaf(p, f, 9.6181291e-3f);
    p = fmaf(p, f, 5.5504109e-2f);
    p = fmaf(p, f, 2.4022651e-1f);
    p = fmaf(p, f, 6.9314718e-1f);
    p = fmaf(p, f, 1.0f);
    const int32_t bits = ((int32_t)r + 127) << 23;
    float two_i;
    memcpy(&two_i, &bits, 4);
    return p * two_i;
}

#define DET_LANES 1024
/* Fixed-order float sum: lane j adds elements j, j+1024, ... in index order,
 * then a pairwise tree over the 1024 lanes (stride 512, 256, ... 1). */
static float det_sum(const float* v, int n) {
    float lane[DET_LANES];
    for (int j = 0; j < DET_LANES; ++j) {
        float s = 0.0f;
        for (int i = j; i < n; i += DET_LANES) s += v[i];
        lane[j] = s;
    }
    for (int st = DET_LANES / 2; st > 0; st >>= 1)
        for (int j = 0; j < st; ++j) lane[j] += lane[j + st];
    return lane[0];
}
/* Temperature softmax following core/src/sampler/sampler.cpp:235-262
 * (v = logit * (1/T); subtract max; exp; * 1/sum) with the deterministic exp
 * and sum above. */
DCO_API void dco_det_softmax(const float* logits, int n, float temperature, float* p) {
    const float inv_t = 1.0f / temperature;
    float mx = -INFINITY;
    for (int i = 0; i < n; ++i) {
        const float v = logits[i] * inv_t;
        if (v > mx) mx = v;
    }
    for (int i = 0; i < n; ++i) p[i] = dco_det_exp(logits[i] * inv_t - mx);
    const float inv = 1.0f / det_sum(p, n);
    for (int i = 0; i < n; ++i) p[i] *= inv;
}

/* The sampler's own temperature softmax, step for step (core/src/sampler/sampler.cpp:235-262):
 * v = logit * (1/T) with T clamped as ClampTemperature does (:21-26), running maximum of v,
 * e = exp(v - max) with the C library's expf, sum in index order, then * (1/sum). */
DCO_API void dco_softmax_temperature(const float* logits, int n, float temperature, float* p) {
    if (!(temperature > 0.0f)) temperature = 1.0f;
    if (temperature < 1e-6f) temperature = 1e-6f;
    const float inv_t = 1.0f / temperature;
    float mx = -INFINITY;
    for (int i = 0; i < n; ++i) {
        const float v = logits[i] * inv_t;
        if (v > mx) mx = v;
    }
    float sum = 0.0f;
    for (int i = 0; i < n; ++i) {
        const float v = logits[i] * inv_t;
        p[i] = expf(v - mx);
        sum += p[i];
    }
    const float inv = 1.0f / sum;
    for (int i = 0; i < n; ++i) p[i] *= inv;
}

/* Inverse CDF in index order over non-negative weights w (not normalised).
 * Sums have a fixed shape: a "run" is 32 consecutive elements added in index
 * order starting from 0; a chunk sum adds its 32 run sums in order; the total
 * adds the chunk sums in order.  target = u * total.  The search walks chunks,
 * then runs, then elements, and returns the first index i with
 * base + prefix_i > target, where base is the accumulated sum of the chunks and
 * runs before and prefix_i the in-run partial sum.  Returns -1 if total <= 0. */
static float run32_sum(const float* w, int lo, int hi) {
    float s = 0.0f;
    for (int i = lo; i < hi; ++i) s += w[i];
    return s;
}
static float chunk_sum(const float* w, int lo, int hi) {
    float s = 0.0f;
    for (int r = lo; r < hi; r += 32) s += run32_sum(w, r, r + 32 < hi ? r + 32 : hi);
    return s;
}
DCO_API int dco_det_inverse_cdf(const float* w, int n, float u) {
    float total = 0.0f;
    for (int c = 0; c < n; c += 1024) total += chunk_sum(w, c, c + 1024 < n ? c + 1024 : n);
    if (!(total > 0.0f)) return -1;
    const float target = u * total;
    float base = 0.0f;
    int last_pos = -1;
    for (int c = 0; c < n; c += 1024) {
        const int hi = c + 1024 < n ? c + 1024 : n;
        const float cs = chunk_sum(w, c, hi);
        if (!(base + cs > target)) {
            base += cs;
            continue;
        }
        float cbase = base;
        for (int r = c; r < hi; r += 32) {
            const int rh = r + 32 < hi ? r + 32 : hi;
            const float rs = run32_sum(w, r, rh);
            if (cbase + rs > target) {
                float prefix = 0.0f;
                for (int i = r; i < rh; ++i) {
                    prefix += w[i];
                    if (cbase + prefix > target) return i;
                }
            }
            cbase += rs;
        }
        base += cs;
    }
    for (int i = 0; i < n; ++i)
        if (w[i] > 0.0f) last_pos = i;
    return last_pos;
}

/* ------------------------------------------------ speculative verify */
/* Standard draft-verify rule (Leviathan et al. 2023; Chen et al. 2023);
 * DenseCore has no implementation (core/src/runtime/engine.cpp:593-645 only
 * loads a draft model).  target_logits: [gamma+1][vocab].  draft_tokens:
 * gamma.  Greedy (mode 0): accept the longest prefix with
 * argmax(target_{i}) == draft_{i}; next token = argmax(target_{n_acc}).
 * Stochastic (mode 1): p_i = softmax(target_i / T); accept draft_i iff
 * u_i * q_i[draft_i] < p_i[draft_i]; on the first rejection sample from
 * max(0, p_i - q_i) by inverse CDF with u[gamma]; if all accepted sample the
 * bonus token from p_gamma with u[gamma].  draft_probs: [gamma][vocab].
 * out_tokens: n_accepted draft tokens followed by the next token. */
DCO_API int dco_verify_accept(const float* target_logits, const int32_t* draft_tokens, const float* draft_probs,
                              const float* u, int gamma, int vocab, int mode, float temperature,
                              int32_t* n_accepted, int32_t* next_token) {
    if (mode == 0) {
        int n = 0;
        while (n < gamma && dco_argmax(target_logits + (size_t)n * vocab, vocab) == draft_tokens[n]) ++n;
        *n_accepted = n;
        *next_token = dco_argmax(target_logits + (size_t)n * vocab, vocab);
        return 1;
    }
    float* p = (float*)malloc(sizeof(float) * (size_t)vocab);
    int n = 0;
    for (; n < gamma; ++n) {
        dco_det_softmax(target_logits + (size_t)n * vocab, vocab, temperature, p);
        const int t = draft_tokens[n];
        const float q = draft_probs[(size_t)n * vocab + t];
        if (u[n] * q < p[t]) continue;
        for (int i = 0; i < vocab; ++i) {
            const float r = p[i] - draft_probs[(size_t)n * vocab + i];
            p[i] = r > 0.0f ? r : 0.0f;
        }
        *n_accepted = n;
        *next_token = dco_det_inverse_cdf(p, vocab, u[gamma]);
        if (*next_token < 0) { /* p == q everywhere: sample from p itself */
            dco_det_softmax(target_logits + (size_t)n * vocab, vocab, temperature, p);
            *next_token = dco_det_inverse_cdf(p, vocab, u[gamma]);
        }
        free(p);
        return 1;
    }
    dco_det_softmax(target_logits + (size_t)gamma * vocab, vocab, temperature, p);
    *n_accepted = gamma;
    *next_token = dco_det_inverse_cdf(p, vocab, u[gamma]);
    free(p);
    return 1;
}

/* ------------------------------------- synthetic weights and quantisers */
/* ggml's K-quant weight quantiser is not in the DenseCore tree; any valid block
 * encoding is a legal input to the dot kernels.  These are this project's own
 * simple min/max quantisers, written so that CPU and GPU produce the same
 * bytes: every float step is a single correctly rounded operation. */

/* Approximately normal value from one Philox block: the eight 16-bit halves
 * are summed (Irwin-Hall, n=8), centred and scaled to unit variance, then
 * multiplied by sigma and rounded through fp16 ("fp16 master weights"). */
static inline float synth_normal(uint64_t seed, uint64_t index, float sigma) {
    const uint32_t key[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
    const uint32_t ctr[4] = {(uint32_t)index, (uint32_t)(index >> 32), 0x5eedu, 0};
    uint32_t o[4];
    dco_philox4x32_10(ctr, key, o);
    int32_t s = 0;
    for (int j = 0; j < 4; ++j) s += (int32_t)(o[j] & 0xFFFFu) + (int32_t)(o[j] >> 16);
    /* mean 8*32767.5 = 262140, std 65536*sqrt(8/12) = 53509.9 */
    const float z = (float)(s - 262140) * (1.0f / 53509.9f);
    return dco_fp16_to_fp32(dco_fp32_to_fp16(z * sigma));
}
DCO_API void dco_synth_normal(uint64_t seed, uint64_t first_index, int64_t n, float sigma, float* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = synth_normal(seed, first_index + (uint64_t)i, sigma);
}

static inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* Q4_K: per 32-sub-block min/max -> (scale, min); super-block d = max scale/63,
 * dmin = max min/63 in fp16; 6-bit codes; q = rne((x + dmin*m) / (d*sc)). */
DCO_API void dco_quantize_block_q4k(const float x[256], void* out) {
    blk_q4k* b = (blk_q4k*)out;
    float sc[8], mn[8], max_sc = 0.0f, max_mn = 0.0f;
    for (int s = 0; s < 8; ++s) {
        float lo = 0.0f, hi = 0.0f;
        for (int l = 0; l < 32; ++l) {
            const float v = x[32 * s + l];
            lo = v < lo ? v : lo;
            hi = v > hi ? v : hi;
        }
        sc[s] = (hi - lo) / 15.0f;
        mn[s] = -lo;
        max_sc = sc[s] > max_sc ? sc[s] : max_sc;
        max_mn = mn[s] > max_mn ? mn[s] : max_mn;
    }
    b->d = dco_fp32_to_fp16(max_sc / 63.0f);
    b->dmin = dco_fp32_to_fp16(max_mn / 63.0f);
    const float d = dco_fp16_to_fp32(b->d), dmin = dco_fp16_to_fp32(b->dmin);
    uint8_t ls[8], lm[8];
    for (int s = 0; s < 8; ++s) {
        ls[s] = (uint8_t)(d > 0.0f ? clampi((int)rintf(sc[s] / d), 0, 63) : 0);
        lm[s] = (uint8_t)(dmin > 0.0f ? clampi((int)rintf(mn[s] / dmin), 0, 63) : 0);
    }
    /* inverse of the 12-byte packing decoded by dco_q4k_decode_scales */
    for (int j = 0; j < 4; ++j) {
        b->scales[j] = (uint8_t)((ls[j] & 63) | ((ls[j + 4] >> 4) << 6));
        b->scales[j + 4] = (uint8_t)((lm[j] & 63) | ((lm[j + 4] >> 4) << 6));
        b->scales[j + 8] = (uint8_t)((ls[j + 4] & 0xF) | ((lm[j + 4] & 0xF) << 4));
    }
    for (int c = 0; c < 4; ++c) {
        const float d1 = d * (float)ls[2 * c], m1 = dmin * (float)lm[2 * c];
        const float d2 = d * (float)ls[2 * c + 1], m2 = dmin * (float)lm[2 * c + 1];
        for (int l = 0; l < 32; ++l) {
            const float a = x[64 * c + l] + m1, bb = x[64 * c + 32 + l] + m2;
            const int q1 = d1 > 0.0f ? clampi((int)rintf(a / d1), 0, 15) : 0;
            const int q2 = d2 > 0.0f ? clampi((int)rintf(bb / d2), 0, 15) : 0;
            b->qs[32 * c + l] = (uint8_t)(q1 | (q2 << 4));
        }
    }
}

/* Q6_K: per 16-sub-block scale = amax/31; d = max scale/127 in fp16; int8 codes;
 * q = rne(x / (d*sc)) in [-32, 31]. */
DCO_API void dco_quantize_block_q6k(const float x[256], void* out) {
    blk_q6k* b = (blk_q6k*)out;
    float sc[16], max_sc = 0.0f;
    for (int g = 0; g < 16; ++g) {
        float am = 0.0f;
        for (int l = 0; l < 16; ++l) {
            const float a = fabsf(x[16 * g + l]);
            am = a > am ? a : am;
        }
        sc[g] = am / 31.0f;
        max_sc = sc[g] > max_sc ? sc[g] : max_sc;
    }
    b->d = dco_fp32_to_fp16(max_sc / 127.0f);
    const float d = dco_fp16_to_fp32(b->d);
    int8_t q[256];
    for (int g = 0; g < 16; ++g) {
        const int s = d > 0.0f ? clampi((int)rintf(sc[g] / d), 0, 127) : 0;
        b->scales[g] = (int8_t)s;
        const float ds = d * (float)s;
        for (int l = 0; l < 16; ++l)
            q[16 * g + l] = (int8_t)(ds > 0.0f ? clampi((int)rintf(x[16 * g + l] / ds), -32, 31) : 0);
    }
    memset(b->ql, 0, 128);
    memset(b->qh, 0, 64);
    for (int j = 0; j < 2; ++j)
        for (int l = 0; l < 32; ++l) {
            const int u0 = q[128 * j + l] + 32, u1 = q[128 * j + 32 + l] + 32;
            const int u2 = q[128 * j + 64 + l] + 32, u3 = q[128 * j + 96 + l] + 32;
            b->ql[64 * j + l] = (uint8_t)((u0 & 15) | ((u2 & 15) << 4));
            b->ql[64 * j + 32 + l] = (uint8_t)((u1 & 15) | ((u3 & 15) << 4));
            b->qh[32 * j + l] = (uint8_t)((u0 >> 4) | ((u1 >> 4) << 2) | ((u2 >> 4) << 4) | ((u3 >> 4) << 6));
        }
}

/* Synthetic quantised tensor: element i of the tensor is
 * synth_normal(seed, i, sigma); rows of K, N rows. */
typedef struct {
    int type;
    uint64_t seed;
    float sigma;
    char* out;
} synth_ctx;
static void synth_blocks(int64_t lo, int64_t hi, void* p) {
    const synth_ctx* c = (const synth_ctx*)p;
    const int bs = c->type == DCO_TYPE_Q4_K ? 144 : 210;
    for (int64_t b = lo; b < hi; ++b) {
        float x[256];
        for (int i = 0; i < 256; ++i) x[i] = synth_normal(c->seed, (uint64_t)(b * 256 + i), c->sigma);
        if (c->type == DCO_TYPE_Q4_K) dco_quantize_block_q4k(x, c->out + b * bs);
        else dco_quantize_block_q6k(x, c->out + b * bs);
    }
}
DCO_API void dco_synth_quantized(int type, uint64_t seed, int64_t N, int64_t K, float sigma, void* out) {
    synth_ctx c = {type, seed, sigma, (char*)out};
    parallel_for(N * K / QK_K, synth_blocks, &c);
}
