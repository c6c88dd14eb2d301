// Drives the three ggml-shaped callbacks of include/dc_ggml_compat.h the way ggml's executor would: fake
// GGML_OP_CUSTOM nodes, every callback entered from nth = 4 host threads, results compared with the CPU
// oracle (test infrastructure), and the fail-closed contract checked on bad nodes.
// Prints one line per check and "ALL PASS" at the end; exit code 0 only then.
#include <fcntl.h>
#include <unistd.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <string>
#include <thread>
#include <vector>

#include "dc_ggml_compat.h"

extern "C" {
int dco_mul_mat(int type, const void* W, int64_t N, int64_t K, const float* x, int64_t M, float* y, void* q8_scratch);
void dco_synth_quantized(int type, uint64_t seed, int64_t N, int64_t K, float sigma, void* out);
void dco_synth_normal(uint64_t seed, uint64_t first_index, int64_t n, float sigma, float* out);
int64_t dco_row_bytes(int type, int64_t K);
int dco_route_stable_topk(const float* logits, int T, int n_experts, int top_k, float scale, int32_t* ids, float* weights);
int dco_moe_forward(int gate_type, int up_type, int down_type, const void* gate_w, const void* up_w, const void* down_w,
                    int n_experts, int hidden, int inter, const float* x, int T, int top_k, const int32_t* ids,
                    const float* weights, int fast_exp, float* out, float* h_out);
void dco_kv_write(uint16_t* k_arena, uint16_t* v_arena, const int32_t* block_table, int pos, int n_kv, int head_dim,
                  const float* k, const float* v);
void dco_paged_attention_blockwise(const float* q, const uint16_t* k_arena, const uint16_t* v_arena, const int32_t* block_table,
                                   int query_pos, int n_head, int n_kv, int head_dim, float scale, float* out);
void dco_set_threads(int n);
}

static int g_failures = 0;
static void check(bool ok, const std::string& what) {
    printf("%s  %s\n", ok ? "ok  " : "FAIL", what.c_str());
    if (!ok) ++g_failures;
}

static ggml_tensor tensor_f32(float* data, int64_t n0, int64_t n1 = 1, int64_t n2 = 1) {
    ggml_tensor t;
    memset(&t, 0, sizeof(t));
    t.type = GGML_TYPE_F32;
    t.ne[0] = n0, t.ne[1] = n1, t.ne[2] = n2, t.ne[3] = 1;
    t.nb[0] = 4, t.nb[1] = 4 * n0, t.nb[2] = 4 * n0 * n1, t.nb[3] = 4 * n0 * n1 * n2;
    t.data = data;
    return t;
}

// The executor's fan-out: nth threads enter the callback with ith = 0..nth-1.
static void run_threads(int nth, const std::function<void(int, int)>& cb) {
    std::vector<std::thread> th;
    for (int i = 0; i < nth; ++i) th.emplace_back(cb, i, nth);
    for (auto& t : th) t.join();
}

// Runs f with stderr redirected to a file; returns how many lines holding "CRITICAL" it wrote.
static int critical_lines(const std::function<void()>& f) {
    char path[] = "/tmp/dc_shims_stderr_XXXXXX";
    const int fd = mkstemp(path);
    fflush(stderr);
    const int saved = dup(2);
    dup2(fd, 2);
    f();
    fflush(stderr);
    dup2(saved, 2);
    close(saved);
    lseek(fd, 0, SEEK_SET);
    std::string all;
    char buf[4096];
    ssize_t n;
    while ((n = read(fd, buf, sizeof(buf))) > 0) all.append(buf, (size_t)n);
    close(fd);
    unlink(path);
    int lines = 0;
    for (size_t p = all.find("CRITICAL"); p != std::string::npos; p = all.find("CRITICAL", p + 1)) ++lines;
    return lines;
}

static float max_rel(const std::vector<float>& a, const std::vector<float>& b) {
    float d = 0, m = 0;
    for (size_t i = 0; i < a.size(); ++i) {
        d = fmaxf(d, fabsf(a[i] - b[i]));
        m = fmaxf(m, fabsf(b[i]));
    }
    return d / (m + 1e-30f);
}

static bool all_equal(const std::vector<float>& a, float v) {
    for (float x : a)
        if (x != v) return false;
    return true;
}

static void test_gemv(dc_ctx* ctx) {
    for (int type : {(int)GGML_TYPE_Q4_K, (int)GGML_TYPE_Q6_K}) {
        for (int M : {1, 5, 19, 70}) {       // 70 rows: the tensor-core kernel (a whole 64-token tile and a ragged one)
            const int64_t n_in = 2048, k_out = 1024;
            std::vector<uint8_t> w((size_t)(k_out * dco_row_bytes(type, n_in)));
            dco_synth_quantized(type, 77 + type, k_out, n_in, 0.02f, w.data());
            std::vector<float> x((size_t)(n_in * M)), y((size_t)(k_out * M), 7.0f), want((size_t)(k_out * M));
            dco_synth_normal(5, 0, n_in * M, 1.0f, x.data());
            ggml_tensor tw;
            memset(&tw, 0, sizeof(tw));
            tw.type = (ggml_type)type;
            tw.ne[0] = n_in, tw.ne[1] = k_out, tw.ne[2] = tw.ne[3] = 1;
            tw.data = w.data();
            ggml_tensor tx = tensor_f32(x.data(), n_in, M), ty = tensor_f32(y.data(), k_out, M);
            ty.src[0] = &tx, ty.src[1] = &tw;
            dc_b200_gemv_userdata ud = {ctx, nullptr};
            // threads other than 0 must leave the result alone
            run_threads(3, [&](int ith, int) { cb_gemv_b200(&ty, ith + 1, 4, &ud); });
            check(all_equal(y, 7.0f), "gemv: threads with ith != 0 write nothing");
            run_threads(4, [&](int ith, int nth) { cb_gemv_b200(&ty, ith, nth, &ud); });
            dco_mul_mat(type, w.data(), k_out, n_in, x.data(), M, want.data(), nullptr);
            // the tensor-core kernel adds one float term per Q6_K block where the CPU kernel keeps eight lane partials:
            // equal integers, a different float order
            const bool exact = !(M >= 32 && type == (int)GGML_TYPE_Q6_K);
            check(exact ? memcmp(y.data(), want.data(), y.size() * 4) == 0 : max_rel(y, want) < 2e-6f,
                  "gemv type " + std::to_string(type) + " M=" + std::to_string(M) + (exact ? ": bit-equal to the CPU kernel" : ": 2e-6 of the CPU kernel"));
            check(ud.weight != nullptr, "gemv: the weight was uploaded once and kept in the userdata");
            // second call reuses the handle
            dc_weight* kept = ud.weight;
            std::fill(y.begin(), y.end(), 3.0f);
            run_threads(4, [&](int ith, int nth) { cb_gemv_b200(&ty, ith, nth, &ud); });
            check(ud.weight == kept && (exact ? memcmp(y.data(), want.data(), y.size() * 4) == 0 : max_rel(y, want) < 2e-6f),
                  "gemv: second call, same handle, same result");
            // wrong output size: zero-fill, one CRITICAL line, one count
            ggml_tensor bad = ty;
            bad.ne[0] = k_out - 256;
            std::fill(y.begin(), y.end(), 3.0f);
            const uint64_t before = dc_b200_shim_fail_closed_count();
            const int lines = critical_lines([&] { run_threads(4, [&](int ith, int nth) { cb_gemv_b200(&bad, ith, nth, &ud); }); });
            bool zero = true;
            for (int64_t i = 0; i < (k_out - 256) * M; ++i) zero &= y[(size_t)i] == 0.0f;
            check(zero && lines == 1 && dc_b200_shim_fail_closed_count() == before + 1,
                  "gemv: output sized wrongly -> zero-filled, one CRITICAL line (" + std::to_string(lines) + ")");
            dc_b200_free_weight(ctx, ud.weight);
        }
    }
}

static void test_moe(dc_ctx* ctx) {
    const int E = 16, H = 512, F = 256, k = 4;
    std::vector<uint8_t> g((size_t)(E * F * dco_row_bytes(12, H))), u(g.size()), d((size_t)(E * H * dco_row_bytes(14, F)));
    dco_synth_quantized(12, 1, (int64_t)E * F, H, 0.05f, g.data());
    dco_synth_quantized(12, 2, (int64_t)E * F, H, 0.05f, u.data());
    dco_synth_quantized(14, 3, (int64_t)E * H, F, 0.05f, d.data());
    dc_weight *wg = nullptr, *wu = nullptr, *wd = nullptr;
    const int64_t ne_gu[4] = {H, F, E, 1}, ne_d[4] = {F, H, E, 1};
    dc_b200_upload_weight(ctx, 12, ne_gu, g.data(), &wg);
    dc_b200_upload_weight(ctx, 12, ne_gu, u.data(), &wu);
    dc_b200_upload_weight(ctx, 14, ne_d, d.data(), &wd);
    for (int T : {1, 3, 21}) {
        std::vector<float> x((size_t)T * H), lg((size_t)T * E), y((size_t)T * H, 7.0f), want((size_t)T * H), wts((size_t)T * k);
        std::vector<int32_t> ids((size_t)T * k);
        dco_synth_normal(11, 0, (int64_t)T * H, 1.0f, x.data());
        dco_synth_normal(12, 0, (int64_t)T * E, 2.0f, lg.data());
        ggml_tensor tx = tensor_f32(x.data(), H, T), tl = tensor_f32(lg.data(), E, T), ty = tensor_f32(y.data(), H, T);
        dc_b200_moe_userdata ud = {ctx, wg, wu, wd, k, 0.0f};
        run_threads(4, [&](int ith, int nth) { cb_moe_forward_b200(&ty, &tx, &tl, ith, nth, &ud); });
        dco_route_stable_topk(lg.data(), T, E, k, 1.0f, ids.data(), wts.data());
        dco_moe_forward(12, 12, 14, g.data(), u.data(), d.data(), E, H, F, x.data(), T, k, ids.data(), wts.data(), 1, want.data(), nullptr);
        const float r = max_rel(y, want);
        check(r < 1e-5f, "moe T=" + std::to_string(T) + ": max rel " + std::to_string(r) + " vs the CPU layer");
        // logits of another token count: zero-fill, one line
        ggml_tensor bad = tl;
        bad.ne[1] = T + 1;
        std::fill(y.begin(), y.end(), 3.0f);
        int lines = critical_lines([&] { run_threads(4, [&](int ith, int nth) { cb_moe_forward_b200(&ty, &tx, &bad, ith, nth, &ud); }); });
        check(all_equal(y, 0.0f) && lines == 1, "moe: logits of another token count -> zero-filled, one CRITICAL line");
        // a failure inside the library (top-k larger than the experts): still one line, zero result
        dc_b200_moe_userdata ud_bad = {ctx, wg, wu, wd, E + 1, 0.0f};
        std::fill(y.begin(), y.end(), 3.0f);
        lines = critical_lines([&] { run_threads(4, [&](int ith, int nth) { cb_moe_forward_b200(&ty, &tx, &tl, ith, nth, &ud_bad); }); });
        check(all_equal(y, 0.0f) && lines == 1, "moe: top-k beyond the expert count -> zero-filled, one CRITICAL line (" + std::to_string(lines) + ")");
    }
    dc_b200_free_weight(ctx, wg);
    dc_b200_free_weight(ctx, wu);
    dc_b200_free_weight(ctx, wd);
}

static void test_attention(dc_ctx* ctx) {
    const int n_head = 8, n_kv = 2, hd = 128, layer = 1, n_layer = 2, max_blocks = 64, bps = 16;
    dc_kv_cache* kv = nullptr;
    check(dc_b200_kv_create(ctx, n_layer, n_kv, hd, max_blocks, 2, bps, &kv) == DC_B200_OK, "attention: cache created");
    int seq = -1;
    dc_b200_kv_seq_alloc(kv, &seq);
    const int total = 75;
    dc_b200_kv_seq_reserve(kv, seq, total);
    std::vector<int32_t> table(bps);
    int nb = 0;
    dc_b200_kv_block_table(kv, seq, table.data(), bps, &nb);
    std::vector<uint16_t> ka((size_t)max_blocks * 16 * n_kv * hd, 0), va(ka.size(), 0);
    const float scale = 1.0f / sqrtf((float)hd);
    int pos = 0;
    float worst = 0;
    // single tokens, then chunks of 3, 16 and 21 (the last one crosses the library's 16-token limit)
    for (int T : {1, 1, 1, 3, 16, 21, 1}) {
        std::vector<float> q((size_t)T * n_head * hd), k((size_t)T * n_kv * hd), v(k.size()), out(q.size(), 7.0f), want(q.size());
        dco_synth_normal(100 + pos, 0, (int64_t)q.size(), 1.0f, q.data());
        dco_synth_normal(200 + pos, 0, (int64_t)k.size(), 1.0f, k.data());
        dco_synth_normal(300 + pos, 0, (int64_t)v.size(), 1.0f, v.data());
        std::vector<int32_t> sid(T, seq), p(T);
        for (int t = 0; t < T; ++t) p[t] = pos + t;
        ggml_tensor tq = tensor_f32(q.data(), hd, n_head, T), tk = tensor_f32(k.data(), hd, n_kv, T),
                    tv = tensor_f32(v.data(), hd, n_kv, T), to = tensor_f32(out.data(), hd, n_head, T);
        to.src[0] = &tq, to.src[1] = &tk, to.src[2] = &tv;
        dc_b200_attn_userdata ud = {ctx, kv, layer, n_head, n_kv, hd, 0.0f, sid.data(), p.data()};
        run_threads(4, [&](int ith, int nth) { cb_paged_attention_decode_b200(&to, ith, nth, &ud); });
        for (int t = 0; t < T; ++t) {
            dco_kv_write(ka.data(), va.data(), table.data(), pos + t, n_kv, hd, k.data() + (size_t)t * n_kv * hd, v.data() + (size_t)t * n_kv * hd);
            dco_paged_attention_blockwise(q.data() + (size_t)t * n_head * hd, ka.data(), va.data(), table.data(), pos + t, n_head, n_kv, hd,
                                          scale, want.data() + (size_t)t * n_head * hd);
        }
        worst = fmaxf(worst, max_rel(out, want));
        if (T == 21) {
            // a node whose q has another head count: zero-filled, one line
            ggml_tensor badq = tq;
            badq.ne[1] = n_head / 2;
            ggml_tensor to2 = to;
            to2.src[0] = &badq;
            std::fill(out.begin(), out.end(), 3.0f);
            const int lines = critical_lines([&] { run_threads(4, [&](int ith, int nth) { cb_paged_attention_decode_b200(&to2, ith, nth, &ud); }); });
            check(all_equal(out, 0.0f) && lines == 1, "attention: q of another head count -> zero-filled, one CRITICAL line");
        }
        pos += T;
    }
    check(worst < 1e-5f, "attention over " + std::to_string(pos) + " positions: max rel " + std::to_string(worst) + " vs the CPU kernel");
    dc_b200_kv_destroy(kv);
}

int main() {
    dc_ctx* ctx = nullptr;
    if (dc_b200_init(0, &ctx) != DC_B200_OK) {
        printf("FAIL  no device context\n");
        return 2;
    }
    dco_set_threads(4);
    test_gemv(ctx);
    test_moe(ctx);
    test_attention(ctx);
    dc_b200_destroy(ctx);
    if (g_failures == 0) printf("ALL PASS\n");
    return g_failures == 0 ? 0 : 1;
}
