// GGUF file -> model on the device.  The file is mapped read-only; metadata gives the
// decoder's shape, every tensor the decoder names is uploaded with its bytes as they lie in
// the file (144-byte Q4_K and 210-byte Q6_K super-blocks stay native, F32 vectors as they
// are).  This is the loader's side of DenseCore's model_loader.cpp:2037-2830 (metadata keys
// "<arch>.block_count", ".embedding_length", ".attention.head_count[_kv]",
// ".attention.layer_norm_rms_epsilon" :2664, ".rope.freq_base" :2679, ".expert_count",
// ".expert_used_count" :2815-2829) for the one model family this library runs (Qwen3-style
// decoders, dense or MoE); the reference goes through ggml's gguf_* API, which is restated
// here from the published GGUF v2/v3 layout because ggml is not part of this library.
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <map>
#include <string>
#include <vector>

#include "dc_common.cuh"
#include "dc_internal.h"
#include "dc_model.h"

namespace {

enum GgufType { U8, I8, U16, I16, U32, I32, F32, BOOL, STR, ARR, U64, I64, F64 };
const size_t kScalarSize[13] = {1, 1, 2, 2, 4, 4, 4, 1, 0, 0, 8, 8, 8};

struct Cursor {
    const uint8_t* p;
    const uint8_t* end;
    bool ok = true;
    bool need(size_t n) {
        if (!ok || (size_t)(end - p) < n) ok = false;
        return ok;
    }
    template <typename T>
    T get() {
        T v{};
        if (need(sizeof(T))) {
            memcpy(&v, p, sizeof(T));
            p += sizeof(T);
        }
        return v;
    }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        if (n > (1u << 20) || !need((size_t)n)) {
            ok = false;
            return {};
        }
        std::string s((const char*)p, (size_t)n);
        p += n;
        return s;
    }
};

struct Meta {
    std::map<std::string, double> num;
    std::map<std::string, std::string> str;
};

struct TensorInfo {
    int type = 0;
    int64_t ne[4] = {1, 1, 1, 1};
    uint64_t offset = 0;
};

// Skips or records one metadata value.
bool read_value(Cursor& c, uint32_t type, const std::string& key, Meta& meta, int depth = 0) {
    if (type > F64) return c.ok = false;
    if (type == STR) {
        std::string s = c.str();
        if (depth == 0) meta.str[key] = s;
        return c.ok;
    }
    if (type == ARR) {
        const uint32_t et = c.get<uint32_t>();
        const uint64_t n = c.get<uint64_t>();
        if (!c.ok || et > F64 || et == ARR) return c.ok = false;
        if (et == STR) {
            for (uint64_t i = 0; i < n && c.ok; ++i) {
                const uint64_t len = c.get<uint64_t>();
                if (!c.need((size_t)len)) return false;
                c.p += len;
            }
            return c.ok;
        }
        const size_t bytes = (size_t)n * kScalarSize[et];
        if (n > (1ull << 32) || !c.need(bytes)) return c.ok = false;
        c.p += bytes;
        return true;
    }
    double v = 0.0;
    switch (type) {
        case U8: v = c.get<uint8_t>(); break;
        case I8: v = c.get<int8_t>(); break;
        case U16: v = c.get<uint16_t>(); break;
        case I16: v = c.get<int16_t>(); break;
        case U32: v = c.get<uint32_t>(); break;
        case I32: v = c.get<int32_t>(); break;
        case F32: v = c.get<float>(); break;
        case BOOL: v = c.get<uint8_t>() ? 1.0 : 0.0; break;
        case U64: v = (double)c.get<uint64_t>(); break;
        case I64: v = (double)c.get<int64_t>(); break;
        case F64: v = c.get<double>(); break;
        default: break;
    }
    if (depth == 0) meta.num[key] = v;
    return c.ok;
}

size_t tensor_bytes(int type, const int64_t ne[4]) {
    const int64_t rows = ne[1] * ne[2] * ne[3];
    switch (type) {
        case DC_TYPE_F32: return (size_t)(ne[0] * rows * 4);
        case DC_TYPE_F16: return (size_t)(ne[0] * rows * 2);
        case DC_TYPE_Q4_K: return (size_t)(ne[0] / DC_QK_K * DC_Q4K_BYTES * rows);
        case DC_TYPE_Q6_K: return (size_t)(ne[0] / DC_QK_K * DC_Q6K_BYTES * rows);
        default: return 0;
    }
}

struct Mapping {
    int fd = -1;
    const uint8_t* base = nullptr;
    size_t size = 0;
    ~Mapping() {
        if (base) munmap((void*)base, size);
        if (fd >= 0) close(fd);
    }
};

}  // namespace

extern "C" int dc_b200_model_from_gguf(dc_ctx* ctx, const char* path, int max_seqs, int max_ctx, int ep_rank, int ep_size,
                                       dc_model** out_model) {
    if (!ctx || !path || !out_model) return DC_B200_INVALID_ARGUMENT;
    *out_model = nullptr;
    Mapping map;
    map.fd = open(path, O_RDONLY);
    if (map.fd < 0) return dc_fail(ctx, DC_B200_MODEL_LOAD_FAILED, "gguf: cannot open '%s'", path);
    struct stat st;
    if (fstat(map.fd, &st) != 0 || st.st_size < 24) return dc_fail(ctx, DC_B200_MODEL_LOAD_FAILED, "gguf: '%s' is too short", path);
    map.size = (size_t)st.st_size;
    void* mm = mmap(nullptr, map.size, PROT_READ, MAP_PRIVATE, map.fd, 0);
    if (mm == MAP_FAILED) return dc_fail(ctx, DC_B200_MODEL_LOAD_FAILED, "gguf: cannot map '%s'", path);
    map.base = (const uint8_t*)mm;

    Cursor c{map.base, map.base + map.size};
    const uint32_t magic = c.get<uint32_t>(), version = c.get<uint32_t>();
    if (magic != 0x46554747u) return dc_fail(ctx, DC_B200_MODEL_LOAD_FAILED, "gguf: '%s' is not a GGUF file", path);
    if (version < 2 || version > 3) return dc_fail(ctx, DC_B200_UNSUPPORTED, "gguf: version %u is not supported (2 and 3 are)", version);
    const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
    if (!c.ok || n_tensors > (1u << 20) || n_kv > (1u << 20)) return dc_fail(ctx, DC_B200_MODEL_LOAD_FAILED, "gguf: bad header");
    Meta meta;
    for (uint64_t i = 0; i < n_kv; ++i) {
        const std::string key = c.str();
        const uint32_t type = c.get<uint32_t>();
        if (!c.ok || !read_value(c, type, key, meta))
            return dc_fail(ctx, DC_B200_MODEL_LOAD_FAILED, "gguf: metadata entry %llu ('%s') is malformed", (unsigned long long)i, key.c_str());
    }
    std::map<std::string, TensorInfo> tensors;
    for (uint64_t i = 0; i < n_tensors; ++i) {
        const std::string name = c.str();
        const uint32_t nd = c.get<uint32_t>();
        if (!c.ok || nd > 4) return dc_fail(ctx, DC_B200_MODEL_LOAD_FAILED, "gguf: tensor %llu is malformed", (unsigned long long)i);
        TensorInfo t;
        for (uint32_t d = 0; d < nd; ++d) t.ne[d] = (int64_t)c.get<uint64_t>();
        t.type = (int)c.get<uint32_t>();
        t.offset = c.get<uint64_t>();
        if (!c.ok) return dc_fail(ctx, DC_B200_MODEL_LOAD_FAILED, "gguf: tensor '%s' is malformed", name.c_str());
        tensors[name] = t;
    }
    uint64_t align = 32;
    if (meta.num.count("general.alignment")) align = (uint64_t)meta.num["general.alignment"];
    if (align == 0 || (align & (align - 1))) return dc_fail(ctx, DC_B200_MODEL_LOAD_FAILED, "gguf: alignment %llu is not a power of two", (unsigned long long)align);
    const uint64_t data0 = ((uint64_t)(c.p - map.base) + align - 1) / align * align;

    // ---- metadata -> configuration
    const std::string arch = meta.str.count("general.architecture") ? meta.str["general.architecture"] : "";
    if (arch.empty()) return dc_fail(ctx, DC_B200_MODEL_LOAD_FAILED, "gguf: general.architecture is missing");
    auto num = [&](const char* key, double dflt, bool* found = nullptr) {
        auto it = meta.num.find(arch + "." + key);
        if (found) *found = it != meta.num.end();
        return it == meta.num.end() ? dflt : it->second;
    };
    dc_model_config cfg = {};
    bool have_layers = false, have_hidden = false, have_heads = false;
    cfg.n_layer = (int)num("block_count", 0, &have_layers);
    cfg.hidden = (int)num("embedding_length", 0, &have_hidden);
    cfg.n_head = (int)num("attention.head_count", 0, &have_heads);
    if (!have_layers || !have_hidden || !have_heads)
        return dc_fail(ctx, DC_B200_MODEL_LOAD_FAILED, "gguf: %s.block_count / embedding_length / attention.head_count missing", arch.c_str());
    cfg.n_kv_head = (int)num("attention.head_count_kv", cfg.n_head);
    cfg.head_dim = (int)num("attention.key_length", cfg.n_head ? cfg.hidden / cfg.n_head : 0);
    cfg.rms_eps = (float)num("attention.layer_norm_rms_epsilon", 1e-6);
    cfg.rope_theta = (float)num("rope.freq_base", 10000.0);
    cfg.n_expert = (int)num("expert_count", 0);
    cfg.n_expert_used = (int)num("expert_used_count", 0);
    cfg.expert_ffn = (int)num("expert_feed_forward_length", 0);
    cfg.ffn = cfg.n_expert > 0 ? 0 : (int)num("feed_forward_length", 0);
    {
        // either name of the routing weights' scale (core/src/models/model_loader.cpp:2849)
        bool have_scale = false;
        cfg.routed_scale = (float)num("expert_weights_scale", 1.0, &have_scale);
        if (!have_scale) cfg.routed_scale = (float)num("routed_scaling_factor", 1.0);
    }
    if (cfg.routed_scale == 0.0f) cfg.routed_scale = 1.0f;
    if (cfg.n_expert > 0) {
        // MoE variants that the reference's loader reads (model_loader.cpp:2833-2850) and this decoder does not
        // compute: refusing them beats decoding wrong tokens silently
        const char* why = nullptr;
        if (num("norm_topk_prob", 1.0) == 0.0) why = "norm_topk_prob = false (routing weights are always renormalised over the top-k here)";
        else if (num("n_shared_experts", 0) > 0 || num("expert_shared_count", 0) > 0) why = "shared experts";
        else if (num("n_group", 0) > 1 || num("topk_group", 0) > 1 || num("expert_group_count", 0) > 1 ||
                 num("expert_group_used_count", 0) > 1)
            why = "grouped routing";
        else if (num("first_k_dense_replace", 0) > 0 || num("leading_dense_block_count", 0) > 0) why = "leading dense layers";
        else {
            for (const auto& kv : tensors)
                if (kv.first.find("_shexp") != std::string::npos) {
                    why = "shared-expert tensors (ffn_*_shexp)";
                    break;
                }
        }
        if (why) return dc_fail(ctx, DC_B200_UNSUPPORTED, "gguf: '%s' uses %s", path, why);
    }
    auto emb = tensors.find("token_embd.weight");
    if (emb == tensors.end()) return dc_fail(ctx, DC_B200_MODEL_LOAD_FAILED, "gguf: token_embd.weight is missing");
    cfg.vocab = (int)emb->second.ne[1];
    cfg.tie_embeddings = tensors.count("output.weight") ? 0 : 1;
    cfg.qk_norm = tensors.count("blk.0.attn_q_norm.weight") ? 1 : 0;
    cfg.max_seqs = max_seqs > 0 ? max_seqs : 4;
    cfg.max_ctx = max_ctx > 0 ? max_ctx : (int)num("context_length", 4096);
    cfg.ep_rank = ep_rank;
    cfg.ep_size = ep_size > 0 ? ep_size : 1;
    if (cfg.n_expert > 0 && cfg.expert_ffn == 0) {
        auto g = tensors.find("blk.0.ffn_gate_exps.weight");
        if (g != tensors.end()) cfg.expert_ffn = (int)g->second.ne[1];
    }

    dc_model* m = nullptr;
    int rc = dc_b200_model_create(ctx, &cfg, &m);
    if (rc != DC_B200_OK) return rc;
    // ---- every tensor the decoder names, straight from the mapping
    int n_names = 0;
    rc = dc_b200_model_tensor_names(m, nullptr, 0, &n_names);
    std::vector<const char*> names((size_t)n_names);
    if (rc == DC_B200_OK) rc = dc_b200_model_tensor_names(m, names.data(), n_names, &n_names);
    for (int i = 0; rc == DC_B200_OK && i < n_names; ++i) {
        auto it = tensors.find(names[i]);
        if (it == tensors.end()) {
            rc = dc_fail(ctx, DC_B200_MODEL_LOAD_FAILED, "gguf: tensor '%s' is missing from '%s'", names[i], path);
            break;
        }
        const TensorInfo& t = it->second;
        const size_t bytes = tensor_bytes(t.type, t.ne);
        if (bytes == 0 || data0 + t.offset > map.size || bytes > map.size - (data0 + t.offset)) {
            rc = dc_fail(ctx, DC_B200_MODEL_LOAD_FAILED, "gguf: tensor '%s' (type %d) is unsupported or runs past the end of the file", names[i], t.type);
            break;
        }
        rc = dc_b200_model_set_tensor(m, names[i], t.type, t.ne, map.base + data0 + t.offset);
    }
    if (rc != DC_B200_OK) {
        dc_b200_model_destroy(m);
        return rc;
    }
    *out_model = m;
    return DC_B200_OK;
}
