// GGUF v3 reader for the qwen35 checkpoint of this path: maps the file, reads the hyper-parameters the
// reference's QwenConfig reads (src/qwen_config.cpp:53-108), lists the tensors (src/gguf.cpp:216-278) and hands
// them to qb_model_create.  Only the two tensor types the reference maps from a GGUF file are accepted
// (F32 = 0, Q8_0 = 8; src/model_source.cpp:120-121).  Host code only.
#include "gguf_reader.h"

using namespace qbgguf;

// Maps and parses the file: configuration, tensor descriptors (pointing into the mapping) and their names.
static int parse_gguf(const char *path, Mapping &mp, qb_model_config &c, std::vector<std::string> &names, std::vector<qb_tensor_desc> &descs) {
    Reader r;
    uint64_t n_tensors = 0;
    std::unordered_map<std::string, Meta> meta;
    QB_TRY(open_and_read_meta(path, mp, r, n_tensors, meta, nullptr));
    struct TInfo { std::string name; uint32_t type; uint64_t rows, cols, elements, rel; };
    if (n_tensors > (r.n - r.at) / 32) return qb_fail(QB_ERR_INVALID, "gguf: %s names more tensors than it has room for", path);   // a header takes 32 bytes at least
    std::vector<TInfo> infos((size_t)n_tensors);
    for (TInfo &t : infos) {
        t.name = r.str();
        const uint32_t nd = r.get<uint32_t>();
        if (r.bad || nd == 0 || nd > 8) return qb_fail(QB_ERR_INVALID, "gguf: bad tensor header near %s", t.name.c_str());
        t.cols = r.get<uint64_t>(); t.rows = 1;
        for (uint32_t d = 1; d < nd; ++d) t.rows *= r.get<uint64_t>();
        t.elements = t.rows * t.cols;
        t.type = r.get<uint32_t>();
        t.rel = r.get<uint64_t>();
    }
    if (r.bad) return qb_fail(QB_ERR_INVALID, "gguf: %s is truncated", path);
    uint64_t align = 32;
    if (auto it = meta.find("general.alignment"); it != meta.end() && it->second.is_num && it->second.num >= 1) align = (uint64_t)it->second.num;
    const uint64_t data0 = (r.at + align - 1) / align * align;

    // hyper-parameters (src/qwen_config.cpp:53-108)
    auto arch_it = meta.find("general.architecture");
    if (arch_it == meta.end() || arch_it->second.s != "qwen35")
        return qb_fail(QB_ERR_UNSUPPORTED, "gguf: architecture '%s' (this path is the qwen35 hybrid model)", arch_it == meta.end() ? "" : arch_it->second.s.c_str());
    const std::string p = "qwen35.";
    bool missing = false; std::string missing_key;
    auto num = [&](const std::string &key, double dflt, bool required) {
        auto it = meta.find(p + key);
        if (it == meta.end() || !it->second.is_num) { if (required && !missing) { missing = true; missing_key = p + key; } return dflt; }
        return it->second.num;
    };
    c = qb_model_config{};
    const uint32_t block_count = (uint32_t)num("block_count", 0, true);
    c.mtp_layers = (uint32_t)num("nextn_predict_layers", 0, false);
    if (c.mtp_layers > block_count) return qb_fail(QB_ERR_INVALID, "gguf: nextn_predict_layers exceeds block_count");
    c.n_layers = block_count - c.mtp_layers;
    c.n_embd = (uint32_t)num("embedding_length", 0, true);
    c.n_ff = (uint32_t)num("feed_forward_length", 0, true);
    c.n_heads = (uint32_t)num("attention.head_count", 0, true);
    c.n_kv_heads = (uint32_t)num("attention.head_count_kv", 0, true);
    c.head_dim = (uint32_t)num("attention.key_length", 0, true);
    c.rms_eps = (float)num("attention.layer_norm_rms_epsilon", 1e-6, false);
    c.rope_dim = (uint32_t)num("rope.dimension_count", c.head_dim, false);
    c.rope_theta = (float)num("rope.freq_base", 1e7, false);
    c.ssm_conv_kernel = (uint32_t)num("ssm.conv_kernel", 4, false);
    c.ssm_head_dim = (uint32_t)num("ssm.state_size", 128, false);
    c.ssm_num_v_heads = (uint32_t)num("ssm.time_step_rank", 0, true);
    c.ssm_num_k_heads = (uint32_t)num("ssm.group_count", 0, true);
    c.full_attention_interval = (uint32_t)num("full_attention_interval", 4, false);
    if (missing) return qb_fail(QB_ERR_INVALID, "gguf: metadata key %s is missing", missing_key.c_str());
    auto tok = meta.find("tokenizer.ggml.tokens");
    if (tok == meta.end() || !tok->second.is_array || tok->second.array_len == 0)
        return qb_fail(QB_ERR_INVALID, "gguf: tokenizer.ggml.tokens is missing (its length is the vocabulary size)");
    c.vocab_size = (uint32_t)tok->second.array_len;
    c.weight_sigma = 0.0f;

    descs.reserve(infos.size());
    names.reserve(infos.size());
    for (const TInfo &t : infos) {
        uint64_t bytes = 0;
        if (t.type == QB_TENSOR_F32) bytes = t.elements * 4;
        else if (t.type == QB_TENSOR_Q8_0) {
            if (t.cols % 32) return qb_fail(QB_ERR_INVALID, "gguf: Q8_0 tensor %s has %llu columns", t.name.c_str(), (unsigned long long)t.cols);
            bytes = t.elements / 32 * 34;
        } else continue;    // other types cannot be bound; qb_model_create reports the tensor as missing if it is needed
        const uint64_t abs = data0 + t.rel;
        if (abs > mp.size || bytes > mp.size - abs) return qb_fail(QB_ERR_INVALID, "gguf: tensor %s points outside the file", t.name.c_str());
        names.push_back(t.name);
        descs.push_back(qb_tensor_desc{nullptr, t.type, t.rows, t.cols, (const uint8_t *)mp.base + abs});
    }
    for (size_t i = 0; i < descs.size(); ++i) descs[i].name = names[i].c_str();
    return QB_OK;
}

extern "C" int qb_model_load_gguf(qb_ctx *ctx, const char *path, qb_model **out, qb_model_config *cfg_out) {
    QB_REQUIRE(ctx && path && out, "qb_model_load_gguf: null argument");
    Mapping mp;
    qb_model_config c{};
    std::vector<std::string> names;
    std::vector<qb_tensor_desc> descs;
    QB_TRY(parse_gguf(path, mp, c, names, descs));
    if (cfg_out) *cfg_out = c;
    return qb_model_create(ctx, &c, descs.data(), descs.size(), out);
}

extern "C" int qb_gguf_read_config(const char *path, qb_model_config *cfg_out, uint64_t *n_tensors_out, uint64_t *tensor_bytes_out) {
    QB_REQUIRE(path && cfg_out, "qb_gguf_read_config: null argument");
    Mapping mp;
    std::vector<std::string> names;
    std::vector<qb_tensor_desc> descs;
    QB_TRY(parse_gguf(path, mp, *cfg_out, names, descs));
    if (n_tensors_out) *n_tensors_out = descs.size();
    if (tensor_bytes_out) {
        uint64_t b = 0;
        for (const qb_tensor_desc &d : descs) b += d.type == QB_TENSOR_F32 ? d.rows * d.cols * 4 : d.rows * d.cols / 32 * 34;
        *tensor_bytes_out = b;
    }
    return QB_OK;
}
