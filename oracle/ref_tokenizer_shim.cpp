// TEST INFRASTRUCTURE ONLY.  The reference's own tokenizer as a callable comparator: qw3::QwenTokenizer built from a GGUF
// file (include/qw3/tokenizer.hpp:30-45, src/tokenizer.cpp:180-216) and its split function
// qw3::detail::qwen_pre_tokenize (src/tokenizer_internal.hpp), called unchanged.  Linked against the reference's
// tokenizer.cpp and gguf.cpp objects, compiled where they lie (oracle/Makefile target ref-tokenizer); nothing here is
// part of the product.  Runs without a GPU.
#include "qw3/gguf.hpp"
#include "qw3/tokenizer.hpp"
#include "tokenizer_internal.hpp"

#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

namespace {
struct Handle {
    std::unique_ptr<qw3::GgufFile> file;
    std::unique_ptr<qw3::QwenTokenizer> tok;
};
}  // namespace

extern "C" {

void *rt_open(const char *path) {
    try {
        auto h = std::make_unique<Handle>();
        h->file = std::make_unique<qw3::GgufFile>(path);
        h->tok = std::make_unique<qw3::QwenTokenizer>(*h->file);
        return h.release();
    } catch (...) {
        return nullptr;
    }
}

void rt_close(void *h) { delete static_cast<Handle *>(h); }

int32_t rt_vocab_size(void *h) { return static_cast<Handle *>(h)->tok->vocab_size(); }

// encode(): returns the number of tokens; writes at most cap of them.
int64_t rt_encode(void *h, const char *text, uint64_t len, int add_bos, int32_t *ids, uint64_t cap) {
    const std::vector<int32_t> v = static_cast<Handle *>(h)->tok->encode(std::string(text, len), add_bos != 0);
    for (uint64_t i = 0; i < v.size() && i < cap; ++i) ids[i] = v[i];
    return (int64_t)v.size();
}

// decode(): returns the number of bytes; writes at most cap of them.
int64_t rt_decode(void *h, const int32_t *ids, uint64_t n, char *out, uint64_t cap) {
    const std::string s = static_cast<Handle *>(h)->tok->decode(std::vector<int32_t>(ids, ids + n));
    memcpy(out, s.data(), s.size() < cap ? s.size() : cap);
    return (int64_t)s.size();
}

// qwen_pre_tokenize(): byte offsets one past each piece; returns the number of pieces.
int64_t rt_split(const char *text, uint64_t len, uint32_t *ends, uint64_t cap) {
    const std::vector<std::string> pieces = qw3::detail::qwen_pre_tokenize(std::string(text, len));
    uint64_t at = 0;
    for (uint64_t i = 0; i < pieces.size(); ++i) {
        at += pieces[i].size();
        if (i < cap) ends[i] = (uint32_t)at;
    }
    return (int64_t)pieces.size();
}

}  // extern "C"
