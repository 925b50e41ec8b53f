// Byte-level BPE tokenizer of the qwen35 checkpoints: the caller side of the path (text -> the token ids qb_prefill
// takes, token ids -> text).  Host code only; no device is needed.
//
// Behaviour follows qw3::QwenTokenizer (include/qw3/tokenizer.hpp:30-45, src/tokenizer.cpp):
//   vocabulary and merge ranks from tokenizer.ggml.tokens / tokenizer.ggml.merges (:180-216): the first of equal
//     token strings keeps the id, the first of equal merge lines keeps the rank, a merge line splits at its first space;
//   the chat-template special tokens that the vocabulary holds are matched as whole tokens before anything else, at the
//     earliest position, the longest first (:327-358, :574-640);
//   the text between them is cut into pieces by the split pattern of the Qwen tokenizer (:376-514)
//       (?i:'s|'t|'re|'ve|'m|'ll|'d) | [^\r\n\p{L}\p{N}]?[\p{L}\p{M}]+ | \p{N} | ?[^\s\p{L}\p{M}\p{N}]+[\r\n]* |
//       \s*[\r\n]+ | \s+(?!\S) | \s+
//     with the reference's character classes (:104-151): ASCII letters and digits, the CJK / kana / hangul / fullwidth
//     blocks as letters, five combining-mark blocks, a short list of spaces, and for every other code point what the
//     process locale's wide-character classification says;
//   every piece is mapped to the GPT-2 visible alphabet byte by byte and merged pair by pair, lowest rank first, leftmost
//     among equals (:516-562); a merged symbol the vocabulary lacks falls back to its single-byte tokens;
//   decoding maps the visible alphabet back to bytes and copies anything else (:719-745).
#include "gguf_reader.h"

#include <algorithm>
#include <clocale>
#include <cwctype>
#include <locale>
#include <mutex>

struct qb_tokenizer {
    std::vector<std::string> tokens;
    std::unordered_map<std::string, int32_t> id_of;
    std::unordered_map<std::string, int32_t> rank;           // key: pair_key(left, right)
    std::string byte_sym[256];                               // UTF-8 of the visible code point of a byte
    std::unordered_map<std::string, uint8_t> byte_of_sym;
    std::vector<std::pair<std::string, int32_t>> specials;   // longest first
    bool initial[256] = {};                                  // first bytes of the special tokens
    int32_t bos = 0, eos = 0;
    bool add_bos = false;
};

namespace {

// Lenient UTF-8 decoding (src/tokenizer.cpp:34-60): a lead byte without its continuation bytes inside the string, or
// any other byte, is one code point of one byte.  Continuation bytes are not checked.
inline uint32_t next_cp(const char *s, size_t n, size_t &pos) {
    const uint8_t c0 = (uint8_t)s[pos];
    auto b = [&](size_t k) { return (uint32_t)((uint8_t)s[pos + k] & 0x3F); };
    if (c0 >= 0x80) {
        if ((c0 & 0xE0) == 0xC0 && pos + 1 < n) { const uint32_t v = ((c0 & 0x1Fu) << 6) | b(1); pos += 2; return v; }
        if ((c0 & 0xF0) == 0xE0 && pos + 2 < n) { const uint32_t v = ((c0 & 0x0Fu) << 12) | (b(1) << 6) | b(2); pos += 3; return v; }
        if ((c0 & 0xF8) == 0xF0 && pos + 3 < n) { const uint32_t v = ((c0 & 0x07u) << 18) | (b(1) << 12) | (b(2) << 6) | b(3); pos += 4; return v; }
    }
    ++pos;
    return c0;
}

std::string utf8_of(uint32_t cp) {
    std::string s;
    if (cp < 0x80) s.push_back((char)cp);
    else if (cp < 0x800) { s.push_back((char)(0xC0 | (cp >> 6))); s.push_back((char)(0x80 | (cp & 0x3F))); }
    else if (cp < 0x10000) { s.push_back((char)(0xE0 | (cp >> 12))); s.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); s.push_back((char)(0x80 | (cp & 0x3F))); }
    else { s.push_back((char)(0xF0 | (cp >> 18))); s.push_back((char)(0x80 | ((cp >> 12) & 0x3F))); s.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); s.push_back((char)(0x80 | (cp & 0x3F))); }
    return s;
}

// The process locale's wide-character classes, as the reference consults them for code points outside its own tables.
const std::ctype<wchar_t> &wide_classes() {
    static const std::locale loc = [] {
        try { return std::locale(""); } catch (...) { return std::locale::classic(); }
    }();
    return std::use_facet<std::ctype<wchar_t>>(loc);
}

enum Cls : uint8_t { C_OTHER = 0, C_LETTER = 1, C_MARK = 2, C_NUMBER = 4, C_SPACE = 8 };

inline bool in(uint32_t cp, uint32_t lo, uint32_t hi) { return cp >= lo && cp <= hi; }

uint8_t classify(uint32_t cp) {
    if (cp < 0x80) {
        if ((cp >= 'a' && cp <= 'z') || (cp >= 'A' && cp <= 'Z')) return C_LETTER;
        if (cp >= '0' && cp <= '9') return C_NUMBER;
        if (cp == ' ' || (cp >= '\t' && cp <= '\r')) return C_SPACE;          // \t \n \v \f \r
        return C_OTHER;
    }
    uint8_t c = C_OTHER;
    const bool block_letter = in(cp, 0x3040, 0x30FF) || in(cp, 0x3400, 0x4DBF) || in(cp, 0x4E00, 0x9FFF) || in(cp, 0xAC00, 0xD7AF) ||
                              in(cp, 0xF900, 0xFAFF) || in(cp, 0xFF00, 0xFFEF);
    const bool wide_ok = cp <= (uint32_t)WCHAR_MAX;
    if (block_letter || (wide_ok && wide_classes().is(std::ctype_base::alpha, (wchar_t)cp))) c |= C_LETTER;
    if (wide_ok && wide_classes().is(std::ctype_base::digit, (wchar_t)cp)) c |= C_NUMBER;
    if (in(cp, 0x0300, 0x036F) || in(cp, 0x1AB0, 0x1AFF) || in(cp, 0x1DC0, 0x1DFF) || in(cp, 0x20D0, 0x20FF) || in(cp, 0xFE20, 0xFE2F)) c |= C_MARK;
    if (cp == 0xA0 || cp == 0x2028 || cp == 0x2029 || in(cp, 0x2000, 0x200A)) c |= C_SPACE;
    return c;
}

// Piece boundaries of a text without special tokens: ends[i] = byte offset one past piece i.
void split_pieces(const char *text, size_t n, std::vector<uint32_t> &ends) {
    struct Cp { uint32_t v, end; uint8_t cls; };
    std::vector<Cp> cps;
    cps.reserve(n);
    for (size_t pos = 0; pos < n;) {
        const uint32_t v = next_cp(text, n, pos);
        cps.push_back({v, (uint32_t)pos, classify(v)});
    }
    const size_t len = cps.size();
    auto word = [&](size_t i) { return i < len && (cps[i].cls & (C_LETTER | C_MARK)); };      // [\p{L}\p{M}]
    auto number = [&](size_t i) { return i < len && (cps[i].cls & C_NUMBER); };
    auto space = [&](size_t i) { return i < len && (cps[i].cls & C_SPACE); };
    auto newline = [&](size_t i) { return i < len && (cps[i].v == '\r' || cps[i].v == '\n'); };
    auto symbol = [&](size_t i) { return i < len && !(cps[i].cls & (C_SPACE | C_LETTER | C_MARK | C_NUMBER)); };
    auto lower = [&](size_t i) -> uint32_t {
        if (i >= len || cps[i].v >= 0x80) return 0;
        const uint32_t v = cps[i].v;
        return v >= 'A' && v <= 'Z' ? v + 32 : v;
    };
    size_t pos = 0;
    auto cut = [&](size_t to) { ends.push_back(cps[to - 1].end); pos = to; };
    while (pos < len) {
        const uint32_t c0 = cps[pos].v;
        // 's 't 'm 'd 're 've 'll, any case
        if (c0 == '\'') {
            const uint32_t a = lower(pos + 1), b = lower(pos + 2);
            if (a == 's' || a == 't' || a == 'm' || a == 'd') { cut(pos + 2); continue; }
            if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e') || (a == 'l' && b == 'l')) { cut(pos + 3); continue; }
        }
        // a run of letters and marks, with at most one leading code point that is no newline, letter or number
        if (!newline(pos) && !number(pos) && (word(pos) || word(pos + 1))) {
            size_t e = pos + 1;
            while (word(e)) ++e;
            cut(e);
            continue;
        }
        // every numeric code point alone
        if (number(pos)) { cut(pos + 1); continue; }
        // a run of symbols with an optional leading blank and its trailing newlines
        {
            const size_t first = c0 == ' ' ? pos + 1 : pos;
            if (symbol(first)) {
                size_t e = first;
                while (symbol(e)) ++e;
                while (newline(e)) ++e;
                cut(e);
                continue;
            }
        }
        // white space: up to the run's last newline; else all but the last character when text follows; else all of it
        if (space(pos)) {
            size_t e = pos, last_nl = 0;
            while (space(e)) { if (newline(e)) last_nl = e + 1; ++e; }
            if (last_nl) cut(last_nl);
            else if (e - pos > 1 && e < len) cut(e - 1);
            else cut(e);
            continue;
        }
        cut(pos + 1);        // nothing above applies (cannot happen with the classes above): one code point
    }
}

inline std::string pair_key(const std::string &l, const std::string &r) {
    std::string k;
    k.reserve(l.size() + r.size() + 4);
    const uint32_t n = (uint32_t)l.size();
    k.append((const char *)&n, 4);
    k += l;
    k += r;
    return k;
}

void bpe_piece(const qb_tokenizer &t, const char *p, size_t n, std::vector<int32_t> &out) {
    std::vector<std::string> sym;
    sym.reserve(n);
    for (size_t i = 0; i < n; ++i) sym.push_back(t.byte_sym[(uint8_t)p[i]]);
    // ranks of the adjacent pairs, kept beside the symbols so that a merge only re-reads its two neighbours
    constexpr int32_t NONE = INT32_MAX;
    auto rank_of = [&](size_t i) -> int32_t {
        const auto it = t.rank.find(pair_key(sym[i], sym[i + 1]));
        return it == t.rank.end() ? NONE : it->second;
    };
    std::vector<int32_t> rk(sym.size() > 1 ? sym.size() - 1 : 0);
    for (size_t i = 0; i + 1 < sym.size(); ++i) rk[i] = rank_of(i);
    while (sym.size() > 1) {
        size_t best = 0;
        for (size_t i = 1; i < rk.size(); ++i)
            if (rk[i] < rk[best]) best = i;                  // lowest rank, leftmost among equals
        if (rk[best] == NONE) break;
        sym[best] += sym[best + 1];
        sym.erase(sym.begin() + (long)best + 1);
        rk.erase(rk.begin() + (long)best);
        if (best > 0) rk[best - 1] = rank_of(best - 1);
        if (best + 1 < sym.size()) rk[best] = rank_of(best);
    }
    for (const std::string &s : sym) {
        const auto it = t.id_of.find(s);
        if (it != t.id_of.end()) { out.push_back(it->second); continue; }
        for (char c : s) {                                    // not in the vocabulary: its single-byte tokens, where they exist
            const auto b = t.id_of.find(std::string(1, c));
            if (b != t.id_of.end()) out.push_back(b->second);
        }
    }
}

void encode_plain(const qb_tokenizer &t, const char *text, size_t n, std::vector<int32_t> &out,
                  std::unordered_map<std::string, std::vector<int32_t>> &cache) {
    std::vector<uint32_t> ends;
    split_pieces(text, n, ends);
    uint32_t begin = 0;
    std::vector<int32_t> ids;
    for (const uint32_t end : ends) {
        std::string piece(text + begin, end - begin);
        auto it = cache.find(piece);
        if (it == cache.end()) {
            ids.clear();
            bpe_piece(t, piece.data(), piece.size(), ids);
            it = cache.emplace(std::move(piece), ids).first;
        }
        out.insert(out.end(), it->second.begin(), it->second.end());
        begin = end;
    }
}

void finish(qb_tokenizer &t) {
    t.id_of.reserve(t.tokens.size() * 2);
    for (size_t i = 0; i < t.tokens.size(); ++i)
        if (!t.tokens[i].empty()) t.id_of.emplace(t.tokens[i], (int32_t)i);
    // the GPT-2 byte <-> visible code point table: printable Latin-1 bytes map to themselves, the others to 256, 257, ...
    uint32_t next = 256;
    for (int b = 0; b < 256; ++b) {
        const bool printable = (b >= 0x21 && b <= 0x7E) || (b >= 0xA1 && b <= 0xAC) || (b >= 0xAE && b <= 0xFF);
        t.byte_sym[b] = utf8_of(printable ? (uint32_t)b : next++);
        t.byte_of_sym[t.byte_sym[b]] = (uint8_t)b;
    }
    static const char *const candidates[] = {
        "<|im_start|>", "<|im_end|>", "<|endoftext|>", "<|fim_prefix|>", "<|fim_middle|>", "<|fim_suffix|>", "<|vision_start|>",
        "<|vision_end|>", "<|image_pad|>", "<|video_pad|>", "<|object_ref_start|>", "<|object_ref_end|>", "<|box_start|>", "<|box_end|>",
        "<|quad_start|>", "<|quad_end|>", "<think>", "</think>", "<tool_call>", "</tool_call>", "<tool_response>", "</tool_response>",
    };
    for (const char *s : candidates) {
        const auto it = t.id_of.find(s);
        if (it != t.id_of.end()) t.specials.emplace_back(s, it->second);
    }
    std::stable_sort(t.specials.begin(), t.specials.end(), [](const auto &a, const auto &b) { return a.first.size() > b.first.size(); });
    for (const auto &s : t.specials) t.initial[(uint8_t)s.first[0]] = true;
}

void add_merges(qb_tokenizer &t, const std::vector<std::string> &lines) {
    t.rank.reserve(lines.size() * 2);
    for (size_t i = 0; i < lines.size(); ++i) {
        const size_t sp = lines[i].find(' ');
        if (sp == std::string::npos) continue;               // the line still takes its rank number
        t.rank.emplace(pair_key(lines[i].substr(0, sp), lines[i].substr(sp + 1)), (int32_t)i);
    }
}

}  // namespace

extern "C" int qb_tokenizer_create(const char *const *tokens, const uint32_t *token_lens, uint32_t n_tokens, const char *const *merges,
                                   const uint32_t *merge_lens, uint32_t n_merges, int32_t bos_id, int32_t eos_id, int add_bos,
                                   qb_tokenizer **out) {
    QB_REQUIRE(tokens && token_lens && n_tokens > 0 && out && (n_merges == 0 || (merges && merge_lens)), "qb_tokenizer_create: bad arguments");
    qb_tokenizer *t = new qb_tokenizer();
    t->tokens.reserve(n_tokens);
    for (uint32_t i = 0; i < n_tokens; ++i) t->tokens.emplace_back(tokens[i], token_lens[i]);
    std::vector<std::string> lines;
    lines.reserve(n_merges);
    for (uint32_t i = 0; i < n_merges; ++i) lines.emplace_back(merges[i], merge_lens[i]);
    add_merges(*t, lines);
    t->bos = bos_id; t->eos = eos_id; t->add_bos = add_bos != 0;
    finish(*t);
    *out = t;
    return QB_OK;
}

extern "C" int qb_tokenizer_load_gguf(const char *path, qb_tokenizer **out) {
    QB_REQUIRE(path && out, "qb_tokenizer_load_gguf: null argument");
    qbgguf::Mapping mp;
    qbgguf::Reader r;
    uint64_t n_tensors = 0;
    std::unordered_map<std::string, qbgguf::Meta> meta;
    QB_TRY(qbgguf::open_and_read_meta(path, mp, r, n_tensors, meta, [](const std::string &k) {
        return k == "tokenizer.ggml.tokens" || k == "tokenizer.ggml.merges";
    }));
    auto tk = meta.find("tokenizer.ggml.tokens");
    if (tk == meta.end() || tk->second.strs.empty()) return qb_fail(QB_ERR_INVALID, "tokenizer: %s has no tokenizer.ggml.tokens", path);
    auto mg = meta.find("tokenizer.ggml.merges");
    if (mg == meta.end() || !mg->second.is_array) return qb_fail(QB_ERR_INVALID, "tokenizer: %s has no tokenizer.ggml.merges (the merge ranks)", path);
    qb_tokenizer *t = new qb_tokenizer();
    t->tokens = std::move(tk->second.strs);
    add_merges(*t, mg->second.strs);
    auto num = [&](const char *key, double dflt) {
        auto it = meta.find(key);
        return it != meta.end() && it->second.is_num ? it->second.num : dflt;
    };
    t->bos = (int32_t)num("tokenizer.ggml.bos_token_id", 0);
    t->eos = (int32_t)num("tokenizer.ggml.eos_token_id", 0);
    t->add_bos = num("tokenizer.ggml.add_bos_token", 0) != 0;
    finish(*t);
    *out = t;
    return QB_OK;
}

extern "C" void qb_tokenizer_destroy(qb_tokenizer *t) { delete t; }

extern "C" int qb_tokenizer_info(const qb_tokenizer *t, int32_t *vocab_size, int32_t *bos_id, int32_t *eos_id, int *add_bos_default,
                                 uint32_t *n_special) {
    QB_REQUIRE(t, "qb_tokenizer_info: null tokenizer");
    if (vocab_size) *vocab_size = (int32_t)t->tokens.size();
    if (bos_id) *bos_id = t->bos;
    if (eos_id) *eos_id = t->eos;
    if (add_bos_default) *add_bos_default = t->add_bos ? 1 : 0;
    if (n_special) *n_special = (uint32_t)t->specials.size();
    return QB_OK;
}

extern "C" int qb_tokenizer_token_id(const qb_tokenizer *t, const char *token, uint32_t len) {
    if (!t || !token) return -1;
    const auto it = t->id_of.find(std::string(token, len));
    return it == t->id_of.end() ? -1 : it->second;
}

extern "C" int qb_tokenizer_encode(const qb_tokenizer *t, const char *text, size_t len, int add_bos, int32_t *ids, size_t cap, size_t *n_out) {
    QB_REQUIRE(t && (text || len == 0) && n_out && (ids || cap == 0), "qb_tokenizer_encode: bad arguments");
    QB_REQUIRE(len < 0xFFFFFFFFull, "qb_tokenizer_encode: texts of 4 GiB and more are not taken in one call");
    std::vector<int32_t> out;
    out.reserve(len / 3 + 4);
    if ((add_bos || t->add_bos) && t->bos < (int32_t)t->tokens.size()) out.push_back(t->bos);
    std::unordered_map<std::string, std::vector<int32_t>> cache;     // pieces repeat: one merge pass per distinct piece and call
    size_t i = 0;
    while (i < len) {
        // the earliest position at which a special token stands, the longest of those that do
        size_t at = i;
        const std::pair<std::string, int32_t> *hit = nullptr;
        for (; at < len && !hit; ++at) {
            if (!t->initial[(uint8_t)text[at]]) continue;
            for (const auto &s : t->specials)
                if (s.first.size() <= len - at && memcmp(text + at, s.first.data(), s.first.size()) == 0) { hit = &s; break; }
            if (hit) break;
        }
        const size_t plain_end = hit ? at : len;
        if (plain_end > i) encode_plain(*t, text + i, plain_end - i, out, cache);
        if (!hit) break;
        out.push_back(hit->second);
        i = at + hit->first.size();
    }
    *n_out = out.size();
    if (out.size() > cap) return qb_fail(QB_ERR_CAPACITY, "qb_tokenizer_encode: %zu tokens, room for %zu", out.size(), cap);
    if (!out.empty()) memcpy(ids, out.data(), out.size() * sizeof(int32_t));
    return QB_OK;
}

extern "C" int qb_tokenizer_decode(const qb_tokenizer *t, const int32_t *ids, size_t n, char *text, size_t cap, size_t *len_out) {
    QB_REQUIRE(t && (ids || n == 0) && len_out && (text || cap == 0), "qb_tokenizer_decode: bad arguments");
    std::string out;
    for (size_t k = 0; k < n; ++k) {
        if (ids[k] < 0 || ids[k] >= (int32_t)t->tokens.size()) continue;          // an id outside the vocabulary decodes to nothing
        const std::string &s = t->tokens[(size_t)ids[k]];
        for (size_t pos = 0; pos < s.size();) {
            const size_t b = pos;
            next_cp(s.data(), s.size(), pos);
            const auto it = t->byte_of_sym.find(s.substr(b, pos - b));
            if (it != t->byte_of_sym.end()) out.push_back((char)it->second);
            else out.append(s, b, pos - b);                                         // e.g. a special token, printed by name
        }
    }
    *len_out = out.size();
    if (out.size() > cap) return qb_fail(QB_ERR_CAPACITY, "qb_tokenizer_decode: %zu bytes, room for %zu", out.size(), cap);
    if (!out.empty()) memcpy(text, out.data(), out.size());
    return QB_OK;
}

extern "C" int qb_tokenizer_split(const char *text, size_t len, uint32_t *piece_ends, size_t cap, size_t *n_out) {
    QB_REQUIRE((text || len == 0) && n_out && (piece_ends || cap == 0) && len < 0xFFFFFFFFull, "qb_tokenizer_split: bad arguments");
    std::vector<uint32_t> ends;
    split_pieces(text, len, ends);
    *n_out = ends.size();
    if (ends.size() > cap) return qb_fail(QB_ERR_CAPACITY, "qb_tokenizer_split: %zu pieces, room for %zu", ends.size(), cap);
    if (!ends.empty()) memcpy(piece_ends, ends.data(), ends.size() * sizeof(uint32_t));
    return QB_OK;
}
