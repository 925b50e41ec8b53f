// GGUF v3 container reader shared by the checkpoint loader and the tokenizer: maps the file, checks magic and
// version, reads the metadata table (src/gguf.cpp:216-278 of the reference reads the same layout).  String arrays
// are skipped unless the caller asks for a key's strings.  Host code only.
#pragma once

#include "qb_internal.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <functional>
#include <string>
#include <unordered_map>
#include <vector>

namespace qbgguf {

struct Reader {
    const uint8_t *p = nullptr; size_t n = 0, at = 0; bool bad = false;
    template <typename T> T get() {
        T v{};
        if (at + sizeof(T) > n) { bad = true; return v; }
        memcpy(&v, p + at, sizeof(T));
        at += sizeof(T);
        return v;
    }
    std::string str() {
        const uint64_t len = get<uint64_t>();
        if (bad || len > n - at) { bad = true; return {}; }
        std::string s((const char *)p + at, (size_t)len);
        at += (size_t)len;
        return s;
    }
    void skip(uint64_t bytes) { if (bytes > n - at) bad = true; else at += (size_t)bytes; }
};

// GGUF metadata value types
enum : uint32_t { GT_U8, GT_I8, GT_U16, GT_I16, GT_U32, GT_I32, GT_F32, GT_BOOL, GT_STR, GT_ARR, GT_U64, GT_I64, GT_F64 };
inline uint32_t scalar_bytes(uint32_t t) {
    switch (t) {
        case GT_U8: case GT_I8: case GT_BOOL: return 1;
        case GT_U16: case GT_I16: return 2;
        case GT_U32: case GT_I32: case GT_F32: return 4;
        case GT_U64: case GT_I64: case GT_F64: return 8;
        default: return 0;
    }
}
struct Meta {
    double num = 0; std::string s; uint64_t array_len = 0; bool is_num = false, is_str = false, is_array = false;
    std::vector<std::string> strs;        // the elements of a string array, when asked for
};

inline bool read_value(Reader &r, uint32_t type, Meta &m, bool keep_strings) {
    switch (type) {
        case GT_U8: m.num = r.get<uint8_t>(); m.is_num = true; return true;
        case GT_I8: m.num = r.get<int8_t>(); m.is_num = true; return true;
        case GT_BOOL: m.num = r.get<uint8_t>() ? 1 : 0; m.is_num = true; return true;
        case GT_U16: m.num = r.get<uint16_t>(); m.is_num = true; return true;
        case GT_I16: m.num = r.get<int16_t>(); m.is_num = true; return true;
        case GT_U32: m.num = r.get<uint32_t>(); m.is_num = true; return true;
        case GT_I32: m.num = r.get<int32_t>(); m.is_num = true; return true;
        case GT_F32: m.num = r.get<float>(); m.is_num = true; return true;
        case GT_U64: m.num = (double)r.get<uint64_t>(); m.is_num = true; return true;
        case GT_I64: m.num = (double)r.get<int64_t>(); m.is_num = true; return true;
        case GT_F64: m.num = r.get<double>(); m.is_num = true; return true;
        case GT_STR: m.s = r.str(); m.is_str = true; return true;
        case GT_ARR: {
            const uint32_t et = r.get<uint32_t>();
            const uint64_t cnt = r.get<uint64_t>();
            m.is_array = true; m.array_len = cnt;
            if (et == GT_STR) {
                if (keep_strings) {
                    if (cnt > r.n) { r.bad = true; return false; }      // every element takes at least its length field
                    m.strs.reserve((size_t)cnt);
                    for (uint64_t i = 0; i < cnt && !r.bad; ++i) m.strs.push_back(r.str());
                } else {
                    for (uint64_t i = 0; i < cnt && !r.bad; ++i) r.skip(r.get<uint64_t>());
                }
                return true;
            }
            const uint32_t sb = scalar_bytes(et);
            if (!sb) return false;                       // nested arrays are not used by this checkpoint format
            r.skip(cnt * sb);
            return true;
        }
        default: return false;
    }
}

struct Mapping {
    int fd = -1; void *base = MAP_FAILED; size_t size = 0;
    ~Mapping() { if (base != MAP_FAILED) munmap(base, size); if (fd >= 0) close(fd); }
};

// Opens and maps the file and reads its metadata table; r is left at the first tensor header.
inline int open_and_read_meta(const char *path, Mapping &mp, Reader &r, uint64_t &n_tensors, std::unordered_map<std::string, Meta> &meta,
                              const std::function<bool(const std::string &)> &keep_strings) {
    mp.fd = open(path, O_RDONLY);
    if (mp.fd < 0) return qb_fail(QB_ERR_INVALID, "gguf: cannot open %s: %s", path, strerror(errno));
    struct stat st {};
    if (fstat(mp.fd, &st) != 0 || st.st_size < 24) return qb_fail(QB_ERR_INVALID, "gguf: %s is not a readable GGUF file", path);
    mp.size = (size_t)st.st_size;
    mp.base = mmap(nullptr, mp.size, PROT_READ, MAP_PRIVATE, mp.fd, 0);
    if (mp.base == MAP_FAILED) return qb_fail(QB_ERR_INVALID, "gguf: mmap of %s failed: %s", path, strerror(errno));
    r = Reader{(const uint8_t *)mp.base, mp.size};
    if (r.get<uint32_t>() != 0x46554747u) return qb_fail(QB_ERR_INVALID, "gguf: %s has no GGUF magic", path);
    const uint32_t version = r.get<uint32_t>();
    if (version != 3) return qb_fail(QB_ERR_UNSUPPORTED, "gguf: version %u (only v3 is read, as in the reference)", version);
    n_tensors = r.get<uint64_t>();
    const uint64_t n_meta = r.get<uint64_t>();
    for (uint64_t i = 0; i < n_meta; ++i) {
        std::string key = r.str();
        const uint32_t type = r.get<uint32_t>();
        Meta m;
        if (r.bad || !read_value(r, type, m, keep_strings && keep_strings(key)) || r.bad)
            return qb_fail(QB_ERR_INVALID, "gguf: bad metadata entry %llu (%s)", (unsigned long long)i, key.c_str());
        meta.emplace(std::move(key), std::move(m));
    }
    return QB_OK;
}

}  // namespace qbgguf
