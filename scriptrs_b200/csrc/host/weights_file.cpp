// safetensors reader (see weights_file.h).  Host only.
#include "weights_file.h"

#include <cerrno>
#include <cstdio>
#include <cstring>

namespace sb {

namespace {

// Minimal JSON reader for the header: objects, strings, integers and arrays of integers.
struct Json {
    const char* p;
    const char* end;
    std::string err;

    void ws() {
        while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
    }
    bool eat(char c) {
        ws();
        if (p < end && *p == c) {
            ++p;
            return true;
        }
        return false;
    }
    bool fail(const char* what) {
        if (err.empty()) err = std::string("malformed header: ") + what;
        return false;
    }
    bool string(std::string* out) {
        ws();
        if (p >= end || *p != '"') return fail("expected a string");
        ++p;
        out->clear();
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (++p >= end) return fail("unterminated escape");
                switch (*p) {
                    case 'n': out->push_back('\n'); break;
                    case 't': out->push_back('\t'); break;
                    case 'r': out->push_back('\r'); break;
                    case 'b': out->push_back('\b'); break;
                    case 'f': out->push_back('\f'); break;
                    case 'u': {
                        if (end - p < 5) return fail("short \\u escape");
                        unsigned v = 0;
                        for (int i = 1; i <= 4; ++i) {
                            const char c = p[i];
                            v = v * 16 + (c >= '0' && c <= '9' ? c - '0' : (c >= 'a' && c <= 'f' ? c - 'a' + 10 : (c >= 'A' && c <= 'F' ? c - 'A' + 10 : 0)));
                        }
                        p += 4;
                        if (v < 0x80) out->push_back((char)v);
                        else if (v < 0x800) { out->push_back((char)(0xC0 | (v >> 6))); out->push_back((char)(0x80 | (v & 0x3F))); }
                        else { out->push_back((char)(0xE0 | (v >> 12))); out->push_back((char)(0x80 | ((v >> 6) & 0x3F))); out->push_back((char)(0x80 | (v & 0x3F))); }
                        break;
                    }
                    default: out->push_back(*p);
                }
                ++p;
            } else {
                out->push_back(*p++);
            }
        }
        if (p >= end) return fail("unterminated string");
        ++p;
        return true;
    }
    bool integer(uint64_t* out) {
        ws();
        if (p >= end || *p < '0' || *p > '9') return fail("expected a non-negative integer");
        uint64_t v = 0;
        while (p < end && *p >= '0' && *p <= '9') v = v * 10 + (uint64_t)(*p++ - '0');
        *out = v;
        return true;
    }
    bool int_array(std::vector<uint64_t>* out) {
        out->clear();
        if (!eat('[')) return fail("expected an array");
        if (eat(']')) return true;
        do {
            uint64_t v;
            if (!integer(&v)) return false;
            out->push_back(v);
        } while (eat(','));
        return eat(']') || fail("unterminated array");
    }
    // skips any value (used for unknown keys)
    bool skip() {
        ws();
        if (p >= end) return fail("unexpected end");
        if (*p == '"') {
            std::string s;
            return string(&s);
        }
        if (*p == '{' || *p == '[') {
            const char open = *p, close = open == '{' ? '}' : ']';
            ++p;
            if (eat(close)) return true;
            do {
                if (open == '{') {
                    std::string k;
                    if (!string(&k) || !eat(':')) return fail("bad object");
                }
                if (!skip()) return false;
            } while (eat(','));
            return eat(close) || fail("unterminated container");
        }
        while (p < end && *p != ',' && *p != '}' && *p != ']') ++p;  // number / literal
        return true;
    }
};

float half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000) << 16;
    uint32_t exp = (h >> 10) & 0x1F, man = h & 0x3FF, bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            exp = 127 - 15 + 1;
            while (!(man & 0x400)) { man <<= 1; --exp; }
            bits = sign | (exp << 23) | ((man & 0x3FF) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

}  // namespace

std::string weight_file_open(const char* path, WeightFile* out, bool* missing) {
    *missing = false;
    std::FILE* f = std::fopen(path, "rb");
    if (!f) {
        *missing = errno == ENOENT || errno == ENOTDIR;
        return std::string(*missing ? "missing model asset: " : "cannot open ") + path;
    }
    auto bail = [&](const std::string& m) {
        std::fclose(f);
        return m + " (" + path + ")";
    };
    unsigned char lenb[8];
    if (std::fread(lenb, 1, 8, f) != 8) return bail("file too short for a header length");
    uint64_t hlen = 0;
    for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | lenb[i];
    if (hlen < 2 || hlen > (1ull << 27)) return bail("unreasonable header length");
    std::string header((size_t)hlen, '\0');
    if (std::fread(&header[0], 1, (size_t)hlen, f) != hlen) return bail("file shorter than its header");
    const long data_start = std::ftell(f);
    if (std::fseek(f, 0, SEEK_END) != 0) return bail("seek failed");
    const long file_end = std::ftell(f);
    if (file_end < data_start) return bail("bad file size");
    const uint64_t data_bytes = (uint64_t)(file_end - data_start);

    Json j{header.data(), header.data() + header.size(), ""};
    if (!j.eat('{')) return bail("malformed header: expected an object");
    if (!j.eat('}')) {
        do {
            std::string name;
            if (!j.string(&name) || !j.eat(':')) return bail(j.err.empty() ? "malformed header" : j.err);
            if (!j.eat('{')) return bail("malformed header: tensor entry is not an object");
            WeightEntry e;
            bool is_meta = name == "__metadata__";
            bool has_dtype = false, has_shape = false, has_off = false;
            if (!j.eat('}')) {
                do {
                    std::string key;
                    if (!j.string(&key) || !j.eat(':')) return bail(j.err.empty() ? "malformed header" : j.err);
                    if (is_meta) {
                        std::string v;
                        j.ws();
                        if (j.p < j.end && *j.p == '"') {
                            if (!j.string(&v)) return bail(j.err);
                            out->metadata[key] = v;
                        } else if (!j.skip()) return bail(j.err);
                    } else if (key == "dtype") {
                        if (!j.string(&e.dtype)) return bail(j.err);
                        has_dtype = true;
                    } else if (key == "shape") {
                        std::vector<uint64_t> s;
                        if (!j.int_array(&s)) return bail(j.err);
                        e.shape.assign(s.begin(), s.end());
                        has_shape = true;
                    } else if (key == "data_offsets") {
                        std::vector<uint64_t> s;
                        if (!j.int_array(&s) || s.size() != 2) return bail("malformed header: data_offsets needs two integers");
                        e.begin = s[0];
                        e.end = s[1];
                        has_off = true;
                    } else if (!j.skip()) {
                        return bail(j.err);
                    }
                } while (j.eat(','));
                if (!j.eat('}')) return bail("malformed header: unterminated tensor entry");
            }
            if (!is_meta) {
                if (!has_dtype || !has_shape || !has_off) return bail("tensor " + name + " lacks dtype, shape or data_offsets");
                const int esz = e.dtype == "F32" ? 4 : ((e.dtype == "F16" || e.dtype == "BF16") ? 2 : 0);
                if (!esz) return bail("tensor " + name + " has dtype " + e.dtype + "; F32, F16 and BF16 are read");
                if (e.end < e.begin || e.end > data_bytes || (uint64_t)e.numel() * esz != e.end - e.begin)
                    return bail("tensor " + name + ": byte range does not match its shape or the file size");
                out->entries[name] = e;
            }
        } while (j.eat(','));
        if (!j.eat('}')) return bail("malformed header: unterminated object");
    }
    out->data.resize((size_t)data_bytes);
    if (std::fseek(f, data_start, SEEK_SET) != 0 ||
        (data_bytes && std::fread(out->data.data(), 1, (size_t)data_bytes, f) != data_bytes))
        return bail("could not read the tensor data");
    std::fclose(f);
    return "";
}

const float* WeightFile::as_f32(const std::string& name) {
    auto it = entries.find(name);
    if (it == entries.end()) return nullptr;
    const WeightEntry& e = it->second;
    const unsigned char* src = data.data() + e.begin;
    if (e.dtype == "F32" && (reinterpret_cast<uintptr_t>(src) & 3) == 0) return reinterpret_cast<const float*>(src);
    auto c = converted.find(name);
    if (c != converted.end()) return c->second.data();
    std::vector<float>& v = converted[name];
    const size_t n = (size_t)e.numel();
    v.resize(n);
    if (e.dtype == "F32") {
        std::memcpy(v.data(), src, n * 4);
    } else if (e.dtype == "BF16") {
        for (size_t i = 0; i < n; ++i) {
            const uint32_t bits = ((uint32_t)src[2 * i] | ((uint32_t)src[2 * i + 1] << 8)) << 16;
            std::memcpy(&v[i], &bits, 4);
        }
    } else {
        for (size_t i = 0; i < n; ++i) v[i] = half_to_float((uint16_t)(src[2 * i] | (src[2 * i + 1] << 8)));
    }
    return v.data();
}

}  // namespace sb
