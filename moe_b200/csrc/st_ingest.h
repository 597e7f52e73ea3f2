// Reading the reference engine's own model container: safetensors files (an 8-byte header length, a JSON directory
// {"name": {"dtype": ..., "shape": [...], "data_offsets": [a, b]}, ...}, then the tensor bytes), one per layer, in which
// every expert is two tensors: `...mlp.experts.E.merged_weight` (the packed nibbles [gate | up | down]) and
// `...mlp.experts.E.qs` (the scale part: F32 group scales, or U8 scale / zero-point bytes followed by the half2 pairs).
// Stands where the reference indexes and maps those files (st.h:19-111, struct Container) and takes an expert's two
// pointers from the map (moex.cu:933-939). Host code only; every offset is checked against the file size, and a
// malformed directory gives an error string instead of the reference's exit(1).
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

namespace moexb {

struct StTensorInfo {
    std::string name, dtype;
    std::vector<long long> shape;
    const uint8_t* data = nullptr;
    long long nbytes = 0;
};

// A cursor over the JSON directory. Only what the format uses: objects, arrays, strings, integers (other scalars are
// stepped over). `ok` turns false at the first thing that is not JSON and stays false.
struct JsonCursor {
    const char* p;
    const char* end;
    bool ok = true;
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++; }
    bool peek(char c) { ws(); return ok && p < end && *p == c; }
    bool eat(char c) {
        if (!peek(c)) return ok = false;
        p++;
        return true;
    }
    bool maybe(char c) {
        if (!peek(c)) return false;
        p++;
        return true;
    }
    std::string string() {
        std::string s;
        if (!eat('"')) return s;
        while (p < end && *p != '"') {
            if (*p == '\\' && p + 1 < end) { s += p[1]; p += 2; }  // names here are ASCII: an escape keeps its character
            else s += *p++;
        }
        if (p >= end) ok = false; else p++;
        return s;
    }
    long long integer() {
        ws();
        const char* q = p;
        if (p < end && *p == '-') p++;
        long long v = 0;
        const char* d = p;
        while (p < end && *p >= '0' && *p <= '9') {
            if (v > (INT64_MAX - 9) / 10) { ok = false; return 0; }
            v = v * 10 + (*p++ - '0');
        }
        if (p == d) ok = false;
        return *q == '-' ? -v : v;
    }
    std::vector<long long> integers() {
        std::vector<long long> v;
        if (!eat('[')) return v;
        if (maybe(']')) return v;
        do v.push_back(integer()); while (ok && maybe(','));
        eat(']');
        return v;
    }
    void skip(int depth = 0) {
        ws();
        if (!ok || p >= end || depth > 16) { ok = false; return; }
        if (*p == '"') { string(); return; }
        if (*p == '{' || *p == '[') {
            const char close = *p == '{' ? '}' : ']';
            const bool object = *p == '{';
            p++;
            if (maybe(close)) return;
            do {
                if (object) { string(); eat(':'); }
                skip(depth + 1);
            } while (ok && maybe(','));
            eat(close);
            return;
        }
        const char* q = p;  // number, true, false, null
        while (p < end && *p != ',' && *p != '}' && *p != ']' && *p != ' ' && *p != '\n' && *p != '\t' && *p != '\r') p++;
        if (p == q) ok = false;
    }
};

}  // namespace moexb

// The handle behind the C ABI: one mapped safetensors file.
struct moexb_st {
    const uint8_t* base = nullptr;
    uint64_t size = 0;
    std::vector<moexb::StTensorInfo> tensors;
    std::unordered_map<std::string, int> by_name;
    ~moexb_st() {
        if (base) munmap(const_cast<uint8_t*>(base), size);
    }
    const moexb::StTensorInfo* find(const std::string& name) const {
        auto it = by_name.find(name);
        return it == by_name.end() ? nullptr : &tensors[it->second];
    }
};

namespace moexb {

// Parses the directory of a mapped file into s. Returns an empty string, or what is wrong with the file.
inline std::string st_parse(moexb_st& s) {
    if (s.size < 8) return "not a safetensors file (shorter than its header length)";
    uint64_t n = 0;
    memcpy(&n, s.base, 8);
    if (n < 2 || n > s.size - 8) return "safetensors header length " + std::to_string(n) + " exceeds the file";
    const uint64_t data_bytes = s.size - 8 - n;
    const uint8_t* data = s.base + 8 + n;
    JsonCursor c{reinterpret_cast<const char*>(s.base) + 8, reinterpret_cast<const char*>(s.base) + 8 + n};
    if (!c.eat('{')) return "safetensors header is not a JSON object";
    if (!c.maybe('}')) {
        do {
            StTensorInfo t;
            t.name = c.string();
            c.eat(':');
            if (!c.ok) break;
            if (t.name == "__metadata__") { c.skip(); continue; }
            std::vector<long long> offs;
            bool have_offs = false;
            c.eat('{');
            if (!c.maybe('}')) {
                do {
                    const std::string k = c.string();
                    c.eat(':');
                    if (k == "dtype") t.dtype = c.string();
                    else if (k == "shape") t.shape = c.integers();
                    else if (k == "data_offsets") { offs = c.integers(); have_offs = true; }
                    else c.skip();
                } while (c.ok && c.maybe(','));
                c.eat('}');
            }
            if (!c.ok) break;
            if (!have_offs || offs.size() != 2 || offs[0] < 0 || offs[1] < offs[0] || (uint64_t)offs[1] > data_bytes)
                return "tensor " + t.name + " has data offsets outside the file";
            for (long long d : t.shape)
                if (d < 0) return "tensor " + t.name + " has a negative dimension";
            t.data = data + offs[0];
            t.nbytes = offs[1] - offs[0];
            s.by_name[t.name] = (int)s.tensors.size();
            s.tensors.push_back(std::move(t));
        } while (c.ok && c.maybe(','));
        c.eat('}');
    }
    if (!c.ok) return "safetensors header is not the JSON directory the format describes (near byte " + std::to_string(c.p - reinterpret_cast<const char*>(s.base)) + ")";
    return std::string();
}

inline moexb_st* st_open(const char* path, std::string& err) {
    const int fd = open(path, O_RDONLY);
    if (fd < 0) { err = std::string("cannot open ") + path; return nullptr; }
    struct stat sb;
    if (fstat(fd, &sb) != 0 || sb.st_size <= 0) { close(fd); err = std::string("cannot size ") + path; return nullptr; }
    void* m = mmap(nullptr, (size_t)sb.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (m == MAP_FAILED) { err = std::string("cannot map ") + path; return nullptr; }
    moexb_st* s = new (std::nothrow) moexb_st;
    if (!s) { munmap(m, (size_t)sb.st_size); err = "out of host memory"; return nullptr; }
    s->base = static_cast<const uint8_t*>(m); s->size = (uint64_t)sb.st_size;
    err = st_parse(*s);
    if (!err.empty()) { delete s; return nullptr; }
    return s;
}

}  // namespace moexb
