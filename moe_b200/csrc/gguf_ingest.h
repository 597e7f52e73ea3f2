// Reading the expert tensors of a GGUF model file (llama.cpp's container) straight into a resident layer image.
// Host code only. The file is mapped read-only; the tensor directory is parsed once, and every length read from the
// file is checked against the mapping before it is used, so a truncated or corrupt file gives an error string, never a
// fault. Stands where the reference's importer reads the file (gguf.h:345-462, struct Gguf) and walks a block's expert
// tensors (gguf.h:666-694, gg_experts), except that nothing is written back to disk: the Q4_K super-blocks go to the
// GPU as they are and are re-packed there.
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

enum : uint32_t { GGML_F32 = 0, GGML_F16 = 1, GGML_Q4_K = 12, GGML_BF16 = 30 };

// Elements and bytes per block of a ggml tensor type (the published ggml table); false for a type not listed.
inline bool ggml_block(uint32_t type, int& elems, int& bytes) {
    struct Row { uint32_t type; int elems, bytes; };
    static const Row rows[] = {
        {0, 1, 4},     {1, 1, 2},     {2, 32, 18},   {3, 32, 20},   {6, 32, 22},    {7, 32, 24},    {8, 32, 34},
        {9, 32, 36},   {10, 256, 84}, {11, 256, 110}, {12, 256, 144}, {13, 256, 176}, {14, 256, 210}, {15, 256, 292},
        {20, 32, 18},  {23, 256, 136}, {24, 1, 1},    {25, 1, 2},    {26, 1, 4},     {27, 1, 8},     {28, 1, 8},
        {30, 1, 2},
    };
    for (const Row& r : rows)
        if (r.type == type) { elems = r.elems; bytes = r.bytes; return true; }
    return false;
}

struct GgufTensor {
    std::string name;
    uint32_t type = 0;
    int n_dims = 0;
    long long ne[4] = {1, 1, 1, 1};
    const uint8_t* data = nullptr;  // null when the type's block size is unknown
    long long nbytes = 0, row_bytes = 0;
};

}  // namespace moexb

// The handle behind the C ABI.
struct moexb_gguf {
    const uint8_t* base = nullptr;
    uint64_t size = 0;
    uint32_t version = 0;
    uint64_t alignment = 32, data_start = 0;
    std::vector<moexb::GgufTensor> tensors;
    std::unordered_map<std::string, int> by_name;

    ~moexb_gguf() {
        if (base) munmap(const_cast<uint8_t*>(base), size);
    }
    const moexb::GgufTensor* find(const std::string& name) const {
        auto it = by_name.find(name);
        return it == by_name.end() ? nullptr : &tensors[it->second];
    }
};

namespace moexb {

// A bounds-checked cursor over the mapped header. Every read reports failure through `ok`; after a failed read the
// cursor stays where it was and all later reads fail too.
struct GgufCursor {
    const uint8_t* base;
    uint64_t size, pos = 0;
    bool ok = true;
    bool take(uint64_t n, const uint8_t*& p) {
        if (!ok || n > size || pos > size - n) { ok = false; return false; }
        p = base + pos; pos += n;
        return true;
    }
    template <class T> T num() {
        T v{};
        const uint8_t* p;
        if (take(sizeof(T), p)) memcpy(&v, p, sizeof(T));
        return v;
    }
    std::string str() {
        const uint64_t n = num<uint64_t>();
        const uint8_t* p;
        return take(n, p) ? std::string(reinterpret_cast<const char*>(p), n) : std::string();
    }
    // bytes of a scalar metadata value of type ty; 0 for string / array / unknown
    static uint64_t scalar_bytes(uint32_t ty) {
        switch (ty) {
            case 0: case 1: case 7: return 1;
            case 2: case 3: return 2;
            case 4: case 5: case 6: return 4;
            case 10: case 11: case 12: return 8;
        }
        return 0;
    }
    // Steps over one metadata value; when `as_u64` is given and the value is an integer scalar, also returns it.
    bool skip_value(uint32_t ty, uint64_t* as_u64 = nullptr, int depth = 0) {
        const uint8_t* p;
        if (ty == 8) { str(); return ok; }
        if (ty == 9) {
            const uint32_t et = num<uint32_t>();
            const uint64_t n = num<uint64_t>();
            if (!ok || depth > 4) return ok = false;
            if (const uint64_t eb = scalar_bytes(et)) return n <= size / eb && take(n * eb, p);
            if (et != 8 && et != 9) return ok = false;
            for (uint64_t i = 0; i < n && ok; i++) skip_value(et, nullptr, depth + 1);
            return ok;
        }
        const uint64_t b = scalar_bytes(ty);
        if (!b) return ok = false;
        if (!take(b, p)) return false;
        if (as_u64 && (ty <= 5 || ty == 10 || ty == 11)) {
            uint64_t v = 0;
            memcpy(&v, p, b);  // little endian
            *as_u64 = v;
        }
        return true;
    }
};

// Parses the header of a mapped file into g. Returns an empty string, or what is wrong with the file.
inline std::string gguf_parse(moexb_gguf& g) {
    GgufCursor c{g.base, g.size};
    const uint8_t* p;
    if (!c.take(4, p) || memcmp(p, "GGUF", 4)) return "not a GGUF file (no GGUF magic)";
    g.version = c.num<uint32_t>();
    if (!c.ok || (g.version != 2 && g.version != 3)) return "GGUF version " + std::to_string(g.version) + " (versions 2 and 3 are read)";
    const uint64_t n_tensors = c.num<uint64_t>(), n_kv = c.num<uint64_t>();
    if (!c.ok || n_tensors > g.size || n_kv > g.size) return "GGUF header is truncated or corrupt";
    for (uint64_t i = 0; i < n_kv; i++) {
        const std::string key = c.str();
        const uint32_t ty = c.num<uint32_t>();
        uint64_t v = 0;
        const bool want = key == "general.alignment";
        if (!c.skip_value(ty, want ? &v : nullptr)) return "GGUF metadata is truncated or has an unknown value type (key " + key + ")";
        if (want) g.alignment = v;
    }
    if (g.alignment == 0 || (g.alignment & (g.alignment - 1)) || g.alignment > 65536)
        return "GGUF general.alignment " + std::to_string(g.alignment) + " is invalid";
    std::vector<uint64_t> offs;
    g.tensors.reserve(n_tensors);
    for (uint64_t i = 0; i < n_tensors; i++) {
        GgufTensor t;
        t.name = c.str();
        const uint32_t nd = c.num<uint32_t>();
        if (!c.ok) return "GGUF tensor directory is truncated";
        if (nd < 1 || nd > 4) return "tensor " + t.name + " has " + std::to_string(nd) + " dimensions";
        t.n_dims = (int)nd;
        long long n = 1;
        for (uint32_t d = 0; d < nd; d++) {
            const uint64_t e = c.num<uint64_t>();
            // no tensor type packs more than 2 elements into a byte
            if (!c.ok || e == 0 || e > 2 * (g.size + 1) || (uint64_t)n > 2 * (g.size + 1) / e) return "tensor " + t.name + " has an invalid shape";
            t.ne[d] = (long long)e; n *= (long long)e;
        }
        t.type = c.num<uint32_t>();
        offs.push_back(c.num<uint64_t>());
        if (!c.ok) return "GGUF tensor directory is truncated";
        int be, bb;
        if (ggml_block(t.type, be, bb)) {
            if (t.ne[0] % be) return "tensor " + t.name + ": row length is not a whole number of blocks";
            t.row_bytes = t.ne[0] / be * bb;
            t.nbytes = n / t.ne[0] * t.row_bytes;
        }
        g.by_name[t.name] = (int)g.tensors.size();
        g.tensors.push_back(std::move(t));
    }
    g.data_start = (c.pos + g.alignment - 1) / g.alignment * g.alignment;
    for (size_t i = 0; i < g.tensors.size(); i++) {
        GgufTensor& t = g.tensors[i];
        if (!t.row_bytes) continue;  // unknown type: listed, but without data
        if (g.data_start > g.size || offs[i] > g.size - g.data_start || (uint64_t)t.nbytes > g.size - g.data_start - offs[i])
            return "tensor " + t.name + " lies past the end of the file";
        t.data = g.base + g.data_start + offs[i];
    }
    return std::string();
}

// Maps path and parses it. On failure returns null and sets err.
inline moexb_gguf* gguf_open(const char* path, std::string& err) {
    const int fd = open(path, O_RDONLY);
    if (fd < 0) { err = std::string("cannot open ") + path; return nullptr; }
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size <= 0) { close(fd); err = std::string("cannot size ") + path; return nullptr; }
    void* m = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (m == MAP_FAILED) { err = std::string("cannot map ") + path; return nullptr; }
    moexb_gguf* g = new (std::nothrow) moexb_gguf;
    if (!g) { munmap(m, (size_t)st.st_size); err = "out of host memory"; return nullptr; }
    g->base = static_cast<const uint8_t*>(m); g->size = (uint64_t)st.st_size;
    err = gguf_parse(*g);
    if (!err.empty()) { delete g; return nullptr; }
    return g;
}

}  // namespace moexb
