// GGUF container reader: header, metadata, tensor table, and the upload of the data
// region into one device allocation.  Replaces GGUF.init (LLM/Base/GGUF.swift:92-158) and
// the buffer windows of MetalContext (LLM/Base/MetalContext.swift:114-185): the file is
// mapped read-only, every tensor is (name, dims with dims[0] fastest, ggml type, byte
// offset from the start of the data region, byte count), and okf_gguf_upload copies the
// data region to the GPU so that a tensor's offset is the `woff` of the matvec / matmul
// calls, as WeightRef.local is in the reference.
//
// Host code only (no kernels); it lives in a .cu file so that one compiler builds the
// whole library.
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <new>
#include <string>
#include <unordered_map>
#include <vector>

#include "okf_internal.h"

namespace {

// GGUF.rowByteCount (LLM/Base/GGUF.swift:160-188): bytes of n elements of a type, and
// whether the type id is one the reference's GGUFType knows (LLM/Base/GGUF.swift:3-14).
bool type_bytes(int32_t ty, uint64_t n, uint64_t *bytes) {
    struct { int32_t ty; uint32_t per, size; } const table[] = {
        {0, 1, 4},      {1, 1, 2},      {30, 1, 2},                                    // f32, f16, bf16
        {2, 32, 18},    {3, 32, 20},    {6, 32, 22},    {7, 32, 24},    {8, 32, 34},   // q4_0 q4_1 q5_0 q5_1 q8_0
        {10, 256, 84},  {11, 256, 110}, {12, 256, 144}, {13, 256, 176}, {14, 256, 210}, {15, 256, 292},  // k-quants
        {16, 256, 66},  {17, 256, 74},  {18, 256, 98},  {19, 256, 50},  {20, 32, 18},  // iq2_xxs iq2_xs iq3_xxs iq1_s iq4_nl
        {21, 256, 110}, {22, 256, 82},  {23, 256, 136}, {29, 256, 56},                 // iq3_s iq2_s iq4_xs iq1_m
        {41, 128, 18},  {42, 128, 34},                                                 // PrismML q1_0, q2_0
    };
    for (const auto &t : table)
        if (t.ty == ty) {
            *bytes = n / t.per * t.size;
            return true;
        }
    // the reference's q8_1 and any integer type fall to "n bytes"; unknown ids are an error
    if (ty == 9) { *bytes = n; return true; }
    return false;
}

struct Value {
    int kind = 0;  // 1 int, 2 double, 3 string, 4 bool, 5 ints, 6 doubles, 7 strings
    int64_t i = 0;
    double d = 0;
    const char *s = nullptr;  // into the mapping, not terminated
    uint64_t len = 0;         // string length, or array count
    std::vector<int64_t> ints;
    std::vector<double> doubles;
    uint64_t table_off = 0;   // strings: where the first length prefix sits in the file
};

struct Tensor {
    std::string name;
    uint32_t nd = 0;
    uint64_t dims[4] = {1, 1, 1, 1};
    int32_t type = 0;
    uint64_t off = 0, bytes = 0;
};

// Reads from the mapping; any read past the end sets `bad` and yields zeros.
struct Cursor {
    const uint8_t *base;
    uint64_t limit, pos = 0;
    bool bad = false;
    template <typename T> T get() {
        T v{};
        if (bad || pos + sizeof(T) > limit) { bad = true; return v; }
        memcpy(&v, base + pos, sizeof(T));
        pos += sizeof(T);
        return v;
    }
    bool str(const char **s, uint64_t *n) {
        *n = get<uint64_t>();
        if (bad || *n > limit - pos) { bad = true; *n = 0; return false; }
        *s = (const char *)(base + pos);
        pos += *n;
        return true;
    }
};

}  // namespace

struct okf_gguf {
    int fd = -1;
    const uint8_t *map = nullptr;
    uint64_t size = 0, data_start = 0, alignment = 32;
    uint32_t version = 0;
    std::vector<Tensor> tensors;
    std::unordered_map<std::string, size_t> by_name;
    std::unordered_map<std::string, Value> meta;
    std::vector<std::string> meta_keys;
};

namespace {

// One metadata value of GGUF value type `vt` (0 u8 .. 12 f64, 8 string, 9 array).
bool read_value(Cursor &c, uint32_t vt, Value &v, int depth) {
    switch (vt) {
    case 0: v.kind = 1; v.i = c.get<uint8_t>(); break;
    case 1: v.kind = 1; v.i = c.get<int8_t>(); break;
    case 2: v.kind = 1; v.i = c.get<uint16_t>(); break;
    case 3: v.kind = 1; v.i = c.get<int16_t>(); break;
    case 4: v.kind = 1; v.i = c.get<uint32_t>(); break;
    case 5: v.kind = 1; v.i = c.get<int32_t>(); break;
    case 10: v.kind = 1; v.i = (int64_t)c.get<uint64_t>(); break;
    case 11: v.kind = 1; v.i = c.get<int64_t>(); break;
    case 6: v.kind = 2; v.d = c.get<float>(); break;
    case 12: v.kind = 2; v.d = c.get<double>(); break;
    case 7: v.kind = 4; v.i = c.get<uint8_t>() != 0; break;
    case 8: v.kind = 3; c.str(&v.s, &v.len); break;
    case 9: {
        if (depth > 0) return false;  // arrays of arrays do not occur in model files
        const uint32_t et = c.get<uint32_t>();
        const uint64_t n = c.get<uint64_t>();
        if (c.bad || n > c.limit) return false;
        v.len = n;
        if (et == 8) {  // a string table stays in the mapping (token lists are large)
            v.kind = 7;
            v.table_off = c.pos;
            for (uint64_t i = 0; i < n && !c.bad; i++) {
                const char *s; uint64_t len;
                c.str(&s, &len);
            }
        } else if (et == 6 || et == 12) {
            v.kind = 6;
            v.doubles.reserve(n);
            for (uint64_t i = 0; i < n && !c.bad; i++) v.doubles.push_back(et == 6 ? (double)c.get<float>() : c.get<double>());
        } else {
            v.kind = 5;
            v.ints.reserve(n);
            for (uint64_t i = 0; i < n && !c.bad; i++) {
                Value e;
                if (!read_value(c, et, e, 1) || (e.kind != 1 && e.kind != 4)) return false;
                v.ints.push_back(e.i);
            }
        }
        break;
    }
    default: return false;
    }
    return !c.bad;
}

int parse(okf_gguf *g) {
    Cursor c{g->map, g->size};
    if (c.get<uint32_t>() != 0x46554747u) return OKF_E_FORMAT;  // "GGUF"
    g->version = c.get<uint32_t>();
    const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
    if (c.bad || n_tensors > g->size || n_kv > g->size) return OKF_E_FORMAT;
    for (uint64_t i = 0; i < n_kv; i++) {
        const char *k; uint64_t kn;
        if (!c.str(&k, &kn)) return OKF_E_FORMAT;
        Value v;
        if (!read_value(c, c.get<uint32_t>(), v, 0)) return OKF_E_FORMAT;
        std::string key(k, kn);
        if (key == "general.alignment" && v.kind == 1 && v.i > 0) g->alignment = (uint64_t)v.i;
        g->meta_keys.push_back(key);
        g->meta[key] = std::move(v);
    }
    g->tensors.reserve(n_tensors);
    for (uint64_t i = 0; i < n_tensors; i++) {
        Tensor t;
        const char *s; uint64_t sn;
        if (!c.str(&s, &sn)) return OKF_E_FORMAT;
        t.name.assign(s, sn);
        t.nd = c.get<uint32_t>();
        if (c.bad || t.nd > 4) return OKF_E_FORMAT;
        uint64_t count = 1;
        for (uint32_t d = 0; d < t.nd; d++) {
            t.dims[d] = c.get<uint64_t>();
            if (t.dims[d] && count > UINT64_MAX / t.dims[d]) return OKF_E_FORMAT;
            count *= t.dims[d];
        }
        t.type = (int32_t)c.get<uint32_t>();
        t.off = c.get<uint64_t>();
        if (c.bad) return OKF_E_FORMAT;
        if (!type_bytes(t.type, count, &t.bytes)) return OKF_E_TYPE;  // "unknown ggml type" in the reference
        g->by_name[t.name] = g->tensors.size();
        g->tensors.push_back(std::move(t));
    }
    g->data_start = (c.pos + g->alignment - 1) / g->alignment * g->alignment;
    if (g->data_start > g->size) return n_tensors ? OKF_E_RANGE : OKF_OK;
    for (const Tensor &t : g->tensors)
        if (t.off > g->size - g->data_start || t.bytes > g->size - g->data_start - t.off) return OKF_E_RANGE;
    return OKF_OK;
}

void fill(const okf_gguf *g, const Tensor &t, okf_gguf_tensor *out) {
    out->name = t.name.c_str();
    out->n_dims = t.nd;
    for (int d = 0; d < 4; d++) out->dims[d] = t.dims[d];
    out->type = t.type;
    out->offset = t.off;
    out->bytes = t.bytes;
    out->host = g->map + g->data_start + t.off;
}

}  // namespace

extern "C" {

int okf_gguf_open(const char *path, okf_gguf **out) {
    if (!path || !out) return OKF_E_ARG;
    *out = nullptr;
    okf_gguf *g = new (std::nothrow) okf_gguf();
    if (!g) return OKF_E_NOMEM;
    struct stat st;
    g->fd = open(path, O_RDONLY);
    if (g->fd < 0 || fstat(g->fd, &st) != 0 || st.st_size < 24) {
        if (g->fd >= 0) close(g->fd);
        const bool small = g->fd >= 0;
        delete g;
        return small ? OKF_E_FORMAT : OKF_E_IO;
    }
    g->size = (uint64_t)st.st_size;
    void *p = mmap(nullptr, g->size, PROT_READ, MAP_PRIVATE, g->fd, 0);
    if (p == MAP_FAILED) {
        close(g->fd);
        delete g;
        return OKF_E_IO;
    }
    g->map = (const uint8_t *)p;
    int rc;
    try {
        rc = parse(g);
    } catch (const std::bad_alloc &) {
        rc = OKF_E_NOMEM;
    }
    if (rc) {
        okf_gguf_close(g);
        return rc;
    }
    *out = g;
    return OKF_OK;
}

void okf_gguf_close(okf_gguf *g) {
    if (!g) return;
    if (g->map) munmap((void *)g->map, g->size);
    if (g->fd >= 0) close(g->fd);
    delete g;
}

uint64_t okf_gguf_tensor_count(const okf_gguf *g) { return g ? g->tensors.size() : 0; }
uint64_t okf_gguf_data_offset(const okf_gguf *g) { return g ? g->data_start : 0; }
uint64_t okf_gguf_data_bytes(const okf_gguf *g) { return g && g->size > g->data_start ? g->size - g->data_start : 0; }
uint32_t okf_gguf_version(const okf_gguf *g) { return g ? g->version : 0; }

int okf_gguf_tensor_at(const okf_gguf *g, uint64_t index, okf_gguf_tensor *out) {
    if (!g || !out) return OKF_E_ARG;
    if (index >= g->tensors.size()) return OKF_E_RANGE;
    fill(g, g->tensors[index], out);
    return OKF_OK;
}

int okf_gguf_find(const okf_gguf *g, const char *name, okf_gguf_tensor *out) {
    if (!g || !name || !out) return OKF_E_ARG;
    auto it = g->by_name.find(name);
    if (it == g->by_name.end()) return OKF_E_RANGE;
    fill(g, g->tensors[it->second], out);
    return OKF_OK;
}

uint64_t okf_gguf_meta_count(const okf_gguf *g) { return g ? g->meta_keys.size() : 0; }
const char *okf_gguf_meta_key(const okf_gguf *g, uint64_t index) {
    return g && index < g->meta_keys.size() ? g->meta_keys[index].c_str() : nullptr;
}

int okf_gguf_meta_kind(const okf_gguf *g, const char *key) {
    if (!g || !key) return 0;
    auto it = g->meta.find(key);
    return it == g->meta.end() ? 0 : it->second.kind;
}

int okf_gguf_meta_int(const okf_gguf *g, const char *key, int64_t *out) {
    if (!g || !key || !out) return OKF_E_ARG;
    auto it = g->meta.find(key);
    if (it == g->meta.end()) return OKF_E_RANGE;
    if (it->second.kind != 1 && it->second.kind != 4) return OKF_E_TYPE;
    *out = it->second.i;
    return OKF_OK;
}

int okf_gguf_meta_double(const okf_gguf *g, const char *key, double *out) {
    if (!g || !key || !out) return OKF_E_ARG;
    auto it = g->meta.find(key);
    if (it == g->meta.end()) return OKF_E_RANGE;
    if (it->second.kind == 2) *out = it->second.d;
    else if (it->second.kind == 1) *out = (double)it->second.i;
    else return OKF_E_TYPE;
    return OKF_OK;
}

int okf_gguf_meta_string(const okf_gguf *g, const char *key, const char **out, uint64_t *len) {
    if (!g || !key || !out || !len) return OKF_E_ARG;
    auto it = g->meta.find(key);
    if (it == g->meta.end()) return OKF_E_RANGE;
    if (it->second.kind != 3) return OKF_E_TYPE;
    *out = it->second.s;
    *len = it->second.len;
    return OKF_OK;
}

int okf_gguf_meta_array(const okf_gguf *g, const char *key, uint64_t *count, const int64_t **ints,
                        const double **doubles) {
    if (!g || !key || !count) return OKF_E_ARG;
    auto it = g->meta.find(key);
    if (it == g->meta.end()) return OKF_E_RANGE;
    const Value &v = it->second;
    if (v.kind < 5) return OKF_E_TYPE;
    *count = v.len;
    if (ints) *ints = v.kind == 5 ? v.ints.data() : nullptr;
    if (doubles) *doubles = v.kind == 6 ? v.doubles.data() : nullptr;
    return OKF_OK;
}

int okf_gguf_meta_string_at(const okf_gguf *g, const char *key, uint64_t index, const char **out, uint64_t *len) {
    if (!g || !key || !out || !len) return OKF_E_ARG;
    auto it = g->meta.find(key);
    if (it == g->meta.end()) return OKF_E_RANGE;
    const Value &v = it->second;
    if (v.kind != 7) return OKF_E_TYPE;
    if (index >= v.len) return OKF_E_RANGE;
    // the table was walked once when the file was opened, so every length is in range
    uint64_t at = v.table_off;
    for (uint64_t i = 0;; i++) {
        uint64_t n;
        memcpy(&n, g->map + at, 8);
        if (i == index) {
            *out = (const char *)(g->map + at + 8);
            *len = n;
            return OKF_OK;
        }
        at += 8 + n;
    }
}

int okf_gguf_upload(okf_ctx *ctx, const okf_gguf *g, okf_weights **out) {
    if (!ctx || !g || !out) return OKF_E_ARG;
    return okf_weights_upload(ctx, g->map + g->data_start, okf_gguf_data_bytes(g), out);
}

}  // extern "C"
