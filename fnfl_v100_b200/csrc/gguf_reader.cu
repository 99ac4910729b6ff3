// Host-only: a minimal GGUF (v2 / v3) tensor-directory reader, enough to find a quantised tensor such as
// token_embd.weight in a model file and read whole rows of it into caller memory for upload.  It plays the part of the
// reference's fn/borrowed/gguf_tensors.h + fn/loader row slicing for this path only: no metadata interpretation, no
// memory mapping, no device work.  Layout per the GGUF specification: header {magic "GGUF", version, tensor count,
// key/value count}, key/value pairs (skipped, except general.alignment), tensor infos {name, n_dims, dims[], ggml type,
// offset}, padding to the alignment, tensor data.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/fnb200.h"

namespace {

inline bool mul_ok(uint64_t a, uint64_t b, uint64_t & out) { return !__builtin_mul_overflow(a, b, &out); }
inline bool add_ok(uint64_t a, uint64_t b, uint64_t & out) { return !__builtin_add_overflow(a, b, &out); }

struct tensor_rec {
    std::string name;
    fnb_gguf_tensor t;
};

struct reader {
    FILE * f = nullptr;
    uint64_t data_start = 0;
    uint64_t file_size = 0;
    std::vector<tensor_rec> tensors;
};

bool rd(FILE * f, void * p, size_t n) { return std::fread(p, 1, n, f) == n; }
template <typename T>
bool rd(FILE * f, T & v) {
    return rd(f, &v, sizeof(T));
}
bool rd_str(FILE * f, std::string & s, uint64_t limit) {
    uint64_t n = 0;
    if (!rd(f, n) || n > limit) return false;
    s.resize(size_t(n));
    return n == 0 || rd(f, &s[0], size_t(n));
}

// bytes of a scalar GGUF metadata value type, 0 for string / array / unknown
size_t scalar_bytes(uint32_t t) {
    switch (t) {
        case 0: case 1: case 7: return 1;   // u8, i8, bool
        case 2: case 3: return 2;           // u16, i16
        case 4: case 5: case 6: return 4;   // u32, i32, f32
        case 10: case 11: case 12: return 8;  // u64, i64, f64
        default: return 0;
    }
}

bool skip_value(FILE * f, uint32_t type, uint64_t file_size, uint64_t * as_u64) {
    if (const size_t n = scalar_bytes(type)) {
        uint64_t v = 0;
        if (!rd(f, &v, n)) return false;
        if (as_u64 != nullptr) *as_u64 = v;
        return true;
    }
    if (type == 8) {  // string
        std::string s;
        return rd_str(f, s, file_size);
    }
    if (type == 9) {  // array: element type, count, elements
        uint32_t et = 0;
        uint64_t cnt = 0;
        if (!rd(f, et) || !rd(f, cnt) || cnt > file_size) return false;
        if (const size_t n = scalar_bytes(et)) {  // cnt <= file_size and n <= 8: the product cannot wrap
            return cnt * n <= file_size && fseeko(f, off_t(cnt * n), SEEK_CUR) == 0;
        }
        for (uint64_t i = 0; i < cnt; ++i) {
            if (!skip_value(f, et, file_size, nullptr)) return false;
        }
        return true;
    }
    return false;
}

// block geometry of the ggml types this library decodes (ggml/include/ggml.h type numbers)
bool block_of(uint32_t type, uint32_t & values, uint32_t & bytes) {
    switch (type) {
        case 0: values = 1, bytes = 4; return true;      // F32
        case 1: values = 1, bytes = 2; return true;      // F16
        case 8: values = 32, bytes = 34; return true;    // Q8_0
        case 12: values = 256, bytes = 144; return true;  // Q4_K
        case 18: values = 256, bytes = 98; return true;   // IQ3_XXS
        case 21: values = 256, bytes = 110; return true;  // IQ3_S
        default: return false;
    }
}

}  // namespace

extern "C" fnb_gguf * fnb_gguf_open(const char * path) {
    if (path == nullptr) return nullptr;
    reader * r = new reader;
    r->f = std::fopen(path, "rb");
    if (r->f == nullptr) {
        delete r;
        return nullptr;
    }
    bool ok = std::fseek(r->f, 0, SEEK_END) == 0;
    r->file_size = ok ? uint64_t(std::ftell(r->f)) : 0;
    ok = ok && std::fseek(r->f, 0, SEEK_SET) == 0;
    uint32_t magic = 0, version = 0;
    uint64_t n_tensors = 0, n_kv = 0, alignment = 32;
    ok = ok && rd(r->f, magic) && magic == 0x46554747u && rd(r->f, version) && (version == 2 || version == 3);
    ok = ok && rd(r->f, n_tensors) && rd(r->f, n_kv) && n_tensors < (1u << 24) && n_kv < (1u << 24);
    for (uint64_t i = 0; ok && i < n_kv; ++i) {
        std::string key;
        uint32_t type = 0;
        uint64_t v = 0;
        ok = rd_str(r->f, key, 1 << 16) && rd(r->f, type) && skip_value(r->f, type, r->file_size, &v);
        if (ok && key == "general.alignment" && v >= 1 && v <= 4096 && (v & (v - 1)) == 0) alignment = v;
    }
    for (uint64_t i = 0; ok && i < n_tensors; ++i) {
        tensor_rec t;
        std::memset(&t.t, 0, sizeof t.t);
        uint32_t n_dims = 0;
        ok = rd_str(r->f, t.name, 1 << 16) && rd(r->f, n_dims) && n_dims >= 1 && n_dims <= 4;
        for (uint32_t d = 0; ok && d < 4; ++d) {
            uint64_t e = 1;
            if (d < n_dims) ok = rd(r->f, e) && e >= 1;
            t.t.ne[d] = int64_t(e);
        }
        uint32_t type = 0;
        uint64_t off = 0;
        ok = ok && rd(r->f, type) && rd(r->f, off);
        t.t.n_dims = int32_t(n_dims);
        t.t.type = int32_t(type);
        t.t.offset = int64_t(off);
        uint32_t bv = 0, bb = 0;
        if (ok && block_of(type, bv, bb) && uint64_t(t.t.ne[0]) % bv == 0) {
            // every product checked: a hostile or corrupt directory must not wrap its way past the bounds test below
            uint64_t rows = 0, row_bytes = 0;
            ok = mul_ok(uint64_t(t.t.ne[1]), uint64_t(t.t.ne[2]), rows) && mul_ok(rows, uint64_t(t.t.ne[3]), rows) &&
                 mul_ok(uint64_t(t.t.ne[0]) / bv, bb, row_bytes) && rows <= uint64_t(INT64_MAX) && row_bytes <= uint64_t(INT64_MAX);
            t.t.row_bytes = int64_t(row_bytes);
            t.t.n_rows = int64_t(rows);
        }  // else row_bytes stays 0: a type this library does not decode
        ok = ok && off % alignment == 0 && off <= uint64_t(INT64_MAX);
        if (ok) r->tensors.push_back(t);
    }
    if (ok) {
        const uint64_t here = uint64_t(std::ftell(r->f));
        r->data_start = (here + alignment - 1) / alignment * alignment;
        for (const tensor_rec & t : r->tensors) {
            uint64_t bytes = 0, end = 0;
            if (t.t.row_bytes > 0 &&
                !(mul_ok(uint64_t(t.t.row_bytes), uint64_t(t.t.n_rows), bytes) && add_ok(r->data_start, uint64_t(t.t.offset), end) &&
                  add_ok(end, bytes, end) && end <= r->file_size)) {
                ok = false;  // a tensor that runs past the end of the file, or whose size does not fit 64 bits
            }
        }
    }
    if (!ok) {
        std::fclose(r->f);
        delete r;
        return nullptr;
    }
    return reinterpret_cast<fnb_gguf *>(r);
}

extern "C" void fnb_gguf_close(fnb_gguf * g) {
    if (g == nullptr) return;
    reader * r = reinterpret_cast<reader *>(g);
    std::fclose(r->f);
    delete r;
}

extern "C" int64_t fnb_gguf_n_tensors(const fnb_gguf * g) {
    return g == nullptr ? -1 : int64_t(reinterpret_cast<const reader *>(g)->tensors.size());
}

extern "C" int32_t fnb_gguf_find(const fnb_gguf * g, const char * name, fnb_gguf_tensor * out) {
    if (g == nullptr || name == nullptr || out == nullptr) return FNB_REJECTED;
    for (const tensor_rec & t : reinterpret_cast<const reader *>(g)->tensors) {
        if (t.name == name) {
            *out = t.t;
            return FNB_OK;
        }
    }
    return FNB_REJECTED;
}

extern "C" int32_t fnb_gguf_read_rows(fnb_gguf * g, const fnb_gguf_tensor * t, int64_t row0, int64_t n_rows, void * dst) {
    if (g == nullptr || t == nullptr || dst == nullptr || t->row_bytes <= 0 || t->offset < 0 || t->n_rows < 0) return FNB_REJECTED;
    if (row0 < 0 || n_rows < 1 || row0 > t->n_rows || n_rows > t->n_rows - row0) return FNB_REJECTED;
    reader * r = reinterpret_cast<reader *>(g);
    // the descriptor is the caller's: it is checked against the file again, whatever the directory said
    uint64_t skip = 0, at = 0, bytes = 0, end = 0;
    if (!mul_ok(uint64_t(row0), uint64_t(t->row_bytes), skip) || !add_ok(r->data_start, uint64_t(t->offset), at) ||
        !add_ok(at, skip, at) || !mul_ok(uint64_t(n_rows), uint64_t(t->row_bytes), bytes) || !add_ok(at, bytes, end) ||
        end > r->file_size || at > uint64_t(INT64_MAX)) {
        return FNB_REJECTED;
    }
    if (fseeko(r->f, off_t(at), SEEK_SET) != 0) return FNB_REJECTED;
    return rd(r->f, dst, size_t(bytes)) ? FNB_OK : FNB_REJECTED;
}
