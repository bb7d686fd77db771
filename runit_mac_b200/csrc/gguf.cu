// GGUF reader and packed-weight upload (C ABI in include/runit_gguf.h).
//
// File layout (GGUF v2 / v3, little endian): magic "GGUF", u32 version, u64 tensor count, u64 metadata count; the metadata
// KV pairs (string key, u32 value type, value; strings are u64 length + bytes, arrays are u32 element type + u64 count +
// elements); the tensor index (string name, u32 n_dims, u64 dims, u32 ggml type, u64 offset into the data region); the
// data region starts at the next multiple of `general.alignment` (default 32).  Behaviour follows
// crates/gguf/src/parser.rs:22-227 and the type tables of crates/gguf/src/types.rs:105-199; the tensor bytes are never
// converted: the fused-dequant kernels read the packed Q8_0 / Q4_0 / Q4_K blocks as they are stored.
#include <cuda_runtime.h>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "runit_gguf.h"
#include "runit_internal.h"

namespace {

thread_local char g_err[512] = "";

int32_t gg_fail(int32_t code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return code;
}

struct DtypeRow {
    uint32_t id;
    const char* name;
    uint32_t block, size;
};
// ggml type ids with elements per block and bytes per block (crates/gguf/src/types.rs:105-190)
const DtypeRow kDtypes[] = {
    {0, "F32", 1, 4},       {1, "F16", 1, 2},       {2, "Q4_0", 32, 18},     {3, "Q4_1", 32, 20},     {6, "Q5_0", 32, 22},
    {7, "Q5_1", 32, 24},    {8, "Q8_0", 32, 34},    {9, "Q8_1", 32, 40},     {10, "Q2_K", 256, 84},   {11, "Q3_K", 256, 110},
    {12, "Q4_K", 256, 144}, {13, "Q5_K", 256, 176}, {14, "Q6_K", 256, 210},  {15, "Q8_K", 256, 292},  {16, "IQ2_XXS", 256, 66},
    {17, "IQ2_XS", 256, 74}, {18, "IQ3_XXS", 256, 98}, {19, "IQ1_S", 256, 50}, {20, "IQ4_NL", 32, 18}, {21, "IQ3_S", 256, 110},
    {22, "IQ2_S", 256, 82}, {23, "IQ4_XS", 32, 36}, {24, "I8", 1, 1},        {25, "I16", 1, 2},       {26, "I32", 1, 4},
    {27, "I64", 1, 8},      {28, "F64", 1, 8},      {29, "IQ1_M", 256, 56},  {30, "BF16", 1, 2},
};
const DtypeRow* dtype_row(uint32_t id) {
    for (const DtypeRow& r : kDtypes)
        if (r.id == id) return &r;
    return nullptr;
}

struct Value {
    uint32_t type = 0, elem_type = 0;
    uint64_t u = 0;             // integers (two's complement for the signed ones) and bool
    double f = 0.0;             // floats
    std::string s;              // string
    std::vector<Value> arr;     // array
};

struct Tensor {
    std::string name;
    uint32_t dtype = 0, n_dims = 0;
    uint64_t ne[4] = {1, 1, 1, 1};
    uint64_t offset = 0, n_elem = 1, bytes = 0;
};

}  // namespace

struct runit_gguf {
    int fd = -1;                       // file-backed
    const uint8_t* image = nullptr;    // memory-backed
    uint64_t size = 0;
    uint32_t version = 0;
    uint64_t alignment = RUNIT_GGUF_DEFAULT_ALIGNMENT, data_offset = 0;
    std::vector<std::string> keys;     // file order
    std::unordered_map<std::string, Value> meta;
    std::vector<Tensor> tensors;
    std::unordered_map<std::string, size_t> by_name;
    void* pinned[2] = {nullptr, nullptr};
    cudaEvent_t ev[2] = {nullptr, nullptr};
};

namespace {

constexpr uint64_t kChunk = 32ull << 20;   // staging buffer size of the upload

// Sequential little-endian reader over the file or the memory image, with the reference's end-of-file report
// (crates/gguf/src/error.rs:20-25).
struct Reader {
    runit_gguf* g;
    uint64_t pos = 0;
    int32_t err = RUNIT_GGUF_OK;
    std::vector<uint8_t> buf;          // read-ahead window of a file
    uint64_t buf_pos = 0;

    bool raw(void* dst, uint64_t n) {
        if (err) return false;
        if (n > g->size || pos > g->size - n) {
            err = gg_fail(RUNIT_GGUF_ERR_UNEXPECTED_EOF, "unexpected end of file at offset %llu (need %llu bytes, have %llu)",
                          (unsigned long long)pos, (unsigned long long)n, (unsigned long long)(g->size - (pos > g->size ? g->size : pos)));
            return false;
        }
        if (g->image) {
            memcpy(dst, g->image + pos, n);
        } else {
            uint8_t* d = static_cast<uint8_t*>(dst);
            uint64_t done = 0;
            while (done < n) {
                if (pos + done < buf_pos || pos + done >= buf_pos + buf.size()) {
                    buf_pos = pos + done;
                    const uint64_t want = g->size - buf_pos < (1u << 20) ? g->size - buf_pos : (1u << 20);
                    buf.resize(want);
                    uint64_t got = 0;
                    while (got < want) {
                        const ssize_t r = pread(g->fd, buf.data() + got, want - got, (off_t)(buf_pos + got));
                        if (r <= 0) {
                            err = gg_fail(RUNIT_GGUF_ERR_IO, "I/O error: read of %llu bytes at offset %llu failed",
                                          (unsigned long long)(want - got), (unsigned long long)(buf_pos + got));
                            return false;
                        }
                        got += (uint64_t)r;
                    }
                }
                const uint64_t off = pos + done - buf_pos;
                const uint64_t take = buf.size() - off < n - done ? buf.size() - off : n - done;
                memcpy(d + done, buf.data() + off, take);
                done += take;
            }
        }
        pos += n;
        return true;
    }
    template <typename T>
    T num() {
        T v{};
        raw(&v, sizeof v);
        return v;
    }
    bool str(std::string* out) {
        const uint64_t at = pos;
        const uint64_t len = num<uint64_t>();
        if (err) return false;
        if (len > g->size) {   // cannot be satisfied: report it as the read that would fail
            err = gg_fail(RUNIT_GGUF_ERR_UNEXPECTED_EOF, "unexpected end of file at offset %llu (need %llu bytes, have %llu)",
                          (unsigned long long)pos, (unsigned long long)len, (unsigned long long)(g->size - pos));
            return false;
        }
        out->resize(len);
        if (len && !raw(&(*out)[0], len)) return false;
        // well-formed UTF-8 only (String::from_utf8 in the reference)
        const unsigned char* p = reinterpret_cast<const unsigned char*>(out->data());
        uint64_t i = 0;
        while (i < len) {
            const unsigned c = p[i];
            int extra;
            unsigned minv;
            if (c < 0x80) { i++; continue; }
            else if ((c & 0xE0) == 0xC0) { extra = 1; minv = 0x80; }
            else if ((c & 0xF0) == 0xE0) { extra = 2; minv = 0x800; }
            else if ((c & 0xF8) == 0xF0) { extra = 3; minv = 0x10000; }
            else { extra = -1; minv = 0; }
            bool ok = extra > 0 && i + (uint64_t)extra < len;   // all continuation bytes inside the string
            unsigned cp = ok ? (c & (0xFFu >> (extra + 2))) : 0;
            for (int k = 1; ok && k <= extra; k++) {
                if ((p[i + k] & 0xC0) != 0x80) ok = false;
                else cp = (cp << 6) | (p[i + k] & 0x3Fu);
            }
            if (ok && (cp < minv || cp > 0x10FFFF || (cp >= 0xD800 && cp <= 0xDFFF))) ok = false;
            if (!ok) {
                err = gg_fail(RUNIT_GGUF_ERR_INVALID_UTF8, "invalid UTF-8 string in metadata at offset %llu", (unsigned long long)at);
                return false;
            }
            i += (uint64_t)extra + 1;
        }
        return true;
    }
};

bool read_value(Reader& r, uint32_t type, Value* v, int depth) {
    v->type = type;
    switch (type) {
        case RUNIT_GGUF_META_UINT8: v->u = r.num<uint8_t>(); break;
        case RUNIT_GGUF_META_INT8: v->u = (uint64_t)(int64_t)r.num<int8_t>(); break;
        case RUNIT_GGUF_META_UINT16: v->u = r.num<uint16_t>(); break;
        case RUNIT_GGUF_META_INT16: v->u = (uint64_t)(int64_t)r.num<int16_t>(); break;
        case RUNIT_GGUF_META_UINT32: v->u = r.num<uint32_t>(); break;
        case RUNIT_GGUF_META_INT32: v->u = (uint64_t)(int64_t)r.num<int32_t>(); break;
        case RUNIT_GGUF_META_FLOAT32: v->f = r.num<float>(); break;
        case RUNIT_GGUF_META_BOOL: v->u = r.num<uint8_t>() != 0; break;
        case RUNIT_GGUF_META_STRING: r.str(&v->s); break;
        case RUNIT_GGUF_META_UINT64: v->u = r.num<uint64_t>(); break;
        case RUNIT_GGUF_META_INT64: v->u = (uint64_t)r.num<int64_t>(); break;
        case RUNIT_GGUF_META_FLOAT64: v->f = r.num<double>(); break;
        case RUNIT_GGUF_META_ARRAY: {
            const uint32_t et = r.num<uint32_t>();
            if (r.err) return false;
            if (et > RUNIT_GGUF_META_FLOAT64) {
                r.err = gg_fail(RUNIT_GGUF_ERR_UNKNOWN_METADATA_TYPE, "unknown metadata value type: %u", et);
                return false;
            }
            if (et == RUNIT_GGUF_META_ARRAY && depth >= 4) {
                r.err = gg_fail(RUNIT_GGUF_ERR_UNKNOWN_METADATA_TYPE, "unknown metadata value type: %u (arrays nested too deep)", et);
                return false;
            }
            v->elem_type = et;
            const uint64_t count = r.num<uint64_t>();
            if (r.err) return false;
            if (count > r.g->size) {   // every element takes at least one byte
                r.err = gg_fail(RUNIT_GGUF_ERR_UNEXPECTED_EOF, "unexpected end of file at offset %llu (need %llu bytes, have %llu)",
                                (unsigned long long)r.pos, (unsigned long long)count, (unsigned long long)(r.g->size - r.pos));
                return false;
            }
            v->arr.resize(count);
            for (uint64_t i = 0; i < count; i++)
                if (!read_value(r, et, &v->arr[i], depth + 1)) return false;
            break;
        }
        default:
            r.err = gg_fail(RUNIT_GGUF_ERR_UNKNOWN_METADATA_TYPE, "unknown metadata value type: %u", type);
            return false;
    }
    return r.err == RUNIT_GGUF_OK;
}

int32_t parse(runit_gguf* g) {
    Reader r{g};
    const uint32_t magic = r.num<uint32_t>();
    if (r.err) return r.err;
    if (magic != RUNIT_GGUF_MAGIC) return gg_fail(RUNIT_GGUF_ERR_INVALID_MAGIC, "invalid GGUF magic: expected 0x46554747 (\"GGUF\"), got 0x%08X", magic);
    g->version = r.num<uint32_t>();
    if (r.err) return r.err;
    if (g->version != 2 && g->version != 3)
        return gg_fail(RUNIT_GGUF_ERR_UNSUPPORTED_VERSION, "unsupported GGUF version: %u (expected 2 or 3)", g->version);
    const uint64_t n_tensors = r.num<uint64_t>(), n_kv = r.num<uint64_t>();
    if (r.err) return r.err;
    for (uint64_t i = 0; i < n_kv; i++) {
        std::string key;
        if (!r.str(&key)) return r.err;
        const uint32_t type = r.num<uint32_t>();
        if (r.err) return r.err;
        Value v;
        if (!read_value(r, type, &v, 0)) return r.err;
        if (!g->meta.count(key)) g->keys.push_back(key);
        g->meta[key] = std::move(v);   // a repeated key keeps the last value, as a HashMap insert does
    }
    auto al = g->meta.find("general.alignment");
    if (al != g->meta.end() && al->second.type == RUNIT_GGUF_META_UINT32 && al->second.u > 0) g->alignment = al->second.u;
    for (uint64_t i = 0; i < n_tensors; i++) {
        Tensor t;
        if (!r.str(&t.name)) return r.err;
        t.n_dims = r.num<uint32_t>();
        if (r.err) return r.err;
        if (t.n_dims > 4) return gg_fail(RUNIT_GGUF_ERR_BAD_ARG, "tensor '%s' has %u dimensions (at most 4)", t.name.c_str(), t.n_dims);
        for (uint32_t d = 0; d < t.n_dims; d++) t.ne[d] = r.num<uint64_t>();
        t.dtype = r.num<uint32_t>();
        t.offset = r.num<uint64_t>();
        if (r.err) return r.err;
        const DtypeRow* row = dtype_row(t.dtype);
        if (!row) return gg_fail(RUNIT_GGUF_ERR_UNKNOWN_DTYPE, "unknown tensor dtype: %u", t.dtype);
        unsigned __int128 n = 1;
        for (uint32_t d = 0; d < t.n_dims; d++) {
            n *= t.ne[d];
            if (n > (unsigned __int128)1 << 62) return gg_fail(RUNIT_GGUF_ERR_DATA_REGION_OVERFLOW, "tensor data region exceeds file size");
        }
        t.n_elem = n > 0 ? (uint64_t)n : 1;   // num_elements(): product, at least 1
        t.bytes = (t.n_elem + row->block - 1) / row->block * row->size;
        g->by_name[t.name] = g->tensors.size();
        g->tensors.push_back(std::move(t));
    }
    g->data_offset = (r.pos + g->alignment - 1) / g->alignment * g->alignment;
    for (const Tensor& t : g->tensors) {
        const uint64_t avail = g->size > g->data_offset ? g->size - g->data_offset : 0;
        if (t.offset > avail || t.bytes > avail - t.offset)
            return gg_fail(RUNIT_GGUF_ERR_DATA_REGION_OVERFLOW, "tensor data region exceeds file size");
    }
    return RUNIT_GGUF_OK;
}

void fill_info(const Tensor& t, runit_gguf_tensor_info* o) {
    o->name = t.name.c_str();
    o->dtype = t.dtype;
    o->n_dims = t.n_dims;
    for (int d = 0; d < 4; d++) o->ne[d] = t.ne[d];
    o->data_offset = t.offset;
    o->num_elements = t.n_elem;
    o->data_size = t.bytes;
}

const Value* find_meta(const runit_gguf* g, const char* key) {
    if (!g || !key) return nullptr;
    auto it = g->meta.find(key);
    return it == g->meta.end() ? nullptr : &it->second;
}
bool is_int(uint32_t t) {
    return t <= RUNIT_GGUF_META_INT32 || t == RUNIT_GGUF_META_UINT64 || t == RUNIT_GGUF_META_INT64;
}
bool is_float(uint32_t t) { return t == RUNIT_GGUF_META_FLOAT32 || t == RUNIT_GGUF_META_FLOAT64; }

int32_t not_found(const char* what, const char* key) {
    return gg_fail(RUNIT_GGUF_ERR_NOT_FOUND, "no %s '%s'", what, key ? key : "(null)");
}

// Copies bytes [off, off + n) of the data source into dst.
int32_t read_at(runit_gguf* g, uint64_t off, void* dst, uint64_t n) {
    if (g->image) {
        memcpy(dst, g->image + off, n);
        return RUNIT_GGUF_OK;
    }
    uint64_t got = 0;
    while (got < n) {
        const ssize_t r = pread(g->fd, static_cast<uint8_t*>(dst) + got, n - got, (off_t)(off + got));
        if (r <= 0) return gg_fail(RUNIT_GGUF_ERR_IO, "I/O error: read of %llu bytes at offset %llu failed", (unsigned long long)(n - got), (unsigned long long)(off + got));
        got += (uint64_t)r;
    }
    return RUNIT_GGUF_OK;
}

}  // namespace

extern "C" {

const char* runit_gguf_last_error(void) { return g_err; }

static int32_t finish_open(runit_gguf* g, runit_gguf_t** out) {
    const int32_t st = parse(g);
    if (st != RUNIT_GGUF_OK) {
        if (g->fd >= 0) close(g->fd);
        delete g;
        return st;
    }
    *out = g;
    return RUNIT_GGUF_OK;
}

int32_t runit_gguf_open(const char* path, runit_gguf_t** out) {
    if (!path || !out) return gg_fail(RUNIT_GGUF_ERR_BAD_ARG, "null argument");
    *out = nullptr;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return gg_fail(RUNIT_GGUF_ERR_IO, "I/O error: cannot open %s", path);
    struct stat sb;
    if (fstat(fd, &sb) != 0) {
        close(fd);
        return gg_fail(RUNIT_GGUF_ERR_IO, "I/O error: cannot stat %s", path);
    }
    runit_gguf* g = new runit_gguf();
    g->fd = fd;
    g->size = (uint64_t)sb.st_size;
    return finish_open(g, out);
}

int32_t runit_gguf_open_memory(const void* image, uint64_t bytes, runit_gguf_t** out) {
    if (!image || !out) return gg_fail(RUNIT_GGUF_ERR_BAD_ARG, "null argument");
    *out = nullptr;
    runit_gguf* g = new runit_gguf();
    g->image = static_cast<const uint8_t*>(image);
    g->size = bytes;
    return finish_open(g, out);
}

void runit_gguf_close(runit_gguf_t* g) {
    if (!g) return;
    for (int i = 0; i < 2; i++) {
        if (g->pinned[i]) cudaFreeHost(g->pinned[i]);
        if (g->ev[i]) cudaEventDestroy(g->ev[i]);
    }
    if (g->fd >= 0) close(g->fd);
    delete g;
}

uint32_t runit_gguf_version(const runit_gguf_t* g) { return g ? g->version : 0; }
uint64_t runit_gguf_alignment(const runit_gguf_t* g) { return g ? g->alignment : 0; }
uint64_t runit_gguf_data_offset(const runit_gguf_t* g) { return g ? g->data_offset : 0; }
uint64_t runit_gguf_tensor_count(const runit_gguf_t* g) { return g ? g->tensors.size() : 0; }
uint64_t runit_gguf_metadata_count(const runit_gguf_t* g) { return g ? g->keys.size() : 0; }

int32_t runit_gguf_tensor_at(const runit_gguf_t* g, uint64_t index, runit_gguf_tensor_info* out) {
    if (!g || !out) return gg_fail(RUNIT_GGUF_ERR_BAD_ARG, "null argument");
    if (index >= g->tensors.size()) return gg_fail(RUNIT_GGUF_ERR_NOT_FOUND, "tensor index %llu out of range", (unsigned long long)index);
    fill_info(g->tensors[index], out);
    return RUNIT_GGUF_OK;
}

int32_t runit_gguf_tensor_find(const runit_gguf_t* g, const char* name, runit_gguf_tensor_info* out) {
    if (!g || !name || !out) return gg_fail(RUNIT_GGUF_ERR_BAD_ARG, "null argument");
    auto it = g->by_name.find(name);
    if (it == g->by_name.end()) return not_found("tensor", name);
    fill_info(g->tensors[it->second], out);
    return RUNIT_GGUF_OK;
}

uint64_t runit_gguf_dtype_block_size(uint32_t dtype) {
    const DtypeRow* r = dtype_row(dtype);
    return r ? r->block : 0;
}
uint64_t runit_gguf_dtype_type_size(uint32_t dtype) {
    const DtypeRow* r = dtype_row(dtype);
    return r ? r->size : 0;
}
uint64_t runit_gguf_dtype_tensor_data_size(uint32_t dtype, uint64_t num_elements) {
    const DtypeRow* r = dtype_row(dtype);
    return r ? (num_elements + r->block - 1) / r->block * r->size : 0;
}
const char* runit_gguf_dtype_name(uint32_t dtype) {
    const DtypeRow* r = dtype_row(dtype);
    return r ? r->name : nullptr;
}

int32_t runit_gguf_meta_key_at(const runit_gguf_t* g, uint64_t index, const char** key) {
    if (!g || !key) return gg_fail(RUNIT_GGUF_ERR_BAD_ARG, "null argument");
    if (index >= g->keys.size()) return gg_fail(RUNIT_GGUF_ERR_NOT_FOUND, "metadata index %llu out of range", (unsigned long long)index);
    *key = g->keys[index].c_str();
    return RUNIT_GGUF_OK;
}

int32_t runit_gguf_meta_type(const runit_gguf_t* g, const char* key, uint32_t* type, uint32_t* elem_type, uint64_t* count) {
    const Value* v = find_meta(g, key);
    if (!v) return not_found("metadata key", key);
    if (type) *type = v->type;
    if (elem_type) *elem_type = v->type == RUNIT_GGUF_META_ARRAY ? v->elem_type : v->type;
    if (count) *count = v->type == RUNIT_GGUF_META_ARRAY ? v->arr.size() : 1;
    return RUNIT_GGUF_OK;
}

static int32_t as_u64(const Value* v, const char* key, uint64_t* out) {
    if (!v || !(is_int(v->type) || v->type == RUNIT_GGUF_META_BOOL) || !out) return not_found("integer metadata value", key);
    *out = v->u;
    return RUNIT_GGUF_OK;
}
static int32_t as_f64(const Value* v, const char* key, double* out) {
    if (!v || !is_float(v->type) || !out) return not_found("float metadata value", key);
    *out = v->f;
    return RUNIT_GGUF_OK;
}
static int32_t as_str(const Value* v, const char* key, const char** out, uint64_t* len) {
    if (!v || v->type != RUNIT_GGUF_META_STRING || !out) return not_found("string metadata value", key);
    *out = v->s.c_str();
    if (len) *len = v->s.size();
    return RUNIT_GGUF_OK;
}
static const Value* elem(const runit_gguf_t* g, const char* key, uint64_t index) {
    const Value* v = find_meta(g, key);
    if (!v || v->type != RUNIT_GGUF_META_ARRAY || index >= v->arr.size()) return nullptr;
    return &v->arr[index];
}

int32_t runit_gguf_meta_u64(const runit_gguf_t* g, const char* key, uint64_t* out) { return as_u64(find_meta(g, key), key, out); }
int32_t runit_gguf_meta_i64(const runit_gguf_t* g, const char* key, int64_t* out) {
    return as_u64(find_meta(g, key), key, reinterpret_cast<uint64_t*>(out));
}
int32_t runit_gguf_meta_f64(const runit_gguf_t* g, const char* key, double* out) { return as_f64(find_meta(g, key), key, out); }
int32_t runit_gguf_meta_bool(const runit_gguf_t* g, const char* key, int32_t* out) {
    const Value* v = find_meta(g, key);
    if (!v || v->type != RUNIT_GGUF_META_BOOL || !out) return not_found("bool metadata value", key);
    *out = v->u != 0;
    return RUNIT_GGUF_OK;
}
int32_t runit_gguf_meta_str(const runit_gguf_t* g, const char* key, const char** out, uint64_t* len) {
    return as_str(find_meta(g, key), key, out, len);
}
int32_t runit_gguf_meta_array_u64(const runit_gguf_t* g, const char* key, uint64_t index, uint64_t* out) {
    return as_u64(elem(g, key, index), key, out);
}
int32_t runit_gguf_meta_array_i64(const runit_gguf_t* g, const char* key, uint64_t index, int64_t* out) {
    return as_u64(elem(g, key, index), key, reinterpret_cast<uint64_t*>(out));
}
int32_t runit_gguf_meta_array_f64(const runit_gguf_t* g, const char* key, uint64_t index, double* out) {
    return as_f64(elem(g, key, index), key, out);
}
int32_t runit_gguf_meta_array_str(const runit_gguf_t* g, const char* key, uint64_t index, const char** out, uint64_t* len) {
    return as_str(elem(g, key, index), key, out, len);
}

int32_t runit_gguf_read_tensor(runit_gguf_t* g, const char* name, void* host_dst, uint64_t capacity) {
    if (!g || !name || !host_dst) return gg_fail(RUNIT_GGUF_ERR_BAD_ARG, "null argument");
    auto it = g->by_name.find(name);
    if (it == g->by_name.end()) return not_found("tensor", name);
    const Tensor& t = g->tensors[it->second];
    if (capacity < t.bytes)
        return gg_fail(RUNIT_GGUF_ERR_BUFFER_SIZE, "tensor '%s' needs %llu bytes, destination has %llu", name, (unsigned long long)t.bytes, (unsigned long long)capacity);
    return read_at(g, g->data_offset + t.offset, host_dst, t.bytes);
}

int32_t runit_gguf_upload_tensor(runit_ctx_t* ctx, runit_gguf_t* g, const char* name, void* device_dst, uint64_t capacity) {
    if (!ctx || !g || !name || !device_dst) return gg_fail(RUNIT_GGUF_ERR_BAD_ARG, "null argument");
    auto it = g->by_name.find(name);
    if (it == g->by_name.end()) return not_found("tensor", name);
    const Tensor& t = g->tensors[it->second];
    if (capacity < t.bytes)
        return gg_fail(RUNIT_GGUF_ERR_BUFFER_SIZE, "tensor '%s' needs %llu bytes, destination has %llu", name, (unsigned long long)t.bytes, (unsigned long long)capacity);
    cudaError_t e = cudaSetDevice(ctx->device);
    for (int i = 0; i < 2 && e == cudaSuccess; i++) {
        if (!g->pinned[i]) e = cudaMallocHost(&g->pinned[i], kChunk);
        if (e == cudaSuccess && !g->ev[i]) e = cudaEventCreateWithFlags(&g->ev[i], cudaEventDisableTiming);
    }
    if (e != cudaSuccess) return gg_fail(RUNIT_GGUF_ERR_CUDA, "staging buffers: %s", cudaGetErrorString(e));
    // chunk c goes through staging buffer c % 2: reading chunk c from the file overlaps the copy of chunk c - 1
    uint64_t done = 0;
    for (uint64_t c = 0; done < t.bytes; c++) {
        const int b = (int)(c & 1);
        const uint64_t n = t.bytes - done < kChunk ? t.bytes - done : kChunk;
        if (c >= 2 && (e = cudaEventSynchronize(g->ev[b])) != cudaSuccess) break;   // buffer b's previous copy has finished
        const int32_t st = read_at(g, g->data_offset + t.offset + done, g->pinned[b], n);
        if (st != RUNIT_GGUF_OK) {
            cudaStreamSynchronize(ctx->stream);
            return st;
        }
        if ((e = cudaMemcpyAsync(static_cast<uint8_t*>(device_dst) + done, g->pinned[b], n, cudaMemcpyHostToDevice, ctx->stream)) != cudaSuccess) break;
        if ((e = cudaEventRecord(g->ev[b], ctx->stream)) != cudaSuccess) break;
        done += n;
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);   // the staging buffers may be reused by the next call
    if (e != cudaSuccess) return gg_fail(RUNIT_GGUF_ERR_CUDA, "upload of '%s': %s", name, cudaGetErrorString(e));
    return RUNIT_GGUF_OK;
}

}  // extern "C"
