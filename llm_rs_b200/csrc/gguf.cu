// GGUF container reader (host code only; see gguf.h).  File format facts follow the reference's
// parser: magic and versions src/gguf/mod.rs:11,182-190; key/value section :192-202 and :256-303;
// tensor directory :204-215; data section at the directory's end rounded up to 32 bytes :217
// (a `general.alignment` key is not consulted there, nor here).
#include "gguf.h"

#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstdio>
#include <cstring>
#include <new>
#include <thread>

#include "../../include/llmrs_cuda.h"

namespace llmrs {

namespace {
constexpr uint32_t GGUF_MAGIC = 0x46554747u;      // "GGUF" read as a little-endian u32
constexpr uint64_t GGUF_ALIGNMENT = 32;
constexpr size_t PREAD_PIECE = 4u << 20;
constexpr uint64_t MAX_DIRECTORY_BYTES = 1ull << 30;   // no honest directory is longer; bounds host memory on a corrupt file

// Thrown by the cursor when the bytes read so far end inside the directory: the caller reads more.
struct NeedMore {};
struct ParseError { std::string what; };

// Bounds-checked little-endian cursor over the header bytes.
struct Cursor {
    const uint8_t *buf;
    size_t len, pos = 0;
    bool whole_file;                               // nothing more to read: running out is an error
    uint64_t file_size;                            // a length that reaches beyond the file is a lie, not a short read
    void need(uint64_t n) const {
        if (n > len - pos) {
            if (whole_file || n > file_size - std::min<uint64_t>(file_size, pos))
                throw ParseError{"file ends inside the GGUF directory"};
            throw NeedMore{};
        }
    }
    template <typename T> T get() {
        need(sizeof(T));
        T v;
        memcpy(&v, buf + pos, sizeof(T));          // x86-64 / aarch64 hosts: little-endian like the file
        pos += sizeof(T);
        return v;
    }
    std::string_view str() {                       // u64 length + bytes, UTF-8 checked (:143-158)
        const uint64_t n = get<uint64_t>();
        need(n);
        std::string_view s((const char *)buf + pos, (size_t)n);
        pos += (size_t)n;
        return s;
    }
};

bool valid_utf8(std::string_view s) {
    const unsigned char *p = (const unsigned char *)s.data(), *e = p + s.size();
    while (p < e) {
        const unsigned c = *p;
        int n;
        uint32_t cp;
        if (c < 0x80) { p++; continue; }
        if (c >= 0xC2 && c <= 0xDF) { n = 1; cp = c & 0x1F; }
        else if (c >= 0xE0 && c <= 0xEF) { n = 2; cp = c & 0x0F; }
        else if (c >= 0xF0 && c <= 0xF4) { n = 3; cp = c & 0x07; }
        else return false;
        if (e - p <= n) return false;
        for (int i = 1; i <= n; i++) {
            if ((p[i] & 0xC0) != 0x80) return false;
            cp = (cp << 6) | (p[i] & 0x3F);
        }
        if ((n == 2 && (cp < 0x800 || (cp >= 0xD800 && cp <= 0xDFFF))) || (n == 3 && (cp < 0x10000 || cp > 0x10FFFF)))
            return false;
        p += n + 1;
    }
    return true;
}

size_t scalar_bytes(uint32_t t) {
    switch (t) {
    case GT_U8: case GT_I8: case GT_BOOL: return 1;
    case GT_U16: case GT_I16: return 2;
    case GT_U32: case GT_I32: case GT_F32: return 4;
    case GT_U64: case GT_I64: case GT_F64: return 8;
    default: return 0;
    }
}

void read_scalar(Cursor &c, uint32_t t, GgufValue &v) {
    switch (t) {
    case GT_U8: v.u = c.get<uint8_t>(); break;
    case GT_I8: v.u = (uint64_t)(int64_t)c.get<int8_t>(); break;
    case GT_U16: v.u = c.get<uint16_t>(); break;
    case GT_I16: v.u = (uint64_t)(int64_t)c.get<int16_t>(); break;
    case GT_U32: v.u = c.get<uint32_t>(); break;
    case GT_I32: v.u = (uint64_t)(int64_t)c.get<int32_t>(); break;
    case GT_F32: v.f = c.get<float>(); break;
    case GT_BOOL: v.u = c.get<uint8_t>() != 0; break;
    case GT_U64: v.u = c.get<uint64_t>(); break;
    case GT_I64: v.u = (uint64_t)c.get<int64_t>(); break;
    case GT_F64: v.f = c.get<double>(); break;
    default: throw ParseError{"unknown metadata type: " + std::to_string(t)};
    }
}

std::string_view checked_str(Cursor &c) {
    std::string_view s = c.str();
    if (!valid_utf8(s)) throw ParseError{"invalid UTF-8 in string"};
    return s;
}

void read_value(Cursor &c, GgufValue &v) {
    v.type = c.get<uint32_t>();
    if (v.type == GT_STRING) {
        v.s = checked_str(c);
    } else if (v.type == GT_ARRAY) {
        v.elem_type = c.get<uint32_t>();
        v.count = c.get<uint64_t>();
        if (v.elem_type == GT_STRING) {
            // a count larger than the bytes left cannot be honest: every string takes eight at least
            c.need(v.count > UINT64_MAX / 8 ? UINT64_MAX : v.count * 8);
            v.strings.reserve((size_t)v.count);
            for (uint64_t i = 0; i < v.count; i++) v.strings.push_back(checked_str(c));
        } else {
            const size_t eb = scalar_bytes(v.elem_type);      // arrays of arrays: as in the reference, an error
            if (!eb) throw ParseError{"unknown metadata type: " + std::to_string(v.elem_type)};
            if (v.count > UINT64_MAX / eb) throw ParseError{"metadata array length overflows"};
            c.need(v.count * eb);
            v.data_pos = c.pos;
            c.pos += (size_t)(v.count * eb);
        }
    } else {
        read_scalar(c, v.type, v);
    }
}

// Parses buf[0, len) into g.  Throws NeedMore when the directory continues beyond len.
void parse(GgufFile &g, const uint8_t *buf, size_t len, bool whole_file) {
    Cursor c{buf, len, 0, whole_file, g.file_size};
    const uint32_t magic = c.get<uint32_t>();
    if (magic != GGUF_MAGIC) {
        char m[48];
        snprintf(m, sizeof m, "invalid GGUF magic: 0x%08x", magic);
        throw ParseError{m};
    }
    g.version = c.get<uint32_t>();
    if (g.version < 2 || g.version > 3) throw ParseError{"unsupported GGUF version: " + std::to_string(g.version)};
    const uint64_t tensor_count = c.get<uint64_t>(), kv_count = c.get<uint64_t>();
    // every entry takes at least 12 (value) / 24 (tensor) bytes of the file
    if (kv_count > g.file_size / 12 || tensor_count > g.file_size / 24) throw ParseError{"directory counts exceed the file size"};
    g.metadata.clear();
    g.tensors.clear();
    g.metadata.reserve((size_t)kv_count);
    for (uint64_t i = 0; i < kv_count; i++) {
        GgufValue v;
        v.key = std::string(checked_str(c));
        read_value(c, v);
        g.metadata.push_back(std::move(v));
    }
    g.tensors.reserve((size_t)tensor_count);
    for (uint64_t i = 0; i < tensor_count; i++) {
        GgufTensor t;
        t.name = std::string(checked_str(c));
        t.n_dims = c.get<uint32_t>();
        if (t.n_dims > 4) throw ParseError{"tensor " + t.name + " has " + std::to_string(t.n_dims) + " dimensions (at most 4)"};
        uint64_t n = 1;
        for (uint32_t d = 0; d < t.n_dims; d++) {
            t.shape[d] = c.get<uint64_t>();
            if (t.shape[d] && n > UINT64_MAX / t.shape[d]) throw ParseError{"tensor " + t.name + ": element count overflows"};
            n *= t.shape[d];
        }
        t.dtype = c.get<uint32_t>();
        uint32_t be = 0, bb = 0;
        if (!gguf_block_layout(t.dtype, &be, &bb)) throw ParseError{"unknown dtype: " + std::to_string(t.dtype)};
        t.offset = c.get<uint64_t>();
        if (n % be) throw ParseError{"tensor " + t.name + ": element count " + std::to_string(n) + " not divisible by block size " + std::to_string(be)};
        t.nbytes = n / be * bb;
        g.tensors.push_back(std::move(t));
    }
    g.data_offset = ((uint64_t)c.pos + GGUF_ALIGNMENT - 1) & ~(GGUF_ALIGNMENT - 1);
}

bool pread_all(int fd, uint8_t *dst, size_t len, uint64_t off) {
    size_t done = 0;
    while (done < len) {
        const ssize_t n = pread(fd, dst + done, len - done, (off_t)(off + done));
        if (n < 0 && errno == EINTR) continue;
        if (n <= 0) return false;
        done += (size_t)n;
    }
    return true;
}
}  // namespace

bool gguf_block_layout(uint32_t dtype, uint32_t *block_elems, uint32_t *block_bytes) {
    // {elements, bytes} per block by GGUF type id; ids 4 and 5 were removed from the format
    static const struct { uint16_t e, b; } T[31] = {
        {1, 4}, {1, 2}, {32, 18}, {32, 20}, {0, 0}, {0, 0}, {32, 22}, {32, 24}, {32, 34}, {32, 40},          // F32 F16 Q4_0 Q4_1 - - Q5_0 Q5_1 Q8_0 Q8_1
        {256, 84}, {256, 110}, {256, 144}, {256, 176}, {256, 210}, {256, 292},                               // Q2_K .. Q6_K, Q8_K
        {256, 66}, {256, 74}, {256, 98}, {256, 50}, {32, 18}, {256, 110}, {256, 82}, {32, 36},               // IQ2_XXS IQ2_XS IQ3_XXS IQ1_S IQ4_NL IQ3_S IQ2_S IQ4_XS
        {1, 1}, {1, 2}, {1, 4}, {1, 8}, {1, 8}, {256, 56}, {1, 2}};                                          // I8 I16 I32 I64 F64 IQ1_M BF16
    if (dtype > 30 || T[dtype].e == 0) return false;
    *block_elems = T[dtype].e;
    *block_bytes = T[dtype].b;
    return true;
}

GgufFile::~GgufFile() {
    if (fd >= 0) close(fd);
}

const GgufValue *GgufFile::find_value(const char *key) const {
    // the reference keeps a map, in which the last of two equal keys wins (:198-202)
    for (size_t i = metadata.size(); i-- > 0;)
        if (metadata[i].key == key) return &metadata[i];
    return nullptr;
}

const GgufTensor *GgufFile::find_tensor(const char *name) const {
    for (const GgufTensor &t : tensors)          // first match, as tensor_view's find (:243)
        if (t.name == name) return &t;
    return nullptr;
}

// The file is untrusted input and this runs below a C ABI: nothing may be thrown out of it.
static GgufFile *gguf_open_impl(const char *path, std::string *error, GgufFile *g) {
    g->fd = open(path, O_RDONLY | O_CLOEXEC);
    struct stat st;
    if (g->fd < 0 || fstat(g->fd, &st) != 0) {
        *error = std::string("IO error: ") + path + ": " + strerror(errno);
        return nullptr;
    }
    g->file_size = (uint64_t)st.st_size;
    // The directory's length is not stored anywhere: read a prefix, parse, and read a longer one
    // when the parser runs out of bytes (token lists make some directories several megabytes).
    size_t want = std::min<uint64_t>(g->file_size, 1u << 20);
    for (;;) {
        const size_t have = g->header.size();
        g->header.resize(want);
        if (!pread_all(g->fd, g->header.data() + have, want - have, have)) {
            *error = std::string("IO error: reading ") + path + ": " + strerror(errno);
            return nullptr;
        }
        try {
            parse(*g, g->header.data(), want, want == g->file_size);
            break;
        } catch (const NeedMore &) {
            if (want >= MAX_DIRECTORY_BYTES) {
                *error = "GGUF directory longer than 1 GiB";
                return nullptr;
            }
            want = (size_t)std::min<uint64_t>(std::min<uint64_t>(g->file_size, MAX_DIRECTORY_BYTES), (uint64_t)want * 4);
        } catch (const ParseError &e) {
            *error = e.what;
            return nullptr;
        }
    }
    // the strings borrow from `header`, whose storage must not move again
    g->header.resize((size_t)std::min<uint64_t>(g->data_offset, g->header.size()));
    for (const GgufTensor &t : g->tensors)
        if (t.offset > g->file_size || t.nbytes > g->file_size - t.offset || g->data_offset > g->file_size - t.offset - t.nbytes) {
            *error = "tensor " + t.name + " lies outside the file";
            return nullptr;
        }
    return g;
}

GgufFile *gguf_open(const char *path, std::string *error) {
    GgufFile *g = new (std::nothrow) GgufFile();
    if (!g) {
        *error = "IO error: out of host memory";
        return nullptr;
    }
    GgufFile *ok = nullptr;
    try {
        ok = gguf_open_impl(path, error, g);
    } catch (const std::bad_alloc &) {
        try { *error = "IO error: out of host memory while reading the GGUF directory"; } catch (...) {}
    } catch (...) {                                // length_error and the like: a directory no host can hold
        try { *error = "malformed GGUF directory"; } catch (...) {}
    }
    if (!ok) delete g;
    return ok;
}

bool gguf_pread_parallel(int fd, void *dst, uint64_t offset, size_t len, int threads) {
    if (len == 0) return true;
    threads = (int)std::max<size_t>(1, std::min<size_t>((size_t)threads, (len + PREAD_PIECE - 1) / PREAD_PIECE));
    const size_t stripe = (len + (size_t)threads - 1) / (size_t)threads;
    std::vector<char> ok((size_t)threads, 1);
    auto work = [&](int t) {
        const size_t a = (size_t)t * stripe, b = std::min(len, a + stripe);
        for (size_t off = a; off < b; off += PREAD_PIECE)
            if (!pread_all(fd, (uint8_t *)dst + off, std::min(PREAD_PIECE, b - off), offset + off)) {
                ok[(size_t)t] = 0;
                return;
            }
    };
    std::vector<std::thread> pool;
    for (int t = 1; t < threads; t++) pool.emplace_back(work, t);
    work(0);
    for (std::thread &th : pool) th.join();
    return std::all_of(ok.begin(), ok.end(), [](char c) { return c != 0; });
}

}  // namespace llmrs

// ---- C ABI: the directory ------------------------------------------------------------------------

struct llmrs_gguf : llmrs::GgufFile {};

namespace {
thread_local std::string g_gguf_error;
int gguf_fail(int code, std::string msg) {
    g_gguf_error = std::move(msg);
    return code;
}
void fill_tensor(const llmrs::GgufTensor &t, llmrs_gguf_tensor *out) {
    out->name = t.name.c_str();
    out->dtype = t.dtype;
    out->n_dims = t.n_dims;
    for (int d = 0; d < 4; d++) out->shape[d] = t.shape[d];
    out->offset = t.offset;
    out->nbytes = t.nbytes;
}
}  // namespace

extern "C" {

const char *llmrs_gguf_last_error(void) { return g_gguf_error.c_str(); }

int llmrs_gguf_open(const char *path, llmrs_gguf **out) {
    if (!path || !out) return gguf_fail(LLMRS_ERR_ARG, "gguf_open: null pointer");
    try {
        std::string err;
        llmrs::GgufFile *g = llmrs::gguf_open(path, &err);
        if (!g) return gguf_fail(err.rfind("IO error", 0) == 0 ? LLMRS_ERR_IO : LLMRS_ERR_FORMAT, err);
        *out = static_cast<llmrs_gguf *>(g);
        return LLMRS_OK;
    } catch (...) {
        return LLMRS_ERR_IO;
    }
}

void llmrs_gguf_close(llmrs_gguf *g) { delete static_cast<llmrs::GgufFile *>(g); }

uint32_t llmrs_gguf_version(const llmrs_gguf *g) { return g ? g->version : 0; }
uint64_t llmrs_gguf_file_size(const llmrs_gguf *g) { return g ? g->file_size : 0; }
uint64_t llmrs_gguf_data_offset(const llmrs_gguf *g) { return g ? g->data_offset : 0; }
uint64_t llmrs_gguf_tensor_count(const llmrs_gguf *g) { return g ? g->tensors.size() : 0; }
uint64_t llmrs_gguf_metadata_count(const llmrs_gguf *g) { return g ? g->metadata.size() : 0; }

int llmrs_gguf_tensor_at(const llmrs_gguf *g, uint64_t index, llmrs_gguf_tensor *out) {
    if (!g || !out) return gguf_fail(LLMRS_ERR_ARG, "gguf_tensor_at: null pointer");
    if (index >= g->tensors.size()) return gguf_fail(LLMRS_ERR_NOT_FOUND, "gguf_tensor_at: index out of range");
    fill_tensor(g->tensors[(size_t)index], out);
    return LLMRS_OK;
}

int llmrs_gguf_find_tensor(const llmrs_gguf *g, const char *name, llmrs_gguf_tensor *out) {
    if (!g || !name || !out) return gguf_fail(LLMRS_ERR_ARG, "gguf_find_tensor: null pointer");
    const llmrs::GgufTensor *t = g->find_tensor(name);
    if (!t) return gguf_fail(LLMRS_ERR_NOT_FOUND, std::string("tensor not found: ") + name);
    fill_tensor(*t, out);
    return LLMRS_OK;
}

int llmrs_gguf_read_tensor(const llmrs_gguf *g, const char *name, void *host, size_t nbytes) {
    if (!g || !name || (!host && nbytes)) return gguf_fail(LLMRS_ERR_ARG, "gguf_read_tensor: null pointer");
    const llmrs::GgufTensor *t = g->find_tensor(name);
    if (!t) return gguf_fail(LLMRS_ERR_NOT_FOUND, std::string("tensor not found: ") + name);
    if (nbytes != t->nbytes)
        return gguf_fail(LLMRS_ERR_SHAPE, "gguf_read_tensor: " + std::to_string(nbytes) + " bytes asked, tensor holds " + std::to_string(t->nbytes));
    if (!llmrs::gguf_pread_parallel(g->fd, host, g->data_offset + t->offset, nbytes, 8))
        return gguf_fail(LLMRS_ERR_IO, std::string("IO error: reading tensor ") + name);
    return LLMRS_OK;
}

int llmrs_gguf_metadata_at(const llmrs_gguf *g, uint64_t index, const char **key, uint32_t *type, uint32_t *elem_type,
                           uint64_t *count) {
    if (!g) return gguf_fail(LLMRS_ERR_ARG, "gguf_metadata_at: null pointer");
    if (index >= g->metadata.size()) return gguf_fail(LLMRS_ERR_NOT_FOUND, "gguf_metadata_at: index out of range");
    const llmrs::GgufValue &v = g->metadata[(size_t)index];
    if (key) *key = v.key.c_str();
    if (type) *type = v.type;
    if (elem_type) *elem_type = v.elem_type;
    if (count) *count = v.count;
    return LLMRS_OK;
}

int llmrs_gguf_get_u64(const llmrs_gguf *g, const char *key, uint64_t *out) {
    if (!g || !key || !out) return gguf_fail(LLMRS_ERR_ARG, "gguf_get_u64: null pointer");
    const llmrs::GgufValue *v = g->find_value(key);
    if (!v) return gguf_fail(LLMRS_ERR_NOT_FOUND, std::string("metadata key not found: ") + key);
    switch (v->type) {
    case llmrs::GT_U8: case llmrs::GT_I8: case llmrs::GT_U16: case llmrs::GT_I16: case llmrs::GT_U32: case llmrs::GT_I32:
    case llmrs::GT_U64: case llmrs::GT_I64: case llmrs::GT_BOOL:
        *out = v->u;
        return LLMRS_OK;
    default:
        return gguf_fail(LLMRS_ERR_DTYPE, std::string("metadata key is not an integer: ") + key);
    }
}

int llmrs_gguf_get_u32(const llmrs_gguf *g, const char *key, uint32_t *out) {
    if (!g || !key || !out) return gguf_fail(LLMRS_ERR_ARG, "gguf_get_u32: null pointer");
    const llmrs::GgufValue *v = g->find_value(key);
    if (!v) return gguf_fail(LLMRS_ERR_NOT_FOUND, std::string("metadata key not found: ") + key);
    // MetadataValue::as_u32 (src/gguf/metadata.rs:38-46): the four wide integer types, truncated
    if (v->type != llmrs::GT_U32 && v->type != llmrs::GT_I32 && v->type != llmrs::GT_U64 && v->type != llmrs::GT_I64)
        return gguf_fail(LLMRS_ERR_DTYPE, std::string("metadata key is not U32/I32/U64/I64: ") + key);
    *out = (uint32_t)v->u;
    return LLMRS_OK;
}

int llmrs_gguf_get_f64(const llmrs_gguf *g, const char *key, double *out) {
    if (!g || !key || !out) return gguf_fail(LLMRS_ERR_ARG, "gguf_get_f64: null pointer");
    const llmrs::GgufValue *v = g->find_value(key);
    if (!v) return gguf_fail(LLMRS_ERR_NOT_FOUND, std::string("metadata key not found: ") + key);
    // MetadataValue::as_f32 (src/gguf/metadata.rs:48-54) accepts F32 and F64
    if (v->type != llmrs::GT_F32 && v->type != llmrs::GT_F64)
        return gguf_fail(LLMRS_ERR_DTYPE, std::string("metadata key is not F32/F64: ") + key);
    *out = v->f;
    return LLMRS_OK;
}

int llmrs_gguf_get_str(const llmrs_gguf *g, const char *key, const char **out, uint64_t *len) {
    if (!g || !key || !out || !len) return gguf_fail(LLMRS_ERR_ARG, "gguf_get_str: null pointer");
    const llmrs::GgufValue *v = g->find_value(key);
    if (!v) return gguf_fail(LLMRS_ERR_NOT_FOUND, std::string("metadata key not found: ") + key);
    if (v->type != llmrs::GT_STRING) return gguf_fail(LLMRS_ERR_DTYPE, std::string("metadata key is not a string: ") + key);
    *out = v->s.data();
    *len = v->s.size();
    return LLMRS_OK;
}

int llmrs_gguf_get_array(const llmrs_gguf *g, const char *key, uint32_t *elem_type, uint64_t *count, const void **data) {
    if (!g || !key) return gguf_fail(LLMRS_ERR_ARG, "gguf_get_array: null pointer");
    const llmrs::GgufValue *v = g->find_value(key);
    if (!v) return gguf_fail(LLMRS_ERR_NOT_FOUND, std::string("metadata key not found: ") + key);
    if (v->type != llmrs::GT_ARRAY) return gguf_fail(LLMRS_ERR_DTYPE, std::string("metadata key is not an array: ") + key);
    if (elem_type) *elem_type = v->elem_type;
    if (count) *count = v->count;
    if (data) *data = v->elem_type == llmrs::GT_STRING ? nullptr : (const void *)(g->header.data() + v->data_pos);
    return LLMRS_OK;
}

int llmrs_gguf_get_array_str(const llmrs_gguf *g, const char *key, uint64_t index, const char **out, uint64_t *len) {
    if (!g || !key || !out || !len) return gguf_fail(LLMRS_ERR_ARG, "gguf_get_array_str: null pointer");
    const llmrs::GgufValue *v = g->find_value(key);
    if (!v) return gguf_fail(LLMRS_ERR_NOT_FOUND, std::string("metadata key not found: ") + key);
    if (v->type != llmrs::GT_ARRAY || v->elem_type != llmrs::GT_STRING)
        return gguf_fail(LLMRS_ERR_DTYPE, std::string("metadata key is not an array of strings: ") + key);
    if (index >= v->strings.size()) return gguf_fail(LLMRS_ERR_NOT_FOUND, "gguf_get_array_str: index out of range");
    *out = v->strings[(size_t)index].data();
    *len = v->strings[(size_t)index].size();
    return LLMRS_OK;
}

}  // extern "C"
