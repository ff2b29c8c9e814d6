// q38b_gguf.cpp -- GGUF v3 reader for the planner: maps a model file and hands its weight tensors to
// q38b_pass_matrix_upload, row-sharded.  Replaces, for this path, the reference's parser and split upload
// (src/runtime/gguf_parser.h:70-146 and src/runtime/engine.cpp:594-629 of the reference project): the file layout is
// the GGUF specification's -- magic "GGUF", version, tensor count, key-value count, the key-value table, the tensor-info
// table (name, n_dims, dims, ggml type, offset), then the tensor data at the next multiple of general.alignment
// (default 32), offsets relative to that point.  Every read is bounds-checked against the mapping; a malformed file
// is an error, never an out-of-range access.  Host code only (no CUDA calls): the upload goes through the C ABI.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "../../include/q38b200.h"

namespace {

constexpr uint32_t GGUF_MAGIC = 0x46554747u;   // "GGUF", little-endian
enum : uint32_t { GT_U8, GT_I8, GT_U16, GT_I16, GT_U32, GT_I32, GT_F32, GT_BOOL, GT_STRING, GT_ARRAY, GT_U64, GT_I64, GT_F64 };

// elements per block and bytes per block of the ggml types this library knows how to size (0: unknown)
bool block_shape(uint32_t type, uint32_t* elems, uint32_t* bytes) {
    switch (type) {
        case 0: *elems = 1; *bytes = 4; return true;      // F32
        case 1: *elems = 1; *bytes = 2; return true;      // F16
        case 30: *elems = 1; *bytes = 2; return true;     // BF16
        case 8: *elems = 32; *bytes = 34; return true;    // Q8_0
        case 10: *elems = 256; *bytes = 84; return true;  // Q2_K
        case 11: *elems = 256; *bytes = 110; return true; // Q3_K
        case 12: *elems = 256; *bytes = 144; return true; // Q4_K
        case 13: *elems = 256; *bytes = 176; return true; // Q5_K
        case 14: *elems = 256; *bytes = 210; return true; // Q6_K
        case 16: *elems = 256; *bytes = 66; return true;  // IQ2_XXS
        case 17: *elems = 256; *bytes = 74; return true;  // IQ2_XS
        case 18: *elems = 256; *bytes = 98; return true;  // IQ3_XXS
        case 19: *elems = 256; *bytes = 50; return true;  // IQ1_S
        case 20: *elems = 32; *bytes = 18; return true;   // IQ4_NL
        case 21: *elems = 256; *bytes = 110; return true; // IQ3_S
        case 22: *elems = 256; *bytes = 82; return true;  // IQ2_S
        case 23: *elems = 256; *bytes = 136; return true; // IQ4_XS
        case 29: *elems = 256; *bytes = 56; return true;  // IQ1_M
        default: return false;
    }
}

struct Tensor {
    std::string name;
    uint32_t type = 0, n_dims = 0;
    uint64_t dims[4] = {1, 1, 1, 1};
    uint64_t offset = 0;    // relative to the data section
    uint64_t nbytes = 0;    // 0 when the type's block shape is unknown
};

}  // namespace

struct q38b_gguf {
    int fd = -1;
    const uint8_t* base = nullptr;
    uint64_t size = 0, pos = 0, data_offset = 0;
    uint32_t version = 0, alignment = 32;
    std::vector<Tensor> tensors;
    bool ok = true;

    bool need(uint64_t n) {
        if (!ok || n > size || pos > size - n) { ok = false; return false; }
        return true;
    }
    template <typename T> T pod() {
        T v{};
        if (need(sizeof(T))) { memcpy(&v, base + pos, sizeof(T)); pos += sizeof(T); }
        return v;
    }
    bool str(std::string* out) {
        const uint64_t n = pod<uint64_t>();
        if (!need(n)) return false;
        if (out) out->assign((const char*)base + pos, (size_t)n);
        pos += n;
        return true;
    }
    // skips (or, for general.alignment, reads) one metadata value
    bool value(uint32_t type, int depth, uint64_t* as_uint) {
        static const uint64_t width[13] = {1, 1, 2, 2, 4, 4, 4, 1, 0, 0, 8, 8, 8};
        if (type == GT_STRING) return str(nullptr);
        if (type == GT_ARRAY) {
            if (depth > 2) { ok = false; return false; }
            const uint32_t et = pod<uint32_t>();
            const uint64_t n = pod<uint64_t>();
            if (!ok || et > GT_F64) { ok = false; return false; }
            if (et != GT_STRING && et != GT_ARRAY) {          // fixed-size elements: one bounds check for the whole array
                if (n > size / width[et] || !need(n * width[et])) { ok = false; return false; }
                pos += n * width[et];
                return true;
            }
            for (uint64_t i = 0; i < n && ok; i++) value(et, depth + 1, nullptr);
            return ok;
        }
        if (type > GT_F64 || !need(width[type])) { ok = false; return false; }
        if (as_uint) {
            uint64_t v = 0;
            memcpy(&v, base + pos, (size_t)width[type]);
            *as_uint = v;
        }
        pos += width[type];
        return true;
    }
};

extern "C" {

void q38b_gguf_close(q38b_gguf* g) {
    if (!g) return;
    if (g->base) munmap((void*)g->base, (size_t)g->size);
    if (g->fd >= 0) close(g->fd);
    delete g;
}

int q38b_gguf_open(const char* path, q38b_gguf** out) {
    if (!path || !out) return Q38B_ERR_ARG;
    *out = nullptr;
    q38b_gguf* g = new (std::nothrow) q38b_gguf;
    if (!g) return Q38B_ERR_NOMEM;
    struct stat st;
    g->fd = open(path, O_RDONLY);
    if (g->fd < 0 || fstat(g->fd, &st) != 0 || st.st_size < 24) { q38b_gguf_close(g); return Q38B_ERR_ARG; }
    g->size = (uint64_t)st.st_size;
    void* m = mmap(nullptr, (size_t)g->size, PROT_READ, MAP_PRIVATE, g->fd, 0);
    if (m == MAP_FAILED) { q38b_gguf_close(g); return Q38B_ERR_NOMEM; }
    g->base = (const uint8_t*)m;
    const uint32_t magic = g->pod<uint32_t>();
    g->version = g->pod<uint32_t>();
    const uint64_t n_tensors = g->pod<uint64_t>(), n_kv = g->pod<uint64_t>();
    if (!g->ok || magic != GGUF_MAGIC || g->version < 2 || g->version > 3 || n_tensors > g->size / 24 || n_kv > g->size / 12) {
        q38b_gguf_close(g);
        return Q38B_ERR_UNSUPPORTED;
    }
    for (uint64_t i = 0; i < n_kv && g->ok; i++) {
        std::string key;
        g->str(&key);
        const uint32_t type = g->pod<uint32_t>();
        uint64_t v = 0;
        const bool is_align = key == "general.alignment" && (type == GT_U32 || type == GT_U64 || type == GT_U16 || type == GT_U8);
        g->value(type, 0, is_align ? &v : nullptr);
        if (is_align && g->ok) {
            if (v == 0 || (v & (v - 1)) || v > (1u << 20)) g->ok = false;   // a power of two
            else g->alignment = (uint32_t)v;
        }
    }
    g->tensors.reserve((size_t)n_tensors);
    for (uint64_t i = 0; i < n_tensors && g->ok; i++) {
        Tensor t;
        g->str(&t.name);
        t.n_dims = g->pod<uint32_t>();
        if (!g->ok || t.n_dims < 1 || t.n_dims > 4) { g->ok = false; break; }
        uint64_t elems = 1;
        for (uint32_t d = 0; d < t.n_dims; d++) {
            t.dims[d] = g->pod<uint64_t>();
            if (t.dims[d] == 0 || t.dims[d] > (1ull << 40) || elems > (1ull << 50) / t.dims[d]) { g->ok = false; break; }
            elems *= t.dims[d];
        }
        t.type = g->pod<uint32_t>();
        t.offset = g->pod<uint64_t>();
        uint32_t be = 0, bb = 0;
        if (g->ok && block_shape(t.type, &be, &bb)) {
            if (t.dims[0] % be) { g->ok = false; break; }     // rows hold whole blocks
            t.nbytes = elems / be * bb;
        }
        if (g->ok) g->tensors.push_back(t);
    }
    if (g->ok) {
        g->data_offset = (g->pos + g->alignment - 1) / g->alignment * g->alignment;
        if (g->data_offset > g->size) g->ok = false;
        for (const Tensor& t : g->tensors)                     // every sized tensor lies inside the file, aligned
            if (t.offset % g->alignment || t.offset > g->size - g->data_offset || t.nbytes > g->size - g->data_offset - t.offset) g->ok = false;
    }
    if (!g->ok) { q38b_gguf_close(g); return Q38B_ERR_ARG; }
    *out = g;
    return Q38B_OK;
}

int q38b_gguf_tensor_count(const q38b_gguf* g) { return g ? (int)g->tensors.size() : 0; }

int q38b_gguf_find(const q38b_gguf* g, const char* name) {
    if (!g || !name) return -1;
    for (size_t i = 0; i < g->tensors.size(); i++)
        if (g->tensors[i].name == name) return (int)i;
    return -1;
}

int q38b_gguf_tensor(const q38b_gguf* g, int index, const char** name, uint32_t* type, int* n_dims, long long dims[4], const void** data,
                     size_t* nbytes) {
    if (!g || index < 0 || index >= (int)g->tensors.size()) return Q38B_ERR_ARG;
    const Tensor& t = g->tensors[(size_t)index];
    if (name) *name = t.name.c_str();
    if (type) *type = t.type;
    if (n_dims) *n_dims = (int)t.n_dims;
    if (dims) for (int d = 0; d < 4; d++) dims[d] = (long long)t.dims[d];
    if (data) *data = g->base + g->data_offset + t.offset;
    if (nbytes) *nbytes = (size_t)t.nbytes;
    return Q38B_OK;
}

int q38b_pass_matrix_from_gguf(q38b_pass* pass, const q38b_gguf* g, int index, int shard, int n_shards) {
    if (!pass || !g || index < 0 || index >= (int)g->tensors.size()) return Q38B_ERR_ARG;
    const Tensor& t = g->tensors[(size_t)index];
    if (t.n_dims != 2 || t.dims[0] > 0x7fffffffull || t.dims[1] > 0x7fffffffull) return Q38B_ERR_ARG;   // a weight matrix: dims[0] = K (row length), dims[1] = rows
    if (!q38b_format_supported(t.type)) return Q38B_ERR_UNSUPPORTED;
    const int K = (int)t.dims[0], M = (int)t.dims[1];
    const size_t row_bytes = q38b_row_bytes(t.type, K);
    if (!row_bytes || row_bytes * (size_t)M != t.nbytes) return Q38B_ERR_ARG;
    return q38b_pass_matrix_upload(pass, t.type, g->base + g->data_offset + t.offset, row_bytes, K, M, shard, n_shards);
}

}  // extern "C"
