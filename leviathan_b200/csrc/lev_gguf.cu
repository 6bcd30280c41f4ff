// GGUF v2/v3 container reader: header, metadata, tensor directory, and a read-only mapping of
// the file from which tensors are uploaded without an intermediate copy.  Host code only.
//
// Written from the public GGUF format description; behaviour follows the reference's reader
// (Sources/LeviathanCore/GGUF.swift:96-406; Rust twin rust/crates/lev-gguf/src/lib.rs):
// little-endian, every untrusted integer is range-checked before use, hard caps on counts,
// string and array lengths and on the header region, alignment from `general.alignment`
// (default 32), every tensor validated when the file is opened (known type, whole blocks,
// aligned offset, inside the file, no two tensors overlapping, no duplicate names).
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <map>
#include <string>
#include <vector>

#include "lev_internal.h"

namespace {

// caps of the reference reader (GGUF.swift:181-189)
constexpr uint64_t kMaxEntries = 100000;
constexpr uint64_t kMaxStringLength = 1u << 20;
constexpr uint64_t kMaxArrayElements = 10000000;
constexpr uint64_t kMaxHeaderBytes = 256ull << 20;
constexpr uint64_t kMaxTensorElements = 1ull << 40;
constexpr uint64_t kMaxAlignment = 1u << 20;

struct Value {
    uint32_t type = 0;        // GGUF value type code; 9 = array
    uint64_t u = 0;           // unsigned / bool payload
    int64_t i = 0;            // signed payload
    double f = 0;             // float payload
    std::string s;            // string payload
    uint32_t elem_type = 0;   // arrays: element type, count and where the payloads lie in the file
    uint64_t count = 0;
    uint64_t payload = 0;               // fixed-size elements: offset of element 0
    std::vector<uint64_t> item_offset;  // strings: offset of each element's length field
};

struct TensorInfo {
    std::string name;
    int n_dims = 0;
    int64_t dims[4] = {1, 1, 1, 1};
    uint32_t type = 0;
    uint64_t offset = 0;   // relative to the data region
    uint64_t bytes = 0;
    uint64_t start = 0;    // absolute file offset
};

struct Failure {
    int status;
    std::string message;
};

// bytes per block / values per block of the tensor types this reader sizes
bool type_geometry(uint32_t type, int* values, int* bytes) {
    switch (type) {
        case 0: *values = 1; *bytes = 4; return true;     // F32
        case 1: *values = 1; *bytes = 2; return true;     // F16
        case 2: *values = 32; *bytes = 18; return true;   // Q4_0
        case 8: *values = 32; *bytes = 34; return true;   // Q8_0
        case 12: *values = 256; *bytes = 144; return true;  // Q4_K
        case 14: *values = 256; *bytes = 210; return true;  // Q6_K
        case 30: *values = 1; *bytes = 2; return true;    // BF16
    }
    return false;
}

class Cursor {
  public:
    Cursor(const uint8_t* p, uint64_t n) : p_(p), n_(n) {}
    uint64_t position() const { return pos_; }
    const uint8_t* take(uint64_t count, const char* what) {
        if (count > n_ - pos_ || pos_ > kMaxHeaderBytes) throw Failure{LEV_GGUF_TRUNCATED, std::string("read of ") + what + " past the end"};
        const uint8_t* r = p_ + pos_;
        pos_ += count;
        return r;
    }
    uint32_t u32(const char* what) {
        const uint8_t* b = take(4, what);
        return (uint32_t)b[0] | (uint32_t)b[1] << 8 | (uint32_t)b[2] << 16 | (uint32_t)b[3] << 24;
    }
    uint64_t u64(const char* what) {
        const uint8_t* b = take(8, what);
        uint64_t v = 0;
        for (int j = 0; j < 8; j++) v |= (uint64_t)b[j] << (8 * j);
        return v;
    }
    std::string str(const char* what) {
        uint64_t len = u64(what);
        if (len > kMaxStringLength) throw Failure{LEV_GGUF_TRUNCATED, std::string(what) + ": string length beyond cap"};
        const uint8_t* b = take(len, what);
        return std::string(reinterpret_cast<const char*>(b), (size_t)len);
    }
    // payload of a value of a known scalar / string type
    void payload(uint32_t type, Value* v) {
        v->type = type;
        switch (type) {
            case 0: v->u = take(1, "uint8")[0]; v->i = (int64_t)v->u; break;
            case 1: v->i = (int8_t)take(1, "int8")[0]; break;
            case 2: { const uint8_t* b = take(2, "uint16"); v->u = (uint64_t)b[0] | (uint64_t)b[1] << 8; v->i = (int64_t)v->u; break; }
            case 3: { const uint8_t* b = take(2, "int16"); v->i = (int16_t)((uint16_t)b[0] | (uint16_t)b[1] << 8); break; }
            case 4: v->u = u32("uint32"); v->i = (int64_t)v->u; break;
            case 5: v->i = (int32_t)u32("int32"); break;
            case 6: { uint32_t bits = u32("float32"); float f; memcpy(&f, &bits, 4); v->f = f; break; }
            case 7: v->u = take(1, "bool")[0] != 0; break;
            case 8: v->s = str("string value"); break;
            case 10: v->u = u64("uint64"); v->i = v->u > (uint64_t)INT64_MAX ? INT64_MAX : (int64_t)v->u; break;
            case 11: v->i = (int64_t)u64("int64"); break;
            case 12: { uint64_t bits = u64("float64"); memcpy(&v->f, &bits, 8); break; }
            default: throw Failure{LEV_GGUF_UNKNOWN_VALUE_TYPE, "value type " + std::to_string(type)};
        }
    }
    void value(Value* v) {
        uint32_t type = u32("value type");
        if (type != 9) {
            payload(type, v);
            return;
        }
        v->type = 9;
        v->elem_type = u32("array element type");
        if (v->elem_type == 9 || v->elem_type > 12) throw Failure{LEV_GGUF_UNKNOWN_VALUE_TYPE, "array element type " + std::to_string(v->elem_type)};
        v->count = u64("array length");
        if (v->count > kMaxArrayElements) throw Failure{LEV_GGUF_TRUNCATED, "array too long"};
        v->payload = pos_;
        Value e;
        if (v->elem_type == 8) v->item_offset.reserve((size_t)std::min<uint64_t>(v->count, (n_ - pos_) / 8));
        for (uint64_t k = 0; k < v->count; k++) {  // validated; contents stay in the file
            if (v->elem_type == 8) v->item_offset.push_back(pos_);
            payload(v->elem_type, &e);
        }
    }

  private:
    const uint8_t* p_;
    uint64_t n_, pos_ = 0;
};

}  // namespace

struct lev_gguf {
    const uint8_t* data = nullptr;
    uint64_t size = 0;
    bool mapped = false;
    uint32_t version = 0;
    uint64_t alignment = 32, data_offset = 0;
    std::map<std::string, Value> meta;
    std::vector<TensorInfo> tensors;
    std::map<std::string, size_t> by_name;
};

namespace {

void parse_into(lev_gguf* g) {
    Cursor c(g->data, g->size);
    if (g->size < 12) throw Failure{LEV_GGUF_TRUNCATED, "header"};
    if (memcmp(c.take(4, "magic"), "GGUF", 4) != 0) throw Failure{LEV_GGUF_BAD_MAGIC, "not a GGUF file"};
    g->version = c.u32("version");
    if (g->version != 2 && g->version != 3) throw Failure{LEV_GGUF_UNSUPPORTED_VERSION, "version " + std::to_string(g->version)};
    const uint64_t n_tensors = c.u64("tensor count"), n_kv = c.u64("metadata count");
    if (n_tensors > kMaxEntries || n_kv > kMaxEntries) throw Failure{LEV_GGUF_TRUNCATED, "implausible tensor/kv counts"};
    for (uint64_t k = 0; k < n_kv; k++) {
        std::string key = c.str("metadata key");
        if (g->meta.count(key)) throw Failure{LEV_GGUF_TRUNCATED, "duplicate metadata key " + key};
        c.value(&g->meta[key]);
    }
    for (uint64_t k = 0; k < n_tensors; k++) {
        TensorInfo t;
        t.name = c.str("tensor name");
        if (g->by_name.count(t.name)) throw Failure{LEV_GGUF_BAD_TENSOR, "duplicate tensor name " + t.name};
        const uint32_t nd = c.u32("dimension count");
        if (nd < 1 || nd > 4) throw Failure{LEV_GGUF_BAD_TENSOR, "tensor " + t.name + ": bad dim count " + std::to_string(nd)};
        t.n_dims = (int)nd;
        for (uint32_t d = 0; d < nd; d++) {
            const uint64_t v = c.u64("dimension");
            if (v == 0 || v > kMaxTensorElements) throw Failure{LEV_GGUF_BAD_TENSOR, "tensor " + t.name + ": invalid dimension"};
            t.dims[d] = (int64_t)v;
        }
        t.type = c.u32("tensor type");
        t.offset = c.u64("tensor offset");
        if (t.offset > (uint64_t)INT64_MAX) throw Failure{LEV_INTEGER_OVERFLOW, "tensor " + t.name + ": offset"};
        g->by_name[t.name] = g->tensors.size();
        g->tensors.push_back(t);
    }
    auto al = g->meta.find("general.alignment");
    if (al != g->meta.end() && al->second.type == 4) {
        if (al->second.u == 0 || al->second.u > kMaxAlignment) throw Failure{LEV_GGUF_TRUNCATED, "invalid general.alignment"};
        g->alignment = al->second.u;
    }
    const uint64_t pos = c.position();
    g->data_offset = (pos + g->alignment - 1) / g->alignment * g->alignment;
    // every tensor: known type, whole blocks, aligned, inside the file
    for (TensorInfo& t : g->tensors) {
        int vals, bytes;
        if (!type_geometry(t.type, &vals, &bytes)) throw Failure{LEV_GGUF_UNSUPPORTED_TENSOR_TYPE, "tensor " + t.name + ": ggml type " + std::to_string(t.type)};
        uint64_t elements = 1;
        for (int d = 0; d < t.n_dims; d++) {
            if ((uint64_t)t.dims[d] > kMaxTensorElements / elements) throw Failure{LEV_INTEGER_OVERFLOW, "tensor " + t.name + ": element count"};
            elements *= (uint64_t)t.dims[d];
        }
        if (elements % (uint64_t)vals != 0 || (uint64_t)t.dims[0] % (uint64_t)vals != 0)
            throw Failure{LEV_GGUF_BAD_TENSOR, "tensor " + t.name + ": element count is not a multiple of the block"};
        t.bytes = elements / (uint64_t)vals * (uint64_t)bytes;
        if (t.offset % g->alignment != 0) throw Failure{LEV_GGUF_BAD_TENSOR, "tensor " + t.name + ": offset " + std::to_string(t.offset) + " misaligned"};
        if (t.offset > g->size || g->data_offset > g->size - t.offset || t.bytes > g->size - g->data_offset - t.offset)
            throw Failure{LEV_GGUF_DATA_BEYOND_EOF, "tensor " + t.name + ": storage reaches beyond the file's " + std::to_string(g->size) + " bytes"};
        t.start = g->data_offset + t.offset;
    }
    // no two tensors overlap
    std::vector<const TensorInfo*> order;
    for (const TensorInfo& t : g->tensors) order.push_back(&t);
    std::stable_sort(order.begin(), order.end(), [](const TensorInfo* a, const TensorInfo* b) { return a->start < b->start; });
    for (size_t k = 1; k < order.size(); k++)
        if (order[k - 1]->start + order[k - 1]->bytes > order[k]->start)
            throw Failure{LEV_GGUF_BAD_TENSOR, "tensor " + order[k]->name + " overlaps " + order[k - 1]->name};
}

int finish(lev_gguf* g, lev_gguf** out, char* err, size_t err_len) {
    try {
        parse_into(g);
    } catch (const Failure& f) {
        if (err && err_len) snprintf(err, err_len, "%s", f.message.c_str());
        if (g->mapped) munmap(const_cast<uint8_t*>(g->data), g->size);
        delete g;
        return f.status;
    } catch (const std::bad_alloc&) {
        if (err && err_len) snprintf(err, err_len, "out of host memory");
        if (g->mapped) munmap(const_cast<uint8_t*>(g->data), g->size);
        delete g;
        return LEV_OUT_OF_MEMORY;
    }
    *out = g;
    return LEV_OK;
}

}  // namespace

extern "C" int lev_gguf_parse(const void* bytes, size_t n_bytes, lev_gguf** out, char* err, size_t err_len) {
    if (!bytes || !out) return LEV_BAD_ARGUMENT;
    *out = nullptr;
    lev_gguf* g = new lev_gguf;
    g->data = static_cast<const uint8_t*>(bytes);
    g->size = n_bytes;
    return finish(g, out, err, err_len);
}

extern "C" int lev_gguf_open(const char* path, lev_gguf** out, char* err, size_t err_len) {
    if (!path || !out) return LEV_BAD_ARGUMENT;
    *out = nullptr;
    int fd = open(path, O_RDONLY);
    if (fd < 0) {
        if (err && err_len) snprintf(err, err_len, "cannot open %s", path);
        return LEV_BAD_ARGUMENT;
    }
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 12) {
        close(fd);
        if (err && err_len) snprintf(err, err_len, "header");
        return LEV_GGUF_TRUNCATED;
    }
    void* p = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (p == MAP_FAILED) {
        if (err && err_len) snprintf(err, err_len, "cannot map %s", path);
        return LEV_OUT_OF_MEMORY;
    }
    lev_gguf* g = new lev_gguf;
    g->data = static_cast<const uint8_t*>(p);
    g->size = (uint64_t)st.st_size;
    g->mapped = true;
    return finish(g, out, err, err_len);
}

extern "C" void lev_gguf_close(lev_gguf* g) {
    if (!g) return;
    if (g->mapped) munmap(const_cast<uint8_t*>(g->data), g->size);
    delete g;
}

extern "C" int lev_gguf_summary(const lev_gguf* g, uint32_t* version, int64_t* n_tensors, int64_t* n_metadata, uint64_t* alignment,
                                uint64_t* data_offset) {
    if (!g) return LEV_BAD_ARGUMENT;
    if (version) *version = g->version;
    if (n_tensors) *n_tensors = (int64_t)g->tensors.size();
    if (n_metadata) *n_metadata = (int64_t)g->meta.size();
    if (alignment) *alignment = g->alignment;
    if (data_offset) *data_offset = g->data_offset;
    return LEV_OK;
}

extern "C" int64_t lev_gguf_find_tensor(const lev_gguf* g, const char* name) {
    if (!g || !name) return -1;
    auto it = g->by_name.find(name);
    return it == g->by_name.end() ? -1 : (int64_t)it->second;
}

extern "C" int lev_gguf_tensor_info(const lev_gguf* g, int64_t index, const char** name, int* ggml_type, int* n_dims, int64_t* dims4,
                                    uint64_t* file_offset, uint64_t* n_bytes) {
    if (!g || index < 0 || index >= (int64_t)g->tensors.size()) return LEV_GGUF_MISSING;
    const TensorInfo& t = g->tensors[(size_t)index];
    if (name) *name = t.name.c_str();
    if (ggml_type) *ggml_type = (int)t.type;
    if (n_dims) *n_dims = t.n_dims;
    if (dims4)
        for (int d = 0; d < 4; d++) dims4[d] = t.dims[d];
    if (file_offset) *file_offset = t.start;
    if (n_bytes) *n_bytes = t.bytes;
    return LEV_OK;
}

extern "C" const void* lev_gguf_tensor_data(const lev_gguf* g, int64_t index) {
    if (!g || index < 0 || index >= (int64_t)g->tensors.size()) return nullptr;
    return g->data + g->tensors[(size_t)index].start;
}

// integer metadata (any integer type; negative values read as 0, like metadataUInt in the reference)
extern "C" int lev_gguf_meta_u64(const lev_gguf* g, const char* key, uint64_t* out) {
    if (!g || !key || !out) return LEV_BAD_ARGUMENT;
    auto it = g->meta.find(key);
    if (it == g->meta.end()) return LEV_GGUF_MISSING;
    const Value& v = it->second;
    switch (v.type) {
        case 0: case 2: case 4: case 10: *out = v.u; return LEV_OK;
        case 1: case 3: case 5: case 11: *out = v.i >= 0 ? (uint64_t)v.i : 0; return LEV_OK;
    }
    return LEV_GGUF_MISSING;
}

extern "C" int lev_gguf_meta_f64(const lev_gguf* g, const char* key, double* out) {
    if (!g || !key || !out) return LEV_BAD_ARGUMENT;
    auto it = g->meta.find(key);
    if (it == g->meta.end() || (it->second.type != 6 && it->second.type != 12)) return LEV_GGUF_MISSING;
    *out = it->second.f;
    return LEV_OK;
}

extern "C" int lev_gguf_meta_string(const lev_gguf* g, const char* key, const char** out, size_t* len) {
    if (!g || !key || !out) return LEV_BAD_ARGUMENT;
    auto it = g->meta.find(key);
    if (it == g->meta.end() || it->second.type != 8) return LEV_GGUF_MISSING;
    *out = it->second.s.c_str();
    if (len) *len = it->second.s.size();
    return LEV_OK;
}

// Arrays: element type and count, then one element at a time as (pointer to its payload in the
// file, payload bytes): little-endian scalars, or the characters of a string element.
extern "C" int lev_gguf_meta_array(const lev_gguf* g, const char* key, int* elem_type, uint64_t* count) {
    if (!g || !key) return LEV_BAD_ARGUMENT;
    auto it = g->meta.find(key);
    if (it == g->meta.end() || it->second.type != 9) return LEV_GGUF_MISSING;
    if (elem_type) *elem_type = (int)it->second.elem_type;
    if (count) *count = it->second.count;
    return LEV_OK;
}

extern "C" int lev_gguf_meta_array_item(const lev_gguf* g, const char* key, uint64_t index, const void** payload, size_t* n_bytes) {
    if (!g || !key || !payload || !n_bytes) return LEV_BAD_ARGUMENT;
    auto it = g->meta.find(key);
    if (it == g->meta.end() || it->second.type != 9 || index >= it->second.count) return LEV_GGUF_MISSING;
    const Value& v = it->second;
    if (v.elem_type == 8) {
        const uint8_t* p = g->data + v.item_offset[(size_t)index];
        uint64_t len = 0;
        for (int j = 0; j < 8; j++) len |= (uint64_t)p[j] << (8 * j);
        *payload = p + 8;
        *n_bytes = (size_t)len;
        return LEV_OK;
    }
    static const int kSize[13] = {1, 1, 2, 2, 4, 4, 4, 1, 0, 0, 8, 8, 8};
    *payload = g->data + v.payload + index * (uint64_t)kSize[v.elem_type];
    *n_bytes = (size_t)kSize[v.elem_type];
    return LEV_OK;
}

// Uploads a Q4_0 / Q4_K / Q6_K tensor straight from the mapping.  GGUF dims are innermost
// first: dims[0] = inDim (cols), dims[1] = outDim (rows); a third dimension (expert tensors
// [in, out, experts], Sources/LeviathanCore/Gemma4.swift:184-284) stacks the experts' rows.
extern "C" int lev_gguf_upload(lev_ctx* ctx, const lev_gguf* g, const char* name, lev_weights** out) {
    if (!ctx || !g || !name || !out) return LEV_BAD_ARGUMENT;
    const int64_t i = lev_gguf_find_tensor(g, name);
    if (i < 0) return lev_fail(ctx, LEV_GGUF_MISSING, "tensor %s is not in the file", name);
    const TensorInfo& t = g->tensors[(size_t)i];
    if (t.type != LEV_GGML_Q4_0 && t.type != LEV_GGML_Q4_K && t.type != LEV_GGML_Q6_K)
        return lev_fail(ctx, LEV_GGUF_UNSUPPORTED_TENSOR_TYPE, "tensor %s: ggml type %u is not a quantized format of this path", name, t.type);
    if (t.n_dims < 2 || t.n_dims > 3) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "tensor %s: %d dimensions", name, t.n_dims);
    const int64_t rows = t.dims[1] * (t.n_dims == 3 ? t.dims[2] : 1);
    return lev_weights_upload(ctx, g->data + t.start, (size_t)t.bytes, (int)t.type, rows, t.dims[0], 0, out);
}

// One layer's routed-expert weights from a model file, with the checks of MoEModelBinding.bind
// (Sources/LeviathanCore/MoEModelBinding.swift:93-166): shape metadata under the architecture's
// prefix, blk.<layer>.ffn_gate_up_exps.weight Q4_0 [hidden, 2*inter, experts],
// blk.<layer>.ffn_down_exps.weight Q4_0 [inter, hidden, experts], and the f32 router
// blk.<layer>.ffn_gate_inp.weight [hidden, experts] (Sources/LeviathanCore/Gemma4.swift:236-246).
extern "C" int lev_gguf_moe_upload(lev_ctx* ctx, const lev_gguf* g, int layer, int local_first, int local_count, lev_moe_weights** out,
                                   int* top_k) {
    if (!ctx || !g || !out) return LEV_BAD_ARGUMENT;
    *out = nullptr;
    auto arch_it = g->meta.find("general.architecture");
    if (arch_it == g->meta.end() || arch_it->second.type != 8) return lev_fail(ctx, LEV_GGUF_MISSING, "general.architecture");
    const std::string arch = arch_it->second.s;
    auto meta_int = [&](const char* suffix, int64_t cap, int64_t* v) -> int {
        const std::string key = arch + "." + suffix;
        uint64_t u = 0;
        if (lev_gguf_meta_u64(g, key.c_str(), &u) != LEV_OK) return lev_fail(ctx, LEV_GGUF_MISSING, "metadata %s", key.c_str());
        if (u == 0 || u > (uint64_t)cap) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "%s = %llu outside (0, %lld]", key.c_str(), (unsigned long long)u, (long long)cap);
        *v = (int64_t)u;
        return LEV_OK;
    };
    int64_t layers = 0, experts = 0, used = 0, hidden = 0, inter = 0;
    int st;
    if ((st = meta_int("block_count", 1 << 16, &layers))) return st;
    if ((st = meta_int("expert_count", LEV_MAX_EXPERTS, &experts))) return st;
    if ((st = meta_int("expert_used_count", LEV_MAX_TOP_K, &used))) return st;
    if ((st = meta_int("embedding_length", 8192, &hidden))) return st;
    if ((st = meta_int("expert_feed_forward_length", 8192, &inter))) return st;
    if (used > experts) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "topK %lld > expert_count %lld", (long long)used, (long long)experts);
    if (layer < 0 || layer >= layers) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "layer %d outside 0..<%lld", layer, (long long)layers);
    if (local_count <= 0) {
        local_first = 0;
        local_count = (int)experts;
    }
    if (local_first < 0 || local_first + (int64_t)local_count > experts)
        return lev_fail(ctx, LEV_BAD_DIMENSIONS, "local experts [%d, +%d) of %lld", local_first, local_count, (long long)experts);
    const std::string p = "blk." + std::to_string(layer) + ".";
    auto find = [&](const std::string& name, uint32_t type, std::vector<int64_t> dims, const TensorInfo** t) -> int {
        auto it = g->by_name.find(name);
        if (it == g->by_name.end()) return lev_fail(ctx, LEV_GGUF_MISSING, "tensor %s is not in the file", name.c_str());
        const TensorInfo& ti = g->tensors[it->second];
        bool same = ti.type == type && ti.n_dims == (int)dims.size();
        for (size_t d = 0; same && d < dims.size(); d++) same = ti.dims[d] == dims[d];
        if (!same) return lev_fail(ctx, LEV_BAD_DIMENSIONS, "%s: type %u, %d dims [%lld, %lld, %lld] do not match the model's shape", name.c_str(),
                                   ti.type, ti.n_dims, (long long)ti.dims[0], (long long)ti.dims[1], (long long)ti.dims[2]);
        *t = &ti;
        return LEV_OK;
    };
    const TensorInfo *gu, *dn, *rw;
    st = find(p + "ffn_gate_up_exps.weight", LEV_GGML_Q4_0, {hidden, 2 * inter, experts}, &gu);
    if (st != LEV_OK) return st;
    st = find(p + "ffn_down_exps.weight", LEV_GGML_Q4_0, {inter, hidden, experts}, &dn);
    if (st != LEV_OK) return st;
    st = find(p + "ffn_gate_inp.weight", LEV_GGML_F32, {hidden, experts}, &rw);
    if (st != LEV_OK) return st;
    const uint64_t gu_stride = gu->bytes / (uint64_t)experts, dn_stride = dn->bytes / (uint64_t)experts;
    if (top_k) *top_k = (int)used;
    return lev_moe_weights_upload(ctx, reinterpret_cast<const float*>(g->data + rw->start),
                                  g->data + gu->start + gu_stride * (uint64_t)local_first, (size_t)(gu_stride * (uint64_t)local_count),
                                  g->data + dn->start + dn_stride * (uint64_t)local_first, (size_t)(dn_stride * (uint64_t)local_count), (int)experts,
                                  (int)hidden, (int)inter, local_first, local_count, 0, out);
}
