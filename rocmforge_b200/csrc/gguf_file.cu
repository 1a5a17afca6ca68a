// GGUF container: header, key/value metadata, tensor directory and memory-mapped tensor data, so that a
// model file feeds the packed-weight kernels directly (no fp32 detour).
//
// Replaces, for the quantized-weight path, the reference's parser and lazy loader:
//   header      src/loader/gguf/header.rs:28-79      magic "GGUF", version 3 only, tensor and KV counts
//   metadata    src/loader/gguf/metadata.rs:20-269   typed values rendered as strings, arrays skipped
//   directory   src/loader/gguf/tensor_info.rs:37-101 name, dims, type id, offset -> LazyTensor handles
//   mapping     src/loader/mmap.rs:38-100            read-only mmap, bounds-checked slices
//   upload      src/loader/gguf/types.rs:199-254     load_tensor_to_gpu (here: packed bytes stay packed)
// Host-only code; nothing here touches the device except b200q_gguf_upload_tensor, which hands the mapped
// bytes to b200q_weight_upload.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cinttypes>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "common.cuh"

namespace {

struct KV {
    std::string key;
    uint32_t type = 0;
    std::string text;   // scalar or string value as text; empty for arrays
    uint32_t array_type = 0;
    uint64_t array_len = 0;
};

struct TensorEntry {
    std::string name;
    uint32_t n_dims = 0;
    uint64_t dims[4] = {1, 1, 1, 1};
    uint32_t ggml_type = 0;
    uint64_t rel_offset = 0;   // as stored in the file
    uint64_t abs_offset = 0;   // file offset of the first byte
    uint64_t nbytes = 0;
    int qtype = -1;            // b200q_qtype, or -1 for types this library has no kernel for (F32, F16)
    int64_t n = 0, k = 0;      // rows x row length as the kernels see them
};

// Limits the reference applies while parsing (metadata.rs:29, :93, :193, :235).
constexpr uint64_t MAX_KEY_LEN = 100000;
constexpr uint64_t MAX_STRING_LEN = 100000000;
constexpr uint64_t MAX_ARRAY_BYTES = 1000000000;
constexpr uint64_t MAX_ARRAY_STRING_LEN = 10000000;
constexpr uint64_t MAX_NAME_LEN = 100000;

}  // namespace

struct b200q_gguf {
    int fd = -1;
    const uint8_t* map = nullptr;
    size_t size = 0;
    uint32_t version = 0;
    int flags = 0;
    uint64_t alignment = 32;
    uint64_t data_start = 0;
    std::vector<KV> kvs;
    std::vector<TensorEntry> tensors;
    std::unordered_map<std::string, int64_t> by_name;
    std::unordered_map<std::string, int64_t> kv_by_key;
};

namespace {

using b200q::fail;

struct Reader {
    const uint8_t* p;
    size_t size, pos = 0;
    bool ok = true;
    bool need(size_t n) {
        if (!ok || n > size - pos) { ok = false; return false; }
        return true;
    }
    template <typename T>
    T get() {
        T v{};
        if (need(sizeof(T))) { memcpy(&v, p + pos, sizeof(T)); pos += sizeof(T); }
        return v;
    }
    std::string str(uint64_t len) {
        std::string s;
        if (need(len)) { s.assign(reinterpret_cast<const char*>(p + pos), len); pos += len; }
        return s;
    }
    void skip(uint64_t n) { if (need(n)) pos += n; }
};

int scalar_size(uint32_t t) {
    switch (t) {
        case 0: case 1: case 7: return 1;
        case 2: case 3: return 2;
        case 4: case 5: case 6: return 4;
        case 10: case 11: case 12: return 8;
        default: return 0;
    }
}

// Scalar of GGUF value type t as text (the reference keeps every value as a String, metadata.rs:56-143).
std::string scalar_text(Reader& r, uint32_t t) {
    char buf[64];
    switch (t) {
        case 0: snprintf(buf, sizeof buf, "%u", (unsigned)r.get<uint8_t>()); break;
        case 1: snprintf(buf, sizeof buf, "%d", (int)r.get<int8_t>()); break;
        case 2: snprintf(buf, sizeof buf, "%u", (unsigned)r.get<uint16_t>()); break;
        case 3: snprintf(buf, sizeof buf, "%d", (int)r.get<int16_t>()); break;
        case 4: snprintf(buf, sizeof buf, "%" PRIu32, r.get<uint32_t>()); break;
        case 5: snprintf(buf, sizeof buf, "%" PRId32, r.get<int32_t>()); break;
        case 6: snprintf(buf, sizeof buf, "%.9g", (double)r.get<float>()); break;
        case 7: snprintf(buf, sizeof buf, "%s", r.get<uint8_t>() ? "true" : "false"); break;
        case 10: snprintf(buf, sizeof buf, "%" PRIu64, r.get<uint64_t>()); break;
        case 11: snprintf(buf, sizeof buf, "%" PRId64, r.get<int64_t>()); break;
        case 12: snprintf(buf, sizeof buf, "%.17g", r.get<double>()); break;
        default: buf[0] = 0; break;
    }
    return buf;
}

// GGUF type id -> (b200q qtype or -1, known). Ids follow GgufTensorType (src/loader/tensor_type.rs:16-61):
// 3, 6, 7 (Q4_1, Q5_0, Q5_1) and unknown ids are errors there and here. Ids 20, 21, 22 mean MXFP4 / MXFP6 only in
// the reference's own enum (tensor_type.rs:31-33), i.e. in files read in its dialect; files written by ggml use
// them for IQ4_NL / IQ3_S / IQ2_S, whose blocks this library has no kernel for, and carry MXFP4 as id 39.
bool map_type(uint32_t id, bool ref_style, int* qtype, int* known_block, int* plain_bytes) {
    *qtype = -1; *known_block = 0; *plain_bytes = 0;
    switch (id) {
        case 0: *plain_bytes = 4; return true;    // F32
        case 1: *plain_bytes = 2; return true;    // F16
        case 2: *qtype = B200Q_Q4_0; return true;
        case 8: *qtype = B200Q_Q8_0; return true;
        case 10: *qtype = B200Q_Q2_K; return true;
        case 11: *qtype = B200Q_Q3_K; return true;
        case 12: *qtype = B200Q_Q4_K; return true;
        case 13: *qtype = B200Q_Q5_K; return true;
        case 14: *qtype = B200Q_Q6_K; return true;
        case 39: if (ref_style) return false; *qtype = B200Q_MXFP4; return true;
        case 20: if (!ref_style) return false; *qtype = B200Q_MXFP4; return true;
        case 21: if (!ref_style) return false; *qtype = B200Q_MXFP6_E2M3; return true;
        case 22: if (!ref_style) return false; *qtype = B200Q_MXFP6_E3M2; return true;
        default: return false;
    }
}

}  // namespace

extern "C" {

int b200q_gguf_open(const char* path, int flags, b200q_gguf** out) {
    if (!out) return fail(B200Q_ERR_INVALID, "gguf_open: out is null");
    *out = nullptr;
    if (!path) return fail(B200Q_ERR_INVALID, "gguf_open: path is null");
    int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(B200Q_ERR_INVALID, "gguf_open: cannot open '%s': %s", path, strerror(errno));
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 24) {
        close(fd);
        return fail(B200Q_ERR_INVALID, "gguf_open: '%s' is too short to hold a GGUF header", path);
    }
    void* m = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    if (m == MAP_FAILED) {
        close(fd);
        return fail(B200Q_ERR_INVALID, "gguf_open: cannot map '%s': %s", path, strerror(errno));
    }
    b200q_gguf* g = new b200q_gguf();
    g->fd = fd; g->map = static_cast<const uint8_t*>(m); g->size = (size_t)st.st_size; g->flags = flags;
    auto bail = [&](int code, const std::string& msg) {
        munmap(const_cast<uint8_t*>(g->map), g->size);
        close(g->fd);
        delete g;
        return fail(code, "gguf_open: %s", msg.c_str());
    };
    Reader r{g->map, g->size};
    if (memcmp(g->map, "GGUF", 4) != 0) return bail(B200Q_ERR_INVALID, "invalid GGUF magic number");
    r.pos = 4;
    g->version = r.get<uint32_t>();
    if (g->version != 3)
        return bail(B200Q_ERR_UNSUPPORTED, "unsupported GGUF version " + std::to_string(g->version) + " (only version 3 is supported)");
    const uint64_t tensor_count = r.get<uint64_t>(), kv_count = r.get<uint64_t>();
    if (tensor_count > g->size / 24 || kv_count > g->size / 12) return bail(B200Q_ERR_INVALID, "tensor or KV count larger than the file");
    // ---- key/value pairs
    for (uint64_t i = 0; i < kv_count; i++) {
        KV kv;
        uint64_t klen = r.get<uint64_t>();
        if (klen > MAX_KEY_LEN) return bail(B200Q_ERR_INVALID, "key_len too large at index " + std::to_string(i));
        kv.key = r.str(klen);
        kv.type = r.get<uint32_t>();
        if (kv.type == 8) {
            uint64_t len = r.get<uint64_t>();
            if (len > MAX_STRING_LEN) return bail(B200Q_ERR_INVALID, "value_len too large for key '" + kv.key + "'");
            kv.text = r.str(len);
        } else if (kv.type == 9) {
            kv.array_type = r.get<uint32_t>();
            kv.array_len = r.get<uint64_t>();
            if (kv.array_type == 8) {
                for (uint64_t j = 0; j < kv.array_len && r.ok; j++) {
                    uint64_t len = r.get<uint64_t>();
                    if (len > MAX_ARRAY_STRING_LEN) return bail(B200Q_ERR_INVALID, "string too large in array '" + kv.key + "'");
                    r.skip(len);
                }
            } else {
                int es = scalar_size(kv.array_type);
                if (es == 0) return bail(B200Q_ERR_INVALID, "unknown array element type in '" + kv.key + "'");
                if (kv.array_len > MAX_ARRAY_BYTES / es) return bail(B200Q_ERR_INVALID, "array too large for key '" + kv.key + "'");
                r.skip(kv.array_len * es);
            }
        } else if (scalar_size(kv.type) != 0) {
            kv.text = scalar_text(r, kv.type);
        } else {
            return bail(B200Q_ERR_INVALID, "unknown value type " + std::to_string(kv.type) + " for key '" + kv.key + "'");
        }
        if (!r.ok) return bail(B200Q_ERR_INVALID, "file ends inside the metadata (key '" + kv.key + "')");
        if (kv.key == "general.alignment" && !kv.text.empty()) {
            uint64_t a = strtoull(kv.text.c_str(), nullptr, 10);
            if (a >= 1 && (a & (a - 1)) == 0) g->alignment = a;
        }
        g->kv_by_key.emplace(kv.key, (int64_t)g->kvs.size());
        g->kvs.push_back(std::move(kv));
    }
    // ---- tensor directory
    const bool ref_style = (flags & B200Q_GGUF_REFERENCE_FIXTURE) != 0;
    const int layout = ref_style ? B200Q_LAYOUT_RF : B200Q_LAYOUT_GGUF;
    for (uint64_t i = 0; i < tensor_count; i++) {
        TensorEntry t;
        uint64_t nlen = r.get<uint64_t>();
        if (nlen > MAX_NAME_LEN) return bail(B200Q_ERR_INVALID, "tensor name too long at index " + std::to_string(i));
        t.name = r.str(nlen);
        t.n_dims = r.get<uint32_t>();
        if (t.n_dims > 4) return bail(B200Q_ERR_INVALID, "tensor '" + t.name + "' has more than 4 dimensions");
        for (uint32_t d = 0; d < t.n_dims; d++) t.dims[d] = r.get<uint64_t>();
        t.ggml_type = r.get<uint32_t>();
        t.rel_offset = r.get<uint64_t>();
        if (!r.ok) return bail(B200Q_ERR_INVALID, "file ends inside the tensor directory");
        int block = 0, plain = 0;
        if (!map_type(t.ggml_type, ref_style, &t.qtype, &block, &plain))
            return bail(B200Q_ERR_UNSUPPORTED, "tensor '" + t.name + "' has unsupported GGUF tensor type " + std::to_string(t.ggml_type));
        unsigned __int128 elems = 1;
        for (uint32_t d = 0; d < t.n_dims; d++) {
            elems *= t.dims[d];
            if (elems > ((unsigned __int128)1 << 62)) return bail(B200Q_ERR_INVALID, "tensor '" + t.name + "' is too large");
        }
        const uint64_t n_el = (uint64_t)elems;
        // ggml stores the contiguous dimension first; the reference's own fixtures store rows first
        // (tests/common/fixtures.rs:125-183) and absolute offsets.
        if (t.n_dims == 0) { t.n = 1; t.k = 1; }
        else if (ref_style) { t.n = (int64_t)t.dims[0]; t.k = (int64_t)(t.dims[0] ? n_el / t.dims[0] : 0); }
        else { t.k = (int64_t)t.dims[0]; t.n = (int64_t)(t.dims[0] ? n_el / t.dims[0] : 0); }
        if (t.qtype >= 0) t.nbytes = b200q_tensor_bytes(t.qtype, layout, (int64_t)n_el);
        else if (plain) t.nbytes = n_el * plain;
        else t.nbytes = ((n_el + 255) / 256) * (ref_style ? 256 : block);
        g->by_name.emplace(t.name, (int64_t)g->tensors.size());
        g->tensors.push_back(std::move(t));
    }
    // ---- data section: aligned after the directory; offsets are relative to it (absolute in fixture style)
    g->data_start = ref_style ? 0 : (r.pos + g->alignment - 1) / g->alignment * g->alignment;
    for (auto& t : g->tensors) {
        t.abs_offset = g->data_start + t.rel_offset;
        if (t.abs_offset > g->size || t.nbytes > g->size - t.abs_offset)
            return bail(B200Q_ERR_INVALID, "slice out of bounds: tensor '" + t.name + "' offset=" + std::to_string(t.abs_offset) +
                                               " size=" + std::to_string(t.nbytes) + " file size=" + std::to_string(g->size));
    }
    *out = g;
    return B200Q_OK;
}

void b200q_gguf_close(b200q_gguf* g) {
    if (!g) return;
    if (g->map) munmap(const_cast<uint8_t*>(g->map), g->size);
    if (g->fd >= 0) close(g->fd);
    delete g;
}

int64_t b200q_gguf_tensor_count(const b200q_gguf* g) { return g ? (int64_t)g->tensors.size() : -1; }
int64_t b200q_gguf_kv_count(const b200q_gguf* g) { return g ? (int64_t)g->kvs.size() : -1; }

int64_t b200q_gguf_find_tensor(const b200q_gguf* g, const char* name) {
    if (!g || !name) return -1;
    auto it = g->by_name.find(name);
    return it == g->by_name.end() ? -1 : it->second;
}

int b200q_gguf_tensor_info(const b200q_gguf* g, int64_t index, b200q_gguf_tensor* out) {
    if (!g || !out) return fail(B200Q_ERR_INVALID, "gguf_tensor_info: null argument");
    if (index < 0 || index >= (int64_t)g->tensors.size()) return fail(B200Q_ERR_INVALID, "gguf_tensor_info: index %lld of %zu", (long long)index, g->tensors.size());
    const TensorEntry& t = g->tensors[(size_t)index];
    out->name = t.name.c_str();
    out->n_dims = (int)t.n_dims;
    for (int d = 0; d < 4; d++) out->dims[d] = (int64_t)t.dims[d];
    out->ggml_type = (int)t.ggml_type;
    out->qtype = t.qtype;
    out->layout = (g->flags & B200Q_GGUF_REFERENCE_FIXTURE) ? B200Q_LAYOUT_RF : B200Q_LAYOUT_GGUF;
    out->n = t.n; out->k = t.k;
    out->file_offset = (int64_t)t.abs_offset;
    out->nbytes = (size_t)t.nbytes;
    return B200Q_OK;
}

int b200q_gguf_kv_key(const b200q_gguf* g, int64_t index, const char** key, int* value_type) {
    if (!g || index < 0 || index >= (int64_t)g->kvs.size()) return fail(B200Q_ERR_INVALID, "gguf_kv_key: bad index");
    if (key) *key = g->kvs[(size_t)index].key.c_str();
    if (value_type) *value_type = (int)g->kvs[(size_t)index].type;
    return B200Q_OK;
}

int b200q_gguf_meta_string(const b200q_gguf* g, const char* key, char* buf, size_t buflen, size_t* needed) {
    if (!g || !key) return fail(B200Q_ERR_INVALID, "gguf_meta_string: null argument");
    auto it = g->kv_by_key.find(key);
    if (it == g->kv_by_key.end()) return fail(B200Q_ERR_INVALID, "gguf_meta_string: key '%s' not found", key);
    const std::string& s = g->kvs[(size_t)it->second].text;
    if (needed) *needed = s.size() + 1;
    if (buf && buflen) {
        size_t n = s.size() < buflen - 1 ? s.size() : buflen - 1;
        memcpy(buf, s.data(), n);
        buf[n] = 0;
    }
    return B200Q_OK;
}

int b200q_gguf_tensor_data(const b200q_gguf* g, int64_t index, const void** h_ptr, size_t* nbytes) {
    if (!g || !h_ptr) return fail(B200Q_ERR_INVALID, "gguf_tensor_data: null argument");
    if (index < 0 || index >= (int64_t)g->tensors.size()) return fail(B200Q_ERR_INVALID, "gguf_tensor_data: index %lld of %zu", (long long)index, g->tensors.size());
    const TensorEntry& t = g->tensors[(size_t)index];
    *h_ptr = g->map + t.abs_offset;
    if (nbytes) *nbytes = (size_t)t.nbytes;
    return B200Q_OK;
}

int b200q_gguf_upload_tensor(b200q_ctx* ctx, const b200q_gguf* g, int64_t index, int shard_rank, int shard_count, b200q_weight** out) {
    if (!g || !out) return fail(B200Q_ERR_INVALID, "gguf_upload_tensor: null argument");
    *out = nullptr;
    if (index < 0 || index >= (int64_t)g->tensors.size()) return fail(B200Q_ERR_INVALID, "gguf_upload_tensor: index %lld of %zu", (long long)index, g->tensors.size());
    const TensorEntry& t = g->tensors[(size_t)index];
    if (t.qtype < 0)
        return fail(B200Q_ERR_UNSUPPORTED, "gguf_upload_tensor: tensor '%s' has GGUF type %u, which this library has no packed kernel for",
                    t.name.c_str(), t.ggml_type);
    const int layout = (g->flags & B200Q_GGUF_REFERENCE_FIXTURE) ? B200Q_LAYOUT_RF : B200Q_LAYOUT_GGUF;
    return b200q_weight_upload(ctx, g->map + t.abs_offset, (size_t)t.nbytes, t.qtype, layout, B200Q_ORIENT_NK, t.n, t.k, shard_rank,
                               shard_count, out);
}

int b200q_gguf_upload_all(b200q_ctx* ctx, const b200q_gguf* g, int shard_rank, int shard_count, b200q_arena** arena_out,
                          b200q_weight** handles, int64_t n_handles) {
    if (!ctx || !g || !arena_out || !handles) return fail(B200Q_ERR_INVALID, "gguf_upload_all: null argument");
    *arena_out = nullptr;
    if (n_handles != (int64_t)g->tensors.size())
        return fail(B200Q_ERR_INVALID, "gguf_upload_all: %lld handle slots for %zu tensors", (long long)n_handles, g->tensors.size());
    if (shard_count < 1 || shard_rank < 0 || shard_rank >= shard_count) return fail(B200Q_ERR_INVALID, "gguf_upload_all: shard %d of %d", shard_rank, shard_count);
    const int layout = (g->flags & B200Q_GGUF_REFERENCE_FIXTURE) ? B200Q_LAYOUT_RF : B200Q_LAYOUT_GGUF;
    for (int64_t i = 0; i < n_handles; i++) handles[i] = nullptr;
    // pass 1: what the arena has to hold (MemoryCalculator's role, src/memory/)
    size_t total = 0;
    for (const TensorEntry& t : g->tensors) {
        if (t.qtype < 0) continue;
        const int64_t n_local = (shard_count > 1 && t.n % shard_count == 0) ? t.n / shard_count : t.n;
        size_t b = 0;
        int rc = b200q_arena_tensor_bytes(t.qtype, layout, B200Q_ORIENT_NK, n_local, t.k, &b);
        if (rc != B200Q_OK) return rc;
        total += b;
    }
    if (total == 0) return fail(B200Q_ERR_UNSUPPORTED, "gguf_upload_all: the file holds no tensor type this library has packed kernels for");
    b200q_arena* arena = nullptr;
    int rc = b200q_arena_create(ctx, total, &arena);
    if (rc != B200Q_OK) return rc;
    // pass 2: queue the uploads
    for (size_t i = 0; i < g->tensors.size() && rc == B200Q_OK; i++) {
        const TensorEntry& t = g->tensors[i];
        if (t.qtype < 0) continue;
        const bool split = shard_count > 1 && t.n % shard_count == 0;
        rc = b200q_arena_upload(ctx, arena, g->map + t.abs_offset, (size_t)t.nbytes, t.qtype, layout, B200Q_ORIENT_NK, t.n, t.k,
                                split ? shard_rank : 0, split ? shard_count : 1, &handles[i]);
    }
    if (rc != B200Q_OK) {
        for (int64_t i = 0; i < n_handles; i++) {
            if (handles[i]) b200q_weight_free(handles[i]);
            handles[i] = nullptr;
        }
        b200q_arena_free(arena);
        return rc;
    }
    *arena_out = arena;
    return B200Q_OK;
}

}  // extern "C"
