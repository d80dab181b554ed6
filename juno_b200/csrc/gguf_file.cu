// GGUF model files on the host: header, metadata, tensor table and raw tensor bytes, as the reference parses them
// (node/GgufReader.java: open :102-180, tensorRaw :329-340, rawByteCount :347-360, readMetadataValue :1189-1244), and
// the model configuration the reference derives from the metadata (node/LlamaConfig.java: from :58-91).
//
// Host code only: the file is mapped read-only and tensors are handed out as pointers into the mapping, so a
// quantised matrix goes from the page cache to the GPU without a copy in between.  The file is not trusted: every
// length and offset is checked against the file size before it is used.  A GGUF embedded in a llamafile ZIP (which the
// reference also scans for) is not supported; the file must start with the GGUF magic.
#include "common.cuh"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <climits>
#include <cstring>
#include <map>
#include <string>
#include <vector>

namespace juno {

constexpr uint32_t kMagicGguf = 0x4A474746;     // handle tag "JGGF"
constexpr uint32_t kGgufFileMagic = 0x46554747; // "GGUF", little endian (GgufReader.java:50)
constexpr int64_t kGgufAlignment = 32;          // GgufReader.java:51

struct GgufValue {
    enum Kind { INT, FLOAT, BOOL, STRING, ARRAY } kind = INT;
    int64_t i = 0;      // INT / BOOL; ARRAY: element count
    double f = 0.0;     // FLOAT
    std::string s;      // STRING
    int32_t elem_type = 0;  // ARRAY
};

struct GgufTensor {
    std::string name;
    int32_t type = 0, ndims = 0;
    int64_t dims[4] = {1, 1, 1, 1};  // innermost first: a weight matrix is [cols (in), rows (out)] (GgufReader.java:246-248)
    int64_t offset = 0;              // relative to the data section
    int64_t nelems = 1, nbytes = 0;
};

}  // namespace juno

struct juno_gguf {
    uint32_t magic = juno::kMagicGguf;
    int fd = -1;
    const uint8_t *base = nullptr;
    int64_t size = 0;
    int32_t version = 0;
    int64_t data_offset = 0;
    std::map<std::string, juno::GgufValue> meta;
    std::vector<juno::GgufTensor> tensors;  // file order
    std::map<std::string, size_t> by_name;
};

namespace juno {

// rawByteCount (GgufReader.java:347-360); -1 for a type without a formula
static int64_t raw_byte_count(int32_t type, int64_t nelems) {
    switch (type) {
        case 0: return nelems * 4;             // F32
        case 1: case 30: return nelems * 2;    // F16, BF16
        case 8: return nelems / 32 * 34;       // Q8_0
        case 2: return nelems / 32 * 18;       // Q4_0
        case 10: return nelems / 256 * 84;     // Q2_K
        case 11: return nelems / 256 * 110;    // Q3_K
        case 12: return nelems / 256 * 144;    // Q4_K
        case 13: return nelems / 256 * 176;    // Q5_K
        case 14: return nelems / 256 * 210;    // Q6_K
        default: return -1;
    }
}

struct Cursor {
    const uint8_t *base;
    int64_t size, pos;
    bool ok = true;
    template <typename T>
    T get() {
        T v{};
        if (!ok || pos + (int64_t)sizeof(T) > size) {
            ok = false;
            return v;
        }
        memcpy(&v, base + pos, sizeof(T));
        pos += sizeof(T);
        return v;
    }
    std::string str() {  // u64 length + UTF-8 bytes (GgufReader.java:1165-1171)
        const uint64_t len = get<uint64_t>();
        if (!ok || len > (uint64_t)(size - pos)) {
            ok = false;
            return {};
        }
        std::string s(reinterpret_cast<const char *>(base + pos), (size_t)len);
        pos += (int64_t)len;
        return s;
    }
};

// One metadata value (readMetadataValue, GgufReader.java:1189-1244).  As there, 8- and 16-bit integers of either
// signedness are read as signed, 32-bit ones as a signed int and 64-bit ones as a signed long.
static bool read_value(Cursor &c, int32_t vtype, GgufValue &out, int depth) {
    switch (vtype) {
        case 0: case 1: out.kind = GgufValue::INT; out.i = c.get<int8_t>(); break;
        case 2: case 3: out.kind = GgufValue::INT; out.i = c.get<int16_t>(); break;
        case 4: case 5: out.kind = GgufValue::INT; out.i = c.get<int32_t>(); break;
        case 6: out.kind = GgufValue::FLOAT; out.f = c.get<float>(); break;
        case 7: out.kind = GgufValue::BOOL; out.i = c.get<int8_t>() != 0; break;
        case 8: out.kind = GgufValue::STRING; out.s = c.str(); break;
        case 10: case 11: out.kind = GgufValue::INT; out.i = c.get<int64_t>(); break;
        case 12: out.kind = GgufValue::FLOAT; out.f = c.get<double>(); break;
        case 9: {  // array: element type, count, elements (readArray :1246-1253); only the count is kept
            if (depth > 2) return false;
            out.kind = GgufValue::ARRAY;
            out.elem_type = c.get<int32_t>();
            const uint64_t n = c.get<uint64_t>();
            if (!c.ok || n > (uint64_t)c.size) return false;
            out.i = (int64_t)n;
            static const int fixed[13] = {1, 1, 2, 2, 4, 4, 4, 1, 0, 0, 8, 8, 8};
            if (out.elem_type >= 0 && out.elem_type <= 12 && fixed[out.elem_type]) {
                const int64_t bytes = (int64_t)n * fixed[out.elem_type];
                if (bytes > c.size - c.pos) return false;
                c.pos += bytes;
            } else {
                GgufValue tmp;
                for (uint64_t k = 0; k < n && c.ok; k++)
                    if (!read_value(c, out.elem_type, tmp, depth + 1)) return false;
            }
            break;
        }
        default: return false;
    }
    return c.ok;
}

static int gguf_check(juno_gguf *g) {
    if (!g) {
        set_error("GGUF handle is null");
        return JUNO_ERR_INVALID_ARG;
    }
    if (g->magic != kMagicGguf) {
        set_error("GGUF handle is closed");
        return JUNO_ERR_CLOSED;
    }
    return JUNO_OK;
}

static void gguf_release(juno_gguf *g) {
    if (g->base) munmap(const_cast<uint8_t *>(g->base), (size_t)g->size);
    if (g->fd >= 0) close(g->fd);
    g->base = nullptr;
    g->fd = -1;
}

static const GgufValue *meta_find(juno_gguf *g, const char *key) {
    auto it = g->meta.find(key);
    return it == g->meta.end() ? nullptr : &it->second;
}
// metaInt / metaLong / metaFloat (GgufReader.java:199-216): any number converts, anything else is the default
static int64_t meta_int(juno_gguf *g, const std::string &key, int64_t dflt) {
    const GgufValue *v = meta_find(g, key.c_str());
    if (!v) return dflt;
    if (v->kind == GgufValue::INT) return v->i;
    if (v->kind == GgufValue::FLOAT) return (int64_t)v->f;
    return dflt;
}
static double meta_float(juno_gguf *g, const std::string &key, double dflt) {
    const GgufValue *v = meta_find(g, key.c_str());
    if (!v) return dflt;
    if (v->kind == GgufValue::INT) return (double)v->i;
    if (v->kind == GgufValue::FLOAT) return v->f;
    return dflt;
}

}  // namespace juno

using namespace juno;

extern "C" {

int juno_gguf_raw_byte_count(int32_t ggml_type, int64_t n_elems, int64_t *bytes) {
    JUNO_REQUIRE(bytes, "bytes is null");
    const int64_t b = raw_byte_count(ggml_type, n_elems);
    if (b < 0) {
        set_error("No byte-size formula for GGML type %d", ggml_type);
        return JUNO_ERR_UNSUPPORTED;
    }
    *bytes = b;
    return JUNO_OK;
}

int juno_gguf_open(const char *path, juno_gguf **out) {
    JUNO_REQUIRE(path && out, "path or out is null");
    *out = nullptr;
    juno_gguf *g = new juno_gguf();
    auto fail = [&](int rc) {
        gguf_release(g);
        g->magic = 0;
        delete g;
        return rc;
    };
    g->fd = open(path, O_RDONLY);
    if (g->fd < 0) {
        set_error("cannot open %s: %s", path, strerror(errno));
        return fail(JUNO_ERR_INVALID_ARG);
    }
    struct stat st;
    if (fstat(g->fd, &st) != 0 || st.st_size < 24) {
        set_error("Not a GGUF file (%s is shorter than a GGUF header)", path);
        return fail(JUNO_ERR_INVALID_ARG);
    }
    g->size = (int64_t)st.st_size;
    void *p = mmap(nullptr, (size_t)g->size, PROT_READ, MAP_PRIVATE, g->fd, 0);
    if (p == MAP_FAILED) {
        set_error("mmap of %s failed: %s", path, strerror(errno));
        return fail(JUNO_ERR_INVALID_ARG);
    }
    g->base = static_cast<const uint8_t *>(p);
    Cursor c{g->base, g->size, 0};
    const uint32_t magic = c.get<uint32_t>();
    g->version = c.get<int32_t>();
    const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
    if (magic != kGgufFileMagic) {
        set_error("Not a GGUF file (magic=0x%x at offset 0)", magic);
        return fail(JUNO_ERR_INVALID_ARG);
    }
    if (g->version < 2 || g->version > 3) {
        set_error("Unsupported GGUF version: %d", g->version);
        return fail(JUNO_ERR_UNSUPPORTED);
    }
    if (n_tensors > (uint64_t)g->size || n_kv > (uint64_t)g->size) {
        set_error("GGUF header counts (%llu tensors, %llu metadata entries) exceed the file", (unsigned long long)n_tensors,
                  (unsigned long long)n_kv);
        return fail(JUNO_ERR_INVALID_ARG);
    }
    for (uint64_t k = 0; k < n_kv; k++) {
        std::string key = c.str();
        const int32_t vtype = c.get<int32_t>();
        GgufValue v;
        if (!c.ok || !read_value(c, vtype, v, 0)) {
            if (c.ok)
                set_error("Unknown metadata type: %d (key %s)", vtype, key.c_str());
            else
                set_error("GGUF metadata runs past the end of the file (entry %llu)", (unsigned long long)k);
            return fail(JUNO_ERR_INVALID_ARG);
        }
        g->meta[key] = std::move(v);  // a repeated key keeps the last value, as HashMap.put does
    }
    g->tensors.reserve((size_t)n_tensors);
    for (uint64_t k = 0; k < n_tensors; k++) {
        GgufTensor t;
        t.name = c.str();
        t.ndims = c.get<int32_t>();
        if (!c.ok || t.ndims < 0 || t.ndims > 4) {
            set_error("GGUF tensor table is damaged at entry %llu", (unsigned long long)k);
            return fail(JUNO_ERR_INVALID_ARG);
        }
        for (int d = 0; d < t.ndims; d++) {
            t.dims[d] = (int64_t)c.get<uint64_t>();
            if (t.dims[d] < 0 || (t.dims[d] && t.nelems > INT64_MAX / t.dims[d])) c.ok = false;
            if (c.ok) t.nelems *= t.dims[d];
        }
        t.type = c.get<int32_t>();
        t.offset = (int64_t)c.get<uint64_t>();
        if (!c.ok || t.offset < 0) {
            set_error("GGUF tensor table is damaged at entry %llu", (unsigned long long)k);
            return fail(JUNO_ERR_INVALID_ARG);
        }
        t.nbytes = raw_byte_count(t.type, t.nelems);  // -1: a type this library has no size for; asking for its bytes fails
        g->by_name[t.name] = g->tensors.size();
        g->tensors.push_back(std::move(t));
    }
    // the data section starts at the next multiple of 32 after the tensor table (GgufReader.java:169-176)
    g->data_offset = (c.pos + kGgufAlignment - 1) / kGgufAlignment * kGgufAlignment;
    for (const GgufTensor &t : g->tensors) {
        if (t.nbytes >= 0 && (t.offset > g->size - g->data_offset || t.nbytes > g->size - g->data_offset - t.offset)) {
            set_error("tensor %s (%lld bytes at data offset %lld) runs past the end of the file", t.name.c_str(), (long long)t.nbytes,
                      (long long)t.offset);
            return fail(JUNO_ERR_INVALID_ARG);
        }
    }
    *out = g;
    return JUNO_OK;
}

int juno_gguf_close(juno_gguf *g) {
    JUNO_TRY(gguf_check(g));
    gguf_release(g);
    g->magic = 0;
    delete g;
    return JUNO_OK;
}

int juno_gguf_info(juno_gguf *g, int32_t *version, int64_t *n_tensors, int64_t *n_meta, int64_t *data_offset) {
    JUNO_TRY(gguf_check(g));
    if (version) *version = g->version;
    if (n_tensors) *n_tensors = (int64_t)g->tensors.size();
    if (n_meta) *n_meta = (int64_t)g->meta.size();
    if (data_offset) *data_offset = g->data_offset;
    return JUNO_OK;
}

int juno_gguf_meta_int(juno_gguf *g, const char *key, int64_t dflt, int64_t *out) {
    JUNO_TRY(gguf_check(g));
    JUNO_REQUIRE(key && out, "key or out is null");
    *out = meta_int(g, key, dflt);
    return JUNO_OK;
}

int juno_gguf_meta_float(juno_gguf *g, const char *key, double dflt, double *out) {
    JUNO_TRY(gguf_check(g));
    JUNO_REQUIRE(key && out, "key or out is null");
    *out = meta_float(g, key, dflt);
    return JUNO_OK;
}

int juno_gguf_meta_string(juno_gguf *g, const char *key, char *buf, int32_t buf_len, int32_t *len) {
    JUNO_TRY(gguf_check(g));
    JUNO_REQUIRE(key && len, "key or len is null");
    const GgufValue *v = meta_find(g, key);
    if (!v || v->kind != GgufValue::STRING) {
        *len = -1;  // metaString returns null for a missing key or another type (GgufReader.java:194-197)
        return JUNO_OK;
    }
    *len = (int32_t)v->s.size();
    if (buf && buf_len > 0) {
        const size_t n = std::min((size_t)buf_len - 1, v->s.size());
        memcpy(buf, v->s.data(), n);
        buf[n] = 0;
    }
    return JUNO_OK;
}

int juno_gguf_meta_array_len(juno_gguf *g, const char *key, int64_t *len) {
    JUNO_TRY(gguf_check(g));
    JUNO_REQUIRE(key && len, "key or len is null");
    const GgufValue *v = meta_find(g, key);
    *len = (v && v->kind == GgufValue::ARRAY) ? v->i : -1;
    return JUNO_OK;
}

int juno_gguf_tensor_name(juno_gguf *g, int64_t index, char *buf, int32_t buf_len) {
    JUNO_TRY(gguf_check(g));
    JUNO_REQUIRE(buf && buf_len > 0, "buf is null or empty");
    JUNO_REQUIRE(index >= 0 && index < (int64_t)g->tensors.size(), "tensor index %lld out of range", (long long)index);
    const std::string &s = g->tensors[(size_t)index].name;
    JUNO_REQUIRE((size_t)buf_len > s.size(), "buffer of %d bytes is too small for a %zu-byte tensor name", buf_len, s.size());
    memcpy(buf, s.c_str(), s.size() + 1);
    return JUNO_OK;
}

int juno_gguf_tensor(juno_gguf *g, const char *name, int32_t *ggml_type, int32_t *n_dims, int64_t *dims4, const void **data,
                     int64_t *n_bytes) {
    JUNO_TRY(gguf_check(g));
    JUNO_REQUIRE(name, "name is null");
    auto it = g->by_name.find(name);
    JUNO_REQUIRE(it != g->by_name.end(), "Tensor not found: %s  (available: %zu tensors)", name, g->tensors.size());
    const GgufTensor &t = g->tensors[it->second];
    if (ggml_type) *ggml_type = t.type;
    if (n_dims) *n_dims = t.ndims;
    if (dims4)
        for (int d = 0; d < 4; d++) dims4[d] = t.dims[d];
    if (data || n_bytes) {
        if (t.nbytes < 0) {
            set_error("No byte-size formula for GGML type %d", t.type);
            return JUNO_ERR_UNSUPPORTED;
        }
        if (data) *data = g->base + g->data_offset + t.offset;
        if (n_bytes) *n_bytes = t.nbytes;
    }
    return JUNO_OK;
}

int juno_gguf_has_tensor(juno_gguf *g, const char *name, int32_t *present) {
    JUNO_TRY(gguf_check(g));
    JUNO_REQUIRE(name && present, "name or present is null");
    *present = g->by_name.count(name) ? 1 : 0;
    return JUNO_OK;
}

// LlamaConfig.from (LlamaConfig.java:58-91): keys under "<general.architecture>." with the "llama." key and then the
// TinyLlama value as defaults; the vocabulary is the larger of <arch>.vocab_size and the tokenizer's token count.
int juno_gguf_model_cfg(juno_gguf *g, juno_model_cfg *cfg) {
    JUNO_TRY(gguf_check(g));
    JUNO_REQUIRE(cfg, "cfg is null");
    std::string arch = "llama";
    if (const GgufValue *v = meta_find(g, "general.architecture"))
        if (v->kind == GgufValue::STRING) arch = v->s;
    const std::string p = arch + ".";
    auto geti = [&](const char *k, int64_t d) { return meta_int(g, p + k, meta_int(g, std::string("llama.") + k, d)); };
    auto getf = [&](const char *k, double d) { return meta_float(g, p + k, meta_float(g, std::string("llama.") + k, d)); };
    const int64_t hidden = geti("embedding_length", 2048);
    const int64_t heads = geti("attention.head_count", 32);
    const GgufValue *toks = meta_find(g, "tokenizer.ggml.tokens");
    const int64_t tok_count = (toks && toks->kind == GgufValue::ARRAY) ? toks->i : 0;
    cfg->hidden = (int32_t)hidden;
    cfg->n_layers = (int32_t)geti("block_count", 22);
    cfg->n_heads = (int32_t)heads;
    cfg->n_kv_heads = (int32_t)geti("attention.head_count_kv", heads);
    cfg->vocab = (int32_t)std::max(geti("vocab_size", 32000), tok_count);
    cfg->inter = (int32_t)geti("feed_forward_length", hidden * 11 / 4);
    cfg->rms_eps = (float)getf("attention.layer_norm_rms_epsilon", 1e-5f);
    cfg->rope_theta = (float)getf("rope.freq_base", 10000.0f);
    return JUNO_OK;
}

}  // extern "C"
