// GGUF model files: header, metadata, tensor directory, alignment, shard and
// byte-range validation over read-only mappings (gguf/reader.go), the model
// hyperparameters of model/qwen35/config.go:48-174, and a loader that uploads
// every tensor of a file into a yuuka_model (engine/gpu/model.go:288-301).
// Host code only; nothing here launches a kernel.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <limits>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "common.cuh"

namespace {

// limits of gguf/reader.go:22-31
constexpr uint32_t MIN_VERSION = 2, MAX_VERSION = 3;
constexpr uint64_t DEFAULT_ALIGN = 32, MAX_METADATA_KEYS = 1ull << 20, MAX_TENSORS = 1ull << 24, MAX_STRING = 1ull << 30;
constexpr uint32_t MAX_RANK = 8;

enum MetaType : uint32_t {
    M_U8 = 0, M_I8 = 1, M_U16 = 2, M_I16 = 3, M_U32 = 4, M_I32 = 5, M_F32 = 6, M_BOOL = 7, M_STR = 8, M_ARR = 9,
    M_U64 = 10, M_I64 = 11, M_F64 = 12
};

// gguf/metadata.go:60-71
struct Value {
    uint32_t type = 0, elem_type = 0;
    bool b = false;
    uint64_t u = 0;
    int64_t i = 0;
    double f = 0;
    std::string s;
    std::vector<Value> arr;
};

bool is_uint(uint32_t t) { return t == M_U8 || t == M_U16 || t == M_U32 || t == M_U64; }
bool is_sint(uint32_t t) { return t == M_I8 || t == M_I16 || t == M_I32 || t == M_I64; }

// Value.AsUint / AsInt (gguf/metadata.go:73-103)
bool as_uint(const Value & v, uint64_t * out) {
    if (is_uint(v.type)) { *out = v.u; return true; }
    if (is_sint(v.type) && v.i >= 0) { *out = (uint64_t)v.i; return true; }
    return false;
}
bool as_int(const Value & v, int64_t * out) {
    if (is_sint(v.type)) { *out = v.i; return true; }
    if (is_uint(v.type) && v.u <= (uint64_t)std::numeric_limits<int64_t>::max()) { *out = (int64_t)v.u; return true; }
    return false;
}

// tensor/dtype.go:101-150: elements and bytes of one storage block; false for an unknown type id
bool block_layout(uint32_t dtype, uint64_t * elements, uint64_t * bytes) {
    static const struct { uint32_t id; uint64_t e, b; } table[] = {
        {0, 1, 4},     {1, 1, 2},     {2, 32, 18},   {3, 32, 20},   {6, 32, 22},   {7, 32, 24},   {8, 32, 34},   {9, 32, 40},
        {10, 256, 84}, {11, 256, 110}, {12, 256, 144}, {13, 256, 176}, {14, 256, 210}, {15, 256, 292}, {16, 256, 66},
        {17, 256, 74}, {18, 256, 98},  {19, 256, 50},  {20, 32, 18},   {21, 256, 110}, {22, 256, 82},  {23, 256, 136},
    };
    for (const auto & t : table)
        if (t.id == dtype) { *elements = t.e; *bytes = t.b; return true; }
    return false;
}

struct Mapping {
    std::string path;
    const uint8_t * data = nullptr;
    size_t size = 0;
    uint64_t data_start = 0;
    ~Mapping() { if (data) munmap(const_cast<uint8_t *>(data), size); }
};

struct TensorInfo {
    std::string name;
    std::vector<uint64_t> dims;
    uint32_t dtype = 0;
    uint64_t offset = 0, absolute = 0, bytes = 0;
    int shard = 0;
};

struct FileMeta {
    uint32_t version = 0;
    uint64_t alignment = DEFAULT_ALIGN;
    std::map<std::string, Value> metadata;
    std::vector<TensorInfo> tensors;
    uint64_t data_start = 0;
};

[[noreturn]] void raise(yuuka_status code, const std::string & msg) {
    yk::fail(code, "%s", msg.c_str());
    throw yk::StatusError{code};
}
// ErrMalformed / ErrUnsupported of gguf/reader.go:33-37
[[noreturn]] void malformed(const std::string & path, const std::string & what) {
    raise(YUUKA_ERR_INVALID_ARGUMENT, "malformed GGUF file: " + path + ": " + what);
}
[[noreturn]] void unsupported(const std::string & path, const std::string & what) {
    raise(YUUKA_ERR_UNSUPPORTED, "unsupported GGUF feature: " + path + ": " + what);
}

// gguf/reader.go:137-215
struct Cursor {
    const std::string & path;
    const uint8_t * data;
    size_t size, off = 0;
    void need(uint64_t n) const {
        if (n > size - off)
            malformed(path, "truncated at byte " + std::to_string(off) + " (need " + std::to_string(n) + ", have " +
                                std::to_string(size - off) + ")");
    }
    template <typename T> T le() {
        need(sizeof(T));
        T v;
        memcpy(&v, data + off, sizeof(T));  // GGUF is little-endian, as is every host this library runs on
        off += sizeof(T);
        return v;
    }
    std::string str() {
        const uint64_t n = le<uint64_t>();
        if (n > MAX_STRING) malformed(path, "string length " + std::to_string(n) + " exceeds limit");
        need(n);
        std::string s(reinterpret_cast<const char *>(data + off), (size_t)n);
        off += (size_t)n;
        return s;
    }
};

Value read_raw(Cursor & c, uint32_t type, int depth);

// gguf/reader.go:395-402
Value read_value(Cursor & c, int depth) { return read_raw(c, c.le<uint32_t>(), depth); }

// gguf/reader.go:404-505
Value read_raw(Cursor & c, uint32_t type, int depth) {
    if (depth > 4) malformed(c.path, "metadata nesting exceeds limit");
    Value v;
    v.type = type;
    switch (type) {
    case M_U8: v.u = c.le<uint8_t>(); break;
    case M_I8: v.i = c.le<int8_t>(); break;
    case M_U16: v.u = c.le<uint16_t>(); break;
    case M_I16: v.i = c.le<int16_t>(); break;
    case M_U32: v.u = c.le<uint32_t>(); break;
    case M_I32: v.i = c.le<int32_t>(); break;
    case M_F32: v.f = (double)c.le<float>(); break;
    case M_BOOL: {
        const uint8_t b = c.le<uint8_t>();
        if (b > 1) malformed(c.path, "invalid bool value " + std::to_string(b));
        v.b = b != 0;
        break;
    }
    case M_STR: v.s = c.str(); break;
    case M_U64: v.u = c.le<uint64_t>(); break;
    case M_I64: v.i = c.le<int64_t>(); break;
    case M_F64: v.f = c.le<double>(); break;
    case M_ARR: {
        v.elem_type = c.le<uint32_t>();
        const uint64_t count = c.le<uint64_t>();
        uint64_t min_size;
        switch (v.elem_type) {
        case M_U8: case M_I8: case M_BOOL: min_size = 1; break;
        case M_U16: case M_I16: min_size = 2; break;
        case M_U32: case M_I32: case M_F32: min_size = 4; break;
        case M_U64: case M_I64: case M_F64: case M_STR: min_size = 8; break;
        case M_ARR: min_size = 16; break;  // a nested array repeats its own type and count
        default: malformed(c.path, "unknown array element type " + std::to_string(v.elem_type));
        }
        if (v.elem_type != M_STR && count > (c.size - c.off) / min_size)
            malformed(c.path, "array length " + std::to_string(count) + " exceeds remaining bytes");
        if (count > (1ull << 31)) malformed(c.path, "array length " + std::to_string(count) + " exceeds limit");
        if (v.elem_type == M_STR && count > (c.size - c.off) / min_size)
            malformed(c.path, "array length " + std::to_string(count) + " exceeds remaining bytes");
        v.arr.reserve((size_t)count);
        for (uint64_t i = 0; i < count; i++) {
            Value item = v.elem_type == M_ARR ? read_value(c, depth + 1) : read_raw(c, v.elem_type, depth + 1);
            if (item.type != v.elem_type) malformed(c.path, "array element " + std::to_string(i) + " has the wrong type");
            v.arr.push_back(std::move(item));
        }
        break;
    }
    default: malformed(c.path, "unknown metadata type " + std::to_string(type));
    }
    return v;
}

uint64_t align_up(uint64_t value, uint64_t alignment) {
    if (alignment <= 1) return value;
    const uint64_t rem = value % alignment;
    if (rem == 0) return value;
    const uint64_t add = alignment - rem;
    if (value > std::numeric_limits<uint64_t>::max() - add) return std::numeric_limits<uint64_t>::max();
    return value + add;
}

// gguf/reader.go:248-393
FileMeta parse_file(const std::string & path, const uint8_t * data, size_t size) {
    Cursor c{path, data, size};
    c.need(4);
    if (memcmp(data, "GGUF", 4) != 0) malformed(path, "bad magic");
    c.off = 4;
    FileMeta m;
    m.version = c.le<uint32_t>();
    if (m.version < MIN_VERSION || m.version > MAX_VERSION)
        unsupported(path, "version " + std::to_string(m.version) + " is not supported (want 2..3)");
    const uint64_t tensor_count = c.le<uint64_t>(), metadata_count = c.le<uint64_t>();
    if (tensor_count > MAX_TENSORS) malformed(path, "tensor count " + std::to_string(tensor_count) + " exceeds limit");
    if (metadata_count > MAX_METADATA_KEYS) malformed(path, "metadata count " + std::to_string(metadata_count) + " exceeds limit");
    for (uint64_t i = 0; i < metadata_count; i++) {
        std::string key = c.str();
        if (key.empty()) malformed(path, "empty metadata key");
        if (m.metadata.count(key)) malformed(path, "duplicate metadata key \"" + key + "\"");
        m.metadata[key] = read_value(c, 0);
    }
    auto al = m.metadata.find("general.alignment");
    if (al != m.metadata.end()) {
        uint64_t a = 0;
        if (!as_uint(al->second, &a)) malformed(path, "general.alignment is not an unsigned integer");
        if (a == 0 || a > (1ull << 20) || (a & (a - 1)) != 0)
            malformed(path, "general.alignment " + std::to_string(a) + " is not a power of two");
        m.alignment = a;
    }
    std::map<std::string, bool> seen;
    m.tensors.reserve((size_t)std::min<uint64_t>(tensor_count, 1 << 16));
    for (uint64_t i = 0; i < tensor_count; i++) {
        TensorInfo t;
        t.name = c.str();
        if (t.name.empty()) malformed(path, "empty tensor name");
        if (seen.count(t.name)) malformed(path, "duplicate tensor name \"" + t.name + "\"");
        seen[t.name] = true;
        const uint32_t rank = c.le<uint32_t>();
        if (rank == 0 || rank > MAX_RANK) malformed(path, "tensor \"" + t.name + "\" has invalid rank " + std::to_string(rank));
        uint64_t elements = 1;
        for (uint32_t d = 0; d < rank; d++) {
            const uint64_t dim = c.le<uint64_t>();
            if (dim == 0) malformed(path, "tensor \"" + t.name + "\" has zero dimension");
            if (elements > std::numeric_limits<uint64_t>::max() / dim) malformed(path, "tensor \"" + t.name + "\" element count overflows");
            elements *= dim;
            t.dims.push_back(dim);
        }
        t.dtype = c.le<uint32_t>();
        t.offset = c.le<uint64_t>();
        uint64_t be = 0, bb = 0;
        if (!block_layout(t.dtype, &be, &bb)) unsupported(path, "tensor \"" + t.name + "\": dtype " + std::to_string(t.dtype));
        if (be > 1 && t.dims[0] % be != 0)
            malformed(path, "tensor \"" + t.name + "\" row width " + std::to_string(t.dims[0]) + " is not a multiple of " + std::to_string(be));
        if (elements / be > std::numeric_limits<uint64_t>::max() / bb) malformed(path, "tensor \"" + t.name + "\" byte size overflows");
        t.bytes = elements / be * bb;
        m.tensors.push_back(std::move(t));
    }
    m.data_start = align_up(c.off, m.alignment);
    if (m.data_start > size) {
        if (tensor_count != 0) malformed(path, "tensor data starts beyond end of file");
        m.data_start = size;
    }
    return m;
}

// gguf/reader.go:217-231
std::unique_ptr<Mapping> map_file(const std::string & path) {
    const int fd = open(path.c_str(), O_RDONLY);
    if (fd < 0) raise(YUUKA_ERR_INVALID_ARGUMENT, "open " + path + ": " + strerror(errno));
    struct stat st;
    if (fstat(fd, &st) != 0) {
        close(fd);
        raise(YUUKA_ERR_INVALID_ARGUMENT, "stat " + path + ": " + strerror(errno));
    }
    if (st.st_size <= 0) {
        close(fd);
        malformed(path, "empty file");
    }
    void * p = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (p == MAP_FAILED) raise(YUUKA_ERR_INTERNAL, "mmap " + path + ": " + strerror(errno));
    auto m = std::make_unique<Mapping>();
    m->path = path;
    m->data = (const uint8_t *)p;
    m->size = (size_t)st.st_size;
    return m;
}

// name-NNNNN-of-NNNNN.gguf (gguf/reader.go:524-545)
std::vector<std::string> split_paths(const std::string & path, uint64_t count) {
    const size_t n = path.size();
    // "-00001-of-00003.gguf" is 20 characters
    bool ok = n > 20 && path.compare(n - 5, 5, ".gguf") == 0 && path[n - 20] == '-' && path.compare(n - 14, 4, "-of-") == 0;
    for (size_t i = 0; ok && i < 5; i++) ok = isdigit((unsigned char)path[n - 19 + i]) && isdigit((unsigned char)path[n - 10 + i]);
    if (!ok) malformed(path, "split model path does not use -NNNNN-of-NNNNN.gguf");
    if (strtoull(path.substr(n - 10, 5).c_str(), nullptr, 10) != count)
        malformed(path, "split count " + std::to_string(count) + " does not match file name");
    const std::string stem = path.substr(0, n - 20);
    std::vector<std::string> out;
    for (uint64_t i = 0; i < count; i++) {
        char buf[32];
        snprintf(buf, sizeof buf, "-%05llu-of-%05llu.gguf", (unsigned long long)(i + 1), (unsigned long long)count);
        out.push_back(stem + buf);
    }
    return out;
}

}  // namespace

struct yuuka_gguf {
    std::string path;
    uint32_t version = 0;
    uint64_t alignment = 0;
    std::map<std::string, Value> metadata;
    std::vector<TensorInfo> order;
    std::map<std::string, size_t> by_name;
    std::vector<std::unique_ptr<Mapping>> shards;
};

namespace {

// gguf/reader.go:547-680
std::unique_ptr<yuuka_gguf> open_gguf(const std::string & path) {
    auto g = std::make_unique<yuuka_gguf>();
    g->path = path;
    auto first = map_file(path);
    FileMeta meta = parse_file(path, first->data, first->size);
    uint64_t shard_count = 1;
    auto sc = meta.metadata.find("split.count");
    if (sc != meta.metadata.end()) {
        if (!as_uint(sc->second, &shard_count)) malformed(path, "split.count is not an unsigned integer");
        if (shard_count == 0 || shard_count > (1ull << 20)) malformed(path, "invalid split.count " + std::to_string(shard_count));
    }
    std::vector<std::string> paths{path};
    if (shard_count > 1) paths = split_paths(path, shard_count);
    g->version = meta.version;
    g->alignment = meta.alignment;
    for (size_t i = 0; i < paths.size(); i++) {
        std::unique_ptr<Mapping> mp;
        FileMeta sm;
        if (i == 0) {
            mp = std::move(first);
            sm = meta;
        } else {
            mp = map_file(paths[i]);
            sm = parse_file(paths[i], mp->data, mp->size);
        }
        if (sm.version != meta.version || sm.alignment != meta.alignment)
            malformed(paths[i], "split shard " + std::to_string(i) + " header differs from shard 0");
        if (shard_count > 1) {
            uint64_t no = 0, cnt = 0;
            auto a = sm.metadata.find("split.no"), b = sm.metadata.find("split.count");
            if (a == sm.metadata.end() || !as_uint(a->second, &no) || no != i)
                malformed(paths[i], "split shard " + std::to_string(i) + " has a missing or wrong split.no");
            if (b == sm.metadata.end() || !as_uint(b->second, &cnt) || cnt != shard_count)
                malformed(paths[i], "split shard " + std::to_string(i) + " has a missing or wrong split.count");
        }
        mp->data_start = sm.data_start;
        for (TensorInfo & t : sm.tensors) {
            if (g->by_name.count(t.name)) malformed(paths[i], "tensor \"" + t.name + "\" appears in more than one shard");
            const uint64_t abs = mp->data_start + t.offset;
            if (abs < mp->data_start) malformed(paths[i], "tensor \"" + t.name + "\" offset overflows");
            if (t.offset % meta.alignment != 0)
                malformed(paths[i], "tensor \"" + t.name + "\" offset " + std::to_string(t.offset) + " is not aligned to " +
                                        std::to_string(meta.alignment));
            const uint64_t end = abs + t.bytes;
            if (end < abs || end > mp->size)
                malformed(paths[i], "tensor \"" + t.name + "\" range [" + std::to_string(abs) + "," + std::to_string(end) +
                                        ") exceeds shard size " + std::to_string(mp->size));
            t.absolute = abs;
            t.shard = (int)i;
            g->by_name[t.name] = g->order.size();
            g->order.push_back(std::move(t));
        }
        g->shards.push_back(std::move(mp));
    }
    g->metadata = std::move(meta.metadata);
    // validateOverlaps (gguf/reader.go:682-704)
    for (size_t s = 0; s < g->shards.size(); s++) {
        std::vector<const TensorInfo *> spans;
        for (const TensorInfo & t : g->order)
            if (t.shard == (int)s) spans.push_back(&t);
        std::sort(spans.begin(), spans.end(), [](const TensorInfo * a, const TensorInfo * b) { return a->absolute < b->absolute; });
        for (size_t k = 1; k < spans.size(); k++)
            if (spans[k]->absolute < spans[k - 1]->absolute + spans[k - 1]->bytes)
                malformed(g->shards[s]->path, "tensors \"" + spans[k - 1]->name + "\" and \"" + spans[k]->name + "\" overlap");
    }
    return g;
}

void fill_tensor(const yuuka_gguf * g, const TensorInfo & t, yuuka_gguf_tensor * out) {
    memset(out, 0, sizeof *out);
    out->name = t.name.c_str();
    out->dtype = t.dtype;
    out->rank = (uint32_t)t.dims.size();
    for (size_t d = 0; d < t.dims.size(); d++) out->dims[d] = t.dims[d];
    out->bytes = t.bytes;
    out->data = g->shards[t.shard]->data + t.absolute;
}

const Value & meta_value(const yuuka_gguf * g, const char * key) {
    YK_REQUIRE(g && key, YUUKA_ERR_INVALID_ARGUMENT, "gguf: null argument");
    auto it = g->metadata.find(key);
    YK_REQUIRE(it != g->metadata.end(), YUUKA_ERR_INVALID_ARGUMENT, "missing required metadata %s", key);
    return it->second;
}

// intKey of model/qwen35/config.go:64-73
int32_t int_key(const yuuka_gguf * g, const std::string & key) {
    int64_t v = 0;
    YK_REQUIRE(as_int(meta_value(g, key.c_str()), &v), YUUKA_ERR_INVALID_ARGUMENT, "metadata %s is not an integer", key.c_str());
    YK_REQUIRE(v > 0 && v <= 0x7fffffffll, YUUKA_ERR_INVALID_ARGUMENT, "metadata %s has invalid value %lld", key.c_str(), (long long)v);
    return (int32_t)v;
}

double float_key(const yuuka_gguf * g, const std::string & key) {
    const Value & v = meta_value(g, key.c_str());
    YK_REQUIRE(v.type == M_F32 || v.type == M_F64, YUUKA_ERR_INVALID_ARGUMENT, "metadata %s is not a float", key.c_str());
    return v.f;
}

// LoadConfig (model/qwen35/config.go:48-174); the remaining range rules are those yuuka_model_create applies
void model_config(const yuuka_gguf * g, yuuka_model_config * cfg) {
    memset(cfg, 0, sizeof *cfg);
    const Value & av = meta_value(g, "general.architecture");
    YK_REQUIRE(av.type == M_STR, YUUKA_ERR_INVALID_ARGUMENT, "general.architecture is not a string");
    const std::string arch = av.s;
    YK_REQUIRE(arch == "qwen35" || arch == "qwen35moe", YUUKA_ERR_UNSUPPORTED,
               "model architecture \"%s\" is not \"qwen35\" or \"qwen35moe\"", arch.c_str());
    auto rs = g->metadata.find(arch + ".rope.scaling.type");
    if (rs != g->metadata.end()) {
        // validateRoPEScaling (config.go:183-194): "", "none" and "default" run unscaled, compared trimmed and lower-cased
        YK_REQUIRE(rs->second.type == M_STR, YUUKA_ERR_INVALID_ARGUMENT, "%s.rope.scaling.type is not a string", arch.c_str());
        std::string text = rs->second.s;
        const size_t b = text.find_first_not_of(" \t\r\n"), e = text.find_last_not_of(" \t\r\n");
        text = b == std::string::npos ? "" : text.substr(b, e - b + 1);
        for (char & ch : text) ch = (char)tolower((unsigned char)ch);
        YK_REQUIRE(text.empty() || text == "none" || text == "default", YUUKA_ERR_UNSUPPORTED,
                   "%s.rope.scaling.type \"%s\" is not supported", arch.c_str(), rs->second.s.c_str());
    }
    auto key = [&](const char * name) { return arch + "." + name; };
    cfg->block_count = int_key(g, key("block_count"));
    cfg->context_length = int_key(g, key("context_length"));
    cfg->hidden = int_key(g, key("embedding_length"));
    if (arch == "qwen35moe") {
        cfg->expert_count = int_key(g, key("expert_count"));
        cfg->expert_used = int_key(g, key("expert_used_count"));
        // scalar, or one width per layer that must not vary (loadExpertFFNSize, config.go:196-231)
        const std::string ek = key("expert_feed_forward_length");
        const Value & ev = meta_value(g, ek.c_str());
        if (ev.type == M_ARR) {
            YK_REQUIRE(!ev.arr.empty(), YUUKA_ERR_INVALID_ARGUMENT, "%s is empty", ek.c_str());
            int64_t w0 = 0;
            for (size_t i = 0; i < ev.arr.size(); i++) {
                int64_t w = 0;
                YK_REQUIRE(as_int(ev.arr[i], &w), YUUKA_ERR_INVALID_ARGUMENT, "%s: element %zu is not an integer", ek.c_str(), i);
                if (i == 0) w0 = w;
                YK_REQUIRE(w == w0, YUUKA_ERR_UNSUPPORTED, "%s varies at layer %zu", ek.c_str(), i);
            }
            YK_REQUIRE(w0 > 0 && w0 <= 0x7fffffffll, YUUKA_ERR_INVALID_ARGUMENT, "metadata %s has invalid value %lld", ek.c_str(), (long long)w0);
            cfg->expert_ffn = (int32_t)w0;
        } else {
            cfg->expert_ffn = int_key(g, ek);
        }
        const std::string sk = key("expert_shared_feed_forward_length");
        cfg->shared_ffn = g->metadata.count(sk) ? int_key(g, sk) : cfg->expert_ffn;
    } else {
        cfg->ffn = int_key(g, key("feed_forward_length"));
    }
    cfg->heads = int_key(g, key("attention.head_count"));
    cfg->kv_heads = int_key(g, key("attention.head_count_kv"));
    cfg->head_dim = int_key(g, key("attention.key_length"));
    const int32_t value_dim = int_key(g, key("attention.value_length"));
    YK_REQUIRE(value_dim == cfg->head_dim, YUUKA_ERR_UNSUPPORTED, "attention value length %d differs from key length %d",
               value_dim, cfg->head_dim);
    cfg->rope_dim = int_key(g, key("rope.dimension_count"));
    cfg->rope_freq_base = float_key(g, key("rope.freq_base"));
    cfg->rms_eps = (float)float_key(g, key("attention.layer_norm_rms_epsilon"));
    cfg->conv_kernel = int_key(g, key("ssm.conv_kernel"));
    cfg->state_size = int_key(g, key("ssm.state_size"));
    cfg->group_count = int_key(g, key("ssm.group_count"));
    cfg->time_step_rank = int_key(g, key("ssm.time_step_rank"));
    cfg->inner_size = int_key(g, key("ssm.inner_size"));
    cfg->full_attention_interval = int_key(g, key("full_attention_interval"));
    auto sec = g->metadata.find(key("rope.dimension_sections"));
    if (sec != g->metadata.end()) {
        const Value & v = sec->second;
        YK_REQUIRE(v.type == M_ARR && v.arr.size() == 4, YUUKA_ERR_INVALID_ARGUMENT, "%s must have 4 entries",
                   key("rope.dimension_sections").c_str());
        int64_t sum = 0;
        for (const Value & e : v.arr) {
            int64_t sv = 0;
            YK_REQUIRE(as_int(e, &sv) && sv >= 0 && sv <= (1 << 20), YUUKA_ERR_INVALID_ARGUMENT, "invalid rope section");
            sum += sv;
        }
        // config.go:243: the sections cover the rotated dimensions pairwise
        YK_REQUIRE(sum == 0 || sum * 2 == cfg->rope_dim, YUUKA_ERR_INVALID_ARGUMENT,
                   "rope sections sum to %lld, want %d", (long long)sum, cfg->rope_dim / 2);
    }
    auto tok = g->metadata.find("tokenizer.ggml.tokens");
    if (tok != g->metadata.end()) {
        YK_REQUIRE(tok->second.type == M_ARR && tok->second.elem_type == M_STR, YUUKA_ERR_INVALID_ARGUMENT,
                   "tokenizer.ggml.tokens is not an array of strings");
        YK_REQUIRE(!tok->second.arr.empty() && tok->second.arr.size() <= 0x7fffffffull, YUUKA_ERR_INVALID_ARGUMENT,
                   "tokenizer.ggml.tokens has an invalid length");
        cfg->vocab = (int32_t)tok->second.arr.size();
    } else {
        YK_REQUIRE(g->metadata.count(key("vocab_size")), YUUKA_ERR_INVALID_ARGUMENT, "vocabulary size is unavailable");
        cfg->vocab = int_key(g, key("vocab_size"));
    }
}

}  // namespace

extern "C" {

yuuka_status yuuka_gguf_open(const char * path, yuuka_gguf ** out) {
    return yk::guard([&] {
        YK_REQUIRE(path && out, YUUKA_ERR_INVALID_ARGUMENT, "gguf_open: null argument");
        *out = nullptr;
        *out = open_gguf(path).release();
    });
}

void yuuka_gguf_close(yuuka_gguf * g) { delete g; }

uint32_t yuuka_gguf_version(const yuuka_gguf * g) { return g ? g->version : 0; }
uint64_t yuuka_gguf_alignment(const yuuka_gguf * g) { return g ? g->alignment : 0; }
uint64_t yuuka_gguf_tensor_count(const yuuka_gguf * g) { return g ? g->order.size() : 0; }
uint64_t yuuka_gguf_metadata_count(const yuuka_gguf * g) { return g ? g->metadata.size() : 0; }

yuuka_status yuuka_gguf_tensor_at(const yuuka_gguf * g, uint64_t index, yuuka_gguf_tensor * out) {
    return yk::guard([&] {
        YK_REQUIRE(g && out, YUUKA_ERR_INVALID_ARGUMENT, "gguf_tensor_at: null argument");
        YK_REQUIRE(index < g->order.size(), YUUKA_ERR_INVALID_ARGUMENT, "gguf_tensor_at: index %llu of %zu",
                   (unsigned long long)index, g->order.size());
        fill_tensor(g, g->order[(size_t)index], out);
    });
}

yuuka_status yuuka_gguf_tensor_find(const yuuka_gguf * g, const char * name, yuuka_gguf_tensor * out) {
    return yk::guard([&] {
        YK_REQUIRE(g && name && out, YUUKA_ERR_INVALID_ARGUMENT, "gguf_tensor_find: null argument");
        auto it = g->by_name.find(name);
        YK_REQUIRE(it != g->by_name.end(), YUUKA_ERR_INVALID_ARGUMENT, "tensor \"%s\" is not in the file", name);
        fill_tensor(g, g->order[it->second], out);
    });
}

yuuka_status yuuka_gguf_meta_int(const yuuka_gguf * g, const char * key, int64_t * out) {
    return yk::guard([&] {
        YK_REQUIRE(out, YUUKA_ERR_INVALID_ARGUMENT, "gguf_meta_int: null argument");
        YK_REQUIRE(as_int(meta_value(g, key), out), YUUKA_ERR_INVALID_ARGUMENT, "metadata %s is not an integer that fits int64", key);
    });
}

yuuka_status yuuka_gguf_meta_float(const yuuka_gguf * g, const char * key, double * out) {
    return yk::guard([&] {
        YK_REQUIRE(out, YUUKA_ERR_INVALID_ARGUMENT, "gguf_meta_float: null argument");
        const Value & v = meta_value(g, key);
        YK_REQUIRE(v.type == M_F32 || v.type == M_F64, YUUKA_ERR_INVALID_ARGUMENT, "metadata %s is not a float", key);
        *out = v.f;
    });
}

yuuka_status yuuka_gguf_meta_string(const yuuka_gguf * g, const char * key, const char ** out, uint64_t * len) {
    return yk::guard([&] {
        YK_REQUIRE(out && len, YUUKA_ERR_INVALID_ARGUMENT, "gguf_meta_string: null argument");
        const Value & v = meta_value(g, key);
        YK_REQUIRE(v.type == M_STR, YUUKA_ERR_INVALID_ARGUMENT, "metadata %s is not a string", key);
        *out = v.s.data();
        *len = v.s.size();
    });
}

yuuka_status yuuka_gguf_meta_array_len(const yuuka_gguf * g, const char * key, uint64_t * out) {
    return yk::guard([&] {
        YK_REQUIRE(out, YUUKA_ERR_INVALID_ARGUMENT, "gguf_meta_array_len: null argument");
        const Value & v = meta_value(g, key);
        YK_REQUIRE(v.type == M_ARR, YUUKA_ERR_INVALID_ARGUMENT, "metadata %s is not an array", key);
        *out = v.arr.size();
    });
}

yuuka_status yuuka_gguf_model_config(const yuuka_gguf * g, yuuka_model_config * out) {
    return yk::guard([&] {
        YK_REQUIRE(g && out, YUUKA_ERR_INVALID_ARGUMENT, "gguf_model_config: null argument");
        model_config(g, out);
    });
}

yuuka_status yuuka_model_load_gguf(yuuka_device * dev, const char * path, yuuka_model ** out) {
    return yk::guard([&] {
        YK_REQUIRE(dev && path && out, YUUKA_ERR_INVALID_ARGUMENT, "model_load_gguf: null argument");
        *out = nullptr;
        std::unique_ptr<yuuka_gguf> g = open_gguf(path);
        yuuka_model_config cfg;
        model_config(g.get(), &cfg);
        yuuka_model * m = nullptr;
        // (the callee has already recorded the message of a failure)
        yuuka_status st = yuuka_model_create(dev, &cfg, &m);
        if (st != YUUKA_OK) throw yk::StatusError{st};
        for (const TensorInfo & t : g->order) {
            uint64_t rows = 1;
            for (size_t d = 1; d < t.dims.size(); d++) rows *= t.dims[d];
            st = yuuka_model_set_tensor(m, t.name.c_str(), t.dtype, g->shards[t.shard]->data + t.absolute, rows, t.dims[0]);
            if (st != YUUKA_OK) {
                const std::string msg = yuuka_last_error();
                yuuka_model_destroy(m);
                raise(st, msg);
            }
        }
        st = yuuka_model_finalize(m);
        if (st != YUUKA_OK) {
            const std::string msg = yuuka_last_error();
            yuuka_model_destroy(m);
            raise(st, msg);
        }
        *out = m;
    });
}

}  // extern "C"
