// GGUF container reader: real model files straight into zq_weight_prepare / zq_moe_experts_create.
//
// Host code only.  What it keeps of the reference's reader (src/weight/container/gguf.rs):
//   open / parse_shard (:364-412, :663-725)   GGUF v3: magic, version, tensor and metadata counts, metadata pairs, tensor
//                                             directory (name, 1..4 dimensions, type, offset); data starts at the next
//                                             multiple of general.alignment (default 32, a power of two); every tensor
//                                             must end inside the file; duplicate names are errors
//   split files (:727-750)                    <prefix>-00001-of-0000N.gguf: the N shards are opened together, split.count
//                                             and split.no are checked, tensor names must be unique across shards
//   storage_bytes (:154-160) + block_layout   bytes of a tensor from its element count and the type's block
//     (src/weight/codec/ggml.rs:33-71)
//   read_matrix (:506-514)                    2-D tensor, GGUF dimension order [columns, rows]
//   read_matrix_slice (:516-534)              matrix `index` of a [columns, rows, count] tensor: expert slicing
//   embedding_rows (:618-629)                 = zq_gather_rows on a loaded matrix (the rows are dequantised on the device)
// Metadata: scalars and strings are kept; arrays are skipped over (their length is kept).
#include <algorithm>
#include <cerrno>
#include <new>
#include <cstdio>
#include <map>
#include <memory>

#include "zq_common.cuh"

namespace {

struct TensorInfo {
    std::string name;
    std::vector<uint64_t> dims;
    uint32_t type = 0;
    uint64_t offset = 0, bytes = 0;
    size_t shard = 0;
};

struct MetaValue {
    int kind = 0;  // 0 unsigned, 1 signed, 2 float, 3 bool, 4 string, 5 array (u = length)
    uint64_t u = 0;
    int64_t i = 0;
    double f = 0;
    std::string s;
};

struct Shard {
    std::string path;
    FILE *file = nullptr;
    uint64_t file_len = 0, data_offset = 0;
    std::map<std::string, MetaValue> metadata;
    std::vector<TensorInfo> tensors;
};

// (elements per block, bytes per block) of every GGML tensor type the reference sizes (src/weight/codec/ggml.rs:33-71)
bool block_layout(uint32_t t, uint64_t *elements, uint64_t *bytes) {
    static const struct { uint32_t t; uint32_t e, b; } table[] = {
        {0, 1, 4}, {1, 1, 2}, {2, 32, 18}, {3, 32, 20}, {6, 32, 22}, {7, 32, 24}, {8, 32, 34}, {9, 32, 36}, {10, 256, 84}, {11, 256, 110}, {12, 256, 144}, {13, 256, 176}, {14, 256, 210},
        {15, 256, 292}, {16, 256, 66}, {17, 256, 74}, {18, 256, 98}, {19, 256, 50}, {20, 32, 18}, {21, 256, 110}, {22, 256, 82}, {23, 256, 136}, {24, 1, 1}, {25, 1, 2}, {26, 1, 4},
        {27, 1, 8}, {28, 1, 8}, {29, 256, 56}, {30, 1, 2}, {34, 256, 54}, {35, 256, 66}, {39, 32, 17}, {40, 64, 36}, {41, 128, 18}, {42, 64, 18}};
    for (const auto &row : table)
        if (row.t == t) {
            *elements = row.e;
            *bytes = row.b;
            return true;
        }
    return false;
}

struct Reader {
    FILE *f;
    std::string error;
    bool ok = true;
    bool read(void *dst, size_t n) {
        if (!ok) return false;
        if (fread(dst, 1, n, f) != n) {
            ok = false;
            error = "unexpected end of file in the GGUF header";
        }
        return ok;
    }
    template <class T> T get() {
        T v{};
        read(&v, sizeof(T));
        return v;
    }
    std::string str() {
        const uint64_t len = get<uint64_t>();
        if (!ok) return {};
        if (len > (uint64_t(1) << 24)) {  // the reference rejects absurd lengths as a damaged file
            ok = false;
            error = "GGUF string length " + std::to_string(len) + " is beyond any sane limit: damaged file?";
            return {};
        }
        std::string s(len, '\0');
        read(&s[0], len);
        return s;
    }
};

bool read_value(Reader &r, uint32_t type, MetaValue &out, int depth = 0) {
    switch (type) {
    case 0: out.kind = 0; out.u = r.get<uint8_t>(); break;
    case 1: out.kind = 1; out.i = r.get<int8_t>(); break;
    case 2: out.kind = 0; out.u = r.get<uint16_t>(); break;
    case 3: out.kind = 1; out.i = r.get<int16_t>(); break;
    case 4: out.kind = 0; out.u = r.get<uint32_t>(); break;
    case 5: out.kind = 1; out.i = r.get<int32_t>(); break;
    case 6: out.kind = 2; out.f = r.get<float>(); break;
    case 7: out.kind = 3; out.u = r.get<uint8_t>() != 0; break;
    case 8: out.kind = 4; out.s = r.str(); break;
    case 10: out.kind = 0; out.u = r.get<uint64_t>(); break;
    case 11: out.kind = 1; out.i = r.get<int64_t>(); break;
    case 12: out.kind = 2; out.f = r.get<double>(); break;
    case 9: {
        if (depth) {
            r.ok = false;
            r.error = "GGUF does not allow nested arrays";
            return false;
        }
        const uint32_t et = r.get<uint32_t>();
        const uint64_t len = r.get<uint64_t>();
        if (!r.ok) return false;
        if (et == 9 || len > (uint64_t(1) << 28)) {
            r.ok = false;
            r.error = "GGUF metadata array is nested or absurdly long";
            return false;
        }
        MetaValue skip;
        for (uint64_t k = 0; k < len && r.ok; ++k) read_value(r, et, skip, 1);
        out.kind = 5;
        out.u = len;
        break;
    }
    default:
        r.ok = false;
        r.error = "unknown GGUF metadata value type " + std::to_string(type);
    }
    return r.ok;
}

int parse_shard(const std::string &path, Shard &sh, zq_error *err) {
    sh.path = path;
    sh.file = fopen(path.c_str(), "rb");
    if (!sh.file) return zq::set_error(err, ZQ_ERR_ARG, "cannot open GGUF file %s: %s", path.c_str(), strerror(errno));
    fseeko(sh.file, 0, SEEK_END);
    sh.file_len = (uint64_t)ftello(sh.file);
    fseeko(sh.file, 0, SEEK_SET);
    Reader r{sh.file};
    char magic[4] = {};
    r.read(magic, 4);
    if (!r.ok || memcmp(magic, "GGUF", 4)) return zq::set_error(err, ZQ_ERR_SHAPE, "%s is not a GGUF file", path.c_str());
    const uint32_t version = r.get<uint32_t>();
    if (r.ok && version != 3) return zq::set_error(err, ZQ_ERR_UNSUPPORTED, "only GGUF v3 is supported, the file is v%u", version);
    const uint64_t tensor_count = r.get<uint64_t>(), metadata_count = r.get<uint64_t>();
    if (r.ok && (tensor_count > (uint64_t(1) << 24) || metadata_count > (uint64_t(1) << 24))) return zq::set_error(err, ZQ_ERR_SHAPE, "GGUF header counts are absurd: damaged file?");
    for (uint64_t k = 0; k < metadata_count && r.ok; ++k) {
        const std::string key = r.str();
        const uint32_t vt = r.get<uint32_t>();
        MetaValue v;
        if (!read_value(r, vt, v)) break;
        if (!sh.metadata.emplace(key, v).second) return zq::set_error(err, ZQ_ERR_SHAPE, "duplicate GGUF metadata key %s", key.c_str());
    }
    for (uint64_t k = 0; k < tensor_count && r.ok; ++k) {
        TensorInfo t;
        t.name = r.str();
        const uint32_t nd = r.get<uint32_t>();
        if (!r.ok) break;
        if (nd == 0 || nd > 4) return zq::set_error(err, ZQ_ERR_SHAPE, "GGUF tensor %s has %u dimensions", t.name.c_str(), nd);
        uint64_t elements = 1;
        for (uint32_t d = 0; d < nd; ++d) {
            const uint64_t v = r.get<uint64_t>();
            if (v != 0 && elements > UINT64_MAX / v) return zq::set_error(err, ZQ_ERR_SHAPE, "GGUF tensor %s: element count overflows", t.name.c_str());
            elements *= v;
            t.dims.push_back(v);
        }
        t.type = r.get<uint32_t>();
        t.offset = r.get<uint64_t>();
        if (!r.ok) break;
        uint64_t be = 0, bb = 0;
        if (!block_layout(t.type, &be, &bb)) return zq::set_error(err, ZQ_ERR_UNSUPPORTED, "GGUF tensor %s has unknown GGML type %u", t.name.c_str(), t.type);
        if (elements % be) return zq::set_error(err, ZQ_ERR_SHAPE, "GGUF tensor %s: %llu elements are not whole blocks of %llu", t.name.c_str(), (unsigned long long)elements, (unsigned long long)be);
        t.bytes = elements / be * bb;
        for (const TensorInfo &o : sh.tensors)
            if (o.name == t.name) return zq::set_error(err, ZQ_ERR_SHAPE, "duplicate GGUF tensor %s", t.name.c_str());
        sh.tensors.push_back(t);
    }
    if (!r.ok) return zq::set_error(err, ZQ_ERR_SHAPE, "%s: %s", path.c_str(), r.error.c_str());
    uint64_t alignment = 32;
    auto al = sh.metadata.find("general.alignment");
    if (al != sh.metadata.end() && (al->second.kind == 0 || al->second.kind == 1)) alignment = al->second.kind == 0 ? al->second.u : (uint64_t)al->second.i;
    if (alignment == 0 || (alignment & (alignment - 1))) return zq::set_error(err, ZQ_ERR_SHAPE, "GGUF alignment %llu is not a power of two", (unsigned long long)alignment);
    const uint64_t directory_end = (uint64_t)ftello(sh.file);
    sh.data_offset = (directory_end + alignment - 1) / alignment * alignment;
    for (const TensorInfo &t : sh.tensors) {
        if (t.offset > sh.file_len || sh.data_offset + t.offset + t.bytes > sh.file_len || sh.data_offset + t.offset + t.bytes < t.bytes)
            return zq::set_error(err, ZQ_ERR_SHAPE, "GGUF tensor %s ends beyond the file (offset %llu + %llu bytes, file %llu)", t.name.c_str(), (unsigned long long)(sh.data_offset + t.offset), (unsigned long long)t.bytes,
                                 (unsigned long long)sh.file_len);
    }
    return ZQ_OK;
}

// "<prefix>-<index>-of-<count>.gguf" with index >= 1 and count > 1 (src/weight/container/gguf.rs:727-735)
bool split_name(const std::string &path, std::string *prefix, size_t *index, size_t *count) {
    const size_t slash = path.find_last_of('/');
    const std::string name = slash == std::string::npos ? path : path.substr(slash + 1);
    if (name.size() < 5 || name.compare(name.size() - 5, 5, ".gguf")) return false;
    const std::string stem = name.substr(0, name.size() - 5);
    const size_t of = stem.rfind("-of-");
    if (of == std::string::npos) return false;
    const std::string left = stem.substr(0, of), cnt = stem.substr(of + 4);
    const size_t dash = left.rfind('-');
    if (dash == std::string::npos) return false;
    const std::string idx = left.substr(dash + 1);
    if (idx.empty() || cnt.empty() || idx.find_first_not_of("0123456789") != std::string::npos || cnt.find_first_not_of("0123456789") != std::string::npos) return false;
    *index = (size_t)strtoull(idx.c_str(), nullptr, 10);
    *count = (size_t)strtoull(cnt.c_str(), nullptr, 10);
    if (*index == 0 || *count <= 1 || *index > *count) return false;
    *prefix = (slash == std::string::npos ? std::string() : path.substr(0, slash + 1)) + left.substr(0, dash);
    return true;
}

}  // namespace

struct zq_gguf {
    std::vector<Shard> shards;
    std::vector<TensorInfo> tensors;
    std::map<std::string, size_t> index;
    ~zq_gguf() {
        for (Shard &s : shards)
            if (s.file) fclose(s.file);
    }
    const TensorInfo *find(const char *name) const {
        auto it = index.find(name);
        return it == index.end() ? nullptr : &tensors[it->second];
    }
};

using namespace zq;

// Reads `bytes` bytes of a tensor starting at `offset` and prepares them as a [rows, columns] weight.
static int load_range(zq_ctx *ctx, const zq_gguf *g, const TensorInfo &t, uint64_t offset, uint64_t bytes, uint64_t rows, uint64_t columns, zq_weight **out, zq_error *err) {
    if (offset + bytes > t.bytes) return set_error(err, ZQ_ERR_SHAPE, "GGUF tensor %s: range %llu..%llu is beyond its %llu bytes", t.name.c_str(), (unsigned long long)offset, (unsigned long long)(offset + bytes), (unsigned long long)t.bytes);
    const Shard &sh = g->shards[t.shard];
    std::unique_ptr<uint8_t[]> host(new (std::nothrow) uint8_t[bytes ? bytes : 1]);
    if (!host) return set_error(err, ZQ_ERR_ARG, "GGUF tensor %s: cannot allocate %llu host bytes", t.name.c_str(), (unsigned long long)bytes);
    if (fseeko(sh.file, (off_t)(sh.data_offset + t.offset + offset), SEEK_SET) != 0 || fread(host.get(), 1, bytes, sh.file) != bytes)
        return set_error(err, ZQ_ERR_ARG, "GGUF tensor %s: reading %llu bytes from %s failed", t.name.c_str(), (unsigned long long)bytes, sh.path.c_str());
    return zq_weight_prepare(ctx, t.type, host.get(), bytes, rows, columns, out, err);
}

extern "C" {

int zq_gguf_open(const char *path, zq_gguf **out, zq_error *err) {
    if (!path || !out) return set_error(err, ZQ_ERR_ARG, "zq_gguf_open: null argument");
    std::vector<std::string> paths;
    std::string prefix;
    size_t index = 0, count = 0;
    if (split_name(path, &prefix, &index, &count)) {
        const int width = (int)std::max<size_t>(5, std::to_string(count).size());
        for (size_t k = 1; k <= count; ++k) {
            char buf[64];
            snprintf(buf, sizeof(buf), "-%0*zu-of-%0*zu.gguf", width, k, width, count);
            paths.push_back(prefix + buf);
        }
    } else {
        paths.push_back(path);
    }
    std::unique_ptr<zq_gguf> g(new zq_gguf());
    g->shards.resize(paths.size());
    for (size_t k = 0; k < paths.size(); ++k) {
        int rc = parse_shard(paths[k], g->shards[k], err);
        if (rc) return rc;
    }
    const auto &meta = g->shards[0].metadata;
    uint64_t expected_shards = 1;
    auto sc = meta.find("split.count");
    if (sc != meta.end() && sc->second.kind == 0) expected_shards = sc->second.u;
    if (expected_shards != paths.size()) return set_error(err, ZQ_ERR_SHAPE, "GGUF split.count is %llu, %zu shard(s) were opened", (unsigned long long)expected_shards, paths.size());
    for (size_t k = 0; k < g->shards.size(); ++k) {
        auto no = g->shards[k].metadata.find("split.no");
        if (no != g->shards[k].metadata.end() && no->second.kind == 0 && no->second.u != k) return set_error(err, ZQ_ERR_SHAPE, "GGUF shard %zu says split.no = %llu", k + 1, (unsigned long long)no->second.u);
        for (TensorInfo &t : g->shards[k].tensors) {
            t.shard = k;
            if (!g->index.emplace(t.name, g->tensors.size()).second) return set_error(err, ZQ_ERR_SHAPE, "GGUF tensor %s appears in two shards", t.name.c_str());
            g->tensors.push_back(t);
        }
    }
    auto tc = meta.find("split.tensors.count");
    if (tc != meta.end() && tc->second.kind == 0 && tc->second.u != g->tensors.size()) return set_error(err, ZQ_ERR_SHAPE, "GGUF split.tensors.count is %llu, %zu tensors were found", (unsigned long long)tc->second.u, g->tensors.size());
    *out = g.release();
    return ZQ_OK;
}

void zq_gguf_close(zq_gguf *g) { delete g; }

size_t zq_gguf_tensor_count(const zq_gguf *g) { return g ? g->tensors.size() : 0; }

int zq_gguf_tensor_name(const zq_gguf *g, size_t index, char *out, size_t capacity, zq_error *err) {
    if (!g || !out || capacity == 0) return set_error(err, ZQ_ERR_ARG, "zq_gguf_tensor_name: null argument");
    if (index >= g->tensors.size()) return set_error(err, ZQ_ERR_ARG, "zq_gguf_tensor_name: index %zu of %zu", index, g->tensors.size());
    snprintf(out, capacity, "%s", g->tensors[index].name.c_str());
    return ZQ_OK;
}

int zq_gguf_tensor_info(const zq_gguf *g, const char *name, uint32_t *type, uint32_t *n_dims, uint64_t *dims4, uint64_t *nbytes, zq_error *err) {
    if (!g || !name) return set_error(err, ZQ_ERR_ARG, "zq_gguf_tensor_info: null argument");
    const TensorInfo *t = g->find(name);
    if (!t) return set_error(err, ZQ_ERR_ARG, "the GGUF file has no tensor %s", name);
    if (type) *type = t->type;
    if (n_dims) *n_dims = (uint32_t)t->dims.size();
    if (dims4)
        for (size_t d = 0; d < 4; ++d) dims4[d] = d < t->dims.size() ? t->dims[d] : 1;
    if (nbytes) *nbytes = t->bytes;
    return ZQ_OK;
}

int zq_gguf_metadata_u64(const zq_gguf *g, const char *key, uint64_t *out, zq_error *err) {
    if (!g || !key || !out) return set_error(err, ZQ_ERR_ARG, "zq_gguf_metadata_u64: null argument");
    auto it = g->shards[0].metadata.find(key);
    if (it == g->shards[0].metadata.end() || !(it->second.kind == 0 || it->second.kind == 3 || (it->second.kind == 1 && it->second.i >= 0) || it->second.kind == 5))
        return set_error(err, ZQ_ERR_ARG, "GGUF metadata %s is missing or not an unsigned value", key);
    *out = it->second.kind == 1 ? (uint64_t)it->second.i : it->second.u;  // for an array: its length
    return ZQ_OK;
}

int zq_gguf_metadata_f64(const zq_gguf *g, const char *key, double *out, zq_error *err) {
    if (!g || !key || !out) return set_error(err, ZQ_ERR_ARG, "zq_gguf_metadata_f64: null argument");
    auto it = g->shards[0].metadata.find(key);
    if (it == g->shards[0].metadata.end() || it->second.kind > 2) return set_error(err, ZQ_ERR_ARG, "GGUF metadata %s is missing or not a number", key);
    *out = it->second.kind == 2 ? it->second.f : (it->second.kind == 1 ? (double)it->second.i : (double)it->second.u);
    return ZQ_OK;
}

int zq_gguf_metadata_str(const zq_gguf *g, const char *key, char *out, size_t capacity, zq_error *err) {
    if (!g || !key || !out || capacity == 0) return set_error(err, ZQ_ERR_ARG, "zq_gguf_metadata_str: null argument");
    auto it = g->shards[0].metadata.find(key);
    if (it == g->shards[0].metadata.end() || it->second.kind != 4) return set_error(err, ZQ_ERR_ARG, "GGUF metadata %s is missing or not a string", key);
    snprintf(out, capacity, "%s", it->second.s.c_str());
    return ZQ_OK;
}

int zq_gguf_load_matrix(zq_ctx *ctx, const zq_gguf *g, const char *name, zq_weight **out, zq_error *err) {
    if (!ctx || !g || !name || !out) return set_error(err, ZQ_ERR_ARG, "zq_gguf_load_matrix: null argument");
    const TensorInfo *t = g->find(name);
    if (!t) return set_error(err, ZQ_ERR_ARG, "the GGUF file has no tensor %s", name);
    if (t->dims.size() != 2) return set_error(err, ZQ_ERR_SHAPE, "GGUF tensor %s has %zu dimensions: not a matrix", name, t->dims.size());
    return load_range(ctx, g, *t, 0, t->bytes, t->dims[1], t->dims[0], out, err);
}

int zq_gguf_load_matrix_slice(zq_ctx *ctx, const zq_gguf *g, const char *name, size_t index, zq_weight **out, zq_error *err) {
    if (!ctx || !g || !name || !out) return set_error(err, ZQ_ERR_ARG, "zq_gguf_load_matrix_slice: null argument");
    const TensorInfo *t = g->find(name);
    if (!t) return set_error(err, ZQ_ERR_ARG, "the GGUF file has no tensor %s", name);
    if (t->dims.size() != 3) return set_error(err, ZQ_ERR_SHAPE, "GGUF tensor %s has %zu dimensions: not an array of matrices", name, t->dims.size());
    const uint64_t columns = t->dims[0], rows = t->dims[1], count = t->dims[2];
    if (index >= count) return set_error(err, ZQ_ERR_ARG, "GGUF tensor %s: matrix %zu of %llu", name, index, (unsigned long long)count);
    uint64_t be = 0, bb = 0;
    block_layout(t->type, &be, &bb);
    if ((rows * columns) % be || (rows * columns / be * bb) * count != t->bytes) return set_error(err, ZQ_ERR_SHAPE, "GGUF tensor %s: its matrices are not separately block-aligned", name);
    const uint64_t slice = rows * columns / be * bb;
    return load_range(ctx, g, *t, index * slice, slice, rows, columns, out, err);
}

}  // extern "C"
