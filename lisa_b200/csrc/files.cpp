// Host-side weight-file readers behind include/lisa_files.h: the GGUF v3 container and the safetensors shard.
// Replaces, for the path's two weight-loading doors, crates/lisa-gguf/src/{lib,header,package}.rs,
// crates/lisa-engine/src/core/gguf_resident.rs:62-115 (view shaping), crates/lisa-engine/src/core/loader.rs:57-160
// and crates/lisa-engine/src/core/quant.rs:273-287,408-432.  Plain C++17 over POSIX files; no CUDA.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <vector>

#include "common.cuh"
#include "lisa_files.h"

namespace lisa {
namespace {

// ------------------------------------------------------------------------------------------ GGUF geometry
struct TypeLayout {
    uint32_t id;
    const char *name;
    uint64_t block, bytes;
};
// GGML's block ABI (crates/lisa-gguf/src/lib.rs:36-70).
const TypeLayout kTypes[] = {
    {0, "F32", 1, 4},      {1, "F16", 1, 2},       {2, "Q4_0", 32, 18},     {3, "Q4_1", 32, 20},    {6, "Q5_0", 32, 22},
    {7, "Q5_1", 32, 24},   {8, "Q8_0", 32, 34},    {9, "Q8_1", 32, 36},     {10, "Q2_K", 256, 84},  {11, "Q3_K", 256, 110},
    {12, "Q4_K", 256, 144}, {13, "Q5_K", 256, 176}, {14, "Q6_K", 256, 210}, {15, "Q8_K", 256, 292}, {16, "IQ2_XXS", 256, 66},
    {17, "IQ2_XS", 256, 74}, {18, "IQ3_XXS", 256, 98}, {19, "IQ1_S", 256, 50}, {20, "IQ4_NL", 32, 18}, {21, "IQ3_S", 256, 110},
    {22, "IQ2_S", 256, 82}, {23, "IQ4_XS", 256, 136}, {24, "I8", 1, 1},      {25, "I16", 1, 2},      {26, "I32", 1, 4},
    {27, "I64", 1, 8},     {28, "F64", 1, 8},      {29, "IQ1_M", 256, 56},  {30, "BF16", 1, 2},     {39, "MXFP4", 32, 17},
};

const TypeLayout *find_type(uint32_t id) {
    for (const TypeLayout &t : kTypes)
        if (t.id == id) return &t;
    return nullptr;
}

int type_row_bytes(uint32_t type, uint64_t columns, uint64_t *out) {
    const TypeLayout *t = find_type(type);
    if (!t) return fail(LISA_ERR_UNSUPPORTED, "unsupported GGUF tensor type " + std::to_string(type));
    if (columns == 0 || columns % t->block != 0)
        return fail(LISA_ERR_BAD_ARG, std::string(t->name) + " row width " + std::to_string(columns) +
                                          " is not a positive multiple of " + std::to_string(t->block));
    const uint64_t blocks = columns / t->block;
    if (blocks > UINT64_MAX / t->bytes) return fail(LISA_ERR_OVERFLOW, "GGUF row byte size overflow");
    *out = blocks * t->bytes;
    return LISA_OK;
}

// ------------------------------------------------------------------------------------------ GGUF values
struct Value {
    int kind = 0;  // 0 unsigned, 1 signed, 2 float, 3 bool, 4 string, 5 array
    uint64_t u = 0;
    int64_t i = 0;
    double f = 0;
    bool b = false;
    std::string s;
    std::vector<Value> a;

    bool as_u64(uint64_t *out) const {
        if (kind == 0) { *out = u; return true; }
        if (kind == 1 && i >= 0) { *out = static_cast<uint64_t>(i); return true; }
        return false;
    }
    bool as_f64(double *out) const {
        if (kind == 2) { *out = f; return true; }
        if (kind == 0) { *out = static_cast<double>(u); return true; }
        if (kind == 1) { *out = static_cast<double>(i); return true; }
        return false;
    }
    bool equals(const Value &o) const {
        if (kind != o.kind) return false;
        switch (kind) {
            case 0: return u == o.u;
            case 1: return i == o.i;
            case 2: return f == o.f;
            case 3: return b == o.b;
            case 4: return s == o.s;
            default:
                if (a.size() != o.a.size()) return false;
                for (size_t n = 0; n < a.size(); ++n)
                    if (!a[n].equals(o.a[n])) return false;
                return true;
        }
    }
};

struct TensorRec {
    std::string name;
    std::vector<uint64_t> dims;
    uint32_t type = 0;
    uint64_t offset = 0, bytes = 0, row_bytes = 0;
    int shard = 0;
};

struct Header {
    std::map<std::string, Value> metadata;
    std::map<std::string, TensorRec> tensors;
    uint64_t data_offset = 0, file_bytes = 0;
};

constexpr uint64_t kMaxHeaderBytes = 256ull << 20;
constexpr uint64_t kMaxEntries = 1000000;
constexpr size_t kMaxValues = 4000000;

// What String::from_utf8 accepts: well-formed sequences of one to four bytes.
bool valid_utf8(const std::string &s) {
    const unsigned char *p = reinterpret_cast<const unsigned char *>(s.data());
    const size_t n = s.size();
    size_t i = 0;
    while (i < n) {
        const unsigned char c = p[i];
        size_t extra;
        if (c < 0x80) extra = 0;
        else if (c >= 0xC2 && c <= 0xDF) extra = 1;
        else if ((c & 0xF0) == 0xE0) extra = 2;
        else if (c >= 0xF0 && c <= 0xF4) extra = 3;
        else return false;
        if (extra > n - 1 - i) return false;
        for (size_t k = 1; k <= extra; ++k)
            if ((p[i + k] & 0xC0) != 0x80) return false;
        if (extra == 2 && c == 0xE0 && p[i + 1] < 0xA0) return false;           // overlong
        if (extra == 2 && c == 0xED && p[i + 1] > 0x9F) return false;           // surrogates
        if (extra == 3 && c == 0xF0 && p[i + 1] < 0x90) return false;           // overlong
        if (extra == 3 && c == 0xF4 && p[i + 1] > 0x8F) return false;           // above U+10FFFF
        i += extra + 1;
    }
    return true;
}

// Cursor over the header bytes in memory; every read is claimed against the limit first.
struct Cursor {
    const uint8_t *data;
    uint64_t have;   // bytes of the buffer
    uint64_t limit;  // min(file_bytes, 256 MiB)
    uint64_t pos = 0;
    size_t values = 0;
    std::string err;

    bool claim(uint64_t n) {
        if (n > UINT64_MAX - pos) { err = "GGUF cursor overflow"; return false; }
        if (pos + n > limit || pos + n > have) { err = "truncated or oversized GGUF header"; return false; }
        return true;
    }
    template <typename T>
    bool num(T *out) {
        if (!claim(sizeof(T))) return false;
        std::memcpy(out, data + pos, sizeof(T));  // little-endian host
        pos += sizeof(T);
        return true;
    }
    bool string(std::string *out) {
        uint64_t size = 0;
        if (!num(&size) || !claim(size)) return false;
        out->assign(reinterpret_cast<const char *>(data + pos), static_cast<size_t>(size));
        pos += size;
        if (!valid_utf8(*out)) { err = "GGUF string is not UTF-8"; return false; }
        return true;
    }
    bool value(uint32_t kind, bool nested, Value *out) {
        if (++values > kMaxValues) { err = "too many GGUF metadata values"; return false; }
        switch (kind) {
            case 0: { uint8_t v; if (!num(&v)) return false; out->kind = 0; out->u = v; return true; }
            case 1: { int8_t v; if (!num(&v)) return false; out->kind = 1; out->i = v; return true; }
            case 2: { uint16_t v; if (!num(&v)) return false; out->kind = 0; out->u = v; return true; }
            case 3: { int16_t v; if (!num(&v)) return false; out->kind = 1; out->i = v; return true; }
            case 4: { uint32_t v; if (!num(&v)) return false; out->kind = 0; out->u = v; return true; }
            case 5: { int32_t v; if (!num(&v)) return false; out->kind = 1; out->i = v; return true; }
            case 6: { float v; if (!num(&v)) return false; out->kind = 2; out->f = v; return true; }
            case 7: {
                uint8_t v;
                if (!num(&v)) return false;
                if (v > 1) { err = "invalid GGUF boolean"; return false; }
                out->kind = 3; out->b = v != 0; return true;
            }
            case 8: out->kind = 4; return string(&out->s);
            case 9: {
                if (nested) { err = "nested GGUF arrays are not supported"; return false; }
                uint32_t element; uint64_t count;
                if (!num(&element)) return false;
                if (element > 12 || element == 9) { err = "invalid GGUF array element type " + std::to_string(element); return false; }
                if (!num(&count)) return false;
                if (count > kMaxValues - values) { err = "oversized GGUF metadata array"; return false; }
                out->kind = 5;
                for (uint64_t n = 0; n < count; ++n) {  // no count-sized reservation before any value was read
                    Value v;
                    if (!value(element, true, &v)) return false;
                    out->a.push_back(std::move(v));
                }
                return true;
            }
            case 10: { uint64_t v; if (!num(&v)) return false; out->kind = 0; out->u = v; return true; }
            case 11: { int64_t v; if (!num(&v)) return false; out->kind = 1; out->i = v; return true; }
            case 12: { double v; if (!num(&v)) return false; out->kind = 2; out->f = v; return true; }
            default: err = "unknown GGUF metadata type " + std::to_string(kind); return false;
        }
    }
};

// Header::read (header.rs:110-214).  Returns a lisa_status; the message is recorded.
int parse_header(const uint8_t *bytes, uint64_t length, uint64_t file_bytes, Header *h) {
    if (file_bytes < 24) return fail(LISA_ERR_BAD_ARG, "truncated GGUF header");
    Cursor r{bytes, length, std::min(file_bytes, kMaxHeaderBytes)};
    auto bad = [&](const std::string &msg) { return fail(LISA_ERR_BAD_ARG, msg); };
    uint8_t magic[4];
    for (int i = 0; i < 4; ++i)
        if (!r.num(&magic[i])) return bad(r.err);
    if (std::memcmp(magic, "GGUF", 4) != 0) return bad("invalid GGUF magic");
    uint32_t version = 0;
    uint64_t tensor_count = 0, metadata_count = 0;
    if (!r.num(&version)) return bad(r.err);
    if (version != 3) return fail(LISA_ERR_UNSUPPORTED, "only GGUF version 3 is supported");
    if (!r.num(&tensor_count) || !r.num(&metadata_count)) return bad(r.err);
    if (tensor_count > kMaxEntries || metadata_count > kMaxEntries) return fail(LISA_ERR_LIMIT, "GGUF header has too many entries");
    for (uint64_t n = 0; n < metadata_count; ++n) {
        std::string key;
        uint32_t kind = 0;
        if (!r.string(&key)) return bad(r.err);
        if (key.empty() || key.size() > 65536) return bad("invalid GGUF metadata key");
        if (!r.num(&kind)) return bad(r.err);
        Value v;
        if (!r.value(kind, false, &v)) return bad(r.err);
        if (!h->metadata.emplace(key, std::move(v)).second) return bad("duplicate GGUF key " + key);
    }
    uint64_t alignment = 32;
    auto al = h->metadata.find("general.alignment");
    if (al != h->metadata.end() && !al->second.as_u64(&alignment)) return bad("invalid GGUF alignment type");
    if (alignment == 0 || (alignment & (alignment - 1)) != 0 || alignment > 65536)
        return bad("invalid GGUF alignment " + std::to_string(alignment));
    for (uint64_t n = 0; n < tensor_count; ++n) {
        TensorRec t;
        uint32_t rank = 0;
        if (!r.string(&t.name)) return bad(r.err);
        if (t.name.empty() || t.name.size() > 65536) return bad("invalid GGUF tensor name");
        if (!r.num(&rank)) return bad(r.err);
        if (rank < 1 || rank > 4) return bad("invalid GGUF rank " + std::to_string(rank) + " for " + t.name);
        uint64_t elements = 1;
        for (uint32_t d = 0; d < rank; ++d) {
            uint64_t dim = 0;
            if (!r.num(&dim)) return bad(r.err);
            if (dim == 0) return bad("zero dimension for GGUF tensor " + t.name);
            if (elements > UINT64_MAX / dim) return fail(LISA_ERR_OVERFLOW, "GGUF shape overflow");
            elements *= dim;
            t.dims.push_back(dim);
        }
        if (!r.num(&t.type) || !r.num(&t.offset)) return bad(r.err);
        if (t.offset % alignment != 0) return bad("unaligned GGUF tensor " + t.name);
        const int rc = type_row_bytes(t.type, t.dims[0], &t.row_bytes);
        if (rc != LISA_OK) return rc;
        const uint64_t rows = elements / t.dims[0];
        if (rows != 0 && t.row_bytes > UINT64_MAX / rows) return fail(LISA_ERR_OVERFLOW, "GGUF tensor size overflow");
        t.bytes = t.row_bytes * rows;
        const std::string name = t.name;
        if (!h->tensors.emplace(name, std::move(t)).second) return bad("duplicate GGUF tensor " + name);
    }
    if (r.pos > UINT64_MAX - (alignment - 1)) return fail(LISA_ERR_OVERFLOW, "GGUF alignment overflow");
    h->data_offset = (r.pos + alignment - 1) & ~(alignment - 1);
    h->file_bytes = file_bytes;
    if (h->data_offset > file_bytes) return bad("truncated GGUF header padding");
    std::vector<std::pair<std::pair<uint64_t, uint64_t>, const std::string *>> ranges;
    for (auto &kv : h->tensors) {
        TensorRec &t = kv.second;
        if (t.offset > UINT64_MAX - h->data_offset) return fail(LISA_ERR_OVERFLOW, "GGUF offset overflow");
        t.offset += h->data_offset;
        if (t.bytes > UINT64_MAX - t.offset) return fail(LISA_ERR_OVERFLOW, "GGUF tensor range overflow");
        const uint64_t end = t.offset + t.bytes;
        if (end > file_bytes) return bad("GGUF tensor " + t.name + " extends beyond file");
        ranges.push_back({{t.offset, end}, &t.name});
    }
    std::sort(ranges.begin(), ranges.end(), [](const auto &a, const auto &b) {
        return a.first != b.first ? a.first < b.first : *a.second < *b.second;
    });
    for (size_t i = 1; i < ranges.size(); ++i)
        if (ranges[i - 1].first.second > ranges[i].first.first)
            return bad("overlapping GGUF tensors " + *ranges[i - 1].second + " and " + *ranges[i].second);
    return LISA_OK;
}


// ------------------------------------------------------------------------------------------ GGUF package
struct ShardFile {
    std::string path;
    int fd = -1;
    uint64_t bytes = 0;
    dev_t dev = 0;
    ino_t ino = 0;
};

}  // namespace
}  // namespace lisa

struct lisa_gguf {
    lisa::Header header;                       // metadata of the first shard; tensors of all shards
    std::vector<lisa::ShardFile> shards;       // empty for a parsed buffer
    std::vector<const lisa::TensorRec *> order;  // tensors sorted by name
    ~lisa_gguf() {
        for (auto &s : shards)
            if (s.fd >= 0) close(s.fd);
    }
};

namespace lisa {
namespace {

constexpr uint64_t kMaxReadBytes = 64ull << 20;

void index_tensors(lisa_gguf *g) {
    g->order.clear();
    for (auto &kv : g->header.tensors) g->order.push_back(&kv.second);
}

// Reads the header of an open file: the first 256 MiB at most, grown in steps so that a small header costs a
// small read.
int read_file_header(int fd, uint64_t file_bytes, Header *h) {
    std::vector<uint8_t> buf;
    uint64_t want = std::min<uint64_t>(file_bytes, 1u << 20);
    for (;;) {
        buf.resize(want);
        uint64_t got = 0;
        while (got < want) {
            const ssize_t n = pread(fd, buf.data() + got, want - got, static_cast<off_t>(got));
            if (n < 0) return fail(LISA_ERR_BAD_ARG, "reading GGUF header failed");
            if (n == 0) break;
            got += static_cast<uint64_t>(n);
        }
        Header trial;
        const int rc = parse_header(buf.data(), got, file_bytes, &trial);
        const bool short_read = rc != LISA_OK && want < std::min(file_bytes, kMaxHeaderBytes) &&
                                std::string(lisa_cuda_last_error_string()) == "truncated or oversized GGUF header";
        if (short_read) {
            want = std::min<uint64_t>(std::min(file_bytes, kMaxHeaderBytes), want * 8);
            continue;
        }
        if (rc == LISA_OK) *h = std::move(trial);
        return rc;
    }
}

bool meta_u64(const Header &h, const char *key, uint64_t *out) {
    auto it = h.metadata.find(key);
    return it != h.metadata.end() && it->second.as_u64(out);
}
const std::string *meta_str(const Header &h, const char *key) {
    auto it = h.metadata.find(key);
    return (it != h.metadata.end() && it->second.kind == 4) ? &it->second.s : nullptr;
}

// Package::open_paths (package.rs:220-292).
int open_paths(const std::vector<std::string> &paths, lisa_gguf **out) {
    if (paths.empty()) return fail(LISA_ERR_BAD_ARG, "GGUF package has no shards");
    std::unique_ptr<lisa_gguf> g(new lisa_gguf);
    std::set<std::pair<dev_t, ino_t>> seen;
    Header first;
    bool have_first = false;
    for (size_t part = 0; part < paths.size(); ++part) {
        ShardFile sf;
        sf.path = paths[part];
        sf.fd = open(sf.path.c_str(), O_RDONLY | O_CLOEXEC);
        if (sf.fd < 0) return fail(LISA_ERR_BAD_ARG, "opening GGUF " + sf.path);
        struct stat st;
        if (fstat(sf.fd, &st) != 0 || !S_ISREG(st.st_mode)) {
            close(sf.fd);
            return fail(LISA_ERR_BAD_ARG, "GGUF shard is not a regular file");
        }
        sf.bytes = static_cast<uint64_t>(st.st_size);
        sf.dev = st.st_dev;
        sf.ino = st.st_ino;
        g->shards.push_back(sf);
        if (!seen.insert({st.st_dev, st.st_ino}).second) return fail(LISA_ERR_BAD_ARG, "duplicate GGUF shard path");
        Header h;
        const int rc = read_file_header(sf.fd, sf.bytes, &h);
        if (rc != LISA_OK) return rc;
        if (paths.size() > 1 || h.metadata.count("split.count")) {
            uint64_t cnt = 0, no = 0;
            if (!meta_u64(h, "split.count", &cnt)) return fail(LISA_ERR_BAD_ARG, "missing or invalid GGUF integer split.count");
            if (!meta_u64(h, "split.no", &no)) return fail(LISA_ERR_BAD_ARG, "missing or invalid GGUF integer split.no");
            if (cnt != paths.size()) return fail(LISA_ERR_BAD_ARG, "GGUF shard count mismatch in " + sf.path);
            if (no != part) return fail(LISA_ERR_BAD_ARG, "GGUF shard number mismatch in " + sf.path);
        }
        if (have_first) {
            uint64_t a = 0, b = 0;
            if (!meta_u64(h, "split.tensors.count", &a) || !meta_u64(first, "split.tensors.count", &b))
                return fail(LISA_ERR_BAD_ARG, "missing or invalid GGUF integer split.tensors.count");
            if (a != b) return fail(LISA_ERR_BAD_ARG, "GGUF total tensor count differs between shards");
            for (const auto &kv : h.metadata) {
                if (kv.first.rfind("split.", 0) == 0 || kv.first.rfind("general.", 0) == 0) continue;
                auto orig = first.metadata.find(kv.first);
                if (orig != first.metadata.end() && !orig->second.equals(kv.second))
                    return fail(LISA_ERR_BAD_ARG, "conflicting GGUF metadata " + kv.first);
            }
            const std::string *arch = meta_str(h, "general.architecture"), *arch0 = meta_str(first, "general.architecture");
            if (h.metadata.count("general.architecture")) {
                if (!arch0) return fail(LISA_ERR_BAD_ARG, "GGUF has no general.architecture");
                if (!arch || *arch != *arch0) return fail(LISA_ERR_BAD_ARG, "conflicting GGUF architectures");
            }
        }
        for (auto &kv : h.tensors) {
            kv.second.shard = static_cast<int>(part);
            const std::string name = kv.first;
            if (!g->header.tensors.emplace(name, std::move(kv.second)).second)
                return fail(LISA_ERR_BAD_ARG, "duplicate GGUF tensor " + name + " across shards");
        }
        if (!have_first) {
            h.tensors.clear();
            first = std::move(h);
            have_first = true;
        }
    }
    if (paths.size() > 1) {
        uint64_t total = 0;
        if (!meta_u64(first, "split.tensors.count", &total)) return fail(LISA_ERR_BAD_ARG, "missing or invalid GGUF integer split.tensors.count");
        if (total != g->header.tensors.size()) return fail(LISA_ERR_BAD_ARG, "GGUF package tensor count mismatch");
    }
    g->header.metadata = std::move(first.metadata);
    g->header.data_offset = first.data_offset;
    g->header.file_bytes = first.file_bytes;
    index_tensors(g.get());
    *out = g.release();
    return LISA_OK;
}

const TensorRec *tensor_at(const lisa_gguf *g, int64_t index) {
    if (!g || index < 0 || index >= static_cast<int64_t>(g->order.size())) return nullptr;
    return g->order[static_cast<size_t>(index)];
}

uint64_t page_size() { return static_cast<uint64_t>(sysconf(_SC_PAGESIZE)); }

}  // namespace
}  // namespace lisa

using namespace lisa;

extern "C" {

int lisa_gguf_type_layout(uint32_t type, const char **name, uint64_t *block_elements, uint64_t *block_bytes) {
    const TypeLayout *t = find_type(type);
    if (!t) return fail(LISA_ERR_UNSUPPORTED, "unsupported GGUF tensor type " + std::to_string(type));
    if (name) *name = t->name;
    if (block_elements) *block_elements = t->block;
    if (block_bytes) *block_bytes = t->bytes;
    return LISA_OK;
}

int lisa_gguf_row_bytes(uint32_t type, uint64_t columns, uint64_t *row_bytes) {
    if (!row_bytes) return fail(LISA_ERR_BAD_ARG, "gguf_row_bytes: null output");
    return type_row_bytes(type, columns, row_bytes);
}

int lisa_gguf_parse(const void *bytes, uint64_t length, uint64_t file_bytes, lisa_gguf **out) {
    if (!bytes || !out) return fail(LISA_ERR_BAD_ARG, "gguf_parse: null pointer");
    std::unique_ptr<lisa_gguf> g(new lisa_gguf);
    const int rc = parse_header(static_cast<const uint8_t *>(bytes), length, file_bytes, &g->header);
    if (rc != LISA_OK) return rc;
    index_tensors(g.get());
    *out = g.release();
    return LISA_OK;
}

int lisa_gguf_open_paths(const char *const *paths, int count, lisa_gguf **out) {
    if (!paths || !out || count < 1) return fail(LISA_ERR_BAD_ARG, "GGUF package has no shards");
    std::vector<std::string> list;
    for (int i = 0; i < count; ++i) {
        if (!paths[i]) return fail(LISA_ERR_BAD_ARG, "gguf_open_paths: null path");
        list.emplace_back(paths[i]);
    }
    return open_paths(list, out);
}

int lisa_gguf_open(const char *path, lisa_gguf **out) {
    if (!path || !out) return fail(LISA_ERR_BAD_ARG, "gguf_open: null pointer");
    // the first shard's header decides how many files there are (package.rs:163-217)
    const int fd = open(path, O_RDONLY | O_CLOEXEC);
    if (fd < 0) return fail(LISA_ERR_BAD_ARG, std::string("opening GGUF ") + path);
    struct stat st;
    if (fstat(fd, &st) != 0 || !S_ISREG(st.st_mode)) {
        close(fd);
        return fail(LISA_ERR_BAD_ARG, std::string("GGUF is not a regular file: ") + path);
    }
    Header h;
    const int rc = read_file_header(fd, static_cast<uint64_t>(st.st_size), &h);
    close(fd);
    if (rc != LISA_OK) return rc;
    uint64_t count = 1;
    if (h.metadata.count("split.count") && !meta_u64(h, "split.count", &count)) return fail(LISA_ERR_BAD_ARG, "invalid split.count");
    if (count < 1 || count > 1024) return fail(LISA_ERR_BAD_ARG, "invalid GGUF shard count " + std::to_string(count));
    std::vector<std::string> paths{path};
    if (count > 1) {
        uint64_t no = 1;
        if (!meta_u64(h, "split.no", &no)) return fail(LISA_ERR_BAD_ARG, "missing or invalid GGUF integer split.no");
        if (no != 0) return fail(LISA_ERR_BAD_ARG, "pass the first GGUF shard (split.no=0)");
        const std::string full(path);
        const size_t slash = full.find_last_of('/');
        const std::string parent = slash == std::string::npos ? "." : full.substr(0, slash);
        const std::string name = slash == std::string::npos ? full : full.substr(slash + 1);
        char suffix[64];
        snprintf(suffix, sizeof(suffix), "-00001-of-%05llu.gguf", static_cast<unsigned long long>(count));
        const std::string suf(suffix);
        if (name.size() < suf.size() || name.compare(name.size() - suf.size(), suf.size(), suf) != 0)
            return fail(LISA_ERR_BAD_ARG, "split GGUF filename does not match metadata");
        const std::string stem = name.substr(0, name.size() - suf.size());
        for (uint64_t part = 2; part <= count; ++part) {
            char tail[64];
            snprintf(tail, sizeof(tail), "-%05llu-of-%05llu.gguf", static_cast<unsigned long long>(part),
                     static_cast<unsigned long long>(count));
            const std::string expected = parent + "/" + stem + tail;
            struct stat ps;
            if (stat(expected.c_str(), &ps) != 0 || !S_ISREG(ps.st_mode)) return fail(LISA_ERR_BAD_ARG, "missing GGUF shard " + expected);
            paths.push_back(expected);
        }
    }
    return open_paths(paths, out);
}

void lisa_gguf_close(lisa_gguf *g) { delete g; }

uint64_t lisa_gguf_data_offset(const lisa_gguf *g) { return g ? g->header.data_offset : 0; }
uint64_t lisa_gguf_file_bytes(const lisa_gguf *g) { return g ? g->header.file_bytes : 0; }
int lisa_gguf_shard_count(const lisa_gguf *g) { return g ? static_cast<int>(g->shards.size()) : 0; }
const char *lisa_gguf_shard_path(const lisa_gguf *g, int shard) {
    if (!g || shard < 0 || shard >= static_cast<int>(g->shards.size())) return nullptr;
    return g->shards[shard].path.c_str();
}
int64_t lisa_gguf_tensor_count(const lisa_gguf *g) { return g ? static_cast<int64_t>(g->order.size()) : 0; }

int lisa_gguf_tensor_at(const lisa_gguf *g, int64_t index, lisa_gguf_tensor *out) {
    const TensorRec *t = tensor_at(g, index);
    if (!t || !out) return fail(LISA_ERR_BAD_ARG, "gguf_tensor_at: index out of range");
    std::memset(out, 0, sizeof(*out));
    out->name = t->name.c_str();
    out->rank = static_cast<uint32_t>(t->dims.size());
    uint64_t rows = 1;
    for (size_t d = 0; d < t->dims.size(); ++d) {
        out->dimensions[d] = t->dims[d];
        if (d > 0) rows *= t->dims[d];  // the header parse has checked the product for overflow
    }
    out->type = t->type;
    out->offset = t->offset;
    out->bytes = t->bytes;
    out->rows = rows;
    out->row_bytes = t->row_bytes;
    out->shard = t->shard;
    return LISA_OK;
}

int64_t lisa_gguf_find_tensor(const lisa_gguf *g, const char *name) {
    if (!g || !name) return fail(LISA_ERR_BAD_ARG, "gguf_find_tensor: null pointer");
    auto it = std::lower_bound(g->order.begin(), g->order.end(), std::string(name),
                               [](const TensorRec *t, const std::string &n) { return t->name < n; });
    if (it == g->order.end() || (*it)->name != name) return fail(LISA_ERR_BAD_ARG, std::string("missing GGUF tensor ") + name);
    return static_cast<int64_t>(it - g->order.begin());
}

static const Value *meta(const lisa_gguf *g, const char *key) {
    if (!g || !key) return nullptr;
    auto it = g->header.metadata.find(key);
    return it == g->header.metadata.end() ? nullptr : &it->second;
}

int lisa_gguf_metadata_kind(const lisa_gguf *g, const char *key) {
    const Value *v = meta(g, key);
    return v ? v->kind : -1;
}
int lisa_gguf_metadata_u64(const lisa_gguf *g, const char *key, uint64_t *out) {
    const Value *v = meta(g, key);
    if (!v || !out || !v->as_u64(out)) return fail(LISA_ERR_BAD_ARG, std::string("missing or invalid GGUF integer ") + (key ? key : ""));
    return LISA_OK;
}
int lisa_gguf_metadata_f64(const lisa_gguf *g, const char *key, double *out) {
    const Value *v = meta(g, key);
    if (!v || !out || !v->as_f64(out)) return fail(LISA_ERR_BAD_ARG, std::string("missing or invalid GGUF number ") + (key ? key : ""));
    return LISA_OK;
}
const char *lisa_gguf_metadata_str(const lisa_gguf *g, const char *key) {
    const Value *v = meta(g, key);
    return (v && v->kind == 4) ? v->s.c_str() : nullptr;
}
int64_t lisa_gguf_metadata_array_len(const lisa_gguf *g, const char *key) {
    const Value *v = meta(g, key);
    return (v && v->kind == 5) ? static_cast<int64_t>(v->a.size()) : -1;
}
int lisa_gguf_metadata_array_u64(const lisa_gguf *g, const char *key, int64_t index, uint64_t *out) {
    const Value *v = meta(g, key);
    if (!v || v->kind != 5 || index < 0 || index >= static_cast<int64_t>(v->a.size()) || !out || !v->a[index].as_u64(out))
        return fail(LISA_ERR_BAD_ARG, "gguf_metadata_array_u64: no such integer element");
    return LISA_OK;
}
const char *lisa_gguf_metadata_array_str(const lisa_gguf *g, const char *key, int64_t index) {
    const Value *v = meta(g, key);
    if (!v || v->kind != 5 || index < 0 || index >= static_cast<int64_t>(v->a.size()) || v->a[index].kind != 4) return nullptr;
    return v->a[index].s.c_str();
}

int lisa_gguf_read_bytes(const lisa_gguf *g, int64_t tensor, uint64_t offset, void *out, uint64_t length) {
    const TensorRec *t = tensor_at(g, tensor);
    if (!t || (!out && length)) return fail(LISA_ERR_BAD_ARG, "gguf_read_bytes: bad tensor or null output");
    if (g->shards.empty()) return fail(LISA_ERR_BAD_ARG, "gguf_read_bytes: the handle was parsed from memory, it has no file");
    if (length > kMaxReadBytes) return fail(LISA_ERR_LIMIT, "GGUF read exceeds 64 MiB staging limit");
    if (offset > UINT64_MAX - length) return fail(LISA_ERR_OVERFLOW, "GGUF read overflow");
    if (offset + length > t->bytes) return fail(LISA_ERR_BAD_ARG, "read outside GGUF tensor " + t->name);
    const ShardFile &sf = g->shards[t->shard];
    uint64_t got = 0;
    while (got < length) {
        const ssize_t n = pread(sf.fd, static_cast<uint8_t *>(out) + got, length - got, static_cast<off_t>(t->offset + offset + got));
        if (n <= 0) return fail(LISA_ERR_BAD_ARG, "reading " + t->name + " in " + sf.path);
        got += static_cast<uint64_t>(n);
    }
    return LISA_OK;
}

int lisa_gguf_read_rows(const lisa_gguf *g, int64_t tensor, const uint64_t *rows, uint64_t count, void *out, uint64_t out_bytes) {
    const TensorRec *t = tensor_at(g, tensor);
    if (!t || (!rows && count)) return fail(LISA_ERR_BAD_ARG, "gguf_read_rows: bad tensor or null rows");
    uint64_t nrows = 1;
    for (size_t d = 1; d < t->dims.size(); ++d) nrows *= t->dims[d];
    if (t->row_bytes != 0 && count > UINT64_MAX / t->row_bytes) return fail(LISA_ERR_OVERFLOW, "GGUF row read size overflow");
    const uint64_t total = count * t->row_bytes;
    if (total != out_bytes || total > kMaxReadBytes) return fail(LISA_ERR_BAD_ARG, "invalid or oversized GGUF row output buffer");
    for (uint64_t i = 0; i < count; ++i)
        if (rows[i] >= nrows) return fail(LISA_ERR_BAD_ARG, "GGUF row index out of range");
    for (uint64_t i = 0; i < count; ++i) {
        const int rc = lisa_gguf_read_bytes(g, tensor, rows[i] * t->row_bytes, static_cast<uint8_t *>(out) + i * t->row_bytes, t->row_bytes);
        if (rc != LISA_OK) return rc;
    }
    return LISA_OK;
}

int lisa_gguf_mapped_region_bytes(const lisa_gguf *g, int64_t tensor, uint64_t *bytes) {
    const TensorRec *t = tensor_at(g, tensor);
    if (!t || !bytes) return fail(LISA_ERR_BAD_ARG, "gguf_mapped_region_bytes: bad tensor or null output");
    const uint64_t page = page_size();
    if (page == 0 || (page & (page - 1)) != 0) return fail(LISA_ERR_BAD_ARG, "invalid host page size");
    const uint64_t inner = t->offset % page;
    if (t->bytes > UINT64_MAX - inner || inner + t->bytes > UINT64_MAX - (page - 1)) return fail(LISA_ERR_OVERFLOW, "GGUF mapping size overflow");
    *bytes = (inner + t->bytes + page - 1) & ~(page - 1);
    return LISA_OK;
}

int lisa_gguf_map_region(const lisa_gguf *g, int64_t tensor, void **mapping, uint64_t *mapped_bytes, uint64_t *inner) {
    const TensorRec *t = tensor_at(g, tensor);
    if (!t || !mapping || !mapped_bytes || !inner) return fail(LISA_ERR_BAD_ARG, "gguf_map_region: bad tensor or null output");
    if (g->shards.empty()) return fail(LISA_ERR_BAD_ARG, "gguf_map_region: the handle was parsed from memory, it has no file");
    uint64_t length = 0;
    const int rc = lisa_gguf_mapped_region_bytes(g, tensor, &length);
    if (rc != LISA_OK) return rc;
    const ShardFile &sf = g->shards[t->shard];
    struct stat st;
    if (fstat(sf.fd, &st) != 0 || static_cast<uint64_t>(st.st_size) < t->offset + t->bytes)
        return fail(LISA_ERR_BAD_ARG, "GGUF shard was truncated: " + sf.path);
    const uint64_t in = t->offset % page_size();
    // the mapping reaches at most to the end of the file's last page; views stay inside the tensor's own bytes
    void *p = mmap(nullptr, length, PROT_READ, MAP_PRIVATE, sf.fd, static_cast<off_t>(t->offset - in));
    if (p == MAP_FAILED) return fail(LISA_ERR_BAD_ARG, "mapping " + t->name + " in " + sf.path + " failed");
    *mapping = p;
    *mapped_bytes = length;
    *inner = in;
    return LISA_OK;
}

int lisa_gguf_unmap(void *mapping, uint64_t mapped_bytes) {
    if (!mapping || munmap(mapping, mapped_bytes) != 0) return fail(LISA_ERR_BAD_ARG, "gguf_unmap: munmap failed");
    return LISA_OK;
}

int lisa_gguf_weight_view(const lisa_gguf *g, int64_t tensor, int64_t *experts, int64_t *rows, int64_t *row_bytes) {
    const TensorRec *t = tensor_at(g, tensor);
    if (!t || !experts || !rows || !row_bytes) return fail(LISA_ERR_BAD_ARG, "gguf_weight_view: bad tensor or null output");
    // shape = reversed(dimensions[1..]) + [row_bytes], every entry an i32 (gguf_resident.rs:95-101)
    uint64_t e = 1;
    const uint64_t r = t->dims.size() > 1 ? t->dims[1] : 1;
    for (size_t d = 2; d < t->dims.size(); ++d) e *= t->dims[d];
    if (e > INT32_MAX || r > INT32_MAX || t->row_bytes > INT32_MAX) return fail(LISA_ERR_OVERFLOW, "GGUF tensor view does not fit 32-bit dimensions");
    *experts = static_cast<int64_t>(e);
    *rows = static_cast<int64_t>(r);
    *row_bytes = static_cast<int64_t>(t->row_bytes);
    return LISA_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------ safetensors
namespace lisa {
namespace {

// The JSON subset a safetensors header uses, parsed into a small tree (objects keep their key order).
struct Json {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool b = false;
    double num = 0;
    bool integral = false;  // a number written without fraction or exponent that fits u64
    uint64_t u = 0;
    std::string s;
    std::vector<Json> items;
    std::vector<std::pair<std::string, Json>> fields;

    const Json *get(const char *key) const {
        for (const auto &f : fields)
            if (f.first == key) return &f.second;
        return nullptr;
    }
};

struct JsonParser {
    const char *p, *end;
    std::string err;
    int depth = 0;

    void ws() {
        while (p < end && (*p == ' ' || *p == '\n' || *p == '\r' || *p == '\t')) ++p;
    }
    bool fail_at(const char *what) {
        if (err.empty()) err = what;
        return false;
    }
    bool string(std::string *out) {
        if (p >= end || *p != '"') return fail_at("expected a string");
        ++p;
        out->clear();
        while (p < end && *p != '"') {
            unsigned char c = static_cast<unsigned char>(*p++);
            if (c < 0x20) return fail_at("control character in string");
            if (c != '\\') {
                out->push_back(static_cast<char>(c));
                continue;
            }
            if (p >= end) return fail_at("truncated escape");
            const char e = *p++;
            switch (e) {
                case '"': out->push_back('"'); break;
                case '\\': out->push_back('\\'); break;
                case '/': out->push_back('/'); break;
                case 'b': out->push_back('\b'); break;
                case 'f': out->push_back('\f'); break;
                case 'n': out->push_back('\n'); break;
                case 'r': out->push_back('\r'); break;
                case 't': out->push_back('\t'); break;
                case 'u': {
                    if (end - p < 4) return fail_at("truncated \\u escape");
                    unsigned cp = 0;
                    for (int i = 0; i < 4; ++i) {
                        const char h = *p++;
                        cp <<= 4;
                        if (h >= '0' && h <= '9') cp |= h - '0';
                        else if (h >= 'a' && h <= 'f') cp |= h - 'a' + 10;
                        else if (h >= 'A' && h <= 'F') cp |= h - 'A' + 10;
                        else return fail_at("bad \\u escape");
                    }
                    // tensor names are ASCII in practice; other code points are encoded as UTF-8 (no surrogate pairing)
                    if (cp < 0x80) out->push_back(static_cast<char>(cp));
                    else if (cp < 0x800) { out->push_back(static_cast<char>(0xC0 | (cp >> 6))); out->push_back(static_cast<char>(0x80 | (cp & 0x3F))); }
                    else { out->push_back(static_cast<char>(0xE0 | (cp >> 12))); out->push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F))); out->push_back(static_cast<char>(0x80 | (cp & 0x3F))); }
                    break;
                }
                default: return fail_at("bad escape");
            }
        }
        if (p >= end) return fail_at("unterminated string");
        ++p;
        return true;
    }
    bool value(Json *out) {
        if (++depth > 64) return fail_at("JSON nested too deeply");
        ws();
        if (p >= end) return fail_at("unexpected end of JSON");
        bool ok = true;
        if (*p == '{') {
            ++p;
            out->kind = Json::Object;
            ws();
            if (p < end && *p == '}') { ++p; --depth; return true; }
            for (;;) {
                ws();
                std::string key;
                if (!string(&key)) return false;
                ws();
                if (p >= end || *p != ':') return fail_at("expected ':'");
                ++p;
                Json v;
                if (!value(&v)) return false;
                out->fields.emplace_back(std::move(key), std::move(v));
                ws();
                if (p < end && *p == ',') { ++p; continue; }
                if (p < end && *p == '}') { ++p; break; }
                return fail_at("expected ',' or '}'");
            }
        } else if (*p == '[') {
            ++p;
            out->kind = Json::Array;
            ws();
            if (p < end && *p == ']') { ++p; --depth; return true; }
            for (;;) {
                Json v;
                if (!value(&v)) return false;
                out->items.push_back(std::move(v));
                ws();
                if (p < end && *p == ',') { ++p; continue; }
                if (p < end && *p == ']') { ++p; break; }
                return fail_at("expected ',' or ']'");
            }
        } else if (*p == '"') {
            out->kind = Json::String;
            ok = string(&out->s);
        } else if (end - p >= 4 && std::memcmp(p, "true", 4) == 0) {
            out->kind = Json::Bool; out->b = true; p += 4;
        } else if (end - p >= 5 && std::memcmp(p, "false", 5) == 0) {
            out->kind = Json::Bool; out->b = false; p += 5;
        } else if (end - p >= 4 && std::memcmp(p, "null", 4) == 0) {
            out->kind = Json::Null; p += 4;
        } else {
            const char *q = p;
            if (q < end && *q == '-') ++q;
            const char *digits = q;
            while (q < end && *q >= '0' && *q <= '9') ++q;
            if (q == digits) return fail_at("unexpected character in JSON");
            bool integral = *p != '-';
            if (q < end && (*q == '.' || *q == 'e' || *q == 'E')) {
                integral = false;
                while (q < end && ((*q >= '0' && *q <= '9') || *q == '.' || *q == 'e' || *q == 'E' || *q == '+' || *q == '-')) ++q;
            }
            const std::string text(p, q);
            out->kind = Json::Number;
            out->num = strtod(text.c_str(), nullptr);
            if (integral && text.size() <= 20) {
                unsigned long long v = 0;
                bool overflow = false;
                for (char c : text) {
                    const unsigned d = static_cast<unsigned>(c - '0');
                    if (v > (UINT64_MAX - d) / 10) { overflow = true; break; }
                    v = v * 10 + d;
                }
                out->integral = !overflow;
                out->u = v;
            }
            p = q;
        }
        --depth;
        return ok;
    }
};

struct StTensor {
    std::string name;
    int dtype = 0;
    std::vector<int64_t> shape;
    uint64_t start = 0, end = 0;  // absolute offsets in the file
};

const struct {
    const char *name;
    int code;
    uint64_t size;
} kStDtypes[] = {{"BF16", LISA_ST_BF16, 2}, {"F32", LISA_ST_F32, 4}, {"F16", LISA_ST_F16, 2}, {"I64", LISA_ST_I64, 8},
                 {"I32", LISA_ST_I32, 4},   {"U32", LISA_ST_U32, 4}, {"U8", LISA_ST_U8, 1},   {"BOOL", LISA_ST_BOOL, 1}};

}  // namespace
}  // namespace lisa

struct lisa_safetensors {
    std::string path;
    void *map = nullptr;
    uint64_t bytes = 0;
    std::vector<lisa::StTensor> tensors;  // sorted by name
    ~lisa_safetensors() {
        if (map) munmap(map, bytes);
    }
};

namespace lisa {
namespace {

void fill_st(const lisa_safetensors *s, const StTensor &t, lisa_st_tensor *out) {
    std::memset(out, 0, sizeof(*out));
    out->name = t.name.c_str();
    out->dtype = t.dtype;
    out->rank = static_cast<int32_t>(t.shape.size());
    for (size_t d = 0; d < t.shape.size(); ++d) out->shape[d] = t.shape[d];
    out->data = static_cast<const uint8_t *>(s->map) + t.start;
    out->bytes = t.end - t.start;
}

const StTensor *st_find(const lisa_safetensors *s, const std::string &name) {
    auto it = std::lower_bound(s->tensors.begin(), s->tensors.end(), name, [](const StTensor &t, const std::string &n) { return t.name < n; });
    return (it != s->tensors.end() && it->name == name) ? &*it : nullptr;
}

}  // namespace
}  // namespace lisa

extern "C" {

int lisa_safetensors_open(const char *path, lisa_safetensors **out) {
    if (!path || !out) return fail(LISA_ERR_BAD_ARG, "safetensors_open: null pointer");
    const std::string where(path);
    const int fd = open(path, O_RDONLY | O_CLOEXEC);
    if (fd < 0) return fail(LISA_ERR_BAD_ARG, "opening shard " + where);
    struct stat st;
    if (fstat(fd, &st) != 0 || !S_ISREG(st.st_mode)) {
        close(fd);
        return fail(LISA_ERR_BAD_ARG, "opening shard " + where);
    }
    std::unique_ptr<lisa_safetensors> s(new lisa_safetensors);
    s->path = where;
    s->bytes = static_cast<uint64_t>(st.st_size);
    if (s->bytes < 8) {
        close(fd);
        s->bytes = 0;
        return fail(LISA_ERR_BAD_ARG, "shard " + where + " too small");
    }
    void *m = mmap(nullptr, s->bytes, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (m == MAP_FAILED) {
        s->bytes = 0;
        return fail(LISA_ERR_BAD_ARG, "mapping shard " + where + " failed");
    }
    s->map = m;
    const uint8_t *base = static_cast<const uint8_t *>(m);
    uint64_t header_len = 0;
    std::memcpy(&header_len, base, 8);
    if (header_len > UINT64_MAX - 8) return fail(LISA_ERR_OVERFLOW, "safetensors header length overflow");
    const uint64_t payload_start = header_len + 8;
    if (payload_start > s->bytes || header_len > (64ull << 20)) return fail(LISA_ERR_BAD_ARG, "shard " + where + " has an invalid or oversized header");
    Json root;
    JsonParser jp{reinterpret_cast<const char *>(base + 8), reinterpret_cast<const char *>(base + payload_start)};
    if (!jp.value(&root)) return fail(LISA_ERR_BAD_ARG, "parsing shard header " + where + ": " + jp.err);
    jp.ws();
    if (jp.p != jp.end) return fail(LISA_ERR_BAD_ARG, "parsing shard header " + where + ": trailing characters");
    if (root.kind != Json::Object) return fail(LISA_ERR_BAD_ARG, "safetensors header must be an object");
    const uint64_t payload = s->bytes - payload_start;
    std::set<std::string> names;
    for (const auto &field : root.fields) {
        const std::string &name = field.first;
        if (name == "__metadata__") continue;
        const Json &info = field.second;
        StTensor t;
        t.name = name;
        const Json *dt = info.kind == Json::Object ? info.get("dtype") : nullptr;
        const std::string dtype = (dt && dt->kind == Json::String) ? dt->s : "";
        uint64_t expected = 0;
        bool known = false;
        for (const auto &d : kStDtypes)
            if (dtype == d.name) {
                t.dtype = d.code;
                expected = d.size;
                known = true;
            }
        if (!known) return fail(LISA_ERR_UNSUPPORTED, "unsupported dtype " + dtype + " for " + name);
        const Json *shape = info.get("shape");
        if (!shape || shape->kind != Json::Array) return fail(LISA_ERR_BAD_ARG, "missing shape for " + name);
        if (shape->items.size() > 8) return fail(LISA_ERR_LIMIT, "more than 8 dimensions for " + name);
        for (const Json &d : shape->items) {
            if (d.kind != Json::Number || !d.integral || d.u > INT32_MAX) return fail(LISA_ERR_BAD_ARG, "invalid dimension for " + name);
            if (d.u != 0 && expected > UINT64_MAX / d.u) return fail(LISA_ERR_OVERFLOW, "tensor shape overflows for " + name);
            expected *= d.u;
            t.shape.push_back(static_cast<int64_t>(d.u));
        }
        const Json *range = info.get("data_offsets");
        if (!range || range->kind != Json::Array) return fail(LISA_ERR_BAD_ARG, "missing data_offsets for " + name);
        if (range->items.size() != 2) return fail(LISA_ERR_BAD_ARG, "data_offsets must have two entries for " + name);
        for (const Json &v : range->items)
            if (v.kind != Json::Number || !v.integral) return fail(LISA_ERR_BAD_ARG, "invalid data offset for " + name);
        const uint64_t start = range->items[0].u, end = range->items[1].u;
        if (!(start <= end && end <= payload)) return fail(LISA_ERR_BAD_ARG, "tensor " + name + " exceeds shard payload bounds");
        if (end - start != expected) return fail(LISA_ERR_BAD_ARG, "tensor byte size differs from shape for " + name);
        t.start = payload_start + start;
        t.end = payload_start + end;
        if (!names.insert(name).second) return fail(LISA_ERR_BAD_ARG, "duplicate tensor " + name);
        s->tensors.push_back(std::move(t));
    }
    std::sort(s->tensors.begin(), s->tensors.end(), [](const StTensor &a, const StTensor &b) { return a.name < b.name; });
    *out = s.release();
    return LISA_OK;
}

void lisa_safetensors_close(lisa_safetensors *s) { delete s; }

int64_t lisa_safetensors_tensor_count(const lisa_safetensors *s) { return s ? static_cast<int64_t>(s->tensors.size()) : 0; }

int lisa_safetensors_tensor_at(const lisa_safetensors *s, int64_t index, lisa_st_tensor *out) {
    if (!s || !out || index < 0 || index >= static_cast<int64_t>(s->tensors.size())) return fail(LISA_ERR_BAD_ARG, "safetensors_tensor_at: index out of range");
    fill_st(s, s->tensors[static_cast<size_t>(index)], out);
    return LISA_OK;
}

int lisa_safetensors_find(const lisa_safetensors *s, const char *name, lisa_st_tensor *out) {
    if (!s || !name || !out) return fail(LISA_ERR_BAD_ARG, "safetensors_find: null pointer");
    const StTensor *t = st_find(s, name);
    if (!t) return fail(LISA_ERR_BAD_ARG, std::string("tensor ") + name + " missing from shard");
    fill_st(s, *t, out);
    return LISA_OK;
}

int32_t lisa_detect_group_size(int32_t weight_cols, int32_t scales_cols, int32_t bits) {
    if (weight_cols <= 0 || scales_cols <= 0 || bits <= 0 || 32 % bits != 0) return 0;
    const int64_t k = static_cast<int64_t>(weight_cols) * (32 / bits);
    if (k > INT32_MAX) return 0;  // checked_mul
    if (k % scales_cols != 0) return 0;
    const int64_t group = k / scales_cols;
    return (group >= 1 && group <= 4096) ? static_cast<int32_t>(group) : 0;
}

int lisa_safetensors_quantized_triplet(const lisa_safetensors *s, const char *prefix, const char *key, int32_t bits,
                                       int32_t group_size_hint, lisa_quantized_triplet *out) {
    if (!s || !prefix || !out) return fail(LISA_ERR_BAD_ARG, "quantized_triplet: null pointer");
    const std::string base = (key && key[0]) ? std::string(prefix) + "." + key : std::string(prefix);
    const StTensor *w = st_find(s, base + ".weight"), *sc = st_find(s, base + ".scales"), *bi = st_find(s, base + ".biases");
    if (!w) return fail(LISA_ERR_BAD_ARG, "tensor " + base + ".weight missing from shard");
    if (!sc) return fail(LISA_ERR_BAD_ARG, "tensor " + base + ".scales missing from shard");
    if (!bi) return fail(LISA_ERR_BAD_ARG, "tensor " + base + ".biases missing from shard");
    if (w->dtype != LISA_ST_U32 || w->shape.size() < 2) return fail(LISA_ERR_BAD_ARG, base + ".weight must be U32 with at least two dimensions");
    if (sc->shape != bi->shape || sc->dtype != bi->dtype || (sc->dtype != LISA_ST_BF16 && sc->dtype != LISA_ST_F16 && sc->dtype != LISA_ST_F32))
        return fail(LISA_ERR_BAD_ARG, base + ": scales and biases must have the same float type and shape");
    if (sc->shape.size() != w->shape.size()) return fail(LISA_ERR_BAD_ARG, base + ": weight and scales ranks differ");
    for (size_t d = 0; d + 1 < w->shape.size(); ++d)
        if (w->shape[d] != sc->shape[d]) return fail(LISA_ERR_BAD_ARG, base + ": weight and scales rows differ");
    const int64_t wc = w->shape.back(), scol = sc->shape.back();
    int32_t group = lisa_detect_group_size(static_cast<int32_t>(wc), static_cast<int32_t>(scol), bits);
    if (group == 0) group = group_size_hint;
    if (bits <= 0 || 32 % bits != 0 || group <= 0) return fail(LISA_ERR_BAD_ARG, base + ": no usable bit width or group size");
    fill_st(s, *w, &out->weight);
    fill_st(s, *sc, &out->scales);
    fill_st(s, *bi, &out->biases);
    out->group_size = group;
    out->bits = bits;
    out->n = w->shape[w->shape.size() - 2];
    out->k = wc * (32 / bits);
    return LISA_OK;
}

}  // extern "C"
