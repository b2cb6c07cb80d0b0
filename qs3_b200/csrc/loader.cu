// Checkpoint loader for the tensors of one MoE layer: safetensors shards -> the device
// layouts the layer call consumes. Upstream has this component only as a trait
// (src/weight_loader.rs:33-38: alloc_tensor / read_exact / zero_fill / seal) and a written
// contract (src/weight_loader.rs:9-32, AGENTS.md:55-67): validate the whole manifest before
// any CUDA-visible memory is touched, then stream file byte ranges through a pinned ring
// (cudaHostAlloc, pread, cudaMemcpyAsync, events) into the final device storage.
//
// Parts of this file:
//   JsonValue / JsonParser      minimal JSON reader (objects keep insertion order and
//                               report duplicate keys, which the manifest check rejects)
//   qs3_checkpoint              parsed shard headers, index and config of one directory
//   LayerManifest               the tensors one MoE layer must have, with the device plan
//   PinnedUploadBackend         the four operations of the upstream trait on a dGPU
//   transpose_bf16_kernel       [n, r, c] -> [n, c, r] for fused tensors stored transposed
#include "common.cuh"

#include <dirent.h>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace qs3 {
namespace ckpt {

// ---- JSON -----------------------------------------------------------------------------

struct JsonValue {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool boolean = false;
    double number = 0.0;
    bool integral = false;     // the literal had no fraction / exponent and fits int64
    int64_t integer = 0;
    std::string text;
    std::vector<JsonValue> items;
    std::vector<std::pair<std::string, JsonValue>> members; // insertion order, duplicates kept

    const JsonValue* get(const char* key) const
    {
        if (kind != Object)
            return nullptr;
        for (const auto& m : members)
            if (m.first == key)
                return &m.second;
        return nullptr;
    }
};

class JsonParser {
public:
    JsonParser(const char* data, size_t size) : p_(data), end_(data + size) {}

    // Parses one document; on failure `error` says what and where.
    bool parse(JsonValue* out, std::string* error)
    {
        if (!value(out, 0) || (skip_ws(), p_ != end_)) {
            if (err_.empty())
                err_ = "trailing characters after the JSON document";
            *error = err_ + " (byte " + std::to_string(pos_of_error()) + ")";
            return false;
        }
        return true;
    }

private:
    static constexpr int kMaxDepth = 64;
    const char* p_;
    const char* end_;
    const char* begin_ = p_;
    std::string err_;

    size_t pos_of_error() const { return static_cast<size_t>(p_ - begin_); }
    bool fail(const char* what)
    {
        if (err_.empty())
            err_ = what;
        return false;
    }
    void skip_ws()
    {
        while (p_ != end_ && (*p_ == ' ' || *p_ == '\t' || *p_ == '\n' || *p_ == '\r'))
            ++p_;
    }
    bool literal(const char* word)
    {
        const size_t n = std::strlen(word);
        if (static_cast<size_t>(end_ - p_) < n || std::memcmp(p_, word, n) != 0)
            return fail("unknown literal");
        p_ += n;
        return true;
    }
    static void append_utf8(std::string* s, uint32_t cp)
    {
        if (cp < 0x80) {
            s->push_back(static_cast<char>(cp));
        } else if (cp < 0x800) {
            s->push_back(static_cast<char>(0xC0 | (cp >> 6)));
            s->push_back(static_cast<char>(0x80 | (cp & 0x3F)));
        } else if (cp < 0x10000) {
            s->push_back(static_cast<char>(0xE0 | (cp >> 12)));
            s->push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
            s->push_back(static_cast<char>(0x80 | (cp & 0x3F)));
        } else {
            s->push_back(static_cast<char>(0xF0 | (cp >> 18)));
            s->push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
            s->push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
            s->push_back(static_cast<char>(0x80 | (cp & 0x3F)));
        }
    }
    bool hex4(uint32_t* out)
    {
        if (end_ - p_ < 4)
            return fail("truncated \\u escape");
        uint32_t v = 0;
        for (int i = 0; i < 4; ++i) {
            const char c = *p_++;
            v <<= 4;
            if (c >= '0' && c <= '9')
                v |= static_cast<uint32_t>(c - '0');
            else if (c >= 'a' && c <= 'f')
                v |= static_cast<uint32_t>(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F')
                v |= static_cast<uint32_t>(c - 'A' + 10);
            else
                return fail("bad \\u escape");
        }
        *out = v;
        return true;
    }
    bool string(std::string* out)
    {
        if (p_ == end_ || *p_ != '"')
            return fail("expected a string");
        ++p_;
        out->clear();
        while (p_ != end_) {
            const unsigned char c = static_cast<unsigned char>(*p_++);
            if (c == '"')
                return true;
            if (c < 0x20)
                return fail("control character inside a string");
            if (c != '\\') {
                out->push_back(static_cast<char>(c));
                continue;
            }
            if (p_ == end_)
                break;
            const char e = *p_++;
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
                uint32_t cp = 0;
                if (!hex4(&cp))
                    return false;
                if (cp >= 0xD800 && cp < 0xDC00) { // surrogate pair
                    uint32_t lo = 0;
                    if (end_ - p_ < 2 || p_[0] != '\\' || p_[1] != 'u')
                        return fail("lone surrogate in a string");
                    p_ += 2;
                    if (!hex4(&lo) || lo < 0xDC00 || lo > 0xDFFF)
                        return fail("bad surrogate pair");
                    cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                }
                append_utf8(out, cp);
                break;
            }
            default: return fail("unknown escape in a string");
            }
        }
        return fail("unterminated string");
    }
    bool number(JsonValue* out)
    {
        const char* start = p_;
        if (p_ != end_ && *p_ == '-')
            ++p_;
        if (p_ == end_ || *p_ < '0' || *p_ > '9')
            return fail("bad number");
        bool integral = true;
        while (p_ != end_ && *p_ >= '0' && *p_ <= '9')
            ++p_;
        if (p_ != end_ && *p_ == '.') {
            integral = false;
            ++p_;
            if (p_ == end_ || *p_ < '0' || *p_ > '9')
                return fail("bad number");
            while (p_ != end_ && *p_ >= '0' && *p_ <= '9')
                ++p_;
        }
        if (p_ != end_ && (*p_ == 'e' || *p_ == 'E')) {
            integral = false;
            ++p_;
            if (p_ != end_ && (*p_ == '+' || *p_ == '-'))
                ++p_;
            if (p_ == end_ || *p_ < '0' || *p_ > '9')
                return fail("bad number");
            while (p_ != end_ && *p_ >= '0' && *p_ <= '9')
                ++p_;
        }
        const std::string lit(start, p_);
        out->kind = JsonValue::Number;
        out->number = std::strtod(lit.c_str(), nullptr);
        out->integral = false;
        if (integral && lit.size() <= 19) { // at most 18 digits and a sign: no overflow
            out->integral = true;
            out->integer = std::strtoll(lit.c_str(), nullptr, 10);
        }
        return true;
    }
    bool value(JsonValue* out, int depth)
    {
        if (depth > kMaxDepth)
            return fail("nesting too deep");
        skip_ws();
        if (p_ == end_)
            return fail("unexpected end of document");
        const char c = *p_;
        if (c == '{') {
            ++p_;
            out->kind = JsonValue::Object;
            skip_ws();
            if (p_ != end_ && *p_ == '}') {
                ++p_;
                return true;
            }
            for (;;) {
                skip_ws();
                std::string key;
                if (!string(&key))
                    return false;
                skip_ws();
                if (p_ == end_ || *p_ != ':')
                    return fail("expected ':'");
                ++p_;
                out->members.emplace_back(std::move(key), JsonValue());
                if (!value(&out->members.back().second, depth + 1))
                    return false;
                skip_ws();
                if (p_ != end_ && *p_ == ',') {
                    ++p_;
                    continue;
                }
                if (p_ != end_ && *p_ == '}') {
                    ++p_;
                    return true;
                }
                return fail("expected ',' or '}'");
            }
        }
        if (c == '[') {
            ++p_;
            out->kind = JsonValue::Array;
            skip_ws();
            if (p_ != end_ && *p_ == ']') {
                ++p_;
                return true;
            }
            for (;;) {
                out->items.emplace_back();
                if (!value(&out->items.back(), depth + 1))
                    return false;
                skip_ws();
                if (p_ != end_ && *p_ == ',') {
                    ++p_;
                    continue;
                }
                if (p_ != end_ && *p_ == ']') {
                    ++p_;
                    return true;
                }
                return fail("expected ',' or ']'");
            }
        }
        if (c == '"') {
            out->kind = JsonValue::String;
            return string(&out->text);
        }
        if (c == 't') {
            out->kind = JsonValue::Bool;
            out->boolean = true;
            return literal("true");
        }
        if (c == 'f') {
            out->kind = JsonValue::Bool;
            out->boolean = false;
            return literal("false");
        }
        if (c == 'n') {
            out->kind = JsonValue::Null;
            return literal("null");
        }
        return number(out);
    }
};

// ---- checkpoint -----------------------------------------------------------------------

struct DtypeName {
    const char* name;
    qsfi_dtype dtype;
    uint32_t bytes;
};
// safetensors dtype spellings; element sizes in bytes.
const DtypeName kDtypes[] = {
    { "F64", QSFI_DTYPE_INVALID, 8 },  { "F32", QSFI_DTYPE_F32, 4 },       { "F16", QSFI_DTYPE_F16, 2 },
    { "BF16", QSFI_DTYPE_BF16, 2 },    { "I64", QSFI_DTYPE_INVALID, 8 },   { "I32", QSFI_DTYPE_I32, 4 },
    { "I16", QSFI_DTYPE_INVALID, 2 },  { "I8", QSFI_DTYPE_I8, 1 },         { "U8", QSFI_DTYPE_U8, 1 },
    { "U16", QSFI_DTYPE_INVALID, 2 },  { "U32", QSFI_DTYPE_U32, 4 },       { "U64", QSFI_DTYPE_INVALID, 8 },
    { "BOOL", QSFI_DTYPE_INVALID, 1 }, { "F8_E4M3", QSFI_DTYPE_FP8_E4M3, 1 }, { "F8_E5M2", QSFI_DTYPE_FP8_E5M2, 1 },
};

struct TensorEntry {
    std::string name;
    uint32_t shard = 0;
    const DtypeName* dtype = nullptr;
    std::vector<int64_t> shape;
    uint64_t offset = 0; // absolute, inside the shard file
    uint64_t bytes = 0;
};

struct Shard {
    std::string path;
    int fd = -1;
    uint64_t size = 0;
};

} // namespace ckpt
} // namespace qs3

struct qs3_checkpoint {
    std::string directory;
    std::vector<qs3::ckpt::Shard> shards;
    std::vector<qs3::ckpt::TensorEntry> tensors; // sorted by name
    bool has_config = false;
    qs3::ckpt::JsonValue config;

    ~qs3_checkpoint()
    {
        for (auto& s : shards)
            if (s.fd >= 0)
                ::close(s.fd);
    }
    const qs3::ckpt::TensorEntry* find(const std::string& name) const
    {
        auto it = std::lower_bound(tensors.begin(), tensors.end(), name,
                                   [](const qs3::ckpt::TensorEntry& t, const std::string& n) { return t.name < n; });
        return it != tensors.end() && it->name == name ? &*it : nullptr;
    }
};

namespace qs3 {
namespace {
using namespace ckpt;

bool read_file(const std::string& path, std::string* out, std::string* error)
{
    const int fd = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
    if (fd < 0) {
        *error = "cannot open " + path + ": " + std::strerror(errno);
        return false;
    }
    struct stat st {};
    if (::fstat(fd, &st) != 0 || st.st_size < 0 || st.st_size > (64ll << 20)) {
        ::close(fd);
        *error = "cannot read " + path + " (missing, or larger than 64 MiB)";
        return false;
    }
    out->resize(static_cast<size_t>(st.st_size));
    size_t done = 0;
    while (done < out->size()) {
        const ssize_t n = ::pread(fd, &(*out)[done], out->size() - done, static_cast<off_t>(done));
        if (n <= 0) {
            ::close(fd);
            *error = "short read on " + path;
            return false;
        }
        done += static_cast<size_t>(n);
    }
    ::close(fd);
    return true;
}

bool file_exists(const std::string& path)
{
    struct stat st {};
    return ::stat(path.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}

// Reads exactly `bytes` bytes at `offset` of a shard; false on a short read or an I/O error.
bool pread_exact(int fd, void* dst, uint64_t bytes, uint64_t offset)
{
    uint64_t done = 0;
    while (done < bytes) {
        const ssize_t n = ::pread(fd, static_cast<char*>(dst) + done, bytes - done, static_cast<off_t>(offset + done));
        if (n < 0 && errno == EINTR)
            continue;
        if (n <= 0)
            return false;
        done += static_cast<uint64_t>(n);
    }
    return true;
}

// Parses and checks the header of one shard, appending its tensors to `out`.
bool parse_shard(uint32_t shard_index, Shard* shard, std::vector<TensorEntry>* out, std::string* error)
{
    const std::string& path = shard->path;
    shard->fd = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
    if (shard->fd < 0) {
        *error = "cannot open shard " + path + ": " + std::strerror(errno);
        return false;
    }
    struct stat st {};
    if (::fstat(shard->fd, &st) != 0 || st.st_size < 8) {
        *error = "shard " + path + " is shorter than a safetensors header";
        return false;
    }
    shard->size = static_cast<uint64_t>(st.st_size);
    unsigned char len8[8];
    if (!pread_exact(shard->fd, len8, 8, 0)) {
        *error = "cannot read the header length of " + path;
        return false;
    }
    uint64_t header_len = 0;
    for (int i = 7; i >= 0; --i)
        header_len = (header_len << 8) | len8[i];
    if (header_len < 2 || header_len > shard->size - 8 || header_len > (256ull << 20)) {
        *error = "shard " + path + ": header length " + std::to_string(header_len) + " is outside the file";
        return false;
    }
    std::string header(header_len, '\0');
    if (!pread_exact(shard->fd, &header[0], header_len, 8)) {
        *error = "cannot read the header of " + path;
        return false;
    }
    JsonValue root;
    std::string jerr;
    if (!JsonParser(header.data(), header.size()).parse(&root, &jerr) || root.kind != JsonValue::Object) {
        *error = "shard " + path + ": header is not a JSON object: " + jerr;
        return false;
    }
    const uint64_t data_begin = 8 + header_len;
    const uint64_t data_size = shard->size - data_begin;
    std::vector<std::pair<uint64_t, uint64_t>> ranges; // [begin, end) with end > begin
    for (const auto& m : root.members) {
        if (m.first == "__metadata__")
            continue;
        const JsonValue& v = m.second;
        const JsonValue* dt = v.get("dtype");
        const JsonValue* sh = v.get("shape");
        const JsonValue* off = v.get("data_offsets");
        if (v.kind != JsonValue::Object || !dt || dt->kind != JsonValue::String || !sh || sh->kind != JsonValue::Array
            || !off || off->kind != JsonValue::Array || off->items.size() != 2) {
            *error = "shard " + path + ": malformed entry for tensor " + m.first;
            return false;
        }
        TensorEntry t;
        t.name = m.first;
        t.shard = shard_index;
        for (const DtypeName& d : kDtypes)
            if (dt->text == d.name)
                t.dtype = &d;
        if (t.dtype == nullptr) {
            *error = "shard " + path + ": tensor " + m.first + " has unknown dtype " + dt->text;
            return false;
        }
        if (sh->items.size() > QS3_CHECKPOINT_MAX_RANK) {
            *error = "shard " + path + ": tensor " + m.first + " has more than 8 dimensions";
            return false;
        }
        uint64_t count = 1;
        for (const JsonValue& dim : sh->items) {
            if (dim.kind != JsonValue::Number || !dim.integral || dim.integer < 0) {
                *error = "shard " + path + ": tensor " + m.first + " has a malformed shape";
                return false;
            }
            const uint64_t d = static_cast<uint64_t>(dim.integer);
            if (d != 0 && count > (1ull << 62) / d) {
                *error = "shard " + path + ": tensor " + m.first + " shape overflows";
                return false;
            }
            count *= d;
            t.shape.push_back(dim.integer);
        }
        const JsonValue& b = off->items[0];
        const JsonValue& e = off->items[1];
        if (b.kind != JsonValue::Number || e.kind != JsonValue::Number || !b.integral || !e.integral || b.integer < 0
            || e.integer < b.integer) {
            *error = "shard " + path + ": tensor " + m.first + " has malformed data_offsets";
            return false;
        }
        const uint64_t begin = static_cast<uint64_t>(b.integer), end = static_cast<uint64_t>(e.integer);
        if (end > data_size) {
            *error = "shard " + path + ": tensor " + m.first + " byte range [" + std::to_string(begin) + ", "
                + std::to_string(end) + ") is out of range (data section has " + std::to_string(data_size) + " bytes)";
            return false;
        }
        if (end - begin != count * t.dtype->bytes) {
            *error = "shard " + path + ": tensor " + m.first + " byte range holds " + std::to_string(end - begin)
                + " bytes but shape and dtype need " + std::to_string(count * t.dtype->bytes);
            return false;
        }
        t.offset = data_begin + begin;
        t.bytes = end - begin;
        out->push_back(std::move(t));
        if (end > begin)
            ranges.emplace_back(begin, end);
    }
    // no name twice in one header (the JSON reader keeps duplicate keys)
    std::vector<const std::string*> names;
    for (const auto& m : root.members)
        names.push_back(&m.first);
    std::sort(names.begin(), names.end(), [](const std::string* a, const std::string* b) { return *a < *b; });
    for (size_t i = 1; i < names.size(); ++i) {
        if (*names[i] == *names[i - 1]) {
            *error = "shard " + path + ": duplicate tensor " + *names[i];
            return false;
        }
    }
    // pairwise disjoint byte ranges: sort by begin, each must start at or after the previous end
    std::vector<size_t> order(ranges.size());
    for (size_t i = 0; i < order.size(); ++i)
        order[i] = i;
    std::sort(order.begin(), order.end(), [&](size_t a, size_t b) { return ranges[a] < ranges[b]; });
    for (size_t i = 1; i < order.size(); ++i) {
        if (ranges[order[i]].first < ranges[order[i - 1]].second) {
            *error = "shard " + path + ": byte ranges of two tensors overlap at offset "
                + std::to_string(ranges[order[i]].first);
            return false;
        }
    }
    return true;
}

// Builds the checkpoint object of a directory; every check of the open call lives here.
bool open_checkpoint(const std::string& directory, qs3_checkpoint* ck, std::string* error)
{
    ck->directory = directory;
    const std::string index_path = directory + "/model.safetensors.index.json";
    std::map<std::string, std::string> weight_map; // tensor -> shard file name
    std::vector<std::string> shard_files;
    const bool has_index = file_exists(index_path);
    if (has_index) {
        std::string text, jerr;
        JsonValue root;
        if (!read_file(index_path, &text, error))
            return false;
        if (!JsonParser(text.data(), text.size()).parse(&root, &jerr)) {
            *error = "index " + index_path + " is not valid JSON: " + jerr;
            return false;
        }
        const JsonValue* wm = root.get("weight_map");
        if (wm == nullptr || wm->kind != JsonValue::Object) {
            *error = "index " + index_path + " has no weight_map object";
            return false;
        }
        for (const auto& m : wm->members) {
            if (m.second.kind != JsonValue::String || m.second.text.empty()
                || m.second.text.find('/') != std::string::npos) {
                *error = "index: weight_map entry of " + m.first + " is not a plain file name";
                return false;
            }
            if (!weight_map.emplace(m.first, m.second.text).second) {
                *error = "index: duplicate tensor " + m.first;
                return false;
            }
            if (std::find(shard_files.begin(), shard_files.end(), m.second.text) == shard_files.end())
                shard_files.push_back(m.second.text);
        }
    } else {
        DIR* dir = ::opendir(directory.c_str());
        if (dir == nullptr) {
            *error = "cannot open checkpoint directory " + directory + ": " + std::strerror(errno);
            return false;
        }
        const std::string suffix = ".safetensors";
        while (const dirent* ent = ::readdir(dir)) {
            const std::string name = ent->d_name;
            if (name.size() > suffix.size() && name.compare(name.size() - suffix.size(), suffix.size(), suffix) == 0)
                shard_files.push_back(name);
        }
        ::closedir(dir);
    }
    if (shard_files.empty()) {
        *error = "no safetensors shard in " + directory;
        return false;
    }
    std::sort(shard_files.begin(), shard_files.end());
    ck->shards.resize(shard_files.size());
    for (size_t i = 0; i < shard_files.size(); ++i) {
        ck->shards[i].path = directory + "/" + shard_files[i];
        if (!parse_shard(static_cast<uint32_t>(i), &ck->shards[i], &ck->tensors, error))
            return false;
    }
    std::sort(ck->tensors.begin(), ck->tensors.end(),
              [](const TensorEntry& a, const TensorEntry& b) { return a.name < b.name; });
    for (size_t i = 1; i < ck->tensors.size(); ++i) {
        if (ck->tensors[i].name == ck->tensors[i - 1].name) {
            *error = "duplicate tensor " + ck->tensors[i].name + " (" + ck->shards[ck->tensors[i - 1].shard].path
                + " and " + ck->shards[ck->tensors[i].shard].path + ")";
            return false;
        }
    }
    if (has_index) {
        for (const auto& m : weight_map) {
            const TensorEntry* t = ck->find(m.first);
            if (t == nullptr || ck->shards[t->shard].path != directory + "/" + m.second) {
                *error = "missing tensor " + m.first + ": the index places it in " + m.second;
                return false;
            }
        }
        for (const TensorEntry& t : ck->tensors) {
            if (weight_map.find(t.name) == weight_map.end()) {
                *error = "unexpected tensor " + t.name + " in " + ck->shards[t.shard].path + ": not in the index";
                return false;
            }
        }
    }
    const std::string config_path = directory + "/config.json";
    if (file_exists(config_path)) {
        std::string text, jerr;
        if (!read_file(config_path, &text, error))
            return false;
        if (!JsonParser(text.data(), text.size()).parse(&ck->config, &jerr) || ck->config.kind != JsonValue::Object) {
            *error = "config.json is not a JSON object: " + jerr;
            return false;
        }
        ck->has_config = true;
    }
    return true;
}

void fill_info(const qs3_checkpoint* ck, const TensorEntry& t, qs3_checkpoint_tensor_info* out)
{
    std::memset(out, 0, sizeof(*out));
    out->name = t.name.c_str();
    out->file = ck->shards[t.shard].path.c_str();
    out->dtype_name = t.dtype->name;
    out->dtype = t.dtype->dtype;
    out->element_bytes = t.dtype->bytes;
    out->rank = static_cast<uint32_t>(t.shape.size());
    for (size_t i = 0; i < t.shape.size(); ++i)
        out->shape[i] = t.shape[i];
    out->file_offset = t.offset;
    out->bytes = t.bytes;
}

// config.json lookup: top level first, then "text_config".
const JsonValue* config_value(const qs3_checkpoint* ck, const char* key)
{
    if (const JsonValue* v = ck->config.get(key))
        return v;
    if (const JsonValue* text = ck->config.get("text_config"))
        return text->get(key);
    return nullptr;
}

bool config_u32(const qs3_checkpoint* ck, const char* key, bool required, uint32_t fallback, uint32_t* out,
                std::string* error)
{
    const JsonValue* v = config_value(ck, key);
    if (v == nullptr || v->kind == JsonValue::Null) {
        if (required) {
            *error = std::string("config.json has no ") + key;
            return false;
        }
        *out = fallback;
        return true;
    }
    if (v->kind == JsonValue::Bool) {
        *out = v->boolean ? 1u : 0u;
        return true;
    }
    if (v->kind != JsonValue::Number || !v->integral || v->integer < 0 || v->integer > 0xffffffffll) {
        *error = std::string("config.json: ") + key + " is not an unsigned 32-bit integer";
        return false;
    }
    *out = static_cast<uint32_t>(v->integer);
    return true;
}

} // namespace
} // namespace qs3

extern "C" {

qsfi_status qs3_checkpoint_open(qsfi_context* ctx, const char* directory, qs3_checkpoint** out)
{
    if (ctx == nullptr || out == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    qs3::clear_error(&ctx->last_error);
    *out = nullptr;
    if (directory == nullptr || directory[0] == '\0')
        return qs3::set_invalid_arg(ctx, "checkpoint directory is empty");
    try {
        std::unique_ptr<qs3_checkpoint> ck(new qs3_checkpoint());
        std::string error;
        std::string dir = directory;
        while (dir.size() > 1 && dir.back() == '/')
            dir.pop_back();
        if (!qs3::open_checkpoint(dir, ck.get(), &error))
            return qs3::set_invalid_arg(ctx, "checkpoint: %s", error.c_str());
        *out = ck.release();
        return QSFI_STATUS_OK;
    } catch (const std::exception& e) {
        return qs3::set_error(ctx, QSFI_STATUS_BACKEND_ERROR, QSFI_ERROR_SOURCE_QSFI, 0, "checkpoint open failed: %s",
                              e.what());
    }
}

void qs3_checkpoint_close(qs3_checkpoint* checkpoint) { delete checkpoint; }

uint64_t qs3_checkpoint_num_tensors(const qs3_checkpoint* checkpoint)
{
    return checkpoint == nullptr ? 0 : checkpoint->tensors.size();
}

qsfi_status qs3_checkpoint_tensor_at(qsfi_context* ctx, const qs3_checkpoint* checkpoint, uint64_t index,
                                     qs3_checkpoint_tensor_info* out)
{
    if (ctx == nullptr || out == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    qs3::clear_error(&ctx->last_error);
    if (checkpoint == nullptr || index >= checkpoint->tensors.size())
        return qs3::set_invalid_arg(ctx, "checkpoint tensor index out of range");
    qs3::fill_info(checkpoint, checkpoint->tensors[index], out);
    return QSFI_STATUS_OK;
}

qsfi_status qs3_checkpoint_find(qsfi_context* ctx, const qs3_checkpoint* checkpoint, const char* name,
                                qs3_checkpoint_tensor_info* out)
{
    if (ctx == nullptr || out == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    qs3::clear_error(&ctx->last_error);
    if (checkpoint == nullptr || name == nullptr)
        return qs3::set_invalid_arg(ctx, "checkpoint and tensor name are required");
    const qs3::ckpt::TensorEntry* t = checkpoint->find(name);
    if (t == nullptr)
        return qs3::set_invalid_arg(ctx, "checkpoint: missing tensor %s", name);
    qs3::fill_info(checkpoint, *t, out);
    return QSFI_STATUS_OK;
}

qsfi_status qs3_checkpoint_read_host(qsfi_context* ctx, const qs3_checkpoint* checkpoint, const char* name, void* dst,
                                     uint64_t dst_bytes)
{
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    qs3::clear_error(&ctx->last_error);
    if (checkpoint == nullptr || name == nullptr || (dst == nullptr && dst_bytes != 0))
        return qs3::set_invalid_arg(ctx, "checkpoint, tensor name and destination are required");
    const qs3::ckpt::TensorEntry* t = checkpoint->find(name);
    if (t == nullptr)
        return qs3::set_invalid_arg(ctx, "checkpoint: missing tensor %s", name);
    if (t->bytes != dst_bytes)
        return qs3::set_invalid_arg(ctx, "checkpoint: tensor %s has %llu bytes, destination %llu", name,
                                    static_cast<unsigned long long>(t->bytes),
                                    static_cast<unsigned long long>(dst_bytes));
    if (!qs3::pread_exact(checkpoint->shards[t->shard].fd, dst, t->bytes, t->offset))
        return qs3::set_error(ctx, QSFI_STATUS_BACKEND_ERROR, QSFI_ERROR_SOURCE_QSFI, errno,
                              "checkpoint: short read of tensor %s", name);
    return QSFI_STATUS_OK;
}

qsfi_status qs3_checkpoint_read_moe_config(qsfi_context* ctx, const qs3_checkpoint* checkpoint,
                                           qs3_checkpoint_moe_config* out)
{
    if (ctx == nullptr || out == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    qs3::clear_error(&ctx->last_error);
    if (checkpoint == nullptr || !checkpoint->has_config)
        return qs3::set_invalid_arg(ctx, "checkpoint has no config.json");
    std::memset(out, 0, sizeof(*out));
    std::string error;
    bool ok = qs3::config_u32(checkpoint, "hidden_size", true, 0, &out->hidden_size, &error)
        && qs3::config_u32(checkpoint, "moe_intermediate_size", true, 0, &out->intermediate_size, &error)
        && qs3::config_u32(checkpoint, "num_experts", true, 0, &out->num_experts, &error)
        && qs3::config_u32(checkpoint, "num_experts_per_tok", true, 0, &out->top_k, &error)
        && qs3::config_u32(checkpoint, "shared_expert_intermediate_size", false, 0, &out->shared_intermediate_size,
                           &error)
        && qs3::config_u32(checkpoint, "num_hidden_layers", true, 0, &out->num_layers, &error)
        && qs3::config_u32(checkpoint, "norm_topk_prob", false, 1, &out->renormalize, &error);
    if (!ok)
        return qs3::set_invalid_arg(ctx, "checkpoint: %s", error.c_str());
    out->rms_norm_eps = 1e-6f;
    if (const qs3::ckpt::JsonValue* v = qs3::config_value(checkpoint, "rms_norm_eps")) {
        if (v->kind != qs3::ckpt::JsonValue::Number || !(v->number > 0.0))
            return qs3::set_invalid_arg(ctx, "checkpoint: config.json: rms_norm_eps is not a positive number");
        out->rms_norm_eps = static_cast<float>(v->number);
    }
    return QSFI_STATUS_OK;
}

} // extern "C"

// ---- layer manifest ---------------------------------------------------------------------
namespace qs3 {
namespace {
using namespace ckpt;

// One NVFP4-quantised projection of a checkpoint (four tensors), or a bf16 one (weight only).
struct Projection {
    const TensorEntry* weight = nullptr;
    const TensorEntry* scale = nullptr;       // weight_scale, e4m3 [rows, k / 16]
    const TensorEntry* scale2 = nullptr;      // weight_scale_2, f32 scalar
    const TensorEntry* input_scale = nullptr; // f32 scalar
};

// Bump allocator over the caller's device block; with a null base it only measures.
class DeviceArena {
public:
    DeviceArena(void* base, size_t capacity) : base_(static_cast<char*>(base)), capacity_(capacity) {}
    // Returns the offset of a 256-byte aligned span of `bytes` bytes.
    size_t take(size_t bytes)
    {
        const size_t at = align_up(used_, kWorkspaceAlign);
        used_ = at + bytes;
        return at;
    }
    char* at(size_t offset) const { return base_ == nullptr ? nullptr : base_ + offset; }
    size_t used() const { return used_; }
    bool contains(size_t offset, size_t bytes) const { return offset <= capacity_ && bytes <= capacity_ - offset; }

private:
    char* base_;
    size_t capacity_;
    size_t used_ = 0;
};

struct LayerManifest {
    const TensorEntry* router = nullptr;
    const TensorEntry* shared_gate = nullptr;
    // BF16_FUSED
    const TensorEntry* gate_up_fused = nullptr;
    const TensorEntry* down_fused = nullptr;
    bool gate_up_transposed = false, down_transposed = false;
    // NVFP4_SPLIT, indexed by checkpoint expert id
    std::vector<Projection> gate, up, down;
    // shared expert (weights bf16, or NVFP4 when `shared_nvfp4`)
    bool shared_nvfp4 = false;
    Projection sh_gate, sh_up, sh_down;
    // device plan (offsets into the weight block / the scratch block)
    uint32_t chunk = 0; // experts staged per half of the scratch block
    size_t router_off = 0, gu_off = 0, gu_sf_off = 0, gu_g_off = 0, d_off = 0, d_sf_off = 0, d_g_off = 0;
    size_t sgu_off = 0, sgu_sf_off = 0, sgu_g_off = 0, sd_off = 0, sd_sf_off = 0, sd_g_off = 0, sgate_off = 0;
    size_t weight_bytes = 0;
    size_t half_bytes = 0;        // one staging half for the routed experts
    size_t half_a = 0, half_b = 0; // within a half: gate_up staging, down staging (then transposed copies)
    size_t half_at = 0, half_bt = 0;
    size_t shared_scratch_off = 0; // after the two halves
    size_t scratch_bytes = 0;
};

bool shape_is(const TensorEntry* t, std::initializer_list<int64_t> want)
{
    return t->shape.size() == want.size() && std::equal(want.begin(), want.end(), t->shape.begin());
}

bool is_scalar(const TensorEntry* t)
{
    return t->shape.empty() || (t->shape.size() == 1 && t->shape[0] == 1);
}

std::string shape_text(const std::vector<int64_t>& shape)
{
    std::string s = "[";
    for (size_t i = 0; i < shape.size(); ++i)
        s += (i ? ", " : "") + std::to_string(shape[i]);
    return s + "]";
}

// Collects the expected tensors of a layer; every lookup records its name so that the
// "unexpected tensor" pass can tell what belongs to the layer.
class ManifestBuilder {
public:
    ManifestBuilder(const qs3_checkpoint* ck, std::string prefix) : ck_(ck), prefix_(std::move(prefix)) {}

    // Tensor <prefix><suffix> with the given dtype; shape checked by the caller.
    const TensorEntry* need(const std::string& suffix, const char* dtype)
    {
        const std::string name = prefix_ + suffix;
        expected_.push_back(name);
        const TensorEntry* t = ck_->find(name);
        if (t == nullptr) {
            fail("missing tensor " + name);
            return nullptr;
        }
        if (std::strcmp(t->dtype->name, dtype) != 0) {
            fail("tensor " + name + " has dtype " + t->dtype->name + ", expected " + dtype);
            return nullptr;
        }
        return t;
    }
    bool has(const std::string& suffix) const { return ck_->find(prefix_ + suffix) != nullptr; }
    void want_shape(const TensorEntry* t, std::initializer_list<int64_t> want)
    {
        if (t != nullptr && !shape_is(t, want))
            fail("tensor " + t->name + " has shape " + shape_text(t->shape) + ", expected "
                 + shape_text(std::vector<int64_t>(want)));
    }
    void want_scalar(const TensorEntry* t)
    {
        if (t != nullptr && !is_scalar(t))
            fail("tensor " + t->name + " has shape " + shape_text(t->shape) + ", expected a scalar");
    }
    // The four tensors of an NVFP4 projection <stem>.{weight, weight_scale, weight_scale_2, input_scale}.
    Projection nvfp4(const std::string& stem, int64_t rows, int64_t k)
    {
        Projection p;
        p.weight = need(stem + ".weight", "U8");
        want_shape(p.weight, { rows, k / 2 });
        p.scale = need(stem + ".weight_scale", "F8_E4M3");
        want_shape(p.scale, { rows, k / 16 });
        p.scale2 = need(stem + ".weight_scale_2", "F32");
        want_scalar(p.scale2);
        p.input_scale = need(stem + ".input_scale", "F32");
        want_scalar(p.input_scale);
        return p;
    }
    // Every tensor of the checkpoint under the prefix must have been asked for.
    void reject_unexpected()
    {
        std::sort(expected_.begin(), expected_.end());
        auto it = std::lower_bound(ck_->tensors.begin(), ck_->tensors.end(), prefix_,
                                   [](const TensorEntry& t, const std::string& n) { return t.name < n; });
        for (; it != ck_->tensors.end() && it->name.compare(0, prefix_.size(), prefix_) == 0; ++it)
            if (!std::binary_search(expected_.begin(), expected_.end(), it->name))
                fail("unexpected tensor " + it->name);
    }
    void fail(const std::string& what)
    {
        if (error_.empty())
            error_ = what;
    }
    const std::string& error() const { return error_; }

private:
    const qs3_checkpoint* ck_;
    std::string prefix_;
    std::vector<std::string> expected_;
    std::string error_;
};

// Validates descriptor and checkpoint and plans the device buffers. No CUDA call.
bool build_manifest(const qs3_checkpoint* ck, const qs3_moe_layer_load_desc& d, LayerManifest* m, std::string* error)
{
    const int64_t h = d.hidden_size, i = d.intermediate_size, e = d.num_experts, is = d.shared_intermediate_size;
    const bool to_nvfp4 = d.backend == QSFI_MOE_BACKEND_FLASHINFER_NVFP4;
    const bool split = d.format == QS3_CHECKPOINT_EXPERTS_NVFP4_SPLIT;
    if (d.layer_prefix == nullptr || h == 0 || i == 0 || e == 0 || d.local_num_experts == 0
        || static_cast<uint64_t>(d.local_expert_offset) + d.local_num_experts > d.num_experts) {
        *error = "invalid layer dimensions or local expert range";
        return false;
    }
    if (d.backend != QSFI_MOE_BACKEND_FLASHINFER_STAGED_BF16 && d.backend != QSFI_MOE_BACKEND_FLASHINFER_FUSED_BF16
        && !to_nvfp4) {
        *error = "the loader produces BF16 or NVFP4 layouts only";
        return false;
    }
    if (d.format != QS3_CHECKPOINT_EXPERTS_BF16_FUSED && !split) {
        *error = "unknown checkpoint expert format";
        return false;
    }
    if (split && !to_nvfp4) {
        *error = "an NVFP4 checkpoint cannot be loaded into a BF16 plan";
        return false;
    }
    if (h % 8 != 0 || i % 8 != 0 || is % 8 != 0 || (to_nvfp4 && (h % 64 != 0 || i % 64 != 0 || is % 64 != 0))) {
        *error = "hidden and intermediate sizes must be multiples of 8 (64 for NVFP4)";
        return false;
    }
    if (d.expert_order != nullptr) {
        std::vector<char> seen(d.num_experts, 0);
        for (uint32_t p = 0; p < d.num_experts; ++p) {
            if (d.expert_order[p] >= d.num_experts || seen[d.expert_order[p]]) {
                *error = "expert_order is not a permutation of the expert ids";
                return false;
            }
            seen[d.expert_order[p]] = 1;
        }
    }
    ManifestBuilder b(ck, d.layer_prefix);
    m->router = b.need("gate.weight", "BF16");
    b.want_shape(m->router, { e, h });
    if (split) {
        m->gate.resize(e);
        m->up.resize(e);
        m->down.resize(e);
        for (int64_t x = 0; x < e; ++x) {
            const std::string stem = "experts." + std::to_string(x) + ".";
            m->gate[x] = b.nvfp4(stem + "gate_proj", i, h);
            m->up[x] = b.nvfp4(stem + "up_proj", i, h);
            m->down[x] = b.nvfp4(stem + "down_proj", h, i);
        }
    } else {
        m->gate_up_fused = b.need("experts.gate_up_proj", "BF16");
        m->down_fused = b.need("experts.down_proj", "BF16");
        if (m->gate_up_fused != nullptr) {
            const bool plain = shape_is(m->gate_up_fused, { e, 2 * i, h });
            const bool transposed = shape_is(m->gate_up_fused, { e, h, 2 * i });
            if (!plain && !transposed)
                b.want_shape(m->gate_up_fused, { e, 2 * i, h });
            m->gate_up_transposed = plain && transposed ? d.fused_transposed != 0 : transposed;
        }
        if (m->down_fused != nullptr) {
            const bool plain = shape_is(m->down_fused, { e, h, i });
            const bool transposed = shape_is(m->down_fused, { e, i, h });
            if (!plain && !transposed)
                b.want_shape(m->down_fused, { e, h, i });
            m->down_transposed = plain && transposed ? d.fused_transposed != 0 : transposed;
        }
    }
    if (is != 0) {
        m->shared_nvfp4 = split && b.has("shared_expert.gate_proj.weight_scale");
        if (m->shared_nvfp4) {
            m->sh_gate = b.nvfp4("shared_expert.gate_proj", is, h);
            m->sh_up = b.nvfp4("shared_expert.up_proj", is, h);
            m->sh_down = b.nvfp4("shared_expert.down_proj", h, is);
        } else {
            m->sh_gate.weight = b.need("shared_expert.gate_proj.weight", "BF16");
            b.want_shape(m->sh_gate.weight, { is, h });
            m->sh_up.weight = b.need("shared_expert.up_proj.weight", "BF16");
            b.want_shape(m->sh_up.weight, { is, h });
            m->sh_down.weight = b.need("shared_expert.down_proj.weight", "BF16");
            b.want_shape(m->sh_down.weight, { h, is });
        }
        m->shared_gate = b.need("shared_expert_gate.weight", "BF16");
        b.want_shape(m->shared_gate, { 1, h });
    }
    b.reject_unexpected();
    if (!b.error().empty()) {
        *error = b.error();
        return false;
    }

    // ---- device plan: the kept tensors ----
    const size_t el = d.local_num_experts;
    const size_t kdiv = to_nvfp4 ? 2 : 1, elem = to_nvfp4 ? 1 : 2;
    DeviceArena w(nullptr, 0);
    m->router_off = w.take(static_cast<size_t>(e) * h * 2);
    m->gu_off = w.take(el * 2 * i * (h / kdiv) * elem);
    m->d_off = w.take(el * h * (i / kdiv) * elem);
    if (to_nvfp4) {
        m->gu_sf_off = w.take(el * qs3_nvfp4_tiled_scale_bytes(2 * i, h));
        m->d_sf_off = w.take(el * qs3_nvfp4_tiled_scale_bytes(h, i));
        m->gu_g_off = w.take(2 * el * sizeof(float));
        m->d_g_off = w.take(el * sizeof(float));
    }
    if (is != 0) {
        m->sgu_off = w.take(static_cast<size_t>(2) * is * (h / kdiv) * elem);
        m->sd_off = w.take(static_cast<size_t>(h) * (is / kdiv) * elem);
        if (to_nvfp4) {
            m->sgu_sf_off = w.take(qs3_nvfp4_tiled_scale_bytes(2 * is, h));
            m->sd_sf_off = w.take(qs3_nvfp4_tiled_scale_bytes(h, is));
            m->sgu_g_off = w.take(2 * sizeof(float));
            m->sd_g_off = w.take(sizeof(float));
        }
        m->sgate_off = w.take(static_cast<size_t>(h) * 2);
    }
    m->weight_bytes = align_up(w.used(), kWorkspaceAlign);

    // ---- device plan: load-time staging ----
    // Two halves, each staging `chunk` experts, so that the copies of one chunk overlap the
    // device pass over the previous one; a region for the shared expert follows.
    m->chunk = static_cast<uint32_t>(std::min<size_t>(el, 8));
    DeviceArena half(nullptr, 0);
    const size_t c = m->chunk;
    if (split) { // linear block scales, re-tiled on the device
        m->half_a = half.take(c * 2 * i * (h / 16));
        m->half_b = half.take(c * h * (i / 16));
    } else if (to_nvfp4 || m->gate_up_transposed || m->down_transposed) {
        if (to_nvfp4 || m->gate_up_transposed)
            m->half_a = half.take(c * 2 * i * h * 2);
        if (to_nvfp4 || m->down_transposed)
            m->half_b = half.take(c * h * i * 2);
        if (to_nvfp4 && m->gate_up_transposed)
            m->half_at = half.take(c * 2 * i * h * 2);
        if (to_nvfp4 && m->down_transposed)
            m->half_bt = half.take(c * h * i * 2);
    }
    m->half_bytes = align_up(half.used(), kWorkspaceAlign);
    DeviceArena s(nullptr, 0);
    s.take(2 * m->half_bytes);
    m->shared_scratch_off = align_up(s.used(), kWorkspaceAlign);
    if (is != 0 && to_nvfp4) {
        if (m->shared_nvfp4)
            s.take(static_cast<size_t>(2) * is * (h / 16) + kWorkspaceAlign + static_cast<size_t>(h) * (is / 16));
        else
            s.take(static_cast<size_t>(2) * is * h * 2 + kWorkspaceAlign + static_cast<size_t>(h) * is * 2);
    }
    m->scratch_bytes = align_up(s.used(), kWorkspaceAlign);
    return true;
}

// ---- upload backend -----------------------------------------------------------------------

// Destination of a load: a span of the caller's device block (upstream WeightLoadSpan,
// src/weight_loader.rs:54-59, memory kind Device).
struct WeightLoadSpan {
    char* ptr = nullptr;
    size_t bytes = 0;
};

// Source of a load: a byte range of an open shard (upstream WeightFileRange,
// src/weight_loader.rs:61-66).
struct WeightFileRange {
    int fd = -1;
    uint64_t offset = 0;
    size_t bytes = 0;
};

// The dGPU implementation upstream describes (src/weight_loader.rs:22-24): final weights in
// device memory, a small ring of pinned host buffers, pread into a free buffer,
// cudaMemcpyAsync from it on a copy stream, one event per buffer for its reuse.
class PinnedUploadBackend {
public:
    static constexpr int kSlots = 4;
    static constexpr size_t kSlotBytes = 8u << 20;

    PinnedUploadBackend(void* block, size_t bytes) : arena_(block, bytes) {}
    PinnedUploadBackend(const PinnedUploadBackend&) = delete;
    PinnedUploadBackend& operator=(const PinnedUploadBackend&) = delete;
    ~PinnedUploadBackend()
    {
        if (stream_ != nullptr)
            cudaStreamSynchronize(stream_);
        for (int s = 0; s < kSlots; ++s)
            if (slot_free_[s] != nullptr)
                cudaEventDestroy(slot_free_[s]);
        if (sealed_ != nullptr)
            cudaEventDestroy(sealed_);
        if (ring_ != nullptr)
            cudaFreeHost(ring_);
        if (stream_ != nullptr)
            cudaStreamDestroy(stream_);
    }

    cudaError_t init()
    {
        cudaError_t err = cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking);
        if (err == cudaSuccess)
            err = cudaHostAlloc(&ring_, kSlots * kSlotBytes, cudaHostAllocDefault);
        for (int s = 0; s < kSlots && err == cudaSuccess; ++s)
            err = cudaEventCreateWithFlags(&slot_free_[s], cudaEventDisableTiming);
        if (err == cudaSuccess)
            err = cudaEventCreateWithFlags(&sealed_, cudaEventDisableTiming);
        return err;
    }

    // alloc_tensor: the span of the device block at an offset the sizing pass
    // (build_manifest) planned; every planned offset is 256-byte aligned.
    WeightLoadSpan alloc_tensor(size_t offset, size_t bytes)
    {
        WeightLoadSpan span;
        if (!arena_.contains(offset, bytes)) {
            fail(cudaSuccess, "alloc_tensor: span outside the device block"); // reads into it then fail too
            return span;
        }
        span.ptr = arena_.at(offset);
        span.bytes = bytes;
        return span;
    }

    // read_exact: file range -> device span (at `dst_offset` inside it), piecewise through the ring.
    bool read_exact(const WeightFileRange& src, const WeightLoadSpan& dst, size_t dst_offset = 0)
    {
        if (dst_offset + src.bytes > dst.bytes)
            return fail(cudaSuccess, "read_exact: destination span too small");
        size_t done = 0;
        while (done < src.bytes) {
            const size_t n = std::min(kSlotBytes, src.bytes - done);
            char* host = acquire_slot();
            if (host == nullptr)
                return false;
            if (!pread_exact(src.fd, host, n, src.offset + done))
                return fail(cudaSuccess, "read_exact: short read from the shard");
            if (!release_slot(cudaMemcpyAsync(dst.ptr + dst_offset + done, host, n, cudaMemcpyHostToDevice, stream_)))
                return false;
            done += n;
        }
        return true;
    }

    // Host bytes -> device span through the ring (small tables the loader builds itself).
    bool upload(const void* src, size_t bytes, const WeightLoadSpan& dst)
    {
        if (bytes > dst.bytes || bytes > kSlotBytes)
            return fail(cudaSuccess, "upload: span too small");
        char* host = acquire_slot();
        if (host == nullptr)
            return false;
        std::memcpy(host, src, bytes);
        return release_slot(cudaMemcpyAsync(dst.ptr, host, bytes, cudaMemcpyHostToDevice, stream_));
    }

    bool zero_fill(const WeightLoadSpan& dst)
    {
        const cudaError_t err = cudaMemsetAsync(dst.ptr, 0, dst.bytes, stream_);
        return err == cudaSuccess || fail(err, "zero_fill");
    }

    // seal: everything copied so far is visible to work enqueued on `stream` afterwards, and
    // the ring is idle when this returns (the one synchronisation point of a load).
    bool seal(cudaStream_t stream)
    {
        cudaError_t err = cudaEventRecord(sealed_, stream_);
        if (err == cudaSuccess)
            err = cudaStreamWaitEvent(stream, sealed_, 0);
        if (err == cudaSuccess)
            err = cudaStreamSynchronize(stream_);
        return err == cudaSuccess || fail(err, "seal");
    }

    cudaStream_t stream() const { return stream_; }
    cudaError_t cuda_error() const { return cuda_error_; }
    const std::string& error() const { return error_; }
    bool fail(cudaError_t err, const char* what)
    {
        if (error_.empty()) {
            error_ = what;
            cuda_error_ = err;
        }
        return false;
    }

private:
    char* acquire_slot()
    {
        const int s = next_;
        if (used_[s]) { // the copy that last read this buffer must have finished
            const cudaError_t err = cudaEventSynchronize(slot_free_[s]);
            if (err != cudaSuccess) {
                fail(err, "waiting for a staging buffer");
                return nullptr;
            }
        }
        return static_cast<char*>(ring_) + static_cast<size_t>(s) * kSlotBytes;
    }
    bool release_slot(cudaError_t copy_status)
    {
        const int s = next_;
        cudaError_t err = copy_status;
        if (err == cudaSuccess)
            err = cudaEventRecord(slot_free_[s], stream_);
        if (err != cudaSuccess)
            return fail(err, "cudaMemcpyAsync from the staging ring");
        used_[s] = true;
        next_ = (next_ + 1) % kSlots;
        return true;
    }

    DeviceArena arena_;
    cudaStream_t stream_ = nullptr;
    void* ring_ = nullptr;
    cudaEvent_t slot_free_[kSlots] = {};
    cudaEvent_t sealed_ = nullptr;
    bool used_[kSlots] = {};
    int next_ = 0;
    cudaError_t cuda_error_ = cudaSuccess;
    std::string error_;
};

// [n, rows, cols] -> [n, cols, rows], bf16, through a padded 32 x 32 shared-memory tile so
// that both the reads and the writes are coalesced.
__global__ void __launch_bounds__(256)
transpose_bf16_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst, uint32_t rows,
                      uint32_t cols)
{
    __shared__ __nv_bfloat16 tile[32][33];
    const uint64_t base = static_cast<uint64_t>(blockIdx.z) * rows * cols;
    const uint32_t c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    const uint32_t tx = threadIdx.x & 31, ty = threadIdx.x >> 5; // 32 x 8
    for (uint32_t r = ty; r < 32; r += 8)
        if (r0 + r < rows && c0 + tx < cols)
            tile[r][tx] = src[base + static_cast<uint64_t>(r0 + r) * cols + c0 + tx];
    __syncthreads();
    for (uint32_t c = ty; c < 32; c += 8)
        if (c0 + c < cols && r0 + tx < rows)
            dst[base + static_cast<uint64_t>(c0 + c) * rows + r0 + tx] = tile[tx][c];
}

cudaError_t launch_transpose_bf16(const void* src, void* dst, uint32_t n, uint32_t rows, uint32_t cols,
                                  cudaStream_t stream)
{
    const dim3 grid((cols + 31) / 32, (rows + 31) / 32, n);
    transpose_bf16_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(src),
                                                    static_cast<__nv_bfloat16*>(dst), rows, cols);
    note_launch();
    return cudaGetLastError();
}

template <int N> struct TensorOf;
template <> struct TensorOf<1> { using type = qsfi_tensor1; };
template <> struct TensorOf<2> { using type = qsfi_tensor2; };
template <> struct TensorOf<3> { using type = qsfi_tensor3; };

// Contiguous view of `data` with the given shape.
template <int N> typename TensorOf<N>::type view(void* data, qsfi_dtype dtype, const int64_t (&shape)[N])
{
    typename TensorOf<N>::type t {};
    t.data = data;
    t.dtype = dtype;
    int64_t stride = 1;
    for (int i = N - 1; i >= 0; --i) {
        t.shape[i] = shape[i];
        t.stride[i] = stride;
        stride *= shape[i];
    }
    return t;
}

// ---- the load -------------------------------------------------------------------------------

class LayerLoad {
public:
    LayerLoad(qsfi_context* ctx, const qs3_checkpoint* ck, const qs3_moe_layer_load_desc& d, const LayerManifest& m,
              void* weights, size_t weight_bytes, void* scratch)
        : ctx_(ctx), ck_(ck), d_(d), m_(m), be_(weights, weight_bytes), scratch_(static_cast<char*>(scratch))
    {
    }
    ~LayerLoad()
    {
        for (cudaEvent_t ev : { copied_[0], copied_[1], consumed_[0], consumed_[1], shared_copied_ })
            if (ev != nullptr)
                cudaEventDestroy(ev);
    }

    qsfi_status run(qs3_moe_layer_weights* out)
    {
        cudaError_t err = be_.init();
        for (cudaEvent_t* ev : { &copied_[0], &copied_[1], &consumed_[0], &consumed_[1], &shared_copied_ })
            if (err == cudaSuccess)
                err = cudaEventCreateWithFlags(ev, cudaEventDisableTiming);
        // the copy stream starts after whatever the context's stream still does with these buffers
        if (err == cudaSuccess)
            err = cudaEventRecord(shared_copied_, ctx_->stream);
        if (err == cudaSuccess)
            err = cudaStreamWaitEvent(be_.stream(), shared_copied_, 0);
        if (err != cudaSuccess)
            return set_cuda_error(ctx_, err, "checkpoint loader setup");
        std::memset(out, 0, sizeof(*out));
        out->act_global_scale = 1.0f;
        out->act2_global_scale = 1.0f;
        qsfi_status status = load_router(out);
        if (status == QSFI_STATUS_OK)
            status = d_.format == QS3_CHECKPOINT_EXPERTS_NVFP4_SPLIT ? load_split_experts(out) : load_fused_experts(out);
        if (status == QSFI_STATUS_OK && d_.shared_intermediate_size != 0)
            status = load_shared(out);
        if (status == QSFI_STATUS_OK && !be_.seal(ctx_->stream))
            status = backend_error();
        return status;
    }

private:
    qsfi_context* ctx_;
    const qs3_checkpoint* ck_;
    const qs3_moe_layer_load_desc& d_;
    const LayerManifest& m_;
    PinnedUploadBackend be_;
    char* scratch_;
    cudaEvent_t copied_[2] = {}, consumed_[2] = {}, shared_copied_ = nullptr;
    bool half_used_[2] = {};
    float act_max_ = 0.0f, act2_max_ = 0.0f;

    bool nvfp4() const { return d_.backend == QSFI_MOE_BACKEND_FLASHINFER_NVFP4; }
    uint32_t expert_at(uint32_t position) const
    {
        return d_.expert_order != nullptr ? d_.expert_order[position] : position;
    }
    WeightFileRange range(const TensorEntry* t, uint64_t offset = 0, size_t bytes = SIZE_MAX) const
    {
        WeightFileRange r;
        r.fd = ck_->shards[t->shard].fd;
        r.offset = t->offset + offset;
        r.bytes = bytes == SIZE_MAX ? static_cast<size_t>(t->bytes) : bytes;
        return r;
    }
    qsfi_status backend_error()
    {
        if (be_.cuda_error() != cudaSuccess)
            return set_cuda_error(ctx_, be_.cuda_error(), be_.error().c_str());
        return set_error(ctx_, QSFI_STATUS_BACKEND_ERROR, QSFI_ERROR_SOURCE_QSFI, errno, "checkpoint loader: %s",
                         be_.error().c_str());
    }
    bool scalar(const TensorEntry* t, float* out)
    {
        return pread_exact(ck_->shards[t->shard].fd, out, sizeof(float), t->offset)
            || be_.fail(cudaSuccess, "short read of a scalar tensor");
    }
    // Copies of a staging half are done -> the context's stream may read it.
    bool publish(cudaEvent_t ev)
    {
        cudaError_t err = cudaEventRecord(ev, be_.stream());
        if (err == cudaSuccess)
            err = cudaStreamWaitEvent(ctx_->stream, ev, 0);
        return err == cudaSuccess || be_.fail(err, "ordering the staging copies before the device pass");
    }
    // The copy stream must not overwrite a staging half the context's stream still reads.
    bool reserve_half(int half)
    {
        if (!half_used_[half])
            return true;
        const cudaError_t err = cudaStreamWaitEvent(be_.stream(), consumed_[half], 0);
        return err == cudaSuccess || be_.fail(err, "waiting for a staging half");
    }
    bool retire_half(int half)
    {
        const cudaError_t err = cudaEventRecord(consumed_[half], ctx_->stream);
        half_used_[half] = true;
        return err == cudaSuccess || be_.fail(err, "marking a staging half as consumed");
    }

    qsfi_status load_router(qs3_moe_layer_weights* out)
    {
        const size_t e = d_.num_experts, row = static_cast<size_t>(d_.hidden_size) * 2;
        const WeightLoadSpan span = be_.alloc_tensor(m_.router_off, e * row);
        bool ok = true;
        if (d_.expert_order == nullptr) {
            ok = be_.read_exact(range(m_.router), span);
        } else {
            for (uint32_t p = 0; p < e && ok; ++p)
                ok = be_.read_exact(range(m_.router, expert_at(p) * row, row), span, p * row);
        }
        if (!ok)
            return backend_error();
        out->router_weight = view<2>(span.ptr, QSFI_DTYPE_BF16, { static_cast<int64_t>(e), d_.hidden_size });
        return QSFI_STATUS_OK;
    }

    qsfi_status tile(const char* linear, int64_t experts, int64_t rows, int64_t k, bool gated, char* tiled)
    {
        qs3_nvfp4_tile_scales_desc t {};
        t.scale_linear = view<3>(const_cast<char*>(linear), QSFI_DTYPE_FP8_E4M3, { experts, rows, k / 16 });
        t.scale_tiled = view<1>(tiled, QSFI_DTYPE_U8,
                                { static_cast<int64_t>(experts * qs3_nvfp4_tiled_scale_bytes(rows, k)) });
        t.gated_rows = gated ? 1 : 0;
        return qs3_nvfp4_tile_scales(ctx_, &t);
    }

    qsfi_status quantize(const char* bf16, int64_t experts, int64_t rows, int64_t k, bool gated, char* packed,
                         char* tiled, char* global)
    {
        qs3_nvfp4_quantize_weight_desc q {};
        q.weight = view<3>(const_cast<char*>(bf16), QSFI_DTYPE_BF16, { experts, rows, k });
        q.packed = view<3>(packed, QSFI_DTYPE_U8, { experts, rows, k / 2 });
        q.scale_tiled = view<1>(tiled, QSFI_DTYPE_U8,
                                { static_cast<int64_t>(experts * qs3_nvfp4_tiled_scale_bytes(rows, k)) });
        q.global_scale = view<1>(global, QSFI_DTYPE_F32, { experts });
        q.gated_rows = gated ? 1 : 0;
        return qs3_nvfp4_quantize_weight(ctx_, &q);
    }

    // NVFP4 checkpoint: codes go straight to their final place (gate rows, then up rows, of
    // the fused gate_up tensor), block scales are staged in the declared linear layout and
    // re-tiled on the device, the scalar scales are gathered on the host.
    qsfi_status load_split_experts(qs3_moe_layer_weights* out)
    {
        const size_t h = d_.hidden_size, i = d_.intermediate_size, el = d_.local_num_experts;
        const size_t gate_codes = i * (h / 2), down_codes = h * (i / 2);
        const size_t gate_sf = i * (h / 16), down_sf = h * (i / 16);
        const size_t gu_tiled = qs3_nvfp4_tiled_scale_bytes(2 * i, h), d_tiled = qs3_nvfp4_tiled_scale_bytes(h, i);
        const WeightLoadSpan gu = be_.alloc_tensor(m_.gu_off, el * 2 * gate_codes);
        const WeightLoadSpan dn = be_.alloc_tensor(m_.d_off, el * down_codes);
        const WeightLoadSpan gu_sf = be_.alloc_tensor(m_.gu_sf_off, el * gu_tiled);
        const WeightLoadSpan dn_sf = be_.alloc_tensor(m_.d_sf_off, el * d_tiled);
        const WeightLoadSpan gu_g = be_.alloc_tensor(m_.gu_g_off, 2 * el * sizeof(float));
        const WeightLoadSpan dn_g = be_.alloc_tensor(m_.d_g_off, el * sizeof(float));
        if (!be_.zero_fill(gu_sf) || !be_.zero_fill(dn_sf))
            return backend_error();
        std::vector<float> gu_global(2 * el), d_global(el);
        for (size_t c0 = 0; c0 < el; c0 += m_.chunk) {
            const size_t n = std::min<size_t>(m_.chunk, el - c0);
            const int half = static_cast<int>((c0 / m_.chunk) & 1);
            char* stage = scratch_ + half * m_.half_bytes;
            const WeightLoadSpan gu_lin { stage + m_.half_a, n * 2 * gate_sf };
            const WeightLoadSpan dn_lin { stage + m_.half_b, n * down_sf };
            bool ok = reserve_half(half);
            for (size_t j = 0; j < n && ok; ++j) {
                const size_t p = c0 + j;
                const uint32_t x = expert_at(d_.local_expert_offset + static_cast<uint32_t>(p));
                const Projection &g = m_.gate[x], &u = m_.up[x], &w = m_.down[x];
                ok = be_.read_exact(range(g.weight), gu, p * 2 * gate_codes)
                    && be_.read_exact(range(u.weight), gu, p * 2 * gate_codes + gate_codes)
                    && be_.read_exact(range(w.weight), dn, p * down_codes)
                    && be_.read_exact(range(g.scale), gu_lin, j * 2 * gate_sf)
                    && be_.read_exact(range(u.scale), gu_lin, j * 2 * gate_sf + gate_sf)
                    && be_.read_exact(range(w.scale), dn_lin, j * down_sf)
                    && scalar(g.scale2, &gu_global[p]) && scalar(u.scale2, &gu_global[el + p])
                    && scalar(w.scale2, &d_global[p]);
            }
            if (!ok || !publish(copied_[half]))
                return backend_error();
            qsfi_status status = tile(gu_lin.ptr, n, 2 * i, h, true, gu_sf.ptr + c0 * gu_tiled);
            if (status == QSFI_STATUS_OK)
                status = tile(dn_lin.ptr, n, h, i, false, dn_sf.ptr + c0 * d_tiled);
            if (status != QSFI_STATUS_OK)
                return status;
            if (!retire_half(half))
                return backend_error();
        }
        // activation scales: one value for all ranks, so every expert of the layer counts
        for (uint32_t x = 0; x < d_.num_experts; ++x) {
            float a = 0.0f, b = 0.0f, c = 0.0f;
            if (!scalar(m_.gate[x].input_scale, &a) || !scalar(m_.up[x].input_scale, &b)
                || !scalar(m_.down[x].input_scale, &c))
                return backend_error();
            act_max_ = std::fmax(act_max_, std::fmax(a, b));
            act2_max_ = std::fmax(act2_max_, c);
        }
        if (!be_.upload(gu_global.data(), gu_global.size() * sizeof(float), gu_g)
            || !be_.upload(d_global.data(), d_global.size() * sizeof(float), dn_g))
            return backend_error();
        const int64_t e64 = static_cast<int64_t>(el);
        out->gate_up_weight = view<3>(gu.ptr, QSFI_DTYPE_U8, { e64, static_cast<int64_t>(2 * i), static_cast<int64_t>(h / 2) });
        out->down_weight = view<3>(dn.ptr, QSFI_DTYPE_U8, { e64, static_cast<int64_t>(h), static_cast<int64_t>(i / 2) });
        out->gate_up_scale_tiled = view<1>(gu_sf.ptr, QSFI_DTYPE_U8, { static_cast<int64_t>(gu_sf.bytes) });
        out->down_scale_tiled = view<1>(dn_sf.ptr, QSFI_DTYPE_U8, { static_cast<int64_t>(dn_sf.bytes) });
        out->gate_up_global_scale = view<1>(gu_g.ptr, QSFI_DTYPE_F32, { 2 * e64 });
        out->down_global_scale = view<1>(dn_g.ptr, QSFI_DTYPE_F32, { e64 });
        if (act_max_ > 0.0f)
            out->act_global_scale = act_max_;
        if (act2_max_ > 0.0f)
            out->act2_global_scale = act2_max_;
        return QSFI_STATUS_OK;
    }

    // BF16 checkpoint with fused expert tensors: one contiguous slice per expert. A slice goes
    // to its final place directly when the plan is BF16 and the file layout is the kernels';
    // otherwise it is staged, transposed and / or quantised on the device.
    qsfi_status load_fused_experts(qs3_moe_layer_weights* out)
    {
        const size_t h = d_.hidden_size, i = d_.intermediate_size, el = d_.local_num_experts;
        const size_t gu_slice = 2 * i * h * 2, d_slice = h * i * 2; // bytes per expert in the file
        const bool q = nvfp4();
        const bool stage_gu = q || m_.gate_up_transposed, stage_d = q || m_.down_transposed;
        const size_t gu_tiled = q ? qs3_nvfp4_tiled_scale_bytes(2 * i, h) : 0;
        const size_t d_tiled = q ? qs3_nvfp4_tiled_scale_bytes(h, i) : 0;
        const WeightLoadSpan gu = be_.alloc_tensor(m_.gu_off, q ? el * 2 * i * (h / 2) : el * gu_slice);
        const WeightLoadSpan dn = be_.alloc_tensor(m_.d_off, q ? el * h * (i / 2) : el * d_slice);
        const WeightLoadSpan gu_sf = be_.alloc_tensor(m_.gu_sf_off, el * gu_tiled);
        const WeightLoadSpan dn_sf = be_.alloc_tensor(m_.d_sf_off, el * d_tiled);
        const WeightLoadSpan gu_g = be_.alloc_tensor(m_.gu_g_off, el * sizeof(float));
        const WeightLoadSpan dn_g = be_.alloc_tensor(m_.d_g_off, el * sizeof(float));
        for (size_t c0 = 0; c0 < el; c0 += m_.chunk) {
            const size_t n = std::min<size_t>(m_.chunk, el - c0);
            const int half = static_cast<int>((c0 / m_.chunk) & 1);
            char* stage = scratch_ + half * m_.half_bytes;
            const WeightLoadSpan gu_raw { stage + m_.half_a, n * gu_slice };
            const WeightLoadSpan d_raw { stage + m_.half_b, n * d_slice };
            bool ok = !(stage_gu || stage_d) || reserve_half(half);
            for (size_t j = 0; j < n && ok; ++j) {
                const size_t p = c0 + j;
                const uint64_t x = expert_at(d_.local_expert_offset + static_cast<uint32_t>(p));
                ok = (stage_gu ? be_.read_exact(range(m_.gate_up_fused, x * gu_slice, gu_slice), gu_raw, j * gu_slice)
                               : be_.read_exact(range(m_.gate_up_fused, x * gu_slice, gu_slice), gu, p * gu_slice))
                    && (stage_d ? be_.read_exact(range(m_.down_fused, x * d_slice, d_slice), d_raw, j * d_slice)
                                : be_.read_exact(range(m_.down_fused, x * d_slice, d_slice), dn, p * d_slice));
            }
            if (!ok)
                return backend_error();
            if (!(stage_gu || stage_d))
                continue;
            if (!publish(copied_[half]))
                return backend_error();
            const uint32_t n32 = static_cast<uint32_t>(n);
            const char* gu_src = gu_raw.ptr;
            const char* d_src = d_raw.ptr;
            cudaError_t err = cudaSuccess;
            if (m_.gate_up_transposed) { // file holds [H, 2I] per expert
                char* dst = q ? stage + m_.half_at : gu.ptr + c0 * gu_slice;
                err = launch_transpose_bf16(gu_raw.ptr, dst, n32, static_cast<uint32_t>(h), static_cast<uint32_t>(2 * i),
                                            ctx_->stream);
                gu_src = dst;
            }
            if (err == cudaSuccess && m_.down_transposed) { // file holds [I, H] per expert
                char* dst = q ? stage + m_.half_bt : dn.ptr + c0 * d_slice;
                err = launch_transpose_bf16(d_raw.ptr, dst, n32, static_cast<uint32_t>(i), static_cast<uint32_t>(h),
                                            ctx_->stream);
                d_src = dst;
            }
            if (err != cudaSuccess)
                return set_cuda_error(ctx_, err, "checkpoint loader transpose");
            if (q) {
                qsfi_status status = quantize(gu_src, n, 2 * i, h, true, gu.ptr + c0 * 2 * i * (h / 2),
                                              gu_sf.ptr + c0 * gu_tiled, gu_g.ptr + c0 * sizeof(float));
                if (status == QSFI_STATUS_OK)
                    status = quantize(d_src, n, h, i, false, dn.ptr + c0 * h * (i / 2), dn_sf.ptr + c0 * d_tiled,
                                      dn_g.ptr + c0 * sizeof(float));
                if (status != QSFI_STATUS_OK)
                    return status;
            }
            if (!retire_half(half))
                return backend_error();
        }
        const int64_t e64 = static_cast<int64_t>(el), h64 = static_cast<int64_t>(h), i64 = static_cast<int64_t>(i);
        if (q) {
            out->gate_up_weight = view<3>(gu.ptr, QSFI_DTYPE_U8, { e64, 2 * i64, h64 / 2 });
            out->down_weight = view<3>(dn.ptr, QSFI_DTYPE_U8, { e64, h64, i64 / 2 });
            out->gate_up_scale_tiled = view<1>(gu_sf.ptr, QSFI_DTYPE_U8, { static_cast<int64_t>(gu_sf.bytes) });
            out->down_scale_tiled = view<1>(dn_sf.ptr, QSFI_DTYPE_U8, { static_cast<int64_t>(dn_sf.bytes) });
            out->gate_up_global_scale = view<1>(gu_g.ptr, QSFI_DTYPE_F32, { e64 });
            out->down_global_scale = view<1>(dn_g.ptr, QSFI_DTYPE_F32, { e64 });
        } else {
            out->gate_up_weight = view<3>(gu.ptr, QSFI_DTYPE_BF16, { e64, 2 * i64, h64 });
            out->down_weight = view<3>(dn.ptr, QSFI_DTYPE_BF16, { e64, h64, i64 });
        }
        return QSFI_STATUS_OK;
    }

    // Shared expert: gate_proj and up_proj rows fused into [1, 2 * Is, H] like the routed experts.
    qsfi_status load_shared(qs3_moe_layer_weights* out)
    {
        const size_t h = d_.hidden_size, is = d_.shared_intermediate_size;
        const bool q = nvfp4();
        const int64_t h64 = static_cast<int64_t>(h), is64 = static_cast<int64_t>(is);
        const WeightLoadSpan gate = be_.alloc_tensor(m_.sgate_off, h * 2);
        if (!be_.read_exact(range(m_.shared_gate), gate))
            return backend_error();
        out->shared_gate_weight = view<2>(gate.ptr, QSFI_DTYPE_BF16, { 1, h64 });
        if (!q) {
            const size_t half_rows = is * h * 2;
            const WeightLoadSpan gu = be_.alloc_tensor(m_.sgu_off, 2 * half_rows);
            const WeightLoadSpan dn = be_.alloc_tensor(m_.sd_off, h * is * 2);
            if (!be_.read_exact(range(m_.sh_gate.weight), gu, 0) || !be_.read_exact(range(m_.sh_up.weight), gu, half_rows)
                || !be_.read_exact(range(m_.sh_down.weight), dn))
                return backend_error();
            out->shared_gate_up_weight = view<3>(gu.ptr, QSFI_DTYPE_BF16, { 1, 2 * is64, h64 });
            out->shared_down_weight = view<3>(dn.ptr, QSFI_DTYPE_BF16, { 1, h64, is64 });
            return QSFI_STATUS_OK;
        }
        const size_t gu_tiled = qs3_nvfp4_tiled_scale_bytes(2 * is, h), d_tiled = qs3_nvfp4_tiled_scale_bytes(h, is);
        const WeightLoadSpan gu = be_.alloc_tensor(m_.sgu_off, 2 * is * (h / 2));
        const WeightLoadSpan dn = be_.alloc_tensor(m_.sd_off, h * (is / 2));
        const WeightLoadSpan gu_sf = be_.alloc_tensor(m_.sgu_sf_off, gu_tiled);
        const WeightLoadSpan dn_sf = be_.alloc_tensor(m_.sd_sf_off, d_tiled);
        const WeightLoadSpan gu_g = be_.alloc_tensor(m_.sgu_g_off, 2 * sizeof(float));
        const WeightLoadSpan dn_g = be_.alloc_tensor(m_.sd_g_off, sizeof(float));
        char* stage_a = scratch_ + m_.shared_scratch_off;
        int64_t gu_globals = 1;
        if (m_.shared_nvfp4) {
            const size_t gate_codes = is * (h / 2), gate_sf = is * (h / 16), down_sf = h * (is / 16);
            char* stage_b = scratch_ + align_up(m_.shared_scratch_off + 2 * gate_sf, kWorkspaceAlign);
            const WeightLoadSpan gu_lin { stage_a, 2 * gate_sf };
            const WeightLoadSpan dn_lin { stage_b, down_sf };
            float globals[3] = {}, inputs[3] = {};
            const bool ok = be_.zero_fill(gu_sf) && be_.zero_fill(dn_sf) && be_.read_exact(range(m_.sh_gate.weight), gu, 0)
                && be_.read_exact(range(m_.sh_up.weight), gu, gate_codes) && be_.read_exact(range(m_.sh_down.weight), dn)
                && be_.read_exact(range(m_.sh_gate.scale), gu_lin, 0) && be_.read_exact(range(m_.sh_up.scale), gu_lin, gate_sf)
                && be_.read_exact(range(m_.sh_down.scale), dn_lin) && scalar(m_.sh_gate.scale2, &globals[0])
                && scalar(m_.sh_up.scale2, &globals[1]) && scalar(m_.sh_down.scale2, &globals[2])
                && scalar(m_.sh_gate.input_scale, &inputs[0]) && scalar(m_.sh_up.input_scale, &inputs[1])
                && scalar(m_.sh_down.input_scale, &inputs[2]) && be_.upload(globals, 2 * sizeof(float), gu_g)
                && be_.upload(globals + 2, sizeof(float), dn_g) && publish(shared_copied_);
            if (!ok)
                return backend_error();
            qsfi_status status = tile(gu_lin.ptr, 1, 2 * is64, h64, true, gu_sf.ptr);
            if (status == QSFI_STATUS_OK)
                status = tile(dn_lin.ptr, 1, h64, is64, false, dn_sf.ptr);
            if (status != QSFI_STATUS_OK)
                return status;
            act_max_ = std::fmax(act_max_, std::fmax(inputs[0], inputs[1]));
            act2_max_ = std::fmax(act2_max_, inputs[2]);
            if (act_max_ > 0.0f)
                out->act_global_scale = act_max_;
            if (act2_max_ > 0.0f)
                out->act2_global_scale = act2_max_;
            gu_globals = 2;
        } else { // bf16 in the file: quantise on the device
            const size_t half_rows = is * h * 2;
            char* stage_b = scratch_ + align_up(m_.shared_scratch_off + 2 * half_rows, kWorkspaceAlign);
            const WeightLoadSpan gu_raw { stage_a, 2 * half_rows };
            const WeightLoadSpan dn_raw { stage_b, h * is * 2 };
            if (!be_.read_exact(range(m_.sh_gate.weight), gu_raw, 0) || !be_.read_exact(range(m_.sh_up.weight), gu_raw, half_rows)
                || !be_.read_exact(range(m_.sh_down.weight), dn_raw) || !publish(shared_copied_))
                return backend_error();
            qsfi_status status = quantize(gu_raw.ptr, 1, 2 * is64, h64, true, gu.ptr, gu_sf.ptr, gu_g.ptr);
            if (status == QSFI_STATUS_OK)
                status = quantize(dn_raw.ptr, 1, h64, is64, false, dn.ptr, dn_sf.ptr, dn_g.ptr);
            if (status != QSFI_STATUS_OK)
                return status;
        }
        out->shared_gate_up_weight = view<3>(gu.ptr, QSFI_DTYPE_U8, { 1, 2 * is64, h64 / 2 });
        out->shared_down_weight = view<3>(dn.ptr, QSFI_DTYPE_U8, { 1, h64, is64 / 2 });
        out->shared_gate_up_scale_tiled = view<1>(gu_sf.ptr, QSFI_DTYPE_U8, { static_cast<int64_t>(gu_tiled) });
        out->shared_down_scale_tiled = view<1>(dn_sf.ptr, QSFI_DTYPE_U8, { static_cast<int64_t>(d_tiled) });
        out->shared_gate_up_global_scale = view<1>(gu_g.ptr, QSFI_DTYPE_F32, { gu_globals });
        out->shared_down_global_scale = view<1>(dn_g.ptr, QSFI_DTYPE_F32, { 1 });
        return QSFI_STATUS_OK;
    }
};

qsfi_status check_load_args(qsfi_context* ctx, const qs3_checkpoint* ck, const qs3_moe_layer_load_desc* d,
                            LayerManifest* m)
{
    if (ck == nullptr || d == nullptr)
        return set_invalid_arg(ctx, "checkpoint and desc are required");
    std::string error;
    if (!build_manifest(ck, *d, m, &error))
        return set_invalid_arg(ctx, "checkpoint layer %s: %s", d->layer_prefix != nullptr ? d->layer_prefix : "(null)",
                               error.c_str());
    return QSFI_STATUS_OK;
}

} // namespace
} // namespace qs3

extern "C" {

qsfi_status qs3_checkpoint_moe_layer_bytes(qsfi_context* ctx, const qs3_checkpoint* checkpoint,
                                           const qs3_moe_layer_load_desc* desc, size_t* weight_bytes,
                                           size_t* scratch_bytes)
{
    if (ctx == nullptr || weight_bytes == nullptr || scratch_bytes == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    qs3::clear_error(&ctx->last_error);
    try {
        qs3::LayerManifest m;
        const qsfi_status status = qs3::check_load_args(ctx, checkpoint, desc, &m);
        if (status != QSFI_STATUS_OK)
            return status;
        *weight_bytes = m.weight_bytes;
        *scratch_bytes = m.scratch_bytes;
        return QSFI_STATUS_OK;
    } catch (const std::exception& e) {
        return qs3::set_error(ctx, QSFI_STATUS_BACKEND_ERROR, QSFI_ERROR_SOURCE_QSFI, 0, "checkpoint layer: %s", e.what());
    }
}

qsfi_status qs3_checkpoint_load_moe_layer(qsfi_context* ctx, const qs3_checkpoint* checkpoint,
                                          const qs3_moe_layer_load_desc* desc, void* weights, size_t weight_bytes,
                                          void* scratch, size_t scratch_bytes, qs3_moe_layer_weights* out)
{
    if (ctx == nullptr || out == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    qs3::clear_error(&ctx->last_error);
    try {
        // the whole manifest is validated before the first CUDA call
        qs3::LayerManifest m;
        qsfi_status status = qs3::check_load_args(ctx, checkpoint, desc, &m);
        if (status != QSFI_STATUS_OK)
            return status;
        if (weights == nullptr || weight_bytes < m.weight_bytes
            || (reinterpret_cast<uintptr_t>(weights) & (qs3::kWorkspaceAlign - 1)) != 0)
            return qs3::set_invalid_arg(ctx, "checkpoint layer: weight block must be 256-byte aligned and hold %zu bytes",
                                        m.weight_bytes);
        if (m.scratch_bytes != 0
            && (scratch == nullptr || scratch_bytes < m.scratch_bytes
                || (reinterpret_cast<uintptr_t>(scratch) & (qs3::kWorkspaceAlign - 1)) != 0))
            return qs3::set_invalid_arg(ctx, "checkpoint layer: scratch block must be 256-byte aligned and hold %zu bytes",
                                        m.scratch_bytes);
        status = qs3::activate_context(ctx);
        if (status != QSFI_STATUS_OK)
            return status;
        qs3::LayerLoad load(ctx, checkpoint, *desc, m, weights, weight_bytes, scratch);
        return load.run(out);
    } catch (const std::exception& e) {
        return qs3::set_error(ctx, QSFI_STATUS_BACKEND_ERROR, QSFI_ERROR_SOURCE_QSFI, 0, "checkpoint layer: %s", e.what());
    }
}

} // extern "C"
