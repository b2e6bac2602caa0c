#include "gguf_file.hpp"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <stdexcept>

namespace mlcb {
namespace gguf {

namespace {

constexpr uint32_t kMagic = 0x46554747u;   // "GGUF", little-endian

[[noreturn]] void fail(const std::string& what) { throw std::runtime_error(what); }

// Reads little-endian scalars from the mapping; every read is checked against the end of the file.
struct Cursor {
    const uint8_t* base;
    uint64_t pos, end;
    template <typename T>
    T get(const char* what) {
        if (end - pos < sizeof(T)) fail(std::string("unexpected end of file while reading ") + what);
        T v;
        std::memcpy(&v, base + pos, sizeof(T));
        pos += sizeof(T);
        return v;
    }
    std::string str(const char* what) {
        const uint64_t n = get<uint64_t>(what);
        if (n > end - pos) fail(std::string("string longer than the rest of the file: ") + what);
        std::string s(reinterpret_cast<const char*>(base + pos), static_cast<size_t>(n));
        pos += n;
        return s;
    }
    // A key or a tensor name: one of more than 1 MiB is taken for damage - its bytes are passed over and the entry
    // it names is dropped (gguf_loader.cpp:187-243 with enforce_soft_limit, 553-554, 590-607).
    std::string name(const char* what, bool* damaged) {
        const uint64_t n = get<uint64_t>(what);
        if (n > end - pos) fail(std::string("string longer than the rest of the file: ") + what);
        *damaged = n > (uint64_t(1) << 20);
        std::string s;
        if (!*damaged) s.assign(reinterpret_cast<const char*>(base + pos), static_cast<size_t>(n));
        pos += n;
        return s;
    }
};

Value parse_value(Cursor& c, uint32_t type, int depth) {
    Value v;
    v.type = type;
    switch (type) {
        case kU8: v.u = c.get<uint8_t>("uint8"); break;
        case kI8: v.i = c.get<int8_t>("int8"); break;
        case kU16: v.u = c.get<uint16_t>("uint16"); break;
        case kI16: v.i = c.get<int16_t>("int16"); break;
        case kU32: v.u = c.get<uint32_t>("uint32"); break;
        case kI32: v.i = c.get<int32_t>("int32"); break;
        case kU64: v.u = c.get<uint64_t>("uint64"); break;
        case kI64: v.i = c.get<int64_t>("int64"); break;
        case kF32: v.f = c.get<float>("float32"); break;
        case kF64: v.f = c.get<double>("float64"); break;
        case kBool: v.u = c.get<uint8_t>("bool") != 0 ? 1 : 0; break;
        case kString: v.s = c.str("string value"); break;
        case kRaw: v.s = c.str("raw value"); break;   // u64 length + bytes, like a string
        case kArray: {
            if (depth > 8) fail("arrays nested too deeply");
            v.elem_type = c.get<uint32_t>("array element type");
            if (v.elem_type > kRaw) fail("Invalid value type " + std::to_string(v.elem_type));
            const uint64_t n = c.get<uint64_t>("array length");
            if (n > c.end - c.pos) fail("array longer than the rest of the file");
            v.arr.reserve(static_cast<size_t>(n));
            for (uint64_t i = 0; i < n; ++i) v.arr.push_back(parse_value(c, v.elem_type, depth + 1));
            break;
        }
        default: fail("Invalid value type " + std::to_string(type));
    }
    return v;
}

struct BlockSize { uint32_t dtype; uint64_t weights, bytes; };
// ggml block formats (weights per block, bytes per block)
constexpr BlockSize kBlocks[] = {
    {0, 1, 4},      // F32
    {1, 1, 2},      // F16
    {2, 32, 18},    // Q4_0
    {3, 32, 20},    // Q4_1
    {6, 32, 22},    // Q5_0
    {7, 32, 24},    // Q5_1
    {8, 32, 34},    // Q8_0
    {9, 32, 36},    // Q8_1
    {10, 256, 84},  // Q2_K: 16 scales + 64 quants + d, dmin
    {11, 256, 110}, // Q3_K: 32 hmask + 64 quants + 12 scales + d
    {12, 256, 144}, // Q4_K: d, dmin + 12 scales + 128 quants
    {13, 256, 176}, // Q5_K: d, dmin + 12 scales + 32 qh + 128 qs
    {14, 256, 210}, // Q6_K: 128 ql + 64 qh + 16 scales + d
    {15, 256, 292}, // Q8_K: f32 d + 256 quants + 16 int16 sums
    {24, 1, 1},     // I8
    {25, 1, 2},     // I16
    {26, 1, 4},     // I32
    {30, 1, 2},     // BF16
};

void json_string(std::string& out, const std::string& s) {
    out += '"';
    for (unsigned char ch : s) {
        if (ch == '"' || ch == '\\') { out += '\\'; out += static_cast<char>(ch); }
        else if (ch < 0x20) { char b[8]; std::snprintf(b, sizeof(b), "\\u%04x", ch); out += b; }
        else out += static_cast<char>(ch);
    }
    out += '"';
}

void json_number(std::string& out, double f, bool single) {
    if (!std::isfinite(f)) { out += std::isnan(f) ? "\"nan\"" : (f > 0 ? "\"inf\"" : "\"-inf\""); return; }
    char b[40];
    std::snprintf(b, sizeof(b), single ? "%.9g" : "%.17g", f);
    out += b;
}

void json_value(std::string& out, const Value& v) {
    switch (v.type) {
        case kU8: case kU16: case kU32: case kU64: out += std::to_string(v.u); break;
        case kI8: case kI16: case kI32: case kI64: out += std::to_string(v.i); break;
        case kF32: json_number(out, v.f, true); break;
        case kF64: json_number(out, v.f, false); break;
        case kBool: out += v.u ? "true" : "false"; break;
        case kString: json_string(out, v.s); break;
        case kRaw: {
            out += '"';
            for (unsigned char ch : v.s) { char b[4]; std::snprintf(b, sizeof(b), "%02x", ch); out += b; }
            out += '"';
            break;
        }
        case kArray: {
            out += '[';
            for (size_t i = 0; i < v.arr.size(); ++i) {
                if (i) out += ',';
                json_value(out, v.arr[i]);
            }
            out += ']';
            break;
        }
        default: out += "null";
    }
}

}  // namespace

const char* value_type_name(uint32_t t) {
    static const char* names[] = {"UINT8", "INT8", "UINT16", "INT16", "UINT32", "INT32", "FLOAT32", "BOOL", "STRING",
                                  "ARRAY", "UINT64", "INT64", "FLOAT64", "RAW"};
    return t <= kRaw ? names[t] : "?";
}

uint64_t Value::as_u64(uint64_t fallback) const {
    if (type == kBool) return u;
    if (!is_integer()) return fallback;
    if (is_signed()) return i >= 0 ? static_cast<uint64_t>(i) : fallback;
    return u;
}

double Value::as_double(double fallback) const {
    if (type == kF32 || type == kF64) return f;
    if (is_integer()) return is_signed() ? static_cast<double>(i) : static_cast<double>(u);
    return fallback;
}

uint64_t tensor_bytes(const std::vector<uint64_t>& shape, uint32_t dtype) {
    if (shape.empty()) return 0;
    uint64_t elements = 1;
    for (uint64_t d : shape)
        if (__builtin_mul_overflow(elements, d, &elements)) fail("Overflow while calculating tensor element count");
    uint64_t weights = 1, bytes = 4;   // a type this table does not know counts as 4 bytes per element
    for (const BlockSize& b : kBlocks)
        if (b.dtype == dtype) { weights = b.weights; bytes = b.bytes; break; }
    uint64_t blocks = elements / weights + (elements % weights ? 1 : 0), total;
    if (__builtin_mul_overflow(blocks, bytes, &total)) fail("Overflow while calculating tensor byte size");
    return total;
}

File::File(const std::string& path) : path_(path) {
    fd_ = ::open(path.c_str(), O_RDONLY);
    if (fd_ < 0) fail("Failed to open GGUF file: " + path);
    struct stat st {};
    if (::fstat(fd_, &st) != 0 || st.st_size < 0) { ::close(fd_); fd_ = -1; fail("Failed to get file size: " + path); }
    size_ = static_cast<uint64_t>(st.st_size);
    if (size_ > 0) {
        void* m = ::mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
        if (m == MAP_FAILED) { ::close(fd_); fd_ = -1; fail("Failed to map GGUF file: " + path); }
        map_ = static_cast<const uint8_t*>(m);
    }
    try {
        Cursor c{map_, 0, size_};
        if (c.get<uint32_t>("magic") != kMagic) fail("Invalid GGUF magic");
        version_ = c.get<uint32_t>("version");
        if (version_ < 1 || version_ > 3) fail("Unsupported GGUF version: " + std::to_string(version_));
        n_tensors_ = c.get<uint64_t>("tensor count");
        n_kv_ = c.get<uint64_t>("metadata count");
        for (uint64_t i = 0; i < n_kv_; ++i) {
            bool damaged = false;
            std::string key = c.name("metadata key", &damaged);
            const uint32_t type = c.get<uint32_t>("metadata value type");
            if (type > kRaw) fail("Invalid value type " + std::to_string(type));
            Value v = parse_value(c, type, 0);
            if (!damaged) kv_[key] = std::move(v);
        }
        if (const Value* q = find_kv("general.quantization_version"))
            if (q->type == kU32 || q->type == kU64) quant_version_ = static_cast<uint32_t>(q->u);
        if (const Value* a = find_kv("general.alignment")) {
            uint64_t v = 32;
            if (a->type == kU32 || a->type == kU64) v = a->u;
            else if ((a->type == kI32 || a->type == kI64) && a->i > 0) v = static_cast<uint64_t>(a->i);
            alignment_ = v ? v : 32;
        }
        for (uint64_t i = 0; i < n_tensors_; ++i) {
            TensorInfo t;
            bool damaged = false;
            t.name = c.name("tensor name", &damaged);
            if (damaged) t.name = "<CORRUPT_STRING>";   // the reference keeps such an entry under this name
            const uint32_t n_dims = c.get<uint32_t>("tensor rank");
            if (n_dims > 16) fail("tensor '" + t.name + "' has " + std::to_string(n_dims) + " dimensions");
            if (version_ == 1) {
                // version 1 as the reference reads it (gguf_loader.cpp:781-807): 32-bit dimensions, optionally behind
                // a 64-bit repeat of the rank
                if (n_dims > 0 && c.end - c.pos >= 8) {
                    uint64_t again;
                    std::memcpy(&again, c.base + c.pos, 8);
                    if (again == n_dims) c.pos += 8;
                }
                for (uint32_t d = 0; d < n_dims; ++d) t.shape.push_back(c.get<uint32_t>("tensor dimension"));
            } else {
                for (uint32_t d = 0; d < n_dims; ++d) t.shape.push_back(c.get<uint64_t>("tensor dimension"));
            }
            t.dtype = c.get<uint32_t>("tensor type");
            t.offset = c.get<uint64_t>("tensor offset");
            t.n_bytes = tensor_bytes(t.shape, t.dtype);
            tensors_[t.name] = std::move(t);   // a repeated name keeps its last entry
        }
        if (version_ == 1) {
            data_start_ = c.pos;   // version 1: offsets are positions in the file, nothing is padded
        } else {
            data_start_ = (c.pos + alignment_ - 1) / alignment_ * alignment_;
            for (auto& kv : tensors_)
                if (__builtin_add_overflow(kv.second.offset, data_start_, &kv.second.offset))
                    fail("tensor '" + kv.first + "': offset overflows");
        }
    } catch (...) {
        if (map_) ::munmap(const_cast<uint8_t*>(map_), size_);
        if (fd_ >= 0) ::close(fd_);
        map_ = nullptr;
        fd_ = -1;
        throw;
    }
}

File::~File() {
    if (map_) ::munmap(const_cast<uint8_t*>(map_), size_);
    if (fd_ >= 0) ::close(fd_);
}

const Value* File::find_kv(const std::string& key) const {
    auto it = kv_.find(key);
    return it == kv_.end() ? nullptr : &it->second;
}

const Value* File::find_kv(std::initializer_list<const char*> keys) const {
    for (const char* k : keys)
        if (const Value* v = find_kv(k)) return v;
    return nullptr;
}

const TensorInfo* File::find_tensor(const std::string& name) const {
    auto it = tensors_.find(name);
    return it == tensors_.end() ? nullptr : &it->second;
}

const uint8_t* File::data(const TensorInfo& t) const {
    if (t.synthetic()) {
        auto it = synthetic_.find(t.name);
        if (it == synthetic_.end()) fail("Synthetic tensor data missing: " + t.name);
        return it->second.data();
    }
    if (t.offset > size_ || t.n_bytes > size_ - t.offset) fail("Failed to read complete tensor data: " + t.name);
    return map_ + t.offset;
}

size_t File::concatenate_block_weights() {
    size_t added = 0;
    auto concat = [&](const std::string& fused, std::initializer_list<std::string> parts) {
        if (tensors_.count(fused)) return;
        std::vector<const TensorInfo*> infos;
        for (const std::string& p : parts) {
            const TensorInfo* t = find_tensor(p);
            if (!t || t->dtype != kGgmlQ4_0 || t->shape.size() != 2) return;
            infos.push_back(t);
        }
        const uint64_t cols = infos[0]->shape[0];
        uint64_t rows = 0, bytes = 0;
        for (const TensorInfo* t : infos) {
            if (t->shape[0] != cols) return;
            rows += t->shape[1];
            bytes += t->n_bytes;
        }
        std::vector<uint8_t> buf;
        buf.reserve(static_cast<size_t>(bytes));
        for (const TensorInfo* t : infos) {
            const uint8_t* p = data(*t);
            buf.insert(buf.end(), p, p + t->n_bytes);
        }
        TensorInfo s;
        s.name = fused;
        s.shape = {cols, rows};
        s.dtype = kGgmlQ4_0;
        s.offset = UINT64_MAX;
        s.n_bytes = buf.size();
        synthetic_[fused] = std::move(buf);
        tensors_[fused] = std::move(s);
        ++added;
    };
    // every block index that has an attn_q weight, in ascending order
    std::vector<uint64_t> layers;
    const std::string prefix = "blk.", suffix = ".attn_q.weight";
    for (const auto& kv : tensors_) {
        const std::string& n = kv.first;
        if (n.size() <= prefix.size() + suffix.size() || n.compare(0, prefix.size(), prefix) != 0 ||
            n.compare(n.size() - suffix.size(), suffix.size(), suffix) != 0)
            continue;
        const std::string idx = n.substr(prefix.size(), n.size() - prefix.size() - suffix.size());
        if (idx.empty() || idx.size() > 9 || idx.find_first_not_of("0123456789") != std::string::npos) continue;
        layers.push_back(std::stoull(idx));
    }
    std::sort(layers.begin(), layers.end());
    layers.erase(std::unique(layers.begin(), layers.end()), layers.end());
    for (uint64_t l : layers) {
        const std::string p = "blk." + std::to_string(l) + ".";
        concat(p + "attn_qkv.weight", {p + "attn_q.weight", p + "attn_k.weight", p + "attn_v.weight"});
        concat(p + "ffn_gate_up.weight", {p + "ffn_gate.weight", p + "ffn_up.weight"});
    }
    return added;
}

std::string File::describe_json() const {
    std::string out = "{";
    out += "\"version\":" + std::to_string(version_);
    out += ",\"n_tensors\":" + std::to_string(n_tensors_);
    out += ",\"n_kv\":" + std::to_string(n_kv_);
    out += ",\"alignment\":" + std::to_string(alignment_);
    out += ",\"data_start\":" + std::to_string(data_start_);
    out += ",\"quantization_version\":" + std::to_string(quant_version_);
    out += ",\"kv\":{";
    bool first = true;
    for (const auto& kv : kv_) {
        if (!first) out += ',';
        first = false;
        json_string(out, kv.first);
        out += ":{\"type\":\"";
        out += value_type_name(kv.second.type);
        out += '"';
        if (kv.second.type == kArray) {
            out += ",\"elem_type\":\"";
            out += value_type_name(kv.second.elem_type);
            out += '"';
        }
        out += ",\"value\":";
        json_value(out, kv.second);
        out += '}';
    }
    out += "},\"tensors\":{";
    first = true;
    for (const auto& kv : tensors_) {
        if (!first) out += ',';
        first = false;
        json_string(out, kv.first);
        out += ":{\"shape\":[";
        for (size_t i = 0; i < kv.second.shape.size(); ++i) {
            if (i) out += ',';
            out += std::to_string(kv.second.shape[i]);
        }
        out += "],\"dtype\":" + std::to_string(kv.second.dtype);
        out += ",\"offset\":" + (kv.second.synthetic() ? std::string("-1") : std::to_string(kv.second.offset));
        out += ",\"n_bytes\":" + std::to_string(kv.second.n_bytes) + "}";
    }
    out += "}}";
    return out;
}

}  // namespace gguf
}  // namespace mlcb
