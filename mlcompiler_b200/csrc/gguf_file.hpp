// GGUF container (versions 1 to 3): header, key/value metadata, tensor directory, tensor bytes.
// Host-only; the file is mapped read-only and tensor bytes are handed out as pointers into the mapping.
//
// Follows what compiler/frontends/gguf_loader.cpp makes of a file (load(): 306-433, parseValue: 463-533,
// calculateTensorSize: 679-752, parseTensorDirectory: 759-838, concatenateBlockWeights: 877-943):
//   * value types on disk are the GGUF enumeration (0 u8 .. 8 string, 9 array, 10 u64, 11 i64, 12 f64; 13 = the
//     legacy raw blob, u64 length + bytes);
//   * general.alignment (u32 / u64 / positive i32 / i64; 0 or absent = 32) pads the end of the tensor directory,
//     and tensor offsets are relative to that point;
//   * a tensor's size is ceil(elements / block) * block bytes of its ggml type; an unknown type counts 4 bytes per
//     element, an empty shape is 0 bytes;
//   * a name that occurs twice keeps its last entry;
//   * per block, attn_q | attn_k | attn_v and ffn_gate | ffn_up (all Q4_0, 2-D, equal column counts) are
//     byte-concatenated into attn_qkv and ffn_gate_up, the tensors the batched walker reads.
//   * version 1 as the reference reads (and its tests write) it: 64-bit counts and string lengths like the later
//     versions, 32-bit tensor dimensions optionally behind a 64-bit repeat of the rank, tensor offsets that are
//     positions in the file, no padding;
//   * a key or tensor name longer than 1 MiB is taken for damage: a key's entry is dropped, its value still read.
// Not taken over: the reference's other recovery heuristics for damaged files (32-bit string lengths, skipping to
// the next 32-byte boundary after an entry that failed to parse, a truncated tensor directory read as far as it
// goes); such files are rejected with a message.
#pragma once

#include <cstdint>
#include <map>
#include <string>
#include <unordered_map>
#include <vector>

namespace mlcb {
namespace gguf {

enum ValueType : uint32_t {
    kU8 = 0, kI8 = 1, kU16 = 2, kI16 = 3, kU32 = 4, kI32 = 5, kF32 = 6, kBool = 7, kString = 8, kArray = 9,
    kU64 = 10, kI64 = 11, kF64 = 12, kRaw = 13,
};
const char* value_type_name(uint32_t t);

struct Value {
    uint32_t type = kU8;
    uint64_t u = 0;          // unsigned integers and bool
    int64_t i = 0;           // signed integers
    double f = 0.0;          // f32 (widened) and f64
    std::string s;           // string, or the bytes of a raw blob
    uint32_t elem_type = 0;  // arrays
    std::vector<Value> arr;
    bool is_integer() const { return type <= kI32 || type == kU64 || type == kI64; }
    bool is_signed() const { return type == kI8 || type == kI16 || type == kI32 || type == kI64; }
    // integer value as unsigned (negative values give `fallback`)
    uint64_t as_u64(uint64_t fallback = 0) const;
    double as_double(double fallback = 0.0) const;
};

enum GgmlType : uint32_t {
    kGgmlF32 = 0, kGgmlF16 = 1, kGgmlQ4_0 = 2, kGgmlQ6_K = 14,
};
// bytes of `elements` weights of a ggml type; throws std::runtime_error on overflow
uint64_t tensor_bytes(const std::vector<uint64_t>& shape, uint32_t dtype);

struct TensorInfo {
    std::string name;
    std::vector<uint64_t> shape;   // shape[0] = columns (fastest), as stored
    uint32_t dtype = 0;
    uint64_t offset = 0;           // absolute file offset; UINT64_MAX for a concatenated tensor
    uint64_t n_bytes = 0;
    bool synthetic() const { return offset == UINT64_MAX; }
};

class File {
public:
    // Throws std::runtime_error with what is wrong with the file.
    explicit File(const std::string& path);
    ~File();
    File(const File&) = delete;
    File& operator=(const File&) = delete;

    uint32_t version() const { return version_; }
    uint64_t n_tensors() const { return n_tensors_; }
    uint64_t n_kv() const { return n_kv_; }
    uint64_t alignment() const { return alignment_; }
    uint32_t quantization_version() const { return quant_version_; }
    uint64_t data_start() const { return data_start_; }
    uint64_t file_size() const { return size_; }
    const std::map<std::string, Value>& kv() const { return kv_; }
    const std::map<std::string, TensorInfo>& tensors() const { return tensors_; }
    const Value* find_kv(const std::string& key) const;
    // first of `keys` that is present
    const Value* find_kv(std::initializer_list<const char*> keys) const;
    const TensorInfo* find_tensor(const std::string& name) const;

    // The tensor's bytes (n_bytes of them). Throws if they lie outside the file.
    const uint8_t* data(const TensorInfo& t) const;

    // gguf_loader.cpp:877-943. Returns how many tensors were added.
    size_t concatenate_block_weights();

    // Everything but the tensor bytes as one JSON object (keys sorted), for tools and tests.
    std::string describe_json() const;

private:
    std::string path_;
    int fd_ = -1;
    const uint8_t* map_ = nullptr;
    uint64_t size_ = 0;
    uint32_t version_ = 0, quant_version_ = 1;
    uint64_t n_tensors_ = 0, n_kv_ = 0, alignment_ = 32, data_start_ = 0;
    std::map<std::string, Value> kv_;
    std::map<std::string, TensorInfo> tensors_;
    std::unordered_map<std::string, std::vector<uint8_t>> synthetic_;
};

}  // namespace gguf
}  // namespace mlcb
