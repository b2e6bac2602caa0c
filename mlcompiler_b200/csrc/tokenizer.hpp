// Text <-> token ids from the vocabulary a GGUF file carries (tokenizer.ggml.*), host-only.
//
// Behaves like the reference's Tokenizer built without llama.cpp (compiler/runtime/tokenizer.{hpp,cpp}: constructor
// 36-126, buildIndices 137-151, encode 153-244, decode 246-283, isControlToken / isEogToken 290-311, bpeEncode
// 327-362, unigramEncode 364-423, decodeTokenString 425-448):
//   * pieces spelled "<0xHH>" stand for the byte HH; lookups go by the decoded bytes, a repeated piece keeps its
//     highest id;
//   * tokenizer.ggml.model "llama" / "spm" / "unigram" -> best-score segmentation over byte positions (scores must
//     cover the vocabulary; a single unknown byte costs the unknown token's score, or -1); "gpt2" / "bpe" -> byte
//     symbols merged lowest rank first (tokenizer.ggml.merges, rank = position in the array); no model key -> merges
//     if there are any, else scores;
//   * when that produced nothing AND no BOS was put in front, the longest piece that matches at every position
//     (longest raw spelling first, lowest id on ties), the unknown token for a byte nothing matches;
//   * decode drops "<s>", "</s>", "<unk>", turns a leading U+2581 into a word break, skips ids past the vocabulary.
#pragma once

#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>

#include "gguf_file.hpp"

namespace mlcb {
namespace text {

constexpr uint64_t kNoToken = UINT64_MAX;

class Tokenizer {
public:
    explicit Tokenizer(const gguf::File& file);

    bool valid() const { return !raw_.empty(); }
    size_t vocab_size() const { return raw_.size(); }
    uint64_t bos() const { return bos_; }
    uint64_t eos() const { return eos_; }
    uint64_t unk() const { return unk_; }

    std::vector<uint64_t> encode(const std::string& text, bool add_bos = true, bool add_eos = false) const;
    std::string decode(const uint64_t* ids, size_t n) const;
    // the piece as spelled in the file ("" past the vocabulary)
    std::string token_string(uint64_t id) const { return id < raw_.size() ? raw_[id] : std::string(); }
    bool is_control(uint64_t id) const;
    bool is_eog(uint64_t id) const { return id == eos_; }

private:
    enum class Model { kNone, kUnigram, kMerges, kOther };
    void segment_by_score(const std::string& text, std::vector<uint64_t>& out) const;
    void segment_by_merges(const std::string& text, std::vector<uint64_t>& out) const;
    void segment_greedy(const std::string& text, std::vector<uint64_t>& out) const;
    uint64_t unknown() const { return unk_ == kNoToken ? 0 : unk_; }

    std::vector<std::string> raw_;     // pieces as spelled
    std::vector<std::string> bytes_;   // pieces as bytes
    std::vector<float> scores_;
    Model model_ = Model::kNone;
    std::unordered_map<std::string, uint64_t> id_of_;        // bytes -> id
    std::unordered_map<std::string, size_t> merge_rank_;     // "left right" -> rank
    std::vector<uint32_t> by_lead_[256];                     // ids whose bytes start with a byte, longest spelling first
    uint64_t bos_ = kNoToken, eos_ = kNoToken, unk_ = kNoToken;
};

}  // namespace text
}  // namespace mlcb
