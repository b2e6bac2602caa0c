#include "tokenizer.hpp"

#include <algorithm>
#include <cctype>
#include <cstring>
#include <limits>

namespace mlcb {
namespace text {

namespace {

int hex_value(unsigned char c) {
    if (c >= '0' && c <= '9') return c - '0';
    if (c >= 'a' && c <= 'f') return c - 'a' + 10;
    if (c >= 'A' && c <= 'F') return c - 'A' + 10;
    return -1;
}

// "<0xHH>" anywhere in a piece stands for the byte HH
std::string piece_bytes(const std::string& raw) {
    std::string out;
    out.reserve(raw.size());
    size_t i = 0;
    while (i < raw.size()) {
        if (raw[i] == '<' && i + 5 < raw.size() && raw[i + 1] == '0' && raw[i + 2] == 'x' && raw[i + 5] == '>') {
            const int hi = hex_value(static_cast<unsigned char>(raw[i + 3])), lo = hex_value(static_cast<unsigned char>(raw[i + 4]));
            if (hi >= 0 && lo >= 0) {
                out.push_back(static_cast<char>(hi * 16 + lo));
                i += 6;
                continue;
            }
        }
        out.push_back(raw[i++]);
    }
    return out;
}

// an id stored as uint32 or uint64; any other type counts as absent
uint64_t id_from(const gguf::File& file, const char* key) {
    const gguf::Value* v = file.find_kv(key);
    if (v && (v->type == gguf::kU32 || v->type == gguf::kU64)) return v->u;
    return kNoToken;
}

bool starts_with_word_mark(const std::string& s) {   // U+2581 in UTF-8
    return s.size() >= 3 && static_cast<unsigned char>(s[0]) == 0xE2 && static_cast<unsigned char>(s[1]) == 0x96 &&
           static_cast<unsigned char>(s[2]) == 0x81;
}

}  // namespace

Tokenizer::Tokenizer(const gguf::File& file) {
    if (const gguf::Value* m = file.find_kv("tokenizer.ggml.model"); m && m->type == gguf::kString) {
        const std::string& name = m->s;
        if (name == "llama" || name == "spm" || name == "unigram") model_ = Model::kUnigram;
        else if (name == "gpt2" || name == "bpe") model_ = Model::kMerges;
        else model_ = name.empty() ? Model::kNone : Model::kOther;
    }
    if (const gguf::Value* t = file.find_kv("tokenizer.ggml.tokens"); t && t->type == gguf::kArray)
        for (const gguf::Value& v : t->arr)
            if (v.type == gguf::kString) {
                raw_.push_back(v.s);
                bytes_.push_back(piece_bytes(v.s));
            }
    if (const gguf::Value* s = file.find_kv("tokenizer.ggml.scores"); s && s->type == gguf::kArray)
        for (const gguf::Value& v : s->arr)
            if (v.type == gguf::kF32 || v.type == gguf::kF64) scores_.push_back(static_cast<float>(v.f));
    bos_ = id_from(file, "tokenizer.ggml.bos_token_id");
    eos_ = id_from(file, "tokenizer.ggml.eos_token_id");
    unk_ = id_from(file, "tokenizer.ggml.unk_token_id");
    for (size_t i = 0; i < bytes_.size(); ++i) id_of_[bytes_[i]] = i;   // a repeated piece keeps its highest id
    if (const gguf::Value* m = file.find_kv("tokenizer.ggml.merges"); m && m->type == gguf::kArray)
        for (size_t rank = 0; rank < m->arr.size(); ++rank) {
            const gguf::Value& v = m->arr[rank];
            if (v.type == gguf::kString && v.s.find(' ') != std::string::npos) merge_rank_[v.s] = rank;
        }
    for (size_t i = 0; i < bytes_.size(); ++i)
        if (!bytes_[i].empty()) by_lead_[static_cast<unsigned char>(bytes_[i][0])].push_back(static_cast<uint32_t>(i));
    for (auto& ids : by_lead_)
        std::sort(ids.begin(), ids.end(), [&](uint32_t a, uint32_t b) {
            return raw_[a].size() != raw_[b].size() ? raw_[a].size() > raw_[b].size() : a < b;
        });
}

std::vector<uint64_t> Tokenizer::encode(const std::string& text, bool add_bos, bool add_eos) const {
    std::vector<uint64_t> ids;
    if (!valid()) return ids;
    if (add_bos && bos_ != kNoToken) ids.push_back(bos_);
    const bool scores_cover = scores_.size() == raw_.size();
    if (model_ == Model::kUnigram) {
        if (scores_cover) segment_by_score(text, ids);
    } else if (model_ == Model::kMerges) {
        if (!merge_rank_.empty()) segment_by_merges(text, ids);
    } else if (!merge_rank_.empty()) {
        segment_by_merges(text, ids);
    } else if (scores_cover) {
        segment_by_score(text, ids);
    }
    if (ids.empty()) segment_greedy(text, ids);
    if (add_eos && eos_ != kNoToken) ids.push_back(eos_);
    return ids;
}

void Tokenizer::segment_by_score(const std::string& text, std::vector<uint64_t>& out) const {
    const size_t n = text.size();
    if (n == 0) return;
    constexpr float kNever = -std::numeric_limits<float>::infinity();
    struct Cell { float score; uint64_t id; size_t from; };
    std::vector<Cell> best(n + 1, Cell{kNever, kNoToken, n + 1});
    best[0].score = 0.0f;
    const float unknown_cost = unk_ < scores_.size() ? scores_[unk_] : -1.0f;
    for (size_t pos = 0; pos < n; ++pos) {
        if (best[pos].score == kNever) continue;
        auto offer = [&](size_t end, float score, uint64_t id) {
            if (score > best[end].score) best[end] = Cell{score, id, pos};
        };
        for (uint32_t id : by_lead_[static_cast<unsigned char>(text[pos])]) {
            const std::string& piece = bytes_[id];
            if (pos + piece.size() > n || std::memcmp(text.data() + pos, piece.data(), piece.size()) != 0) continue;
            float score = best[pos].score;
            if (id < scores_.size()) score += scores_[id];
            offer(pos + piece.size(), score, id);
        }
        offer(pos + 1, best[pos].score + unknown_cost, unknown());   // one byte as the unknown token
    }
    if (best[n].id == kNoToken) return;
    const size_t first = out.size();
    for (size_t cur = n; cur > 0 && cur <= n;) {
        out.push_back(best[cur].id);
        if (best[cur].from >= cur) break;
        cur = best[cur].from;
    }
    std::reverse(out.begin() + static_cast<std::ptrdiff_t>(first), out.end());
}

void Tokenizer::segment_by_merges(const std::string& text, std::vector<uint64_t>& out) const {
    if (text.empty()) return;
    // symbols are consecutive stretches of the text: [cut[i], cut[i + 1])
    std::vector<size_t> cut(text.size() + 1);
    for (size_t i = 0; i <= text.size(); ++i) cut[i] = i;
    std::string key;
    while (cut.size() > 2) {
        size_t best_rank = std::numeric_limits<size_t>::max(), best_at = 0;
        for (size_t i = 0; i + 2 < cut.size(); ++i) {
            key.assign(text, cut[i], cut[i + 1] - cut[i]);
            key.push_back(' ');
            key.append(text, cut[i + 1], cut[i + 2] - cut[i + 1]);
            auto it = merge_rank_.find(key);
            if (it != merge_rank_.end() && it->second < best_rank) {
                best_rank = it->second;
                best_at = i;
            }
        }
        if (best_rank == std::numeric_limits<size_t>::max()) break;
        cut.erase(cut.begin() + static_cast<std::ptrdiff_t>(best_at) + 1);   // the two symbols become one
    }
    for (size_t i = 0; i + 1 < cut.size(); ++i) {
        auto it = id_of_.find(text.substr(cut[i], cut[i + 1] - cut[i]));
        out.push_back(it != id_of_.end() ? it->second : unknown());
    }
}

void Tokenizer::segment_greedy(const std::string& text, std::vector<uint64_t>& out) const {
    size_t pos = 0;
    while (pos < text.size()) {
        size_t taken = 0;
        for (uint32_t id : by_lead_[static_cast<unsigned char>(text[pos])]) {
            const std::string& piece = bytes_[id];
            if (piece.size() <= text.size() - pos && std::memcmp(text.data() + pos, piece.data(), piece.size()) == 0) {
                out.push_back(id);
                taken = piece.size();
                break;
            }
        }
        if (!taken) {
            out.push_back(unknown());
            taken = 1;
        }
        pos += taken;
    }
}

std::string Tokenizer::decode(const uint64_t* ids, size_t n) const {
    std::string out;
    for (size_t i = 0; i < n; ++i) {
        if (ids[i] >= bytes_.size()) continue;
        const std::string& piece = bytes_[ids[i]];
        if (piece == "<s>" || piece == "</s>" || piece == "<unk>") continue;
        if (starts_with_word_mark(piece)) {
            if (piece.size() > 3) {
                if (!out.empty()) out.push_back(' ');
                out.append(piece, 3, std::string::npos);
            }
        } else {
            out.append(piece);
        }
    }
    return out;
}

bool Tokenizer::is_control(uint64_t id) const {
    if (id >= raw_.size()) return false;
    const std::string& t = raw_[id];
    if (t == "<s>" || t == "</s>" || t == "<unk>") return true;
    return t.size() >= 3 && t[0] == '<' && t[1] == '|' && t.back() == '>';
}

}  // namespace text
}  // namespace mlcb
