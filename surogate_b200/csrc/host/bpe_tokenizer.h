// Byte-level BPE tokenizer reading HuggingFace `tokenizer.json` (GPT-2 / Qwen / Llama-3 style vocabularies).
// The hot path (pre-tokenisation, merges, batch encode on a thread pool) is native; chat templates are rendered by the
// Python wrapper, which calls `encode` per rendered span to build loss masks.
// Reference counterpart: csrc/src/tokenizer/tokenizer.h:39-122, bpe.h.
#pragma once
#include <cstdint>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace sg {

struct PreTokenizerStyle {
    bool legacy_gpt2 = false;           // " ?\p{L}+" alternatives instead of "[^\r\n\p{L}\p{N}]?\p{L}+"
    bool contractions_ignore_case = true;
    int max_digits = 1;                 // digits per number piece; 0 = unlimited
};

class BpeTokenizer {
public:
    static std::shared_ptr<BpeTokenizer> from_file(const std::string& tokenizer_json_path);
    static std::shared_ptr<BpeTokenizer> from_json(const std::string& json_text);

    std::vector<int32_t> encode(const std::string& text, bool allow_added_tokens = true) const;
    std::vector<std::vector<int32_t>> encode_batch(const std::vector<std::string>& texts, bool allow_added_tokens, int threads) const;
    std::string decode(const std::vector<int32_t>& ids, bool skip_special = false) const;
    std::vector<std::string> pre_tokenize(const std::string& text) const;

    int32_t vocab_size() const { return static_cast<int32_t>(id_to_bytes_.size()); }
    int32_t token_to_id(const std::string& token_bytes) const;
    const std::string& id_to_token(int32_t id) const;
    bool is_special(int32_t id) const;
    const std::vector<std::pair<std::string, int32_t>>& added_tokens() const { return added_; }
    PreTokenizerStyle style() const { return style_; }

private:
    void encode_word(const std::string& word, std::vector<int32_t>& out) const;
    void encode_plain(const std::string& text, std::vector<int32_t>& out) const;

    PreTokenizerStyle style_;
    bool ignore_merges_ = false;
    std::unordered_map<std::string, int32_t> bytes_to_id_;
    std::vector<std::string> id_to_bytes_;
    std::vector<uint8_t> special_;
    std::unordered_map<uint64_t, std::pair<int32_t, int32_t>> merges_;  // (left id << 32 | right id) -> (rank, merged id)
    std::vector<std::pair<std::string, int32_t>> added_;                // content -> id, longest first
    int32_t byte_id_[256];
    mutable std::unordered_map<std::string, std::vector<int32_t>> cache_;
    mutable std::mutex cache_mu_;
};

// Unicode helpers shared with tests.
bool unicode_is_letter(uint32_t cp);
bool unicode_is_number(uint32_t cp);
bool unicode_is_space(uint32_t cp);

}  // namespace sg
