// Byte-level BPE tokenizer for the DeepSeek ("deepseek-llm" pre-tokenizer, tokenizer.ggml.model = "gpt2").
//
// Same behaviour as the reference's llm_tokenizer_bpe (src/llama-vocab.cpp:76-98 pre-split rules, 142-236 merge
// loop, 956-1087 special-token partition, 1112-1239 detokenisation) with a hand-written scanner for the six
// pre-split rules instead of std::regex over collapsed code points (src/unicode.cpp:678-857).
#pragma once
#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>

namespace jib {

enum TokenType : int32_t { TOK_UNDEFINED = 0, TOK_NORMAL = 1, TOK_UNKNOWN = 2, TOK_CONTROL = 3, TOK_USER_DEFINED = 4, TOK_UNUSED = 5, TOK_BYTE = 6 };

struct TokenizerConfig {
    int32_t bos = 11, eos = 11, eot = -1, pad = -1;     // reference defaults for BPE vocabularies: bos = eos = 11
    bool add_bos = false, add_eos = false;
};

class Tokenizer {
  public:
    Tokenizer(std::vector<std::string> tokens, std::vector<int32_t> types, const std::vector<std::string> & merges, TokenizerConfig cfg);

    int n_tokens() const { return (int) tokens_.size(); }
    const TokenizerConfig & config() const { return cfg_; }
    bool is_eog(int32_t id) const;
    bool is_control(int32_t id) const { return id >= 0 && id < n_tokens() && (types_[id] == TOK_CONTROL || types_[id] == TOK_UNKNOWN); }

    std::vector<int32_t> encode(const std::string & text, bool add_special, bool parse_special) const;
    // Bytes of one token ("piece"). Control / unknown tokens render only when `special`.
    std::string token_to_piece(int32_t id, bool special) const;
    std::string decode(const std::vector<int32_t> & ids, bool remove_special, bool unparse_special) const;

    // Pre-split of raw text into BPE "words" (exposed for tests).
    static std::vector<std::string> pre_split(const std::string & text);

  private:
    void bpe_word(const std::string & word, std::vector<int32_t> & out) const;

    std::vector<std::string> tokens_;
    std::vector<int32_t> types_;
    std::unordered_map<std::string, int32_t> token_id_;
    std::unordered_map<std::string, int32_t> rank_;          // "left right" -> merge rank
    std::vector<int32_t> special_ids_;                        // control/user-defined/unknown, longest text first
    std::vector<std::string> piece_cache_;                    // decoded bytes per token
    std::vector<int32_t> eog_;
    TokenizerConfig cfg_;
};

// UTF-8 helpers shared with the server (hold back output that ends in an incomplete sequence:
// reference examples/server/server.cpp:1078-1107, common/utils.hpp:160-193).
size_t utf8_incomplete_tail(const std::string & s);
bool utf8_valid(const std::string & s);

}  // namespace jib
