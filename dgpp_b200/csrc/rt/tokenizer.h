// Byte-level BPE tokenizer reading Hugging Face `tokenizer.json`:
//   * optional NFC normalisation (canonical decomposition, reordering, composition)
//   * added / special tokens split off first (longest match at each position)
//   * pre-tokenisation by one of the pinned split patterns, implemented as hand-written scanners over
//     Unicode categories (no regex engine):
//        Gpt2      's|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+
//        Cl100k    (?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+
//        Qwen2     as Cl100k with single digits (\p{N})
//        Whole     no split (the whole segment is one word)
//   * bytes -> printable code points (the GPT-2 table), then rank-ordered pair merges with a heap;
//     `ignore_merges` looks the whole word up in the vocabulary first
//   * a bounded word cache
//   * decoding is incremental and never emits a partial UTF-8 sequence
// (behavioural spec: src/text/tokenizer.cpp:1-1135, src/text/bpe.hpp, docs/tokenization.md of the reference)
#pragma once
#include <cstdint>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace dgpp {

enum class SplitPattern { Gpt2, Cl100k, Qwen2, Whole };

struct AddedToken {
  std::string content;
  int32_t id;
  bool special;
};

class Tokenizer {
 public:
  // Builds from the text of a tokenizer.json.  Throws std::runtime_error on malformed input.
  static Tokenizer from_json(const std::string& json_text);
  // A self-contained byte-level tokenizer (256 byte tokens + the given merges), for tests and synthetic runs.
  static Tokenizer byte_level(const std::vector<std::pair<std::string, std::string>>& merges,
                              const std::vector<AddedToken>& added, SplitPattern pattern);

  std::vector<int32_t> encode(const std::string& text, bool allow_special = true) const;
  std::string decode(const std::vector<int32_t>& ids, bool skip_special = false) const;
  // Bytes of one token (after undoing the byte -> code point table); empty for unknown ids.
  const std::string& token_bytes(int32_t id) const;
  int32_t token_to_id(const std::string& token) const;  // -1 when absent (raw bytes or added-token text)
  int32_t vocab_size() const { return static_cast<int32_t>(id_to_bytes_.size()); }
  bool is_special(int32_t id) const;
  SplitPattern pattern() const { return pattern_; }
  bool nfc() const { return nfc_; }
  std::vector<std::string> pre_tokenize(const std::string& text) const;  // exposed for tests
  static std::string normalize_nfc(const std::string& utf8);
  uint64_t fingerprint() const;  // hash of vocabulary + merges (keys golden files)

 private:
  void finish();
  void encode_word(const std::string& word, std::vector<int32_t>& out) const;
  void encode_segment(const std::string& text, std::vector<int32_t>& out) const;

  std::unordered_map<std::string, int32_t> vocab_;        // mapped (printable) token string -> id
  std::unordered_map<std::string, int32_t> merge_rank_;   // "left\x01right" -> rank
  std::vector<std::string> id_to_bytes_;                  // raw bytes per id
  std::vector<uint8_t> special_;                          // per id
  std::vector<AddedToken> added_;
  std::unordered_map<std::string, int32_t> added_lookup_;
  std::vector<uint8_t> added_first_byte_;                 // 256 flags
  size_t added_max_len_ = 0;
  SplitPattern pattern_ = SplitPattern::Gpt2;
  bool nfc_ = false;
  bool ignore_merges_ = false;
  mutable std::unordered_map<std::string, std::vector<int32_t>> cache_;
  std::string empty_;
};

// Incremental detokeniser: feed ids, get text that is always valid UTF-8 (an incomplete trailing
// sequence is held back until its continuation bytes arrive).
class StreamDecoder {
 public:
  explicit StreamDecoder(const Tokenizer* tok, bool skip_special = true) : tok_(tok), skip_special_(skip_special) {}
  std::string push(int32_t id);
  std::string flush();

 private:
  const Tokenizer* tok_;
  bool skip_special_;
  std::string pending_;
};

}  // namespace dgpp
