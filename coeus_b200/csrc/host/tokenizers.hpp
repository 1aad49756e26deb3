// Native tokenizers: whitespace, byte-level BPE (with trainer) and WordPiece.
// Observable behaviour follows the reference plugins (plugins/tokenizer-basic/src/lib.rs,
// plugins/tokenizer-bpe/src/lib.rs, plugins/tokenizer-wordpiece/src/lib.rs); the data structures
// do not: ids instead of heap strings per byte, a per-word cache, merge lookup by hashed pair.
#pragma once
#include <cstdint>
#include <string>
#include <string_view>
#include <unordered_map>
#include <utility>
#include <vector>

namespace coeus {

// ---- whitespace helpers (Rust's char::is_whitespace on the code points that matter here)
bool is_unicode_whitespace(uint32_t cp);
// Decodes one UTF-8 code point at s[i]; advances i.  Invalid bytes yield U+FFFD and advance by 1.
uint32_t utf8_next(std::string_view s, size_t& i);
void utf8_append(std::string& out, uint32_t cp);
std::vector<std::string_view> split_whitespace(std::string_view text);

// ------------------------------------------------------------------------------------------
class BasicTokenizer {
 public:
  std::vector<std::string_view> tokenize(std::string_view text) const { return split_whitespace(text); }
  std::string decode(const std::vector<std::string>& tokens) const;
};

// ------------------------------------------------------------------------------------------
struct PairHash {
  size_t operator()(const std::pair<uint32_t, uint32_t>& p) const {
    return (static_cast<uint64_t>(p.first) << 32 | p.second) * 0x9E3779B97F4A7C15ull >> 13;
  }
};

class BpeTokenizer {
 public:
  BpeTokenizer();
  // Learns up to num_merges merges from whitespace-split words of the corpus.  Ties between
  // equally frequent pairs go to the pair with the smallest (first string, second string); the
  // reference leaves ties to hash-map iteration order.
  void train(const std::vector<std::string>& corpus, size_t num_merges);
  // Replays merges learned elsewhere, in order, on a fresh tokenizer: the vocabulary ids come
  // out as training assigned them (persistence of a trained tokenizer).
  void load_merges(const std::vector<std::pair<std::string, std::string>>& pairs);
  // ids with a space token (id 32) between words; `strings` (optional) receives the token text.
  void encode(std::string_view text, std::vector<uint32_t>& ids,
              std::vector<std::string>* strings = nullptr);
  std::string decode_strings(const std::vector<std::string>& tokens) const;
  std::string decode_ids(const std::vector<uint32_t>& ids) const;
  // Raw bytes: byte tokens stay bytes (no per-byte lossy conversion); may be invalid UTF-8.
  std::string decode_ids_bytes(const std::vector<uint32_t>& ids) const;
  size_t vocab_size() const { return vocab_.size(); }
  uint32_t add_token(const std::string& token);
  bool remove_token(const std::string& token);
  bool contains_token(const std::string& token) const { return vocab_.count(token) != 0; }
  bool token_from_id(uint32_t id, std::string& out) const;
  bool id_from_token(const std::string& token, uint32_t& out) const;
  size_t num_merges() const { return merges_.size(); }
  std::pair<std::string, std::string> merge_at(size_t i) const;
  void clear_cache() { cache_.clear(); }

 private:
  uint32_t intern(const std::string& s);        // id of a working token string
  void bpe_word(std::vector<uint32_t>& toks) const;
  // Working token space: every distinct token string that can occur while merging has a dense
  // "tok" index; tok_str_ holds the strings, tok_vocab_id_ the vocabulary id (or UNK = 1).
  std::vector<std::string> tok_str_;
  std::unordered_map<std::string, uint32_t> tok_index_;
  uint32_t byte_tok_[256];
  struct Merge { uint32_t a, b, merged; };
  std::vector<Merge> merges_;
  std::unordered_map<std::pair<uint32_t, uint32_t>, uint32_t, PairHash> merge_rank_;
  std::unordered_map<std::string, uint32_t> vocab_;
  std::unordered_map<uint32_t, std::string> reverse_vocab_;
  uint32_t next_id_ = 0;
  std::unordered_map<std::string, std::vector<uint32_t>> cache_;  // word -> toks
};

// ------------------------------------------------------------------------------------------
std::string nfd(std::string_view text);
bool is_nfd(std::string_view text);
// UAX-29-style word segmentation restricted to what unicode_words() returns: maximal runs that
// contain a letter or digit, allowing ' . : between letters and , . ; between digits.
std::vector<std::string> unicode_words(std::string_view text);

class WordPieceTokenizer {
 public:
  WordPieceTokenizer();
  void add_token(const std::string& token, uint32_t id);
  // [CLS] ... [SEP] ids of the NFD-normalised text.
  std::vector<uint32_t> encode(std::string_view text) const;
  std::vector<uint32_t> tokenize_word(std::string_view word) const;
  std::string decode_strings(const std::vector<std::string>& tokens) const;
  bool id_to_token(uint32_t id, std::string& out) const;
  bool token_to_id(const std::string& t, uint32_t& out) const;
  size_t vocab_size() const { return id_to_token_.size(); }
  // (id, code points matched) of the longest vocabulary entry that prefixes `text`
  bool longest_match(std::string_view text, uint32_t& id, size_t& chars) const;

 private:
  struct Node {
    std::unordered_map<uint32_t, int> next;
    int64_t token_id = -1;
  };
  std::vector<Node> trie_;
  std::unordered_map<std::string, uint32_t> token_to_id_;
  std::unordered_map<uint32_t, std::string> id_to_token_;
};

}  // namespace coeus
