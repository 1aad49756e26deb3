#include "tokenizers.hpp"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <limits>

namespace coeus {

// ------------------------------------------------------------------------------ UTF-8
bool is_unicode_whitespace(uint32_t cp) {
  return (cp >= 0x9 && cp <= 0xD) || cp == 0x20 || cp == 0x85 || cp == 0xA0 || cp == 0x1680 ||
         (cp >= 0x2000 && cp <= 0x200A) || cp == 0x2028 || cp == 0x2029 || cp == 0x202F ||
         cp == 0x205F || cp == 0x3000;
}

uint32_t utf8_next(std::string_view s, size_t& i) {
  const unsigned char c = static_cast<unsigned char>(s[i]);
  auto cont = [&](size_t k) {
    return i + k < s.size() && (static_cast<unsigned char>(s[i + k]) & 0xC0) == 0x80;
  };
  if (c < 0x80) { i += 1; return c; }
  if ((c & 0xE0) == 0xC0 && cont(1)) {
    const uint32_t cp = ((c & 0x1Fu) << 6) | (static_cast<unsigned char>(s[i + 1]) & 0x3Fu);
    i += 2;
    return cp;
  }
  if ((c & 0xF0) == 0xE0 && cont(1) && cont(2)) {
    const uint32_t cp = ((c & 0x0Fu) << 12) | ((static_cast<unsigned char>(s[i + 1]) & 0x3Fu) << 6) |
                        (static_cast<unsigned char>(s[i + 2]) & 0x3Fu);
    i += 3;
    return cp;
  }
  if ((c & 0xF8) == 0xF0 && cont(1) && cont(2) && cont(3)) {
    const uint32_t cp = ((c & 0x07u) << 18) | ((static_cast<unsigned char>(s[i + 1]) & 0x3Fu) << 12) |
                        ((static_cast<unsigned char>(s[i + 2]) & 0x3Fu) << 6) |
                        (static_cast<unsigned char>(s[i + 3]) & 0x3Fu);
    i += 4;
    return cp;
  }
  i += 1;
  return 0xFFFD;
}

void utf8_append(std::string& out, uint32_t cp) {
  if (cp < 0x80) {
    out.push_back(static_cast<char>(cp));
  } else if (cp < 0x800) {
    out.push_back(static_cast<char>(0xC0 | (cp >> 6)));
    out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
  } else if (cp < 0x10000) {
    out.push_back(static_cast<char>(0xE0 | (cp >> 12)));
    out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
    out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
  } else {
    out.push_back(static_cast<char>(0xF0 | (cp >> 18)));
    out.push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
    out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
    out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
  }
}

std::vector<std::string_view> split_whitespace(std::string_view text) {
  std::vector<std::string_view> out;
  size_t i = 0, start = std::string_view::npos;
  while (i < text.size()) {
    const size_t at = i;
    const unsigned char c = static_cast<unsigned char>(text[i]);
    uint32_t cp;
    if (c < 0x80) { cp = c; ++i; } else { cp = utf8_next(text, i); }
    if (is_unicode_whitespace(cp)) {
      if (start != std::string_view::npos) {
        out.push_back(text.substr(start, at - start));
        start = std::string_view::npos;
      }
    } else if (start == std::string_view::npos) {
      start = at;
    }
  }
  if (start != std::string_view::npos) out.push_back(text.substr(start));
  return out;
}

std::string BasicTokenizer::decode(const std::vector<std::string>& tokens) const {
  std::string out;
  for (size_t i = 0; i < tokens.size(); ++i) {
    if (i) out.push_back(' ');
    out += tokens[i];
  }
  return out;
}

// ------------------------------------------------------------------------------ BPE
static std::string byte_token_string(unsigned b) {
  if (b < 0x80) return std::string(1, static_cast<char>(b));
  char buf[8];
  std::snprintf(buf, sizeof(buf), "<0x%02X>", b);
  return buf;
}

BpeTokenizer::BpeTokenizer() {
  for (unsigned b = 0; b < 256; ++b) {
    const std::string s = byte_token_string(b);
    byte_tok_[b] = intern(s);
    add_token(s);  // ids 0..255 in order
  }
  const char* specials[4] = {"<PAD>", "<UNK>", "<BOS>", "<EOS>"};
  for (uint32_t id = 0; id < 4; ++id) {  // overlay: same ids as the control bytes 0..3
    vocab_[specials[id]] = id;
    reverse_vocab_[id] = specials[id];
  }
}

uint32_t BpeTokenizer::intern(const std::string& s) {
  auto it = tok_index_.find(s);
  if (it != tok_index_.end()) return it->second;
  const uint32_t idx = static_cast<uint32_t>(tok_str_.size());
  tok_str_.push_back(s);
  tok_index_.emplace(s, idx);
  return idx;
}

uint32_t BpeTokenizer::add_token(const std::string& token) {
  auto it = vocab_.find(token);
  if (it != vocab_.end()) return it->second;
  const uint32_t id = next_id_++;
  vocab_.emplace(token, id);
  reverse_vocab_[id] = token;
  cache_.clear();
  return id;
}

bool BpeTokenizer::remove_token(const std::string& token) {
  auto it = vocab_.find(token);
  if (it == vocab_.end()) return false;
  reverse_vocab_.erase(it->second);
  vocab_.erase(it);
  cache_.clear();
  return true;
}

bool BpeTokenizer::token_from_id(uint32_t id, std::string& out) const {
  auto it = reverse_vocab_.find(id);
  if (it == reverse_vocab_.end()) return false;
  out = it->second;
  return true;
}

bool BpeTokenizer::id_from_token(const std::string& token, uint32_t& out) const {
  auto it = vocab_.find(token);
  if (it == vocab_.end()) return false;
  out = it->second;
  return true;
}

std::pair<std::string, std::string> BpeTokenizer::merge_at(size_t i) const {
  return {tok_str_[merges_[i].a], tok_str_[merges_[i].b]};
}

static void apply_merge(std::vector<uint32_t>& toks, uint32_t a, uint32_t b, uint32_t merged) {
  size_t w = 0;
  for (size_t i = 0; i < toks.size();) {
    if (i + 1 < toks.size() && toks[i] == a && toks[i + 1] == b) {
      toks[w++] = merged;
      i += 2;
    } else {
      toks[w++] = toks[i++];
    }
  }
  toks.resize(w);
}

// Same result as the reference's "for each merge in learned order: one left-to-right pass"
// (lib.rs:245-271): merges are visited in increasing rank, and a rank that was passed is never
// revisited, but ranks with no occurrence in the word are skipped without a pass.
void BpeTokenizer::bpe_word(std::vector<uint32_t>& toks) const {
  int64_t last_rank = -1;
  while (toks.size() >= 2) {
    int64_t best = std::numeric_limits<int64_t>::max();
    for (size_t i = 0; i + 1 < toks.size(); ++i) {
      auto it = merge_rank_.find({toks[i], toks[i + 1]});
      if (it != merge_rank_.end() && static_cast<int64_t>(it->second) > last_rank &&
          static_cast<int64_t>(it->second) < best)
        best = it->second;
    }
    if (best == std::numeric_limits<int64_t>::max()) break;
    const Merge& m = merges_[static_cast<size_t>(best)];
    apply_merge(toks, m.a, m.b, m.merged);
    last_rank = best;
  }
}

void BpeTokenizer::train(const std::vector<std::string>& corpus, size_t num_merges) {
  std::unordered_map<std::string, size_t> word_count;
  for (const std::string& text : corpus)
    for (std::string_view w : split_whitespace(text)) ++word_count[std::string(w)];
  std::vector<std::pair<std::vector<uint32_t>, size_t>> words;
  words.reserve(word_count.size());
  for (auto& kv : word_count) {
    std::vector<uint32_t> toks;
    toks.reserve(kv.first.size());
    for (unsigned char c : kv.first) toks.push_back(byte_tok_[c]);
    words.emplace_back(std::move(toks), kv.second);
  }
  for (size_t step = 0; step < num_merges; ++step) {
    std::unordered_map<std::pair<uint32_t, uint32_t>, size_t, PairHash> freq;
    for (auto& w : words)
      for (size_t i = 0; i + 1 < w.first.size(); ++i) freq[{w.first[i], w.first[i + 1]}] += w.second;
    if (freq.empty()) break;
    std::pair<uint32_t, uint32_t> best{0, 0};
    size_t best_n = 0;
    for (auto& kv : freq) {
      bool better = kv.second > best_n;
      if (!better && kv.second == best_n) {
        const int c = tok_str_[kv.first.first].compare(tok_str_[best.first]);
        better = c < 0 || (c == 0 && tok_str_[kv.first.second] < tok_str_[best.second]);
      }
      if (better) { best = kv.first; best_n = kv.second; }
    }
    const std::string merged_str = tok_str_[best.first] + tok_str_[best.second];
    const uint32_t merged = intern(merged_str);
    merges_.push_back({best.first, best.second, merged});
    merge_rank_.emplace(best, static_cast<uint32_t>(merges_.size() - 1));  // keeps the first rank
    add_token(merged_str);
    for (auto& w : words) apply_merge(w.first, best.first, best.second, merged);
  }
  cache_.clear();
}

void BpeTokenizer::load_merges(const std::vector<std::pair<std::string, std::string>>& pairs) {
  for (const auto& pr : pairs) {
    const uint32_t a = intern(pr.first), b = intern(pr.second);
    const std::string merged_str = pr.first + pr.second;
    const uint32_t merged = intern(merged_str);
    merges_.push_back({a, b, merged});
    merge_rank_.emplace(std::make_pair(a, b), static_cast<uint32_t>(merges_.size() - 1));
    add_token(merged_str);
  }
  cache_.clear();
}

void BpeTokenizer::encode(std::string_view text, std::vector<uint32_t>& ids,
                          std::vector<std::string>* strings) {
  bool first = true;
  std::string key;
  for (std::string_view word : split_whitespace(text)) {
    if (!first) {
      ids.push_back(32);
      if (strings) strings->emplace_back(" ");
    }
    first = false;
    key.assign(word);
    auto it = cache_.find(key);
    if (it == cache_.end()) {
      std::vector<uint32_t> toks;
      toks.reserve(word.size());
      for (unsigned char c : word) toks.push_back(byte_tok_[c]);
      bpe_word(toks);
      if (cache_.size() > (1u << 20)) cache_.clear();
      it = cache_.emplace(key, std::move(toks)).first;
    }
    for (uint32_t t : it->second) {
      auto v = vocab_.find(tok_str_[t]);
      ids.push_back(v == vocab_.end() ? 1u : v->second);  // 1 = <UNK>
      if (strings) strings->push_back(tok_str_[t]);
    }
  }
}

static int hex_val(char c) {
  if (c >= '0' && c <= '9') return c - '0';
  if (c >= 'a' && c <= 'f') return c - 'a' + 10;
  if (c >= 'A' && c <= 'F') return c - 'A' + 10;
  return -1;
}

// A token of the form "<0xNN...>" decodes to the single byte NN read lossily: bytes >= 0x80
// become U+FFFD, exactly like String::from_utf8_lossy(&[byte]) in the reference (lib.rs:319-342).
static void decode_one(const std::string& s, std::string& out) {
  if (s.size() >= 6 && s.compare(0, 3, "<0x") == 0 && s.back() == '>') {
    const int hi = hex_val(s[3]), lo = hex_val(s[4]);
    if (hi >= 0 && lo >= 0) {
      const unsigned b = static_cast<unsigned>(hi * 16 + lo);
      if (b < 0x80) out.push_back(static_cast<char>(b)); else utf8_append(out, 0xFFFD);
      return;
    }
  }
  out += s;
}

// The same walk keeping every byte token as its byte, so that a multi-byte character whose bytes
// were never merged comes back whole (the caller validates the UTF-8 once, at the end).
std::string BpeTokenizer::decode_ids_bytes(const std::vector<uint32_t>& ids) const {
  std::string out;
  for (uint32_t id : ids) {
    if (id < 4) {   // the special tokens share the ids of the control bytes 0..3: bytes here
      out.push_back(static_cast<char>(id));
      continue;
    }
    auto it = reverse_vocab_.find(id);
    if (it == reverse_vocab_.end()) continue;
    const std::string& s = it->second;
    // a merged token is the concatenation of its parts' strings: every "<0xNN>" with NN >= 0x80
    // inside it is a byte token (bytes below 0x80 are stored as themselves, so a lower NN can
    // only be literal text)
    for (size_t i = 0; i < s.size();) {
      if (i + 6 <= s.size() && s.compare(i, 3, "<0x") == 0 && s[i + 5] == '>') {
        // byte tokens are written with upper-case digits; anything else is literal text
        auto up = [](char c) { return (c >= '0' && c <= '9') || (c >= 'A' && c <= 'F'); };
        const int hi = up(s[i + 3]) ? hex_val(s[i + 3]) : -1;
        const int lo = up(s[i + 4]) ? hex_val(s[i + 4]) : -1;
        if (hi >= 8 && lo >= 0) {
          out.push_back(static_cast<char>(hi * 16 + lo));
          i += 6;
          continue;
        }
      }
      out.push_back(s[i++]);
    }
  }
  return out;
}

std::string BpeTokenizer::decode_strings(const std::vector<std::string>& tokens) const {
  std::string out;
  for (const std::string& s : tokens) decode_one(s, out);
  return out;
}

std::string BpeTokenizer::decode_ids(const std::vector<uint32_t>& ids) const {
  std::string out;
  for (uint32_t id : ids) {
    auto it = reverse_vocab_.find(id);
    if (it != reverse_vocab_.end()) decode_one(it->second, out);
  }
  return out;
}

// ------------------------------------------------------------------------------ NFD
struct NfdEntry { uint32_t cp; uint32_t d[4]; };
struct CccEntry { uint32_t cp; int ccc; };
#include "unicode_tables.inc"

static const NfdEntry* find_nfd(uint32_t cp) {
  const NfdEntry* lo = kNfd;
  const NfdEntry* hi = kNfd + sizeof(kNfd) / sizeof(kNfd[0]);
  const NfdEntry* it = std::lower_bound(lo, hi, cp, [](const NfdEntry& e, uint32_t v) { return e.cp < v; });
  return (it != hi && it->cp == cp) ? it : nullptr;
}
static int ccc_of(uint32_t cp) {
  const CccEntry* lo = kCcc;
  const CccEntry* hi = kCcc + sizeof(kCcc) / sizeof(kCcc[0]);
  const CccEntry* it = std::lower_bound(lo, hi, cp, [](const CccEntry& e, uint32_t v) { return e.cp < v; });
  return (it != hi && it->cp == cp) ? it->ccc : 0;
}

static void decompose(uint32_t cp, std::vector<uint32_t>& out) {
  if (cp >= 0xAC00 && cp <= 0xD7A3) {  // Hangul syllables
    const uint32_t s = cp - 0xAC00;
    out.push_back(0x1100 + s / 588);
    out.push_back(0x1161 + (s % 588) / 28);
    if (s % 28) out.push_back(0x11A7 + s % 28);
    return;
  }
  if (cp >= 0x80 && cp < 0x10000) {
    if (const NfdEntry* e = find_nfd(cp)) {
      for (int i = 0; i < 4 && e->d[i]; ++i) out.push_back(e->d[i]);
      return;
    }
  }
  out.push_back(cp);
}

static std::vector<uint32_t> nfd_codepoints(std::string_view text) {
  std::vector<uint32_t> cps;
  for (size_t i = 0; i < text.size();) decompose(utf8_next(text, i), cps);
  // canonical ordering: stable sort of each run of non-starters by combining class
  size_t i = 0;
  while (i < cps.size()) {
    if (ccc_of(cps[i]) == 0) { ++i; continue; }
    size_t j = i;
    while (j < cps.size() && ccc_of(cps[j]) != 0) ++j;
    std::stable_sort(cps.begin() + i, cps.begin() + j,
                     [](uint32_t a, uint32_t b) { return ccc_of(a) < ccc_of(b); });
    i = j;
  }
  return cps;
}

std::string nfd(std::string_view text) {
  std::string out;
  for (uint32_t cp : nfd_codepoints(text)) utf8_append(out, cp);
  return out;
}

bool is_nfd(std::string_view text) { return nfd(text) == text; }

// ------------------------------------------------------------------------------ words
static bool is_digit_cp(uint32_t cp) { return cp >= '0' && cp <= '9'; }
static bool is_extend(uint32_t cp) {
  return (cp >= 0x300 && cp <= 0x36F) || (cp >= 0x1AB0 && cp <= 0x1AFF) ||
         (cp >= 0x1DC0 && cp <= 0x1DFF) || (cp >= 0x20D0 && cp <= 0x20FF) || cp == 0x200D;
}
static bool is_letter_cp(uint32_t cp) {
  if ((cp >= 'a' && cp <= 'z') || (cp >= 'A' && cp <= 'Z')) return true;
  if (cp < 0xAA) return false;
  if (cp == 0xAA || cp == 0xB5 || cp == 0xBA) return true;
  if (cp < 0xC0) return false;
  if (cp == 0xD7 || cp == 0xF7) return false;
  if (cp >= 0x2000 && cp <= 0x2BFF) return false;   // punctuation, symbols, arrows, ...
  if (cp >= 0x3000 && cp <= 0x303F) return false;   // CJK punctuation
  if (cp >= 0xFE00 && cp <= 0xFE6F) return false;
  if (cp >= 0xFF00 && cp <= 0xFF0F) return false;
  if (is_extend(cp) || is_unicode_whitespace(cp)) return false;
  return true;
}

std::vector<std::string> unicode_words(std::string_view text) {
  std::vector<uint32_t> cps;
  for (size_t i = 0; i < text.size();) cps.push_back(utf8_next(text, i));
  std::vector<std::string> out;
  size_t i = 0;
  const size_t n = cps.size();
  auto alnum = [&](uint32_t c) { return is_letter_cp(c) || is_digit_cp(c) || c == '_'; };
  while (i < n) {
    if (!alnum(cps[i])) { ++i; continue; }
    std::string w;
    bool has_alnum = false;
    while (i < n) {
      const uint32_t c = cps[i];
      if (alnum(c)) {
        utf8_append(w, c);
        has_alnum = has_alnum || c != '_';
        ++i;
      } else if (is_extend(c)) {
        utf8_append(w, c);
        ++i;
      } else if (i + 1 < n && i > 0) {
        const uint32_t prev = cps[i - 1], next = cps[i + 1];
        const bool mid_letter = (c == '\'' || c == '.' || c == ':' || c == 0xB7 || c == 0x2019) &&
                                is_letter_cp(prev) && is_letter_cp(next);
        const bool mid_num = (c == ',' || c == '.' || c == ';' || c == '\'') && is_digit_cp(prev) &&
                             is_digit_cp(next);
        if (mid_letter || mid_num) {
          utf8_append(w, c);
          ++i;
        } else {
          break;
        }
      } else {
        break;
      }
    }
    if (has_alnum || !w.empty()) out.push_back(std::move(w));
  }
  return out;
}

// ------------------------------------------------------------------------------ WordPiece
WordPieceTokenizer::WordPieceTokenizer() {
  trie_.emplace_back();
  const char* specials[5] = {"[UNK]", "[CLS]", "[SEP]", "[PAD]", "[MASK]"};
  for (uint32_t i = 0; i < 5; ++i) add_token(specials[i], i);
  uint32_t id = 100;
  for (char c = 'a'; c <= 'z'; ++c) add_token(std::string(1, c), id++);
  for (char c = 'A'; c <= 'Z'; ++c) add_token(std::string(1, c), id++);
  const char* subwords[13] = {"##ing", "##ed", "##er", "##est", "##ly", "##tion", "##ness",
                              "##ment", "##able", "##ible", "##ful", "##less", "##ous"};
  for (const char* s : subwords) add_token(s, id++);
}

void WordPieceTokenizer::add_token(const std::string& token, uint32_t id) {
  int node = 0;
  for (size_t i = 0; i < token.size();) {
    const uint32_t cp = utf8_next(token, i);
    auto it = trie_[node].next.find(cp);
    if (it == trie_[node].next.end()) {
      trie_.emplace_back();
      const int nn = static_cast<int>(trie_.size()) - 1;
      trie_[node].next.emplace(cp, nn);
      node = nn;
    } else {
      node = it->second;
    }
  }
  trie_[node].token_id = id;
  token_to_id_[token] = id;
  id_to_token_[id] = token;
}

bool WordPieceTokenizer::longest_match(std::string_view text, uint32_t& id, size_t& chars) const {
  int node = 0;
  bool found = false;
  size_t count = 0;
  for (size_t i = 0; i < text.size();) {
    const uint32_t cp = utf8_next(text, i);
    auto it = trie_[node].next.find(cp);
    if (it == trie_[node].next.end()) break;
    node = it->second;
    ++count;
    if (trie_[node].token_id >= 0) {
      found = true;
      id = static_cast<uint32_t>(trie_[node].token_id);
      chars = count;
    }
  }
  return found;
}

std::vector<uint32_t> WordPieceTokenizer::tokenize_word(std::string_view word) const {
  std::vector<uint32_t> out;
  std::string_view remaining = word;
  bool first = true;
  while (!remaining.empty()) {
    const size_t prefix_chars = first ? 0 : 2;
    std::string search = first ? std::string() : std::string("##");
    search.append(remaining);
    uint32_t id = 0;
    size_t chars = 0;
    if (!longest_match(search, id, chars) || chars <= prefix_chars) {
      out.push_back(0);  // [UNK]; the rest of the word is abandoned (lib.rs:281-285)
      break;
    }
    out.push_back(id);
    size_t consumed = chars - prefix_chars, pos = 0;
    while (consumed-- > 0 && pos < remaining.size()) utf8_next(remaining, pos);
    remaining = remaining.substr(pos);
    first = false;
  }
  return out;
}

std::vector<uint32_t> WordPieceTokenizer::encode(std::string_view text) const {
  const std::string normalized = nfd(text);
  std::vector<uint32_t> out{1};  // [CLS]
  for (const std::string& w : unicode_words(normalized))
    for (uint32_t id : tokenize_word(w))
      if (id_to_token_.count(id)) out.push_back(id);
  out.push_back(2);  // [SEP]
  return out;
}

std::string WordPieceTokenizer::decode_strings(const std::vector<std::string>& tokens) const {
  std::string out;
  bool first = true;
  for (const std::string& t : tokens) {
    if (!t.empty() && t.front() == '[' && t.back() == ']') continue;
    if (t.compare(0, 2, "##") == 0) {
      out.append(t, 2, std::string::npos);
    } else {
      if (!first) out.push_back(' ');
      out += t;
      first = false;
    }
  }
  return out;
}

bool WordPieceTokenizer::id_to_token(uint32_t id, std::string& out) const {
  auto it = id_to_token_.find(id);
  if (it == id_to_token_.end()) return false;
  out = it->second;
  return true;
}

bool WordPieceTokenizer::token_to_id(const std::string& t, uint32_t& out) const {
  auto it = token_to_id_.find(t);
  if (it == token_to_id_.end()) return false;
  out = it->second;
  return true;
}

}  // namespace coeus
