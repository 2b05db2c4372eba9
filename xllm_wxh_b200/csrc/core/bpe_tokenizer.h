// Byte-level BPE tokenizer (GPT-2 / Qwen / tiktoken family) in C++.
//
// The reference links the Rust HF `tokenizers` crate through a C ABI
// (xllm/core/framework/tokenizer/tokenizers/src/lib.rs:77-224) and a tiktoken loader
// (tokenizer/tiktoken_tokenizer.cpp).  This implementation covers the same two file
// formats for byte-level BPE models: the caller hands over the vocabulary as raw byte
// strings with ids (ranks) plus the merge list, and picks the pre-tokenizer flavour.
//
// Pre-tokenizer: a hand-written scanner equivalent to the regular expression
//   (?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,D}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+
// with D = 1 (Qwen2/Qwen3) or D = 3 (cl100k-style).
#pragma once
#include <algorithm>
#include <cstdint>
#include <limits>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "unicode_tables.h"

namespace xl {

namespace detail {
inline bool in_ranges(const uint32_t (*tab)[2], int n, uint32_t cp) {
  int lo = 0, hi = n - 1;
  while (lo <= hi) {
    int mid = (lo + hi) >> 1;
    if (cp < tab[mid][0]) hi = mid - 1;
    else if (cp > tab[mid][1]) lo = mid + 1;
    else return true;
  }
  return false;
}
inline bool is_letter(uint32_t cp) {
  if (cp < 128) return (cp >= 'a' && cp <= 'z') || (cp >= 'A' && cp <= 'Z');
  return in_ranges(unicode::kLetter, unicode::kLetter_len, cp);
}
inline bool is_number(uint32_t cp) {
  if (cp < 128) return cp >= '0' && cp <= '9';
  return in_ranges(unicode::kNumber, unicode::kNumber_len, cp);
}
inline bool is_space(uint32_t cp) {
  if (cp < 128) return cp == ' ' || (cp >= 9 && cp <= 13);
  return in_ranges(unicode::kSpace, unicode::kSpace_len, cp);
}
// Decode one UTF-8 code point at s[i]; invalid bytes decode as themselves (length 1).
inline uint32_t utf8_at(const std::string& s, size_t i, int* len) {
  unsigned char c = s[i];
  auto cont = [&](size_t k) { return i + k < s.size() && (static_cast<unsigned char>(s[i + k]) & 0xC0) == 0x80; };
  if (c < 0x80) { *len = 1; return c; }
  if ((c >> 5) == 6 && cont(1)) { *len = 2; return ((c & 0x1F) << 6) | (s[i + 1] & 0x3F); }
  if ((c >> 4) == 14 && cont(1) && cont(2)) {
    *len = 3;
    return ((c & 0x0F) << 12) | ((s[i + 1] & 0x3F) << 6) | (s[i + 2] & 0x3F);
  }
  if ((c >> 3) == 30 && cont(1) && cont(2) && cont(3)) {
    *len = 4;
    return ((c & 0x07) << 18) | ((s[i + 1] & 0x3F) << 12) | ((s[i + 2] & 0x3F) << 6) | (s[i + 3] & 0x3F);
  }
  *len = 1;
  return 0xFFFD;  // treated as "other"
}
}  // namespace detail

class BpeTokenizer {
 public:
  // vocab: (token bytes, id); merges: (left bytes, right bytes) in priority order.  When `merges` is
  // empty the ids themselves are the merge ranks (tiktoken files).
  void load_vocab(const std::vector<std::pair<std::string, int>>& vocab,
                  const std::vector<std::pair<std::string, std::string>>& merges, int max_digits) {
    max_digits_ = std::max(1, max_digits);
    tok2id_.clear();
    id2tok_.clear();
    ranks_.clear();
    int max_id = -1;
    for (auto& kv : vocab) max_id = std::max(max_id, kv.second);
    id2tok_.assign(max_id + 1, std::string());
    for (auto& kv : vocab) {
      tok2id_[kv.first] = kv.second;
      id2tok_[kv.second] = kv.first;
    }
    use_id_as_rank_ = merges.empty();
    int r = 0;
    for (auto& m : merges) ranks_[m.first + '\x01' + std::to_string(m.first.size()) + '\x01' + m.second] = r++;
    merge_keys_exact_ = true;
    cache_.clear();
  }

  void add_special(const std::string& tok, int id) {
    specials_.emplace_back(tok, id);
    std::sort(specials_.begin(), specials_.end(),
              [](const auto& a, const auto& b) { return a.first.size() > b.first.size(); });
    if (id >= static_cast<int>(id2tok_.size())) id2tok_.resize(id + 1);
    id2tok_[id] = tok;
    special_ids_.resize(std::max<size_t>(special_ids_.size(), id + 1), 0);
    special_ids_[id] = 1;
    special_first_[static_cast<unsigned char>(tok[0])] = true;
  }

  int vocab_size() const { return static_cast<int>(id2tok_.size()); }
  int token_to_id(const std::string& t) const {
    auto it = tok2id_.find(t);
    if (it != tok2id_.end()) return it->second;
    for (auto& s : specials_) if (s.first == t) return s.second;
    return -1;
  }
  std::string id_to_token(int id) const {
    if (id < 0 || id >= static_cast<int>(id2tok_.size())) return std::string();
    return id2tok_[id];
  }

  std::vector<int32_t> encode(const std::string& text, bool allow_special) const {
    std::vector<int32_t> out;
    size_t i = 0, seg = 0;
    while (allow_special && !specials_.empty() && i < text.size()) {
      if (special_first_[static_cast<unsigned char>(text[i])]) {
        bool hit = false;
        for (auto& s : specials_) {
          if (text.compare(i, s.first.size(), s.first) == 0) {
            if (i > seg) encode_ordinary(text.substr(seg, i - seg), out);
            out.push_back(s.second);
            i += s.first.size();
            seg = i;
            hit = true;
            break;
          }
        }
        if (hit) continue;
      }
      ++i;
    }
    if (seg < text.size()) encode_ordinary(text.substr(seg), out);
    return out;
  }

  std::string decode(const std::vector<int32_t>& ids, bool skip_special) const {
    std::string out;
    for (int32_t id : ids) {
      if (id < 0 || id >= static_cast<int>(id2tok_.size())) continue;
      if (skip_special && id < static_cast<int>(special_ids_.size()) && special_ids_[id]) continue;
      out += id2tok_[id];
    }
    return out;
  }

  // exposed for tests
  std::vector<std::string> pretokenize(const std::string& s) const {
    std::vector<std::string> out;
    split(s, [&](size_t a, size_t b) { out.push_back(s.substr(a, b - a)); });
    return out;
  }

 private:
  template <class F>
  void split(const std::string& s, F&& emit) const {
    using namespace detail;
    const size_t n = s.size();
    size_t i = 0;
    auto cp_at = [&](size_t p, int* len) { return utf8_at(s, p, len); };
    while (i < n) {
      int l0;
      uint32_t c0 = cp_at(i, &l0);
      // 1. contractions
      if (c0 == '\'' && i + 1 < n) {
        auto lower = [](char ch) { return (ch >= 'A' && ch <= 'Z') ? char(ch + 32) : ch; };
        char a = lower(s[i + 1]);
        char b = (i + 2 < n) ? lower(s[i + 2]) : 0;
        size_t len = 0;
        if (a == 's' || a == 't' || a == 'm' || a == 'd') len = 2;
        if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e') || (a == 'l' && b == 'l')) len = 3;
        if (len) {
          emit(i, i + len);
          i += len;
          continue;
        }
      }
      // 2. [^\r\n\p{L}\p{N}]?\p{L}+
      {
        size_t p = i;
        bool c0_letter = is_letter(c0);
        if (!c0_letter && c0 != '\r' && c0 != '\n' && !is_number(c0)) p = i + l0;  // optional prefix char
        size_t q = p;
        while (q < n) {
          int l;
          uint32_t c = cp_at(q, &l);
          if (!is_letter(c)) break;
          q += l;
        }
        if (q > p) {
          emit(i, q);
          i = q;
          continue;
        }
      }
      // 3. \p{N}{1,D}
      if (is_number(c0)) {
        size_t q = i;
        int cnt = 0;
        while (q < n && cnt < max_digits_) {
          int l;
          uint32_t c = cp_at(q, &l);
          if (!is_number(c)) break;
          q += l;
          ++cnt;
        }
        emit(i, q);
        i = q;
        continue;
      }
      // 4. ' '?[^\s\p{L}\p{N}]+[\r\n]*
      {
        size_t p = i;
        if (c0 == ' ') p = i + 1;
        size_t q = p;
        while (q < n) {
          int l;
          uint32_t c = cp_at(q, &l);
          if (is_space(c) || is_letter(c) || is_number(c)) break;
          q += l;
        }
        if (q > p) {
          while (q < n && (s[q] == '\r' || s[q] == '\n')) ++q;
          emit(i, q);
          i = q;
          continue;
        }
      }
      // whitespace alternatives: c0 is white space here
      {
        size_t q = i, last_nl_end = 0, last_char_start = i;
        bool has_nl = false;
        while (q < n) {
          int l;
          uint32_t c = cp_at(q, &l);
          if (!is_space(c)) break;
          if (c == '\r' || c == '\n') {
            has_nl = true;
            last_nl_end = q + l;
          }
          last_char_start = q;
          q += l;
        }
        if (q == i) {  // not white space either (e.g. invalid byte): emit as is
          emit(i, i + l0);
          i += l0;
          continue;
        }
        // 5. \s*[\r\n]+
        if (has_nl) {
          emit(i, last_nl_end);
          i = last_nl_end;
          continue;
        }
        // 6. \s+(?!\S): leave the last white-space char to the next token unless at end of text
        if (q < n && last_char_start > i) {
          emit(i, last_char_start);
          i = last_char_start;
          continue;
        }
        // 7. \s+
        emit(i, q);
        i = q;
      }
    }
  }

  void encode_ordinary(const std::string& text, std::vector<int32_t>& out) const {
    split(text, [&](size_t a, size_t b) { bpe_piece(text.substr(a, b - a), out); });
  }

  int pair_rank(const std::string& l, const std::string& r) const {
    if (use_id_as_rank_) {
      auto it = tok2id_.find(l + r);
      return it == tok2id_.end() ? std::numeric_limits<int>::max() : it->second;
    }
    auto it = ranks_.find(l + '\x01' + std::to_string(l.size()) + '\x01' + r);
    return it == ranks_.end() ? std::numeric_limits<int>::max() : it->second;
  }

  void bpe_piece(const std::string& piece, std::vector<int32_t>& out) const {
    {
      auto whole = tok2id_.find(piece);
      if (whole != tok2id_.end() && (use_id_as_rank_ || piece.size() == 1)) {
        out.push_back(whole->second);
        return;
      }
      std::lock_guard<std::mutex> g(cache_mu_);
      auto it = cache_.find(piece);
      if (it != cache_.end()) {
        out.insert(out.end(), it->second.begin(), it->second.end());
        return;
      }
    }
    std::vector<std::string> parts;
    parts.reserve(piece.size());
    for (char ch : piece) parts.emplace_back(1, ch);
    while (parts.size() > 1) {
      int best = std::numeric_limits<int>::max();
      size_t at = 0;
      for (size_t k = 0; k + 1 < parts.size(); ++k) {
        int r = pair_rank(parts[k], parts[k + 1]);
        if (r < best) {
          best = r;
          at = k;
        }
      }
      if (best == std::numeric_limits<int>::max()) break;
      parts[at] += parts[at + 1];
      parts.erase(parts.begin() + at + 1);
    }
    std::vector<int32_t> ids;
    for (auto& p : parts) {
      auto it = tok2id_.find(p);
      if (it != tok2id_.end()) {
        ids.push_back(it->second);
      } else {
        for (char ch : p) {  // unknown merge result: fall back to bytes
          auto b = tok2id_.find(std::string(1, ch));
          if (b != tok2id_.end()) ids.push_back(b->second);
        }
      }
    }
    out.insert(out.end(), ids.begin(), ids.end());
    std::lock_guard<std::mutex> g(cache_mu_);
    if (cache_.size() < (1u << 20)) cache_.emplace(piece, std::move(ids));
  }

  std::unordered_map<std::string, int> tok2id_;
  std::vector<std::string> id2tok_;
  std::unordered_map<std::string, int> ranks_;
  std::vector<std::pair<std::string, int>> specials_;
  std::vector<uint8_t> special_ids_;
  bool special_first_[256] = {false};
  bool use_id_as_rank_ = false;
  bool merge_keys_exact_ = true;
  int max_digits_ = 1;
  mutable std::mutex cache_mu_;
  mutable std::unordered_map<std::string, std::vector<int32_t>> cache_;
};

}  // namespace xl
