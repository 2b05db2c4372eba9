// Suffix-pattern cache for model-free speculative decoding ("Suffix" algorithm).
//
// Role of xllm/core/util/suffix_tree.cpp + suffix_decoding_cache.cpp in the reference: remember
// token patterns seen in prompts and generations, and propose a continuation for a sequence by
// matching the longest recent suffix of its context.  Stored as a depth-bounded trie of token
// windows with hit counts; each live sequence keeps cursors into the trie so that appending a
// token costs O(max_depth).
#pragma once
#include <cstdint>
#include <unordered_map>
#include <vector>

namespace xl {

class SuffixCache {
 public:
  SuffixCache(int max_depth, int max_sequences) : max_depth_(max_depth), max_seqs_(max_sequences) { nodes_.emplace_back(); }

  void append(int64_t seq_id, const std::vector<int32_t>& tokens) {
    if (static_cast<int>(cursors_.size()) >= max_seqs_ && !cursors_.count(seq_id)) cursors_.erase(cursors_.begin());
    auto& cur = cursors_[seq_id];
    for (int32_t t : tokens) {
      cur.push_back({0, 0});
      size_t w = 0;
      for (size_t i = 0; i < cur.size(); ++i) {
        if (cur[i].depth >= max_depth_) continue;  // window full: drop
        int child = step(cur[i].node, t, /*create=*/true);
        nodes_[child].count++;
        cur[w++] = {child, cur[i].depth + 1};
      }
      cur.resize(w);
    }
    if (nodes_.size() > kMaxNodes) {  // bounded memory: start over
      nodes_.clear();
      nodes_.emplace_back();
      cursors_.clear();
    }
  }

  void evict(int64_t seq_id) { cursors_.erase(seq_id); }

  // Longest suffix of `context` (at least min_match tokens) that is a known pattern; follow the
  // most frequent continuation for up to max_tokens tokens.
  std::vector<int32_t> speculate(int64_t /*seq_id*/, const std::vector<int32_t>& context, int max_tokens,
                                 int min_match) const {
    std::vector<int32_t> out;
    const int n = static_cast<int>(context.size());
    const int longest = std::min(n, max_depth_ - 1);
    for (int m = longest; m >= std::max(1, min_match); --m) {
      int node = 0;
      bool ok = true;
      for (int i = n - m; i < n && ok; ++i) {
        node = step_const(node, context[i]);
        ok = node >= 0;
      }
      if (!ok) continue;
      int depth = m;
      while (static_cast<int>(out.size()) < max_tokens && depth < max_depth_) {
        int best = -1, best_cnt = 0;
        int32_t best_tok = 0;
        for (auto& kv : nodes_[node].children)
          if (nodes_[kv.second].count > best_cnt) {
            best_cnt = nodes_[kv.second].count;
            best = kv.second;
            best_tok = kv.first;
          }
        if (best < 0) break;
        out.push_back(best_tok);
        node = best;
        ++depth;
      }
      if (!out.empty()) return out;
    }
    return out;
  }

  // The reference's rule (core/util/suffix_tree.cpp:602-633,836-870): for every suffix of `context` that is a known
  // pattern, from one token up, follow the most frequent continuation; a match of m tokens may propose at most
  // m * max_spec_factor + max_spec_offset tokens, and a token is proposed only while the product of the branch
  // frequencies on the way to it is at least min_token_prob.  The proposal with the highest sum of those products wins
  // (the longer match on a tie).
  std::vector<int32_t> speculate_scored(const std::vector<int32_t>& context, int max_spec_tokens, float max_spec_factor,
                                        float max_spec_offset, float min_token_prob) const {
    std::vector<int32_t> best;
    float best_score = 0.f;
    const int n = static_cast<int>(context.size());
    const int longest = std::min(n, max_depth_ - 1);
    for (int m = 1; m <= longest; ++m) {
      int node = 0;
      bool ok = true;
      for (int i = n - m; i < n && ok; ++i) {
        node = step_const(node, context[i]);
        ok = node >= 0;
      }
      if (!ok) break;                       // a longer suffix contains this one: it cannot match either
      int max_tokens = std::min(max_spec_tokens, static_cast<int>(m * max_spec_factor + max_spec_offset + 1e-6f));
      max_tokens = std::max(max_tokens, 0);
      std::vector<int32_t> out;
      float prob = 1.f, score = 0.f;
      int depth = m;
      while (static_cast<int>(out.size()) < max_tokens && depth < max_depth_) {
        int child = -1, child_cnt = 0;
        int32_t child_tok = 0;
        for (auto& kv : nodes_[node].children) {
          const int c = nodes_[kv.second].count;
          if (c > child_cnt || (c == child_cnt && child >= 0 && kv.first < child_tok)) {
            child_cnt = c;
            child = kv.second;
            child_tok = kv.first;
          }
        }
        if (child < 0 || nodes_[node].count <= 0) break;
        prob *= static_cast<float>(child_cnt) / static_cast<float>(nodes_[node].count);
        if (prob < min_token_prob) break;
        out.push_back(child_tok);
        score += prob;
        node = child;
        ++depth;
      }
      if (score >= best_score) {
        best_score = score;
        best = std::move(out);
      }
    }
    return best;
  }

  size_t num_nodes() const { return nodes_.size(); }

 private:
  static constexpr size_t kMaxNodes = 8u << 20;
  struct Node {
    std::unordered_map<int32_t, int> children;
    int count = 0;
  };
  struct Cursor {
    int node;
    int depth;
  };
  int step(int node, int32_t t, bool create) {
    auto it = nodes_[node].children.find(t);
    if (it != nodes_[node].children.end()) return it->second;
    if (!create) return -1;
    int id = static_cast<int>(nodes_.size());
    nodes_.emplace_back();
    nodes_[node].children.emplace(t, id);
    return id;
  }
  int step_const(int node, int32_t t) const {
    auto it = nodes_[node].children.find(t);
    return it == nodes_[node].children.end() ? -1 : it->second;
  }
  int max_depth_, max_seqs_;
  std::vector<Node> nodes_;
  std::unordered_map<int64_t, std::vector<Cursor>> cursors_;
};

}  // namespace xl
