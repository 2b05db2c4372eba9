// Flattens a scheduled Batch into one packed int32 staging buffer (pinned host memory owned
// by the caller) so that a step needs a single host->device copy.
//
// The reference builds the same information as separate tensors in BatchInputBuilder
// (xllm/core/framework/batch/batch_input_builder.cpp: flatten_tokens, new_token_slot_ids,
// block tables, cumulative q_seq_lens / seq_lens, sampling indexes, unique-token counts).
// Here every section lives at a fixed offset that depends only on the capacities
// (T_cap tokens, B_cap sequences, MB_cap blocks per sequence, S_cap sample rows, P_cap
// penalty entries), which is what lets a captured CUDA graph replay on the same device
// buffer with new contents.
#pragma once
#include <cstring>
#include <map>
#include <unordered_map>

#include "scheduler.h"

namespace xl {

struct BatchLayout {
  int T_cap, B_cap, MB_cap, S_cap, P_cap;
  // offsets in int32 words
  int header, tokens, positions, slots, token_seq, next_tokens, q_cu, kv_lens, block_tables, sample_idx, temperature, top_p, top_k,
      rep_pen, freq_pen, pres_pen, seed_lo, seed_hi, want_logprobs, pen_cu, pen_ids, pen_counts, total_words;
  static int align(int x) { return (x + 31) & ~31; }
  BatchLayout(int T, int B, int MB, int S, int P) : T_cap(T), B_cap(B), MB_cap(MB), S_cap(S), P_cap(P) {
    int o = 0;
    auto sec = [&](int n) { int at = o; o = align(o + n); return at; };
    header = sec(32);
    tokens = sec(T);
    positions = sec(T);
    slots = sec(T);
    token_seq = sec(T);
    next_tokens = sec(T);
    q_cu = sec(B + 1);
    kv_lens = sec(B);
    block_tables = sec(B * MB);
    sample_idx = sec(S);
    temperature = sec(S);
    top_p = sec(S);
    top_k = sec(S);
    rep_pen = sec(S);
    freq_pen = sec(S);
    pres_pen = sec(S);
    seed_lo = sec(S);
    seed_hi = sec(S);
    want_logprobs = sec(S);
    pen_cu = sec(S + 1);
    pen_ids = sec(P);
    pen_counts = sec(P);
    total_words = o;
  }
};

enum HeaderField : int {
  H_NUM_TOKENS = 0, H_NUM_SEQS = 1, H_NUM_SAMPLE = 2, H_NUM_DECODE = 3, H_NUM_PREFILL = 4, H_MAX_Q = 5, H_MAX_KV = 6,
  H_FWD_TYPE = 7, H_NUM_SPEC = 8, H_T_CAP = 9, H_B_CAP = 10, H_MB_CAP = 11, H_BATCH_LO = 12, H_BATCH_HI = 13,
  H_ANY_PENALTY = 14, H_ALL_GREEDY = 15, H_ANY_LOGPROBS = 16, H_BLOCK_SIZE = 17, H_PEN_TOTAL = 18, H_S_CAP = 19,
  H_MAX_TOP_LOGPROBS = 20, H_NUM_PREFILL_TOKENS = 21,
  H_MAX_TOP_K = 22       // largest top_k among the rows that sample (a row that samples without top-k counts as 2^30; 0: none sample)
};

// Returns 0 on success, or a negative number: -1 capacity overflow (tokens / seqs / blocks /
// samples), -(needed P_cap) - 16 when only the penalty section is too small.
inline long build_batch(const Batch& b, const BatchLayout& L, int32_t* buf, int block_size) {
  auto as_f = [](float f) { int32_t i; std::memcpy(&i, &f, 4); return i; };
  const int n_seq = static_cast<int>(b.entries.size());
  int n_rows = 0;
  for (auto& e : b.entries) if (e.sample) n_rows += 1 + e.n_spec;
  if (b.num_tokens > L.T_cap || n_seq > L.B_cap || n_rows > L.S_cap) return -1;
  int32_t* H = buf + L.header;
  std::memset(H, 0, 32 * 4);
  int32_t *tok = buf + L.tokens, *pos = buf + L.positions, *slot = buf + L.slots, *tseq = buf + L.token_seq;
  int32_t* nxt = buf + L.next_tokens;   // token that follows each position (-1: not known yet = the one sampled this step)
  int32_t *qcu = buf + L.q_cu, *kvl = buf + L.kv_lens, *bt = buf + L.block_tables, *sidx = buf + L.sample_idx;
  int t = 0, row = 0, max_q = 0, max_kv = 0, n_spec = 0, pen_total = 0, n_prefill_tokens = 0;
  bool any_pen = false, all_greedy = true, any_lp = false;
  int max_top_lp = 0, max_top_k = 0;
  qcu[0] = 0;
  buf[L.pen_cu] = 0;
  for (int i = 0; i < n_seq; ++i) {
    const BatchEntry& e = b.entries[i];
    const Sequence* s = e.seq;
    const int n_blocks = static_cast<int>(s->blocks.size());
    const int kv_after = e.kv_before + e.n_tokens;
    const int used_blocks = (kv_after + block_size - 1) / block_size;
    if (used_blocks > L.MB_cap || used_blocks > n_blocks) return -1;
    const int real = e.n_tokens - e.n_spec;
    for (int j = 0; j < e.n_tokens; ++j) {
      const int p = e.kv_before + j;
      tok[t] = (j < real) ? s->tokens[p] : 0;  // draft slots are filled in by the worker
      pos[t] = p;
      slot[t] = s->blocks[p / block_size] * block_size + p % block_size;
      tseq[t] = i;
      nxt[t] = (p + 1 < s->num_tokens() && j < real) ? s->tokens[p + 1] : -1;
      ++t;
    }
    qcu[i + 1] = t;
    kvl[i] = kv_after;
    std::memcpy(bt + size_t(i) * L.MB_cap, s->blocks.data(), size_t(used_blocks) * 4);
    for (int j = used_blocks; j < L.MB_cap; ++j) bt[size_t(i) * L.MB_cap + j] = 0;
    max_q = std::max(max_q, e.n_tokens);
    max_kv = std::max(max_kv, kv_after);
    n_spec = std::max(n_spec, e.n_spec);
    const bool is_dec = (real == 1 && e.sample && e.kv_before > 0);
    if (!is_dec) n_prefill_tokens += e.n_tokens;
    if (e.sample) {
      const SamplingParams& sp = s->req->sampling;
      const int rows = 1 + e.n_spec;
      for (int j = 0; j < rows; ++j) {
        sidx[row] = t - rows + j;
        buf[L.temperature + row] = as_f(sp.temperature);
        buf[L.top_p + row] = as_f(sp.top_p);
        buf[L.top_k + row] = sp.top_k;
        buf[L.rep_pen + row] = as_f(sp.repetition_penalty);
        buf[L.freq_pen + row] = as_f(sp.frequency_penalty);
        buf[L.pres_pen + row] = as_f(sp.presence_penalty);
        // per-step stream: seed (or sequence id) mixed with the position being sampled
        uint64_t seed = sp.seed >= 0 ? uint64_t(sp.seed) * 0x9e3779b97f4a7c15ULL + uint64_t(s->index)
                                     : uint64_t(s->id) * 0xd1342543de82ef95ULL + 0x632be59bd9b4e019ULL;
        seed ^= (uint64_t(kv_after + j) + 1) * 0xbf58476d1ce4e5b9ULL;
        buf[L.seed_lo + row] = int32_t(uint32_t(seed));
        buf[L.seed_hi + row] = int32_t(uint32_t(seed >> 32));
        buf[L.want_logprobs + row] = sp.logprobs ? 1 + sp.top_logprobs : 0;
        if (sp.needs_penalties()) {
          any_pen = true;
          // unique token ids with counts; generated tokens are flagged in the high bit of the count
          // (frequency / presence penalties apply to generated tokens only, the repetition penalty to all).
          // The counts live on the sequence and take in only the tokens that are new since the last step; a negative id
          // is a schedule-overlap placeholder at the tail, counted once its real token has replaced it (so under overlap
          // the newest token starts to be penalised one step later, as with the reference's token_to_count_map_:
          // core/framework/request/sequence.cpp:234-241,280-283).
          Sequence* ms = e.seq;
          if (ms->pen_counted > ms->num_tokens()) {          // the sequence was cut back: recount
            ms->pen_counts.clear();
            ms->pen_counted = 0;
          }
          while (ms->pen_counted < ms->num_tokens() && ms->tokens[ms->pen_counted] >= 0) {
            auto& c = ms->pen_counts[ms->tokens[ms->pen_counted]];
            c.first++;
            if (ms->pen_counted >= ms->num_prompt_tokens) c.second++;
            ++ms->pen_counted;
          }
          const auto& cnt = ms->pen_counts;
          for (auto& kv : cnt) {
            if (pen_total < L.P_cap) {
              buf[L.pen_ids + pen_total] = kv.first;
              buf[L.pen_counts + pen_total] = std::min(kv.second.first, 0xffff) | (std::min(kv.second.second, 0xffff) << 16);   // saturating halves
            }
            ++pen_total;
          }
        }
        buf[L.pen_cu + row + 1] = pen_total;
        if (sp.temperature != 0.0f) {
          all_greedy = false;
          max_top_k = std::max(max_top_k, sp.top_k > 0 ? int(sp.top_k) : (1 << 30));
        }
        if (sp.logprobs) { any_lp = true; max_top_lp = std::max(max_top_lp, sp.top_logprobs); }
        ++row;
      }
    }
  }
  // padding: tokens hit the reserved block 0, sequences are empty
  for (int i = t; i < L.T_cap; ++i) {
    tok[i] = 0;
    pos[i] = 0;
    slot[i] = i % block_size;
    tseq[i] = -1;
    nxt[i] = 0;
  }
  for (int i = n_seq; i < L.B_cap; ++i) {
    qcu[i + 1] = t;
    kvl[i] = 0;
  }
  for (int i = row; i < L.S_cap; ++i) {
    sidx[i] = 0;
    buf[L.temperature + i] = 0;
    buf[L.top_p + i] = as_f(1.0f);
    buf[L.top_k + i] = -1;
    buf[L.rep_pen + i] = as_f(1.0f);
    buf[L.freq_pen + i] = 0;
    buf[L.pres_pen + i] = 0;
    buf[L.seed_lo + i] = buf[L.seed_hi + i] = 0;
    buf[L.want_logprobs + i] = 0;
    buf[L.pen_cu + i + 1] = std::min(pen_total, L.P_cap);
  }
  H[H_NUM_TOKENS] = t;
  H[H_NUM_SEQS] = n_seq;
  H[H_NUM_SAMPLE] = row;
  H[H_NUM_DECODE] = b.num_decode_seqs;
  H[H_NUM_PREFILL] = b.num_prefill_seqs;
  H[H_MAX_Q] = max_q;
  H[H_MAX_KV] = max_kv;
  H[H_FWD_TYPE] = static_cast<int>(b.forward_type());
  H[H_NUM_SPEC] = n_spec;
  H[H_T_CAP] = L.T_cap;
  H[H_B_CAP] = L.B_cap;
  H[H_MB_CAP] = L.MB_cap;
  H[H_BATCH_LO] = int32_t(uint32_t(uint64_t(b.id)));
  H[H_BATCH_HI] = int32_t(uint32_t(uint64_t(b.id) >> 32));
  H[H_ANY_PENALTY] = any_pen;
  H[H_ALL_GREEDY] = all_greedy;
  H[H_ANY_LOGPROBS] = any_lp;
  H[H_BLOCK_SIZE] = block_size;
  H[H_PEN_TOTAL] = std::min(pen_total, L.P_cap);
  H[H_S_CAP] = L.S_cap;
  H[H_MAX_TOP_LOGPROBS] = max_top_lp;
  H[H_NUM_PREFILL_TOKENS] = n_prefill_tokens;
  H[H_MAX_TOP_K] = max_top_k;
  if (pen_total > L.P_cap) return -(long(pen_total) + 16);
  return 0;
}

}  // namespace xl
