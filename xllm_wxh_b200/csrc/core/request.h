// Request / Sequence state kept by the scheduler.
//
// Mirrors the roles of xllm/core/framework/request/{request,sequence,
// sequence_kv_state,stopping_checker,request_params}.h in the reference:
// a Request owns 1..best_of Sequences; a Sequence owns its token ids, its paged-KV
// blocks and the number of tokens whose KV is already in the cache.
#pragma once
#include <algorithm>
#include <chrono>
#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace xl {

enum class FinishReason : int { NONE = 0, STOP = 1, LENGTH = 2, CANCELLED = 3, RESOURCE_EXHAUSTED = 4, HANDOFF = 5 };

// Defaults follow request_params.h:77-112 of the reference.
struct SamplingParams {
  float temperature = 0.0f;
  float top_p = 1.0f;
  int top_k = -1;
  float repetition_penalty = 1.0f;
  float frequency_penalty = 0.0f;
  float presence_penalty = 0.0f;
  bool logprobs = false;
  int top_logprobs = 0;
  int64_t seed = -1;
  bool needs_penalties() const {
    return repetition_penalty != 1.0f || frequency_penalty != 0.0f || presence_penalty != 0.0f;
  }
};

// stopping_checker.h:27-92 of the reference: max_tokens, context length, eos,
// stop token ids, stop token sequences.
struct StopCriteria {
  int max_tokens = 5120;
  int max_context_len = 1 << 30;
  int eos_token_id = -1;
  bool ignore_eos = false;
  std::vector<int32_t> stop_token_ids;
  std::vector<std::vector<int32_t>> stop_sequences;
};

struct Request;

struct Sequence {
  int64_t id = 0;
  int index = 0;  // index inside the request (0..best_of-1)
  Request* req = nullptr;
  std::vector<int32_t> tokens;
  std::vector<float> logprobs;  // one per generated token when requested
  int num_prompt_tokens = 0;
  std::vector<int> blocks;
  int kv_tokens = 0;            // tokens whose KV is in the cache
  int num_cached_tokens = 0;    // prompt tokens served by the prefix cache at admission
  int dp_rank = -1;
  bool finished = false;
  FinishReason reason = FinishReason::NONE;
  int reported = 0;             // generated tokens already handed to the caller
  int num_placeholders = 0;     // trailing tokens that are schedule-overlap placeholders
  int preempt_count = 0;
  int chunks_since_match = 0;
  // sampling penalties: occurrences of every token id among tokens[0, pen_counted) as (all, of which generated); grown
  // by the batch builder with the tokens that arrived since the last step instead of recounted from the start
  std::map<int32_t, std::pair<int, int>> pen_counts;
  int pen_counted = 0;

  int num_tokens() const { return static_cast<int>(tokens.size()); }
  int num_generated() const { return num_tokens() - num_prompt_tokens; }
  int remaining() const { return num_tokens() - kv_tokens; }
  bool in_decode() const { return remaining() == 1 && num_tokens() > num_prompt_tokens; }
};

struct Request {
  int64_t id = 0;
  std::string ext_id;
  std::vector<std::unique_ptr<Sequence>> seqs;
  int n = 1, best_of = 1;
  int priority = 0;          // smaller = more urgent
  bool offline = false;
  bool cancelled = false;
  bool expanded = false;     // siblings of seq 0 created
  bool preempted = false;
  bool handoff_after_prefill = false;  // prefill instance of a disaggregated pair
  double arrival = 0;        // seconds, monotonic
  double deadline = 0;       // arrival + ttft slo (deadline strategy)
  double first_token_time = 0;
  // service-level targets of the request (scheduler_param in request_params.h:148-158 of the reference); 0 = none
  double ttft_slo_ms = 0, tpot_slo_ms = 0;
  int ttft_weight = 1, tpot_weight = 1;
  // scratch of the urgency-ordered (mix) policy, recomputed every step
  double est_ms = 0, remaining_ms = 0;
  bool urgent = false, starved = false;
  SamplingParams sampling;
  StopCriteria stop;
  std::vector<int32_t> prompt;

  bool finished() const {
    if (!expanded && best_of > 1 && !cancelled) {
      // siblings not created yet: the request is only done if seq 0 ended abnormally
      return !seqs.empty() && seqs[0]->finished &&
             (seqs[0]->reason == FinishReason::RESOURCE_EXHAUSTED || seqs[0]->reason == FinishReason::CANCELLED);
    }
    for (auto& s : seqs)
      if (!s->finished) return false;
    return true;
  }
};

inline double now_seconds() {
  using namespace std::chrono;
  return duration<double>(steady_clock::now().time_since_epoch()).count();
}

// Returns the finish reason triggered by the last token of `s`, or NONE.
inline FinishReason check_stop(const Sequence& s, const StopCriteria& c) {
  const int n_gen = s.num_generated();
  if (n_gen <= 0) return FinishReason::NONE;
  const int32_t last = s.tokens.back();
  if (last >= 0) {
    if (!c.ignore_eos && c.eos_token_id >= 0 && last == c.eos_token_id) return FinishReason::STOP;
    for (int32_t t : c.stop_token_ids)
      if (t == last) return FinishReason::STOP;
    for (auto& seq : c.stop_sequences) {
      const int m = static_cast<int>(seq.size());
      if (m == 0 || m > n_gen) continue;
      if (std::equal(seq.begin(), seq.end(), s.tokens.end() - m)) return FinishReason::STOP;
    }
  }
  if (n_gen >= c.max_tokens) return FinishReason::LENGTH;
  if (s.num_tokens() >= c.max_context_len) return FinishReason::LENGTH;
  return FinishReason::NONE;
}

}  // namespace xl
