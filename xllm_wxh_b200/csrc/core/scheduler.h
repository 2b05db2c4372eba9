// Continuous-batching scheduler family (one class, policy flags).
//
// Behavioural spec taken from the reference schedulers:
//   * ContinuousScheduler: prefill-first, decode only when no prefill was
//     scheduled; token / sequence / memory budgets; online requests may evict
//     offline decodes; on block exhaustion the lowest-priority running request
//     is preempted for recompute (xllm/core/scheduler/continuous_scheduler.cpp:
//     231-436 prefill, 438-688 decode, 805-1022 prepare_batch);
//   * ChunkedPrefillScheduler: decode-maximal batches, prefill in chunks of
//     max_tokens_per_chunk_for_prefill, leftover budget tops chunks up
//     (chunked_prefill_scheduler.cpp:490-716);
//   * PrefillOnlyScheduler: chunked, but a batch is pure prefill or pure decode
//     (scheduler_factory.cpp:46-53);
//   * ZeroEvictionScheduler: admit a prefill only if simulated future block usage
//     never forces an eviction (zero_eviction_scheduler.h:23-80);
//   * schedule-overlap: a step's tokens may be appended as placeholders (-k) and
//     patched one step later (continuous_scheduler.cpp:1085-1115,
//     sequence.cpp:255-296).
#pragma once
#include <deque>
#include <mutex>
#include <unordered_map>

#include "block_manager.h"
#include "request.h"
#include "step_time_model.h"

namespace xl {

struct SchedulerOptions {
  int max_tokens_per_batch = 10240;
  int max_seqs_per_batch = 1024;
  bool enable_chunked_prefill = true;
  int max_tokens_per_chunk_for_prefill = -1;  // -1: whole budget
  bool prefill_only_batches = false;
  bool use_zero_evict = false;
  int max_decode_token_per_sequence = 256;
  int num_speculative_tokens = 0;
  int spec_extra_slots = 0;   // KV slots reserved beyond a step's rows (a draft model that proposes several tokens writes its own KV ahead)
  double prefill_scheduling_memory_usage_threshold = 0.95;
  bool enable_online_preempt_offline = true;
  std::string priority_strategy = "fcfs";  // fcfs | priority | deadline
  int chunked_match_frequency = 2;
  int dp_size = 1;
  bool handoff_after_prefill = false;  // instance_role == PREFILL in a disaggregated pair
  // urgency-ordered single queue ("mix" policy; global_flags.cpp:188-208,254-280 of the reference)
  bool use_mix_scheduler = false;
  bool enable_latency_aware_schedule = false;
  double max_global_ttft_ms = 0, max_global_tpot_ms = 0;  // 0 = none; used by requests without targets of their own
  double aggressive_coeff = 1.0, starve_threshold = 1.0;
  bool enable_starve_prevent = true;
  int min_prefill_chunk = 50;  // a latency-bounded chunk smaller than this is not worth a step
  // host-memory tier of the prefix cache: host blocks = host_blocks_factor x device blocks (global_flags.cpp:439-442)
  double host_blocks_factor = 0.0;
};

enum class ForwardType : int { PREFILL = 0, CHUNKED_PREFILL = 1, DECODE = 2, MIXED = 3, EMPTY = 4 };

struct BatchEntry {
  Sequence* seq = nullptr;
  int n_tokens = 0;    // tokens processed this step (incl. speculative draft slots)
  int n_spec = 0;      // draft tokens among them (filled in by the worker)
  bool sample = false; // step ends at the sequence tail -> a token is sampled
  int kv_before = 0;   // seq->kv_tokens when scheduled
  int sample_slot = -1;  // index among the sampling entries of the batch
  int placeholder_pos = -1;  // position in seq->tokens of the overlap placeholder
};

struct Batch {
  int64_t id = 0;
  int dp_rank = 0;
  std::vector<BatchEntry> entries;
  int num_tokens = 0, num_prefill_seqs = 0, num_decode_seqs = 0, num_sample = 0;
  bool output_pending = false;  // placeholders appended, real tokens not yet applied
  ForwardType forward_type() const {
    if (entries.empty()) return ForwardType::EMPTY;
    if (num_prefill_seqs == 0) return ForwardType::DECODE;
    if (num_decode_seqs > 0) return ForwardType::MIXED;
    for (auto& e : entries)
      if (e.kv_before > 0 || !e.sample) return ForwardType::CHUNKED_PREFILL;
    return ForwardType::PREFILL;
  }
};

struct SeqOutput {
  int64_t request_id = 0;
  std::string ext_id;
  int seq_index = 0;
  int64_t seq_id = 0;         // scheduler-wide id of the sequence (the key of per-sequence state kept outside)
  std::vector<int32_t> new_tokens;
  std::vector<float> new_logprobs;
  bool finished = false;
  int finish_reason = 0;
  int num_prompt_tokens = 0, num_generated = 0, num_cached_tokens = 0;
  bool request_finished = false;
};

// One block copy between the device cache and the host tier.
struct BlockCopy {
  int src = 0, dst = 0;
};

struct SchedulerStats {
  int64_t num_preemptions = 0, num_offline_evictions = 0;
  int64_t host_offloaded_blocks = 0, host_loaded_blocks = 0, host_adopted_blocks = 0;
  int64_t prompt_tokens = 0, generated_tokens = 0;
  int64_t steps = 0;
};

class Scheduler {
 public:
  Scheduler(const SchedulerOptions& opt, int num_blocks, int block_size, bool enable_prefix_cache, uint64_t seed = 1024)
      : opt_(opt), pool_(opt.dp_size, num_blocks, block_size, enable_prefix_cache, seed) {
    if (opt_.max_tokens_per_chunk_for_prefill <= 0) opt_.max_tokens_per_chunk_for_prefill = opt_.max_tokens_per_batch;
    const int host_blocks = static_cast<int>(opt_.host_blocks_factor * (num_blocks - 1));
    if (enable_prefix_cache && host_blocks >= 1) {
      for (int i = 0; i < opt_.dp_size; ++i) host_.emplace_back(host_blocks + 1, block_size, true, seed);
      loads_.resize(opt_.dp_size);
      offloads_.resize(opt_.dp_size);
    }
  }

  // ---- host tier of the prefix cache (HierarchyBlockManagerPool in the reference,
  // hierarchy_block_manager_pool.cpp:58-120 offload at release, :122-215 load at allocation).
  // Blocks that enter the device prefix cache are also copied to host blocks under the same chained keys; a prompt whose
  // prefix has left the device cache but is still on the host gets device blocks and a list of host->device copies
  // instead of a recompute.  The scheduler only keeps the books: the copies of a step are handed to the engine with
  // `take_transfers`, which runs the device->host ones before the host->device ones, before the step's forward.
  bool host_tier_enabled() const { return !host_.empty(); }
  int num_host_blocks() const { return host_.empty() ? 0 : host_[0].num_blocks() - 1; }
  BlockManager& host_manager(int dp_rank) { return host_.at(dp_rank); }
  // Leading full blocks of a prompt that the device cache / the host tier hold (for a third tier that fetches the rest).
  std::pair<int, int> prefix_presence(int dp_rank, const std::vector<int32_t>& tokens) const {
    const BlockManager& bm = pool_.at(dp_rank);
    const int n = static_cast<int>(tokens.size());
    const int max_blocks = n > 0 ? (n - 1) / bm.block_size() : 0;
    int dev = bm.count_prefix(tokens.data(), n, max_blocks);
    int host = host_.empty() ? 0 : host_.at(dp_rank).count_prefix(tokens.data(), n, max_blocks);
    return {dev, host};
  }
  // Make room in the host tier for the blocks [its current prefix, upto_blocks) of `tokens`, publish them under their
  // keys and return (block index, host block) for each: the caller fills the records before the next step is built
  // (content fetched from a remote store, which holds the blocks from `from_block` on).  Returns nothing when the host
  // tier cannot take all of them, or when its prefix has shrunk below `from_block` meanwhile.
  std::vector<std::pair<int, int>> host_adopt(int dp_rank, const std::vector<int32_t>& tokens, int from_block,
                                              int upto_blocks) {
    std::vector<std::pair<int, int>> out;
    if (host_.empty()) return out;
    BlockManager& hm = host_.at(dp_rank);
    const int bs = hm.block_size();
    upto_blocks = std::min<int>(upto_blocks, static_cast<int>(tokens.size()) / bs);
    std::vector<int> held = hm.match(tokens.data(), upto_blocks * bs, upto_blocks);
    const int have = static_cast<int>(held.size());
    const int want = upto_blocks - have;
    if (have >= from_block && want > 0 && want <= hm.num_available_blocks() && hm.allocate(want, held)) {
      hm.insert(tokens.data(), upto_blocks * bs, held);
      for (int i = have; i < upto_blocks; ++i) out.emplace_back(i, held[i]);
      stats_.host_adopted_blocks += want;
    }
    hm.release(held);
    return out;
  }
  // True while copies wait to be handed over or device blocks are still held for copies in flight: the engine then
  // keeps calling `take_transfers` every step (publishing a copy-only message when no batch was built), so that the
  // held blocks return to the pool.
  bool has_pending_transfers() const {
    for (auto& v : offloads_) if (!v.empty()) return true;
    for (auto& v : loads_) if (!v.empty()) return true;
    return pins_outstanding();
  }
  bool pins_outstanding() const {
    if (!pins_now_.empty()) return true;
    for (auto& v : offload_pins_) if (!v.empty()) return true;
    return false;
  }
  // Per DP rank: (offloads device->host, loads host->device) recorded since the last call.  Device blocks that are
  // being copied out stay referenced until two later calls, by which time every rank has finished reading them.
  std::vector<std::pair<std::vector<BlockCopy>, std::vector<BlockCopy>>> take_transfers() {
    std::vector<std::pair<std::vector<BlockCopy>, std::vector<BlockCopy>>> out(host_.size());
    if (host_.empty()) return out;
    for (size_t d = 0; d < host_.size(); ++d) {
      out[d].first.swap(offloads_[d]);
      out[d].second.swap(loads_[d]);
    }
    offload_pins_.push_back(std::move(pins_now_));
    pins_now_.clear();
    while (offload_pins_.size() > 2) {
      for (auto& pr : offload_pins_.front()) pool_.at(pr.first).release(pr.second);
      offload_pins_.pop_front();
    }
    return out;
  }

  const SchedulerOptions& options() const { return opt_; }
  BlockManagerPool& pool() { return pool_; }
  const SchedulerStats& stats() const { return stats_; }

  // Thread-safe: API threads enqueue, the scheduler thread drains.
  int64_t add_request(std::unique_ptr<Request> r) {
    std::lock_guard<std::mutex> g(mu_);
    r->id = next_request_id_++;
    if (r->arrival == 0) r->arrival = now_seconds();
    if (clock_override_ >= 0) {  // hand-driven clock: arrivals are stamped with it too
      r->deadline += clock_override_ - r->arrival;
      r->arrival = clock_override_;
    }
    int64_t id = r->id;
    incoming_.push_back(std::move(r));
    return id;
  }
  void cancel(int64_t id) {
    std::lock_guard<std::mutex> g(mu_);
    cancels_.push_back(id);
  }

  // A request whose prompt KV was produced elsewhere (decode side of a
  // disaggregated pair): blocks are reserved now, the request starts running once
  // `activate_remote` delivers the first token.
  // Returns the reserved block ids (empty on failure) and the dp rank in *dp_rank.
  std::vector<int> reserve_remote(std::unique_ptr<Request> r, int* dp_rank) {
    int rank = pool_.pick_dp_rank();
    BlockManager& bm = pool_.at(rank);
    const int bs = bm.block_size();
    int n_tok = static_cast<int>(r->prompt.size());
    int need = (n_tok + 1 + opt_.num_speculative_tokens + bs - 1) / bs;
    std::vector<int> blocks;
    if (!bm.allocate(need, blocks)) return {};
    {
      std::lock_guard<std::mutex> g(mu_);
      r->id = next_request_id_++;
    }
    if (r->arrival == 0) r->arrival = now_seconds();
    auto s = std::make_unique<Sequence>();
    s->id = next_seq_id_++;
    s->req = r.get();
    s->tokens = r->prompt;
    s->num_prompt_tokens = n_tok;
    s->blocks = blocks;
    s->dp_rank = rank;
    r->seqs.push_back(std::move(s));
    r->expanded = true;
    r->best_of = r->n = 1;
    if (dp_rank) *dp_rank = rank;
    int64_t id = r->id;
    remote_pending_[id] = std::move(r);
    return blocks;
  }
  int64_t last_reserved_id() const { return next_request_id_ - 1; }

  bool activate_remote(int64_t id, int32_t first_token, float logprob) {
    auto it = remote_pending_.find(id);
    if (it == remote_pending_.end()) return false;
    std::unique_ptr<Request> r = std::move(it->second);
    remote_pending_.erase(it);
    Sequence* s = r->seqs[0].get();
    s->kv_tokens = s->num_prompt_tokens;
    s->tokens.push_back(first_token);
    if (r->sampling.logprobs) s->logprobs.push_back(logprob);
    r->first_token_time = clock_now();
    Request* raw = r.get();
    requests_[id] = std::move(r);
    FinishReason fr = check_stop(*s, raw->stop);
    if (fr != FinishReason::NONE) finish_sequence(s, fr);
    running_.push_back(raw);
    emit(s);
    return true;
  }
  void drop_remote(int64_t id) {
    auto it = remote_pending_.find(id);
    if (it == remote_pending_.end()) return;
    Sequence* s = it->second->seqs[0].get();
    pool_.at(s->dp_rank).release(s->blocks);
    remote_pending_.erase(it);
  }

  bool has_unfinished() {
    std::lock_guard<std::mutex> g(mu_);
    return !incoming_.empty() || !waiting_online_.empty() || !waiting_offline_.empty() || !running_.empty();
  }
  int num_waiting() const { return static_cast<int>(waiting_online_.size() + waiting_offline_.size()); }
  // Token budget of a step, as fitted by the start-up profiler for a latency target (never above the configured
  // `max_tokens_per_batch`, never below one chunk of 16 tokens).
  void set_token_budget(int tokens) {
    if (configured_max_tokens_ <= 0) configured_max_tokens_ = opt_.max_tokens_per_batch;
    opt_.max_tokens_per_batch = std::max(16, std::min(tokens, configured_max_tokens_));
  }
  int token_budget() const { return opt_.max_tokens_per_batch; }
  // Step-time model of the latency-aware policies (fitted by the start-up profiler).
  void set_step_time_model(const StepTimeModel& m) { model_ = m; }
  const StepTimeModel& step_time_model() const { return model_; }
  // Tests drive the policy clock by hand; a negative value returns to the monotonic clock.
  void set_clock_override(double seconds) { clock_override_ = seconds; }
  // Order in which the mix policy would serve the unfinished requests now (ids, most urgent first).
  std::vector<int64_t> mix_order() {
    drain_incoming();
    std::vector<Request*> order;
    double budget = 0;
    mix_rank(order, &budget);
    std::vector<int64_t> ids;
    for (auto* r : order) ids.push_back(r->id);
    return ids;
  }
  double mix_latency_budget() {
    drain_incoming();
    std::vector<Request*> order;
    double budget = 0;
    mix_rank(order, &budget);
    return budget;
  }
  int num_running() const { return static_cast<int>(running_.size()); }
  int num_pending() {
    std::lock_guard<std::mutex> g(mu_);
    return static_cast<int>(incoming_.size());
  }

  // Build the next step: one Batch per DP rank (possibly empty).
  std::vector<Batch*> schedule() {
    drain_incoming();
    reap_finished();
    current_.clear();
    batches_storage_.emplace_back();
    std::vector<Batch>& bs = batches_storage_.back();
    bs.resize(opt_.dp_size);
    for (int i = 0; i < opt_.dp_size; ++i) {
      bs[i].id = next_batch_id_++;
      bs[i].dp_rank = i;
    }
    budget_tokens_.assign(opt_.dp_size, opt_.max_tokens_per_batch);
    budget_seqs_.assign(opt_.dp_size, opt_.max_seqs_per_batch);
    if (opt_.use_mix_scheduler)
      schedule_mix(bs);
    else if (opt_.enable_chunked_prefill)
      schedule_chunked(bs);
    else
      schedule_prefill_first(bs);
    for (auto& pr : host_pins_) host_[pr.first].release(pr.second);
    host_pins_.clear();
    std::vector<Batch*> out;
    for (auto& b : bs) {
      finalize(b);
      live_batches_[b.id] = &b;
      out.push_back(&b);
    }
    // keep storage bounded: batches older than 4 steps can no longer be referenced
    while (batches_storage_.size() > 4) {
      for (auto& b : batches_storage_.front()) live_batches_.erase(b.id);
      batches_storage_.pop_front();
    }
    ++stats_.steps;
    return out;
  }

  // Apply sampled tokens.  `tokens` is [num_sample, width]; width = 1 + n_spec, -1 marks a
  // rejected speculative position.  `logprobs` may be null.
  void process_output(int64_t batch_id, const int32_t* tokens, const float* logprobs, int width) {
    Batch* b = find_batch(batch_id);
    if (!b) return;
    for (auto& e : b->entries) {
      Sequence* s = e.seq;
      if (s->finished) continue;  // cancelled / finished while in flight
      if (!e.sample) {
        s->kv_tokens = e.kv_before + e.n_tokens;
        continue;
      }
      const int32_t* row = tokens + size_t(e.sample_slot) * width;
      const float* lrow = logprobs ? logprobs + size_t(e.sample_slot) * width : nullptr;
      int accepted = 0;
      s->kv_tokens = e.kv_before + (e.n_tokens - e.n_spec);
      const bool first = (s->num_generated() == 0);
      for (int j = 0; j < std::min(width, 1 + e.n_spec); ++j) {
        if (row[j] < 0) break;
        s->tokens.push_back(row[j]);
        if (s->req->sampling.logprobs) s->logprobs.push_back(lrow ? lrow[j] : 0.f);
        if (j > 0) s->kv_tokens += 1;  // draft token j-1 was accepted: its KV is valid
        ++accepted;
        ++stats_.generated_tokens;
        FinishReason fr = check_stop(*s, s->req->stop);
        if (fr != FinishReason::NONE) {
          finish_sequence(s, fr);
          break;
        }
      }
      (void)accepted;
      if (first) after_first_token(s);
      emit(s);
    }
    b->output_pending = false;
  }

  // Schedule-overlap, first half: pretend the step produced tokens.  Placeholder for the
  // j-th sampling entry is -(j+1); the worker replaces it on the device.
  void process_placeholder_output(int64_t batch_id) {
    Batch* b = find_batch(batch_id);
    if (!b) return;
    for (auto& e : b->entries) {
      Sequence* s = e.seq;
      if (s->finished) continue;
      s->kv_tokens = e.kv_before + e.n_tokens;
      if (!e.sample) continue;
      e.placeholder_pos = s->num_tokens();
      s->tokens.push_back(-(e.sample_slot + 1));
      ++s->num_placeholders;
      // length limits are known without the token value: do not schedule past them
      const StopCriteria& c = s->req->stop;
      if (s->num_generated() >= c.max_tokens || s->num_tokens() >= c.max_context_len) s->finished = true;  // provisional
    }
    b->output_pending = true;
  }

  // Schedule-overlap, second half: real tokens of a step whose placeholders are in place.
  void update_output(int64_t batch_id, const int32_t* tokens, const float* logprobs) {
    Batch* b = find_batch(batch_id);
    if (!b || !b->output_pending) return;
    for (auto& e : b->entries) {
      Sequence* s = e.seq;
      if (!e.sample || e.placeholder_pos < 0) continue;
      if (e.placeholder_pos >= s->num_tokens()) continue;  // truncated by an earlier finish
      if (s->reason != FinishReason::NONE) continue;       // really finished already
      s->tokens[e.placeholder_pos] = tokens[e.sample_slot];
      --s->num_placeholders;
      if (s->req->sampling.logprobs) s->logprobs.push_back(logprobs ? logprobs[e.sample_slot] : 0.f);
      ++stats_.generated_tokens;
      const bool first = (e.placeholder_pos == s->num_prompt_tokens);
      // stop check as if the sequence ended at this token
      std::vector<int32_t> tail(s->tokens.begin() + e.placeholder_pos + 1, s->tokens.end());
      s->tokens.resize(e.placeholder_pos + 1);
      FinishReason fr = check_stop(*s, s->req->stop);
      if (fr != FinishReason::NONE) {
        s->finished = false;
        s->num_placeholders = 0;
        s->kv_tokens = std::min(s->kv_tokens, s->num_tokens());
        finish_sequence(s, fr);
      } else {
        s->tokens.insert(s->tokens.end(), tail.begin(), tail.end());
      }
      if (first) after_first_token(s);
      emit(s);
    }
    b->output_pending = false;
  }

  std::vector<SeqOutput> take_outputs() {
    std::vector<SeqOutput> out;
    out.swap(outputs_);
    return out;
  }

  Batch* find_batch(int64_t id) {
    auto it = live_batches_.find(id);
    return it == live_batches_.end() ? nullptr : it->second;
  }

  // test / introspection helpers
  std::vector<int64_t> running_ids() const {
    std::vector<int64_t> v;
    for (auto* r : running_) v.push_back(r->id);
    return v;
  }
  std::vector<int64_t> waiting_ids() const {
    std::vector<int64_t> v;
    for (auto* r : waiting_online_) v.push_back(r->id);
    for (auto* r : waiting_offline_) v.push_back(r->id);
    return v;
  }
  Request* find_request(int64_t id) {
    auto it = requests_.find(id);
    return it == requests_.end() ? nullptr : it->second.get();
  }

 private:
  // ---------------------------------------------------------------- queues
  bool before(const Request* a, const Request* b) const {
    if (opt_.priority_strategy == "priority") {
      if (a->priority != b->priority) return a->priority < b->priority;
    } else if (opt_.priority_strategy == "deadline") {
      if (a->deadline != b->deadline) return a->deadline < b->deadline;
    }
    if (a->arrival != b->arrival) return a->arrival < b->arrival;
    return a->id < b->id;
  }
  void push_waiting(Request* r, bool front = false) {
    auto& q = r->offline ? waiting_offline_ : waiting_online_;
    if (front && opt_.priority_strategy == "fcfs") {
      q.push_front(r);
      return;
    }
    auto it = std::upper_bound(q.begin(), q.end(), r, [this](const Request* a, const Request* b) { return before(a, b); });
    q.insert(it, r);
  }

  void drain_incoming() {
    std::deque<std::unique_ptr<Request>> in;
    std::vector<int64_t> cancels;
    {
      std::lock_guard<std::mutex> g(mu_);
      in.swap(incoming_);
      cancels.swap(cancels_);
    }
    for (auto& r : in) {
      Request* raw = r.get();
      raw->handoff_after_prefill = raw->handoff_after_prefill || opt_.handoff_after_prefill;
      auto s = std::make_unique<Sequence>();
      s->id = next_seq_id_++;
      s->index = 0;
      s->req = raw;
      s->tokens = raw->prompt;
      s->num_prompt_tokens = static_cast<int>(raw->prompt.size());
      raw->seqs.push_back(std::move(s));
      raw->best_of = std::max(raw->best_of, raw->n);
      if (raw->best_of <= 1) raw->expanded = true;
      stats_.prompt_tokens += raw->prompt.size();
      requests_[raw->id] = std::move(r);
      push_waiting(raw);
    }
    for (int64_t id : cancels) {
      auto it = requests_.find(id);
      if (it != requests_.end()) it->second->cancelled = true;
      auto rp = remote_pending_.find(id);
      if (rp != remote_pending_.end()) drop_remote(id);
    }
  }

  void release_blocks(Sequence* s, bool publish) {
    if (s->blocks.empty()) return;
    BlockManager& bm = pool_.at(s->dp_rank);
    if (publish && s->num_placeholders == 0) {
      int valid = std::min(s->kv_tokens, s->num_tokens());
      bm.insert(s->tokens.data(), valid, s->blocks);
      if (!host_.empty()) offload_to_host(s, valid);
    }
    drop_loads_into(s);
    bm.release(s->blocks);
    s->blocks.clear();
  }

  // Copy the full blocks of `s` that the host tier does not hold yet (same chained keys as the device cache).
  void offload_to_host(Sequence* s, int valid_tokens) {
    BlockManager& hm = host_[s->dp_rank];
    BlockManager& bm = pool_.at(s->dp_rank);
    const int bs = bm.block_size();
    const int full = std::min<int>(valid_tokens / bs, static_cast<int>(s->blocks.size()));
    if (full <= 0) return;
    std::vector<int> held = hm.match(s->tokens.data(), full * bs, full);
    const int have = static_cast<int>(held.size());
    int want = std::min(full - have, hm.num_available_blocks());
    if (want > 0 && hm.allocate(want, held)) {
      hm.insert(s->tokens.data(), (have + want) * bs, held);
      for (int i = have; i < have + want; ++i) {
        offloads_[s->dp_rank].push_back({s->blocks[i], held[i]});
        bm.add_ref(s->blocks[i]);  // the copy reads the block after the sequence is gone
        pins_now_.push_back({s->dp_rank, s->blocks[i]});
      }
      stats_.host_offloaded_blocks += want;
    }
    hm.release(held);
  }

  // Extend a fresh device match with blocks that only the host tier still holds.
  void match_host(Sequence* s) {
    if (host_.empty() || s->num_placeholders > 0) return;
    BlockManager& hm = host_[s->dp_rank];
    BlockManager& bm = pool_.at(s->dp_rank);
    const int bs = bm.block_size();
    const int max_blocks = (s->num_tokens() - 1) / bs;
    const int have = static_cast<int>(s->blocks.size());
    if (max_blocks <= have || s->kv_tokens != have * bs) return;
    std::vector<int> held = hm.match(s->tokens.data(), s->num_tokens(), max_blocks);
    const int upto = static_cast<int>(held.size());
    if (upto > have && bm.allocate(upto - have, s->blocks)) {
      for (int i = have; i < upto; ++i) loads_[s->dp_rank].push_back({held[i], s->blocks[i]});
      s->kv_tokens = upto * bs;
      s->num_cached_tokens = std::min(s->kv_tokens, s->num_prompt_tokens);
      stats_.host_loaded_blocks += upto - have;
    }
    // the host blocks stay referenced until the step is built: an offload recorded later in this step must not
    // evict and overwrite a block that a load of the same step still has to read (offloads run first)
    for (int id : held) host_pins_.push_back({s->dp_rank, id});
  }

  // A sequence that gives its blocks back before the step ran must not leave copies into them behind.
  void drop_loads_into(Sequence* s) {
    if (host_.empty() || s->dp_rank < 0 || loads_[s->dp_rank].empty()) return;
    auto& v = loads_[s->dp_rank];
    v.erase(std::remove_if(v.begin(), v.end(),
                           [&](const BlockCopy& c) {
                             return std::find(s->blocks.begin(), s->blocks.end(), c.dst) != s->blocks.end();
                           }),
            v.end());
  }

  void finish_sequence(Sequence* s, FinishReason fr) {
    s->finished = true;
    s->reason = fr;
    release_blocks(s, fr == FinishReason::STOP || fr == FinishReason::LENGTH || fr == FinishReason::HANDOFF);
  }

  void emit(Sequence* s) {
    SeqOutput o;
    o.request_id = s->req->id;
    o.ext_id = s->req->ext_id;
    o.seq_index = s->index;
    o.seq_id = s->id;
    int gen = s->num_generated() - s->num_placeholders;
    if (gen > s->reported) {
      o.new_tokens.assign(s->tokens.begin() + s->num_prompt_tokens + s->reported,
                          s->tokens.begin() + s->num_prompt_tokens + gen);
      if (s->req->sampling.logprobs && static_cast<int>(s->logprobs.size()) >= gen)
        o.new_logprobs.assign(s->logprobs.begin() + s->reported, s->logprobs.begin() + gen);
      s->reported = gen;
    }
    o.finished = s->finished && s->reason != FinishReason::NONE;
    o.finish_reason = static_cast<int>(s->reason);
    o.num_prompt_tokens = s->num_prompt_tokens;
    o.num_generated = gen;
    o.num_cached_tokens = s->num_cached_tokens;
    o.request_finished = o.finished && s->req->finished();
    outputs_.push_back(std::move(o));
  }

  // After the first generated token: hand-off (disaggregated prefill) or sibling expansion.
  void after_first_token(Sequence* s) {
    Request* r = s->req;
    if (r->first_token_time == 0) r->first_token_time = clock_now();
    if (r->handoff_after_prefill && !s->finished) {
      finish_sequence(s, FinishReason::HANDOFF);
      return;
    }
    if (!r->expanded && s->index == 0) {
      // publish the prompt so that the siblings share its blocks (handle_running_requests :783-803)
      if (!s->blocks.empty() && s->num_placeholders == 0)
        pool_.at(s->dp_rank).insert(s->tokens.data(), std::min(s->kv_tokens, s->num_prompt_tokens), s->blocks);
      for (int i = 1; i < r->best_of; ++i) {
        auto c = std::make_unique<Sequence>();
        c->id = next_seq_id_++;
        c->index = i;
        c->req = r;
        c->tokens = r->prompt;
        c->num_prompt_tokens = static_cast<int>(r->prompt.size());
        c->dp_rank = s->dp_rank;
        r->seqs.push_back(std::move(c));
      }
      r->expanded = true;
    }
  }

  void reap_finished() {
    auto reap = [this](std::deque<Request*>& q) {
      for (auto it = q.begin(); it != q.end();) {
        Request* r = *it;
        if (r->cancelled) {
          for (auto& s : r->seqs)
            if (!s->finished || s->reason == FinishReason::NONE) {
              s->num_placeholders = 0;
              finish_sequence(s.get(), FinishReason::CANCELLED);
              emit(s.get());
            }
        }
        if (r->finished()) {
          it = q.erase(it);
          graveyard_.push_back(r->id);
        } else {
          ++it;
        }
      }
    };
    reap(running_);
    reap(waiting_online_);
    reap(waiting_offline_);
    // Requests are destroyed one schedule() later so that batches in flight may still
    // dereference their sequences.
    for (int64_t id : graveyard_prev_) requests_.erase(id);
    graveyard_prev_.swap(graveyard_);
    graveyard_.clear();
  }

  // ---------------------------------------------------------------- block helpers
  int blocks_needed(const Sequence* s, int upto_tokens) const {
    const int bs = pool_.at(0).block_size();
    int need = (upto_tokens + bs - 1) / bs;
    return std::max(0, need - static_cast<int>(s->blocks.size()));
  }

  // Attention-DP rank of a new sequence.  The reference takes the rank with the most free blocks
  // (block_manager_pool.cpp:97-106); here a rank that already caches the beginning of the prompt (on the device or in
  // its host tier) is preferred, as long as it has room for the rest, because a prefix cached on the other rank is
  // worth nothing.  Ties and prompts nobody caches fall back to the most free blocks.
  int choose_dp_rank(const Sequence* s) const {
    const int dp = pool_.dp_size();
    int fallback = pool_.pick_dp_rank();
    if (dp <= 1 || !pool_.at(0).prefix_cache_enabled() || s->num_placeholders > 0) return fallback;
    const int bs = pool_.at(0).block_size();
    const int n = s->num_tokens();
    const int max_blocks = n > 0 ? (n - 1) / bs : 0;
    if (max_blocks <= 0) return fallback;
    int best = fallback, best_hit = 0;
    for (int r = 0; r < dp; ++r) {
      int hit = pool_.at(r).count_prefix(s->tokens.data(), n, max_blocks);
      if (!host_.empty()) hit = std::max(hit, host_[r].count_prefix(s->tokens.data(), n, max_blocks));
      const int need = (n + bs - 1) / bs - hit + 1;
      if (hit > best_hit && pool_.at(r).num_available_blocks() >= need) {
        best = r;
        best_hit = hit;
      }
    }
    return best;
  }

  // Prefix-cache match for a sequence with no KV yet.
  void match_prefix(Sequence* s) {
    if (s->dp_rank < 0) s->dp_rank = choose_dp_rank(s);
    BlockManager& bm = pool_.at(s->dp_rank);
    if (!bm.prefix_cache_enabled() || !s->blocks.empty() || s->kv_tokens != 0) return;
    const int bs = bm.block_size();
    // leave at least one token to compute so that logits exist
    int max_blocks = (s->num_tokens() - 1) / bs;
    if (max_blocks <= 0) return;
    // placeholders can't be hashed
    if (s->num_placeholders > 0) return;
    std::vector<int> hit = bm.match(s->tokens.data(), s->num_tokens(), max_blocks);
    if (!hit.empty()) {
      s->blocks = hit;
      s->kv_tokens = static_cast<int>(hit.size()) * bs;
      s->num_cached_tokens = std::min(s->kv_tokens, s->num_prompt_tokens);
    }
    match_host(s);
  }

  // Re-match while a chunked prefill is in progress (chunked_prefill_scheduler.cpp:753-781):
  // another request may have published the same prefix meanwhile.
  void rematch_prefix(Sequence* s) {
    BlockManager& bm = pool_.at(s->dp_rank);
    if (!bm.prefix_cache_enabled() || s->num_placeholders > 0) return;
    const int bs = bm.block_size();
    if (s->kv_tokens % bs != 0) return;
    int max_blocks = (s->num_tokens() - 1) / bs;
    int have = s->kv_tokens / bs;
    if (max_blocks <= have) return;
    std::vector<int> hit = bm.match(s->tokens.data(), s->num_tokens(), max_blocks);
    if (static_cast<int>(hit.size()) > have) {
      // adopt the shared blocks beyond what we computed; give back our own duplicates
      for (int i = 0; i < static_cast<int>(hit.size()); ++i) {
        if (i < static_cast<int>(s->blocks.size())) {
          if (s->blocks[i] != hit[i]) {
            bm.release(s->blocks[i]);
            s->blocks[i] = hit[i];
          } else {
            bm.release(hit[i]);  // drop the extra reference match() took
          }
        } else {
          s->blocks.push_back(hit[i]);
        }
      }
      s->kv_tokens = static_cast<int>(hit.size()) * bs;
      s->num_cached_tokens = std::min(s->kv_tokens, s->num_prompt_tokens);
    } else {
      bm.release(hit);
    }
  }

  bool ensure_blocks(Sequence* s, int upto_tokens) {
    int need = blocks_needed(s, upto_tokens);
    if (need == 0) return true;
    return pool_.at(s->dp_rank).allocate(need, s->blocks);
  }

  void preempt(Request* r) {
    for (auto& s : r->seqs) {
      if (s->finished) continue;
      // publish what is complete so that the recompute can hit the cache
      release_blocks(s.get(), true);
      s->kv_tokens = 0;
      ++s->preempt_count;
    }
    r->preempted = true;
    ++stats_.num_preemptions;
  }

  // Evict one victim from the back of the running queue (offline first).  Never evicts `keep`
  // nor a request that already has entries in the batch being built.
  bool preempt_one(Request* keep, bool offline_only) {
    for (int pass = 0; pass < 2; ++pass) {
      for (auto it = running_.rbegin(); it != running_.rend(); ++it) {
        Request* v = *it;
        if (v == keep || in_current(v)) continue;
        if (pass == 0 && !v->offline) continue;
        if (pass == 1 && (offline_only || v->offline)) continue;
        bool has_blocks = false;
        for (auto& s : v->seqs) has_blocks |= !s->blocks.empty();
        if (!has_blocks) continue;
        preempt(v);
        if (v->offline) ++stats_.num_offline_evictions;
        running_.erase(std::next(it).base());
        push_waiting(v, /*front=*/true);
        return true;
      }
      if (offline_only) break;
    }
    return false;
  }

  bool in_current(Request* r) const { return current_.count(r->id) > 0; }

  void add_entry(std::vector<Batch>& bs, Sequence* s, int n_tokens, int n_spec) {
    Batch& b = bs[s->dp_rank];
    BatchEntry e;
    e.seq = s;
    e.n_tokens = n_tokens;
    e.n_spec = n_spec;
    e.kv_before = s->kv_tokens;
    e.sample = (s->kv_tokens + n_tokens - n_spec == s->num_tokens());
    b.entries.push_back(e);
    budget_tokens_[s->dp_rank] -= n_tokens;
    budget_seqs_[s->dp_rank] -= 1;
    current_[s->req->id] += 1;
  }

  // zero-evict admission test: would every running sequence still fit at its projected length?
  bool zero_evict_admits(const Sequence* cand, int dp_rank) const {
    const BlockManager& bm = pool_.at(dp_rank);
    const int bs = bm.block_size();
    long total = 0;
    auto projected = [&](const Sequence* s) {
      int left = std::min(s->req->stop.max_tokens - s->num_generated(), opt_.max_decode_token_per_sequence);
      int len = s->num_tokens() + std::max(left, 0);
      return (len + bs - 1) / bs;
    };
    for (auto* r : running_)
      for (auto& s : r->seqs)
        if (!s->finished && s->dp_rank == dp_rank) total += projected(s.get());
    total += projected(cand);
    return total <= bm.num_blocks() - 1;
  }

  // ---------------------------------------------------------------- policies
  // Try to admit the head of a waiting queue; returns false when admission must stop.
  bool admit_prefill(std::deque<Request*>& q, std::vector<Batch>& bs, bool chunked) {
    Request* r = q.front();
    bool any = false, blocked = false;
    for (auto& sp : r->seqs) {
      Sequence* s = sp.get();
      if (s->finished) continue;
      if (s->blocks.empty() && s->kv_tokens == 0) match_prefix(s);
      if (s->dp_rank < 0) s->dp_rank = choose_dp_rank(s);
      const int rank = s->dp_rank;
      const int remaining = s->remaining();
      int n = remaining;
      if (chunked) n = std::min({remaining, opt_.max_tokens_per_chunk_for_prefill, budget_tokens_[rank]});
      const bool alone = running_.empty() && !has_any_entry(bs);
      if (!chunked && alone && n > opt_.max_tokens_per_batch) {
        // can never be scheduled in one piece (continuous_scheduler.cpp:398-431)
        undo_match(s);
        finish_sequence(s, FinishReason::RESOURCE_EXHAUSTED);
        emit(s);
        continue;
      }
      if (budget_seqs_[rank] <= 0 || n <= 0 || n > budget_tokens_[rank] ||
          (opt_.use_zero_evict && !running_.empty() && !zero_evict_admits(s, rank))) {
        undo_match(s);
        blocked = true;
        break;
      }
      bool ok = true;
      while (!ensure_blocks(s, s->kv_tokens + n + opt_.spec_extra_slots)) {
        bool freed = false;
        if (!r->offline && opt_.enable_online_preempt_offline) freed = preempt_one(r, /*offline_only=*/true);
        if (!freed) {
          ok = false;
          break;
        }
      }
      if (!ok) {
        undo_match(s);
        if (alone && !any && !pins_outstanding()) {
          // nothing else holds memory: the request can never fit
          finish_sequence(s, FinishReason::RESOURCE_EXHAUSTED);
          emit(s);
          continue;
        }
        blocked = true;
        break;
      }
      add_entry(bs, s, n, 0);
      any = true;
    }
    if (blocked && !any) return false;
    q.pop_front();
    if (!r->finished()) {
      running_.push_back(r);
      r->preempted = false;
    } else {
      graveyard_.push_back(r->id);
    }
    return !blocked;
  }
  bool has_any_entry(const std::vector<Batch>& bs) const {
    for (auto& b : bs)
      if (!b.entries.empty()) return true;
    return false;
  }
  // A sequence that was matched against the prefix cache but not admitted must not pin blocks.
  void undo_match(Sequence* s) {
    if (s->blocks.empty()) return;
    drop_loads_into(s);
    pool_.at(s->dp_rank).release(s->blocks);
    s->blocks.clear();
    s->kv_tokens = 0;
    s->num_cached_tokens = 0;
  }
  bool is_running(const Request* r) const {
    return std::find(running_.begin(), running_.end(), r) != running_.end();
  }

  bool memory_pressure() const {
    return pool_.utilization() >= opt_.prefill_scheduling_memory_usage_threshold;
  }

  // `which`: 0 = both classes, 1 = online requests only, 2 = offline requests only
  void admit_waiting(std::vector<Batch>& bs, bool chunked, int which = 0) {
    for (auto* q : {&waiting_online_, &waiting_offline_}) {
      if ((which == 1 && q == &waiting_offline_) || (which == 2 && q == &waiting_online_)) continue;
      while (!q->empty()) {
        if (memory_pressure() && (!running_.empty() || has_any_entry(bs))) return;
        bool tokens_left = false;
        for (int i = 0; i < opt_.dp_size; ++i) tokens_left |= (budget_tokens_[i] > 0 && budget_seqs_[i] > 0);
        if (!tokens_left) return;
        if (!admit_prefill(*q, bs, chunked)) return;
      }
    }
  }

  // Decode (and running-prefill chunks in chunked mode) for the running queue.
  // `want_prefill`/`want_decode` select which stages may be scheduled.
  void schedule_running(std::vector<Batch>& bs, bool chunked, bool want_prefill, bool want_decode, int which = 0) {
    const int k = opt_.num_speculative_tokens;
    // iterate over a snapshot: preemption edits running_
    std::vector<Request*> snap(running_.begin(), running_.end());
    for (Request* r : snap) {
      if ((which == 1 && r->offline) || (which == 2 && !r->offline)) continue;
      if (!is_running(r)) continue;  // preempted meanwhile
      for (auto& sp : r->seqs) {
        Sequence* s = sp.get();
        if (s->finished) continue;
        if (s->dp_rank < 0) s->dp_rank = choose_dp_rank(s);
        const int rank = s->dp_rank;
        if (budget_seqs_[rank] <= 0) continue;
        int n, n_spec = 0;
        if (s->in_decode()) {
          if (!want_decode) continue;
          n = 1 + k;
          n_spec = k;
          if (budget_tokens_[rank] < n) continue;
        } else {
          if (!want_prefill) continue;
          if (s->blocks.empty() && s->kv_tokens == 0)
            match_prefix(s);
          else if (chunked && opt_.chunked_match_frequency > 0 && ++s->chunks_since_match >= opt_.chunked_match_frequency) {
            s->chunks_since_match = 0;
            rematch_prefix(s);
          }
          n = s->remaining();
          if (chunked) n = std::min({n, opt_.max_tokens_per_chunk_for_prefill, budget_tokens_[rank]});
          if (n <= 0 || n > budget_tokens_[rank]) continue;
        }
        bool ok = true;
        while (!ensure_blocks(s, s->kv_tokens + n + opt_.spec_extra_slots)) {
          if (!preempt_one(r, /*offline_only=*/false)) {
            ok = false;
            break;
          }
        }
        if (!ok) {
          // nothing else to evict: this request itself yields, unless it is alone
          if (!in_current(r)) {
            if (running_.size() == 1 && !has_any_entry(bs)) {
              // alone: either it can never fit, or blocks held for copies in flight come back within two steps
              if (!pins_outstanding()) {
                finish_sequence(s, FinishReason::RESOURCE_EXHAUSTED);
                emit(s);
              }
            } else {
              preempt(r);
              running_.erase(std::find(running_.begin(), running_.end(), r));
              push_waiting(r, true);
            }
          }
          break;
        }
        add_entry(bs, s, n, n_spec);
      }
    }
  }

  void schedule_prefill_first(std::vector<Batch>& bs) {
    // siblings created by expansion and recompute-after-preemption live in running_: they are prefills too
    schedule_running(bs, /*chunked=*/false, /*want_prefill=*/true, /*want_decode=*/false);
    admit_waiting(bs, /*chunked=*/false);
    if (has_any_entry(bs)) return;
    schedule_running(bs, false, false, true);
  }

  void schedule_chunked(std::vector<Batch>& bs) {
    if (opt_.prefill_only_batches) {
      schedule_running(bs, true, true, false);
      admit_waiting(bs, true);
      if (has_any_entry(bs)) return;
      schedule_running(bs, true, false, true);
      return;
    }
    // online work first: a new online prefill may still evict offline decodes, which join the step only afterwards
    // (chunked_prefill_scheduler.cpp:605-668)
    schedule_running(bs, true, false, true, 1);  // decode-maximal
    schedule_running(bs, true, true, false, 1);  // chunks of prefills already running
    admit_waiting(bs, true, 1);
    schedule_running(bs, true, false, true, 2);
    schedule_running(bs, true, true, false, 2);
    admit_waiting(bs, true, 2);
  }

  // ---------------------------------------------------------------- urgency-ordered single queue ("mix" policy)
  // Prefills and decodes of all unfinished requests, waiting or running, are ranked in one list every step
  // (the reference's MixScheduler / ProSched, mix_scheduler.cpp:41-114, with the orderings of
  // priority_comparator.cpp:24-227): requests whose slack is smaller than the work queued in front of the
  // deadline are URGENT and served by value density (weight / predicted step cost, decodes first, starved
  // prefills before the rest), the others by earliest deadline.  The step then takes requests from the front
  // until the token, sequence or latency budget is used up; when blocks run out the least important request
  // that holds KV is recomputed later.
  static constexpr double kNoSlo = 1e15;
  double clock_now() const { return clock_override_ >= 0 ? clock_override_ : now_seconds(); }
  static const Sequence* lead_seq(const Request* r) {
    for (auto& s : r->seqs)
      if (!s->finished) return s.get();
    return r->seqs.empty() ? nullptr : r->seqs[0].get();
  }
  static bool decoding(const Request* r) {
    const Sequence* s = lead_seq(r);
    return s && s->in_decode();
  }
  double ttft_slo(const Request* r) const {
    return r->ttft_slo_ms > 0 ? r->ttft_slo_ms : (opt_.max_global_ttft_ms > 0 ? opt_.max_global_ttft_ms : kNoSlo);
  }
  double tpot_slo(const Request* r) const {
    return r->tpot_slo_ms > 0 ? r->tpot_slo_ms : (opt_.max_global_tpot_ms > 0 ? opt_.max_global_tpot_ms : kNoSlo);
  }
  static double density(const Request* r) {
    const double w = decoding(r) ? r->tpot_weight : r->ttft_weight;
    return w / std::max(r->est_ms, 1e-9);
  }
  static bool earlier(const Request* a, const Request* b) {
    if (a->arrival != b->arrival) return a->arrival < b->arrival;
    return a->id < b->id;
  }
  static bool by_deadline(const Request* a, const Request* b) {
    if (a->remaining_ms != b->remaining_ms) return a->remaining_ms < b->remaining_ms;
    return earlier(a, b);
  }
  static bool by_density(const Request* a, const Request* b) {
    const double da = density(a), db = density(b);
    if (da != db) return da > db;
    return earlier(a, b);
  }
  static bool by_density_anti_starve(const Request* a, const Request* b) {
    if (a->starved != b->starved) return a->starved;
    return a->starved ? by_deadline(a, b) : by_density(a, b);
  }
  static bool by_priority(const Request* a, const Request* b) {
    if (a->priority != b->priority) return a->priority < b->priority;
    return earlier(a, b);
  }
  // true when `a` is served before `b`
  bool mix_before(const Request* a, const Request* b, const std::string& strategy) const {
    const bool da = decoding(a), db = decoding(b);
    if (strategy == "priority") return by_priority(a, b);
    if (strategy == "deadline") return by_deadline(a, b);
    if (strategy == "density") return by_density(a, b);
    if (strategy == "sjf") return a->est_ms != b->est_ms ? a->est_ms < b->est_ms : earlier(a, b);
    if (strategy == "decode_deadline") return da != db ? da : by_deadline(a, b);
    if (strategy == "decode_density") return da != db ? da : by_density(a, b);
    if (strategy == "urgency_priority") {
      if (a->urgent != b->urgent) return a->urgent;
      return a->urgent ? by_priority(a, b) : by_deadline(a, b);
    }
    if (strategy == "decode_urgency_density" && (da || db)) {
      if (da != db) return da;
      return earlier(a, b);
    }
    // urgency_density (the default of this policy)
    if (a->urgent != b->urgent) return a->urgent;
    if (!a->urgent) return by_deadline(a, b);
    if (da != db) return da;
    return da ? by_density(a, b) : by_density_anti_starve(a, b);
  }

  // Refresh the per-request metrics, derive the latency budget of the step and rank every unfinished request.
  void mix_rank(std::vector<Request*>& order, double* latency_budget) {
    order.clear();
    for (auto* r : running_) order.push_back(r);
    for (auto* r : waiting_online_) order.push_back(r);
    for (auto* r : waiting_offline_) order.push_back(r);
    const double now = clock_now(), overhead = model_.constant_overhead();
    double total_est = 0, min_remaining = kNoSlo, min_tpot = kNoSlo;
    for (auto* r : order) {
      const Sequence* s = lead_seq(r);
      const bool dec = s && s->in_decode();
      r->est_ms = !s ? 0 : (dec ? model_.decode_ms(s->kv_tokens) : model_.prefill_ms(s->num_tokens(), s->kv_tokens));
      const double elapsed = (now - r->arrival) * 1e3;
      double deadline;
      if (!dec) {
        deadline = ttft_slo(r);
      } else {
        const double ttft = r->first_token_time > 0 ? (r->first_token_time - r->arrival) * 1e3 : elapsed;
        deadline = ttft + s->num_generated() * tpot_slo(r);
      }
      r->remaining_ms = std::min(deadline, kNoSlo) - elapsed;
      r->starved = false;
      total_est += r->est_ms;
      min_tpot = std::min(min_tpot, tpot_slo(r));
      // requests that are already late do not shrink the budget of everybody else
      if (r->remaining_ms >= r->est_ms + overhead) min_remaining = std::min(min_remaining, r->remaining_ms);
    }
    double budget = std::max(min_remaining >= kNoSlo / 2 ? 0.0 : min_remaining, min_tpot >= kNoSlo / 2 ? 0.0 : 0.65 * min_tpot);
    if (min_remaining >= kNoSlo / 2 && min_tpot >= kNoSlo / 2) budget = kNoSlo;
    const double load = budget >= kNoSlo / 2 ? total_est
                                             : (budget - overhead > 1e-9 ? total_est * budget / (budget - overhead) : kNoSlo);
    for (auto* r : order) {
      if (opt_.enable_starve_prevent) {
        const double unit = decoding(r) ? tpot_slo(r) : ttft_slo(r);
        r->starved = unit < kNoSlo / 2 && r->remaining_ms < -opt_.starve_threshold * unit;
      }
      r->urgent = r->remaining_ms < opt_.aggressive_coeff * load;
    }
    const std::string strategy = opt_.priority_strategy == "fcfs" ? "urgency_density" : opt_.priority_strategy;
    std::stable_sort(order.begin(), order.end(),
                     [&](const Request* a, const Request* b) { return mix_before(a, b, strategy); });
    if (latency_budget) *latency_budget = budget;
  }

  void remove_from_queues(Request* r) {
    for (auto* q : {&running_, &waiting_online_, &waiting_offline_}) {
      auto it = std::find(q->begin(), q->end(), r);
      if (it != q->end()) {
        q->erase(it);
        return;
      }
    }
  }

  void schedule_mix(std::vector<Batch>& bs) {
    std::vector<Request*> order;
    double latency_budget = kNoSlo;
    mix_rank(order, &latency_budget);
    const bool latency_aware = opt_.enable_latency_aware_schedule && model_.fitted() && latency_budget < kNoSlo / 2;
    const int k = opt_.num_speculative_tokens;
    double spent_ms = model_.constant_overhead();
    size_t victim = order.size();  // victims are taken from the back of the ranking
    std::vector<Request*> evicted;
    // With prefill_only_batches (speculative decoding, prefill sequence parallelism) a step is all prefill or all
    // decode: its kind is that of the most urgent sequence that fits, and sequences of the other kind wait a step.
    int step_kind = -1;            // -1 undecided, 0 prefill, 1 decode
    for (size_t i = 0; i < order.size() && i < victim; ++i) {
      Request* r = order[i];
      bool stop = false, any = false;
      for (auto& sp : r->seqs) {
        Sequence* s = sp.get();
        if (s->finished) continue;
        if (opt_.prefill_only_batches && step_kind >= 0 && step_kind != int(s->in_decode())) continue;
        if (s->dp_rank < 0) s->dp_rank = choose_dp_rank(s);
        const int rank = s->dp_rank;
        int n, n_spec = 0;
        double cost = 0;
        if (s->in_decode()) {
          n = 1 + k;
          n_spec = k;
          cost = model_.decode_ms(s->kv_tokens);
          if (latency_aware && spent_ms + cost > latency_budget && has_any_entry(bs)) stop = true;
        } else {
          if (s->blocks.empty() && s->kv_tokens == 0) match_prefix(s);
          n = std::min({s->remaining(), opt_.max_tokens_per_chunk_for_prefill, budget_tokens_[rank]});
          if (latency_aware) {
            const int upto = model_.max_chunk(s->kv_tokens + n, s->kv_tokens, latency_budget - spent_ms);
            const int fit = upto - s->kv_tokens;
            // nothing fits, or only a sliver of a long prompt: leave it for a step with more slack
            if (fit < n && (fit <= 0 || fit < opt_.min_prefill_chunk)) {
              if (has_any_entry(bs)) stop = true; else n = std::max(1, std::min(n, std::max(fit, opt_.min_prefill_chunk)));
            } else {
              n = fit;
            }
          }
          cost = model_.prefill_ms(s->kv_tokens + n, s->kv_tokens);
        }
        if (!stop && (n <= 0 || budget_seqs_[rank] <= 0 || n > budget_tokens_[rank])) stop = true;
        if (stop) {
          if (!any && s->kv_tokens > 0 && !is_running(r)) undo_match(s);
          break;
        }
        bool ok = true;
        while (!ensure_blocks(s, s->kv_tokens + n + opt_.spec_extra_slots)) {
          // recompute the least important request that holds KV and is not part of this step
          bool freed = false;
          while (victim > i + 1) {
            Request* v = order[--victim];
            if (in_current(v)) continue;
            bool has_blocks = false;
            for (auto& vs : v->seqs) has_blocks |= !vs->blocks.empty();
            if (!has_blocks) continue;
            preempt(v);
            if (v->offline) ++stats_.num_offline_evictions;
            evicted.push_back(v);
            freed = true;
            break;
          }
          if (!freed) {
            ok = false;
            break;
          }
        }
        if (!ok) {
          if (!any && !has_any_entry(bs) && !pins_outstanding()) {
            // nothing else holds memory: the request can never fit
            finish_sequence(s, FinishReason::RESOURCE_EXHAUSTED);
            emit(s);
            continue;
          }
          if (!any && !is_running(r)) undo_match(s);
          stop = true;
          break;
        }
        add_entry(bs, s, n, n_spec);
        if (opt_.prefill_only_batches) step_kind = n_spec > 0 || s->in_decode() ? 1 : 0;
        spent_ms += cost;
        any = true;
      }
      if (any && !is_running(r)) {
        remove_from_queues(r);
        running_.push_back(r);
        r->preempted = false;
      }
      if (stop) break;
    }
    for (Request* v : evicted) {
      remove_from_queues(v);
      push_waiting(v, /*front=*/true);
    }
  }

  void finalize(Batch& b) {
    // decode entries first, then prefill chunks: kernels see the single-token rows contiguously
    std::stable_partition(b.entries.begin(), b.entries.end(),
                          [](const BatchEntry& e) { return e.n_tokens - e.n_spec == 1 && e.sample && e.kv_before > 0; });
    b.num_tokens = b.num_prefill_seqs = b.num_decode_seqs = b.num_sample = 0;
    for (auto& e : b.entries) {
      b.num_tokens += e.n_tokens;
      const bool dec = (e.n_tokens - e.n_spec == 1 && e.sample && e.kv_before > 0);
      if (dec) ++b.num_decode_seqs; else ++b.num_prefill_seqs;
      if (e.sample) e.sample_slot = b.num_sample++;
    }
  }

  std::vector<BlockManager> host_;                              // host tier, one per DP rank (empty: off)
  std::vector<std::vector<BlockCopy>> loads_, offloads_;        // copies of the step being built, per DP rank
  std::vector<std::pair<int, int>> host_pins_, pins_now_;       // (dp rank, block) references held for copies
  std::deque<std::vector<std::pair<int, int>>> offload_pins_;   // device blocks of the last two hand-overs
  SchedulerOptions opt_;
  StepTimeModel model_;
  double clock_override_ = -1.0;
  BlockManagerPool pool_;
  std::mutex mu_;
  std::deque<std::unique_ptr<Request>> incoming_;
  std::vector<int64_t> cancels_;
  std::unordered_map<int64_t, std::unique_ptr<Request>> requests_;
  std::unordered_map<int64_t, std::unique_ptr<Request>> remote_pending_;
  std::deque<Request*> waiting_online_, waiting_offline_, running_;
  std::deque<std::vector<Batch>> batches_storage_;
  std::unordered_map<int64_t, Batch*> live_batches_;
  std::unordered_map<int64_t, int> current_;
  int configured_max_tokens_ = 0;
  std::vector<int> budget_tokens_, budget_seqs_;
  std::vector<SeqOutput> outputs_;
  std::vector<int64_t> graveyard_, graveyard_prev_;
  SchedulerStats stats_;
  int64_t next_request_id_ = 1, next_seq_id_ = 1, next_batch_id_ = 1;
};

}  // namespace xl
