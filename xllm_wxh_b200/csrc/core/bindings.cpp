// pybind11 module `xllm_wxh_b200._core`: host-side runtime in C++
// (scheduler, block manager, prefix cache, batch builder, safetensors index, BPE tokenizer,
// shared-memory step channel, EPLB policy, suffix-tree drafter).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "batch_builder.h"
#include "bpe_tokenizer.h"
#include "eplb_policy.h"
#include "safetensors.h"
#include "scheduler.h"
#include "shm_channel.h"
#include "suffix_tree.h"

namespace py = pybind11;
using namespace xl;

namespace {

std::unique_ptr<Request> make_request(const std::vector<int32_t>& prompt, const SamplingParams& sp, const StopCriteria& st,
                                      int n, int best_of, int priority, bool offline, const std::string& ext_id,
                                      double ttft_slo_ms, double tpot_slo_ms = 0.0, int ttft_weight = 1,
                                      int tpot_weight = 1) {
  auto r = std::make_unique<Request>();
  r->prompt = prompt;
  r->sampling = sp;
  r->stop = st;
  r->n = std::max(1, n);
  r->best_of = std::max(r->n, best_of);
  r->priority = priority;
  r->offline = offline;
  r->ext_id = ext_id;
  r->arrival = now_seconds();
  r->deadline = r->arrival + (ttft_slo_ms > 0 ? ttft_slo_ms * 1e-3 : 1e9);
  r->ttft_slo_ms = std::max(0.0, ttft_slo_ms);
  r->tpot_slo_ms = std::max(0.0, tpot_slo_ms);
  r->ttft_weight = std::max(1, ttft_weight);
  r->tpot_weight = std::max(1, tpot_weight);
  return r;
}

}  // namespace

PYBIND11_MODULE(_core, m) {
  m.doc() = "host-side runtime of the B200-native xLLM engine";

  py::class_<SamplingParams>(m, "SamplingParams")
      .def(py::init<>())
      .def_readwrite("temperature", &SamplingParams::temperature)
      .def_readwrite("top_p", &SamplingParams::top_p)
      .def_readwrite("top_k", &SamplingParams::top_k)
      .def_readwrite("repetition_penalty", &SamplingParams::repetition_penalty)
      .def_readwrite("frequency_penalty", &SamplingParams::frequency_penalty)
      .def_readwrite("presence_penalty", &SamplingParams::presence_penalty)
      .def_readwrite("logprobs", &SamplingParams::logprobs)
      .def_readwrite("top_logprobs", &SamplingParams::top_logprobs)
      .def_readwrite("seed", &SamplingParams::seed);

  py::class_<StopCriteria>(m, "StopCriteria")
      .def(py::init<>())
      .def_readwrite("max_tokens", &StopCriteria::max_tokens)
      .def_readwrite("max_context_len", &StopCriteria::max_context_len)
      .def_readwrite("eos_token_id", &StopCriteria::eos_token_id)
      .def_readwrite("ignore_eos", &StopCriteria::ignore_eos)
      .def_readwrite("stop_token_ids", &StopCriteria::stop_token_ids)
      .def_readwrite("stop_sequences", &StopCriteria::stop_sequences);

  py::class_<SchedulerOptions>(m, "SchedulerOptions")
      .def(py::init<>())
      .def_readwrite("max_tokens_per_batch", &SchedulerOptions::max_tokens_per_batch)
      .def_readwrite("max_seqs_per_batch", &SchedulerOptions::max_seqs_per_batch)
      .def_readwrite("enable_chunked_prefill", &SchedulerOptions::enable_chunked_prefill)
      .def_readwrite("max_tokens_per_chunk_for_prefill", &SchedulerOptions::max_tokens_per_chunk_for_prefill)
      .def_readwrite("prefill_only_batches", &SchedulerOptions::prefill_only_batches)
      .def_readwrite("use_zero_evict", &SchedulerOptions::use_zero_evict)
      .def_readwrite("max_decode_token_per_sequence", &SchedulerOptions::max_decode_token_per_sequence)
      .def_readwrite("num_speculative_tokens", &SchedulerOptions::num_speculative_tokens)
      .def_readwrite("spec_extra_slots", &SchedulerOptions::spec_extra_slots)
      .def_readwrite("prefill_scheduling_memory_usage_threshold", &SchedulerOptions::prefill_scheduling_memory_usage_threshold)
      .def_readwrite("enable_online_preempt_offline", &SchedulerOptions::enable_online_preempt_offline)
      .def_readwrite("priority_strategy", &SchedulerOptions::priority_strategy)
      .def_readwrite("chunked_match_frequency", &SchedulerOptions::chunked_match_frequency)
      .def_readwrite("dp_size", &SchedulerOptions::dp_size)
      .def_readwrite("handoff_after_prefill", &SchedulerOptions::handoff_after_prefill)
      .def_readwrite("use_mix_scheduler", &SchedulerOptions::use_mix_scheduler)
      .def_readwrite("enable_latency_aware_schedule", &SchedulerOptions::enable_latency_aware_schedule)
      .def_readwrite("max_global_ttft_ms", &SchedulerOptions::max_global_ttft_ms)
      .def_readwrite("max_global_tpot_ms", &SchedulerOptions::max_global_tpot_ms)
      .def_readwrite("aggressive_coeff", &SchedulerOptions::aggressive_coeff)
      .def_readwrite("starve_threshold", &SchedulerOptions::starve_threshold)
      .def_readwrite("enable_starve_prevent", &SchedulerOptions::enable_starve_prevent)
      .def_readwrite("min_prefill_chunk", &SchedulerOptions::min_prefill_chunk)
      .def_readwrite("host_blocks_factor", &SchedulerOptions::host_blocks_factor);

  py::class_<StepTimeModel>(m, "StepTimeModel")
      .def(py::init<>())
      .def_readwrite("a0", &StepTimeModel::a0)
      .def_readwrite("a1", &StepTimeModel::a1)
      .def_readwrite("a2", &StepTimeModel::a2)
      .def_readwrite("b0", &StepTimeModel::b0)
      .def_readwrite("b1", &StepTimeModel::b1)
      .def_readwrite("b2", &StepTimeModel::b2)
      .def("prefill_ms", &StepTimeModel::prefill_ms, py::arg("upto"), py::arg("kv") = 0)
      .def("decode_ms", &StepTimeModel::decode_ms)
      .def("max_chunk", &StepTimeModel::max_chunk)
      .def_property_readonly("constant_overhead", &StepTimeModel::constant_overhead);

  py::class_<SeqOutput>(m, "SeqOutput")
      .def_readonly("request_id", &SeqOutput::request_id)
      .def_readonly("ext_id", &SeqOutput::ext_id)
      .def_readonly("seq_index", &SeqOutput::seq_index)
      .def_readonly("seq_id", &SeqOutput::seq_id)
      .def_readonly("new_tokens", &SeqOutput::new_tokens)
      .def_readonly("new_logprobs", &SeqOutput::new_logprobs)
      .def_readonly("finished", &SeqOutput::finished)
      .def_readonly("finish_reason", &SeqOutput::finish_reason)
      .def_readonly("num_prompt_tokens", &SeqOutput::num_prompt_tokens)
      .def_readonly("num_generated", &SeqOutput::num_generated)
      .def_readonly("num_cached_tokens", &SeqOutput::num_cached_tokens)
      .def_readonly("request_finished", &SeqOutput::request_finished);

  py::class_<BatchLayout>(m, "BatchLayout")
      .def(py::init<int, int, int, int, int>(), py::arg("T_cap"), py::arg("B_cap"), py::arg("MB_cap"), py::arg("S_cap"),
           py::arg("P_cap"))
#define RO(f) .def_readonly(#f, &BatchLayout::f)
      RO(T_cap) RO(B_cap) RO(MB_cap) RO(S_cap) RO(P_cap) RO(header) RO(tokens) RO(positions) RO(slots) RO(token_seq) RO(next_tokens)
      RO(q_cu) RO(kv_lens) RO(block_tables) RO(sample_idx) RO(temperature) RO(top_p) RO(top_k) RO(rep_pen) RO(freq_pen)
      RO(pres_pen) RO(seed_lo) RO(seed_hi) RO(want_logprobs) RO(pen_cu) RO(pen_ids) RO(pen_counts) RO(total_words)
#undef RO
      ;

  py::class_<Batch>(m, "Batch")
      .def_readonly("id", &Batch::id)
      .def_readonly("dp_rank", &Batch::dp_rank)
      .def_readonly("num_tokens", &Batch::num_tokens)
      .def_readonly("num_prefill_seqs", &Batch::num_prefill_seqs)
      .def_readonly("num_decode_seqs", &Batch::num_decode_seqs)
      .def_readonly("num_sample", &Batch::num_sample)
      .def_property_readonly("num_seqs", [](const Batch& b) { return b.entries.size(); })
      .def_property_readonly("forward_type", [](const Batch& b) { return static_cast<int>(b.forward_type()); })
      .def_property_readonly("empty", [](const Batch& b) { return b.entries.empty(); })
      .def_property_readonly("num_sample_rows",
                             [](const Batch& b) {
                               int r = 0;
                               for (auto& e : b.entries) if (e.sample) r += 1 + e.n_spec;
                               return r;
                             })
      .def_property_readonly("max_blocks",
                             [](const Batch& b) {
                               size_t mb = 0;
                               for (auto& e : b.entries) mb = std::max(mb, e.seq->blocks.size());
                               return mb;
                             })
      .def_property_readonly("num_spec",
                             [](const Batch& b) {
                               int k = 0;
                               for (auto& e : b.entries) k = std::max(k, e.n_spec);
                               return k;
                             })
      // (seq_id, request_id, n_tokens, n_spec, sample, kv_before, sample_slot, seq_index) per entry
      .def("entries", [](const Batch& b) {
        std::vector<std::tuple<int64_t, int64_t, int, int, bool, int, int, int>> v;
        for (auto& e : b.entries)
          v.emplace_back(e.seq->id, e.seq->req->id, e.n_tokens, e.n_spec, e.sample, e.kv_before, e.sample_slot,
                         e.seq->index);
        return v;
      })
      // (request_id, seq_index, first sampling row, top_logprobs) of the sampling entries that asked for alternatives
      .def("top_logprob_rows", [](const Batch& b) {
        std::vector<std::tuple<int64_t, int, int, int>> v;
        int row = 0;
        for (auto& e : b.entries) {
          if (!e.sample) continue;
          const auto& sp = e.seq->req->sampling;
          if (sp.logprobs && sp.top_logprobs > 0) v.emplace_back(e.seq->req->id, e.seq->index, row, sp.top_logprobs);
          row += 1 + e.n_spec;
        }
        return v;
      })
      .def("seq_tokens", [](const Batch& b, int i) { return b.entries.at(i).seq->tokens; })
      .def("seq_num_tokens", [](const Batch& b, int i) { return b.entries.at(i).seq->num_tokens(); })
      .def("seq_tokens_from", [](const Batch& b, int i, int start) {
        // the tokens of entry i's sequence from position `start` on (callers that follow a sequence step by step)
        const auto& t = b.entries.at(i).seq->tokens;
        const int n = static_cast<int>(t.size());
        start = std::max(0, std::min(start, n));
        return std::vector<int32_t>(t.begin() + start, t.end());
      })
      .def("seq_blocks", [](const Batch& b, int i) { return b.entries.at(i).seq->blocks; })
      .def("build", [](const Batch& b, const BatchLayout& L, uintptr_t ptr, size_t capacity_words, int block_size) {
        if (capacity_words < size_t(L.total_words)) throw std::runtime_error("staging buffer too small for layout");
        return build_batch(b, L, reinterpret_cast<int32_t*>(ptr), block_size);
      });

  py::class_<BlockManager>(m, "BlockManager")
      .def(py::init<int, int, bool, uint64_t>(), py::arg("num_blocks"), py::arg("block_size"),
           py::arg("enable_prefix_cache") = true, py::arg("seed") = 1024)
      .def_property_readonly("block_size", &BlockManager::block_size)
      .def_property_readonly("num_blocks", &BlockManager::num_blocks)
      .def_property_readonly("num_free_blocks", &BlockManager::num_free_blocks)
      .def_property_readonly("num_used_blocks", &BlockManager::num_used_blocks)
      .def_property_readonly("num_available_blocks", &BlockManager::num_available_blocks)
      .def_property_readonly("num_blocks_in_prefix_cache", &BlockManager::num_blocks_in_prefix_cache)
      .def_property_readonly("utilization", &BlockManager::utilization)
      .def_property_readonly("match_queries", &BlockManager::match_queries)
      .def_property_readonly("match_hits", &BlockManager::match_hits)
      .def("ref_count", &BlockManager::ref_count)
      .def("allocate", [](BlockManager& bm, int n) {
        std::vector<int> out;
        if (!bm.allocate(n, out)) return std::vector<int>{};
        return out;
      })
      .def("release", [](BlockManager& bm, const std::vector<int>& ids) { bm.release(ids); })
      .def("match", [](BlockManager& bm, const std::vector<int32_t>& t, int max_blocks) {
        return bm.match(t.data(), static_cast<int>(t.size()), max_blocks);
      }, py::arg("tokens"), py::arg("max_blocks") = 1 << 30)
      .def("insert", [](BlockManager& bm, const std::vector<int32_t>& t, const std::vector<int>& blocks) {
        return bm.insert(t.data(), static_cast<int>(t.size()), blocks);
      })
      .def("evict", &BlockManager::evict)
      .def("drop_cached", &BlockManager::drop_cached)
      // prefix key of a cached block as (lo, hi); (0, 0) for a block outside the cache
      .def("block_hash", [](BlockManager& bm, int id) {
        Hash128 h = bm.hash_of(id);
        return std::make_pair(h.lo, h.hi);
      })
      .def("count_prefix", [](BlockManager& bm, const std::vector<int32_t>& t, int max_blocks) {
        return bm.count_prefix(t.data(), static_cast<int>(t.size()), max_blocks);
      }, py::arg("tokens"), py::arg("max_blocks") = 1 << 30)
      .def("record_cache_events", &BlockManager::record_cache_events)
      // (stored, removed) prefix keys since the last call, each key as (lo, hi)
      .def("take_cache_events", [](BlockManager& bm) {
        auto ev = bm.take_cache_events();
        std::vector<std::pair<uint64_t, uint64_t>> st, rm;
        for (auto& h : ev.first) st.emplace_back(h.lo, h.hi);
        for (auto& h : ev.second) rm.emplace_back(h.lo, h.hi);
        return std::make_pair(st, rm);
      });

  // chained keys of the full blocks of a token sequence, as the prefix cache computes them
  m.def("prefix_block_keys", [](const std::vector<int32_t>& tokens, int block_size, uint64_t seed) {
    std::vector<std::pair<uint64_t, uint64_t>> out;
    Hash128 prev;
    const int full = block_size > 0 ? static_cast<int>(tokens.size()) / block_size : 0;
    for (int b = 0; b < full; ++b) {
      Hash128 h = chain_block_hash(b ? &prev : nullptr, tokens.data() + size_t(b) * block_size, block_size, seed);
      out.emplace_back(h.lo, h.hi);
      prev = h;
    }
    return out;
  }, py::arg("tokens"), py::arg("block_size"), py::arg("seed") = 1024);

  m.def("hash128", [](py::bytes data, uint64_t seed) {
    std::string s = data;
    Hash128 h = hash128(s.data(), s.size(), seed);
    return std::make_pair(h.lo, h.hi);
  });

  py::class_<Scheduler>(m, "Scheduler")
      .def(py::init<const SchedulerOptions&, int, int, bool, uint64_t>(), py::arg("options"), py::arg("num_blocks"),
           py::arg("block_size"), py::arg("enable_prefix_cache") = true, py::arg("seed") = 1024)
      .def("add_request",
           [](Scheduler& s, const std::vector<int32_t>& prompt, const SamplingParams& sp, const StopCriteria& st, int n,
              int best_of, int priority, bool offline, const std::string& ext_id, double ttft_slo_ms, double tpot_slo_ms,
              int ttft_weight, int tpot_weight) {
             return s.add_request(make_request(prompt, sp, st, n, best_of, priority, offline, ext_id, ttft_slo_ms,
                                               tpot_slo_ms, ttft_weight, tpot_weight));
           },
           py::arg("prompt"), py::arg("sampling") = SamplingParams(), py::arg("stop") = StopCriteria(), py::arg("n") = 1,
           py::arg("best_of") = 1, py::arg("priority") = 0, py::arg("offline") = false, py::arg("ext_id") = "",
           py::arg("ttft_slo_ms") = 0.0, py::arg("tpot_slo_ms") = 0.0, py::arg("ttft_weight") = 1,
           py::arg("tpot_weight") = 1, py::call_guard<py::gil_scoped_release>())
      .def("reserve_remote",
           [](Scheduler& s, const std::vector<int32_t>& prompt, const SamplingParams& sp, const StopCriteria& st,
              const std::string& ext_id) {
             int rank = 0;
             auto blocks = s.reserve_remote(make_request(prompt, sp, st, 1, 1, 0, false, ext_id, 0), &rank);
             return py::make_tuple(blocks.empty() ? int64_t(-1) : s.last_reserved_id(), blocks, rank);
           })
      .def("activate_remote", &Scheduler::activate_remote)
      .def("drop_remote", &Scheduler::drop_remote)
      .def("cancel", &Scheduler::cancel)
      .def("has_unfinished", &Scheduler::has_unfinished)
      .def_property_readonly("num_waiting", &Scheduler::num_waiting)
      .def("set_token_budget", &Scheduler::set_token_budget)
      .def_property_readonly("token_budget", &Scheduler::token_budget)
      .def_property_readonly("host_tier_enabled", &Scheduler::host_tier_enabled)
      .def_property_readonly("num_host_blocks", &Scheduler::num_host_blocks)
      .def_property_readonly("has_pending_transfers", &Scheduler::has_pending_transfers)
      .def("host_manager", &Scheduler::host_manager, py::return_value_policy::reference_internal, py::arg("dp_rank") = 0)
      .def("prefix_presence", &Scheduler::prefix_presence, py::arg("dp_rank"), py::arg("tokens"))
      .def("host_adopt", &Scheduler::host_adopt, py::arg("dp_rank"), py::arg("tokens"), py::arg("from_block"),
           py::arg("upto_blocks"))
      // per DP rank: (offloads [(device block, host block)], loads [(host block, device block)]) since the last call
      .def("take_transfers", [](Scheduler& s) {
        std::vector<std::pair<std::vector<std::pair<int, int>>, std::vector<std::pair<int, int>>>> out;
        for (auto& pr : s.take_transfers()) {
          out.emplace_back();
          for (auto& c : pr.first) out.back().first.emplace_back(c.src, c.dst);
          for (auto& c : pr.second) out.back().second.emplace_back(c.src, c.dst);
        }
        return out;
      })
      .def("set_step_time_model", &Scheduler::set_step_time_model)
      .def("step_time_model", &Scheduler::step_time_model)
      .def("set_clock_override", &Scheduler::set_clock_override)
      .def("mix_order", &Scheduler::mix_order)
      .def("mix_latency_budget", &Scheduler::mix_latency_budget)
      .def_property_readonly("num_running", &Scheduler::num_running)
      .def_property_readonly("num_pending", &Scheduler::num_pending)
      .def("schedule", &Scheduler::schedule, py::return_value_policy::reference_internal)
      .def("process_output",
           [](Scheduler& s, int64_t batch_id, py::array_t<int32_t, py::array::c_style | py::array::forcecast> tokens,
              py::object logprobs) {
             int width = tokens.ndim() == 2 ? static_cast<int>(tokens.shape(1)) : 1;
             const float* lp = nullptr;
             py::array_t<float, py::array::c_style | py::array::forcecast> lpa;
             if (!logprobs.is_none()) {
               lpa = logprobs.cast<py::array_t<float, py::array::c_style | py::array::forcecast>>();
               lp = lpa.data();
             }
             Batch* b = s.find_batch(batch_id);
             if (b) {
               int rows = 0;
               for (auto& e : b->entries) if (e.sample) ++rows;
               if (tokens.size() < py::ssize_t(rows) * width) throw std::runtime_error("process_output: too few tokens");
             }
             s.process_output(batch_id, tokens.data(), lp, width);
           },
           py::arg("batch_id"), py::arg("tokens"), py::arg("logprobs") = py::none())
      .def("process_placeholder_output", &Scheduler::process_placeholder_output)
      .def("update_output",
           [](Scheduler& s, int64_t batch_id, py::array_t<int32_t, py::array::c_style | py::array::forcecast> tokens,
              py::object logprobs) {
             const float* lp = nullptr;
             py::array_t<float, py::array::c_style | py::array::forcecast> lpa;
             if (!logprobs.is_none()) {
               lpa = logprobs.cast<py::array_t<float, py::array::c_style | py::array::forcecast>>();
               lp = lpa.data();
             }
             s.update_output(batch_id, tokens.data(), lp);
           },
           py::arg("batch_id"), py::arg("tokens"), py::arg("logprobs") = py::none())
      .def("take_outputs", &Scheduler::take_outputs)
      .def("running_ids", &Scheduler::running_ids)
      .def("waiting_ids", &Scheduler::waiting_ids)
      .def("block_manager", [](Scheduler& s, int dp_rank) -> BlockManager& { return s.pool().at(dp_rank); },
           py::return_value_policy::reference_internal, py::arg("dp_rank") = 0)
      .def_property_readonly("kv_utilization", [](Scheduler& s) { return s.pool().utilization(); })
      .def("request_tokens",
           [](Scheduler& s, int64_t id, int seq) {
             Request* r = s.find_request(id);
             if (!r || seq >= static_cast<int>(r->seqs.size())) return std::vector<int32_t>{};
             return r->seqs[seq]->tokens;
           })
      .def("stats", [](Scheduler& s) {
        py::dict d;
        const auto& st = s.stats();
        d["num_preemptions"] = st.num_preemptions;
        d["num_offline_evictions"] = st.num_offline_evictions;
        d["prompt_tokens"] = st.prompt_tokens;
        d["generated_tokens"] = st.generated_tokens;
        d["steps"] = st.steps;
        d["host_offloaded_blocks"] = st.host_offloaded_blocks;
        d["host_loaded_blocks"] = st.host_loaded_blocks;
        d["host_adopted_blocks"] = st.host_adopted_blocks;
        return d;
      });

  // ---- safetensors
  py::class_<SafeTensorInfo>(m, "SafeTensorInfo")
      .def_readonly("name", &SafeTensorInfo::name)
      .def_readonly("dtype", &SafeTensorInfo::dtype)
      .def_readonly("shape", &SafeTensorInfo::shape)
      .def_readonly("begin", &SafeTensorInfo::begin)
      .def_readonly("end", &SafeTensorInfo::end);
  py::class_<SafeTensorsFile>(m, "SafeTensorsFile")
      .def(py::init<const std::string&>())
      .def("keys", &SafeTensorsFile::keys)
      .def("info", &SafeTensorsFile::info)
      .def("has", &SafeTensorsFile::has)
      .def_property_readonly("metadata", &SafeTensorsFile::metadata)
      .def_property_readonly("data_ptr", [](SafeTensorsFile& f) { return reinterpret_cast<uintptr_t>(f.data()); })
      .def_property_readonly("data_size", &SafeTensorsFile::data_size)
      // zero-copy view of one tensor's bytes; the file object must outlive the array
      .def("view", [](py::object self, const std::string& name) {
        auto& f = self.cast<SafeTensorsFile&>();
        const SafeTensorInfo& ti = f.info(name);
        return py::array_t<uint8_t>({py::ssize_t(ti.end - ti.begin)}, {1}, f.data() + ti.begin, self);
      });

  // ---- tokenizer
  py::class_<BpeTokenizer>(m, "BpeTokenizer")
      .def(py::init<>())
      .def("load_vocab", &BpeTokenizer::load_vocab)
      .def("add_special", &BpeTokenizer::add_special)
      .def("encode", &BpeTokenizer::encode, py::arg("text"), py::arg("allow_special") = true,
           py::call_guard<py::gil_scoped_release>())
      .def("decode", [](const BpeTokenizer& t, const std::vector<int32_t>& ids, bool skip_special) {
        return py::bytes(t.decode(ids, skip_special));
      }, py::arg("ids"), py::arg("skip_special") = true)
      .def("token_to_id", &BpeTokenizer::token_to_id)
      .def("id_to_token", [](const BpeTokenizer& t, int id) { return py::bytes(t.id_to_token(id)); })
      .def_property_readonly("vocab_size", &BpeTokenizer::vocab_size);

  // ---- shared-memory step channel
  py::class_<ShmChannel>(m, "ShmChannel")
      .def(py::init<const std::string&, size_t, int, bool>(), py::arg("name"), py::arg("capacity_bytes"),
           py::arg("num_readers"), py::arg("create"))
      .def("write", [](ShmChannel& c, py::bytes data, double timeout_s) {
        std::string s = data;
        py::gil_scoped_release rel;
        return c.write(s.data(), s.size(), timeout_s);
      }, py::arg("data"), py::arg("timeout_s") = 10.0)
      .def("write_ptr", [](ShmChannel& c, uintptr_t p, size_t n, double timeout_s) {
        py::gil_scoped_release rel;
        return c.write(reinterpret_cast<const void*>(p), n, timeout_s);
      }, py::arg("ptr"), py::arg("nbytes"), py::arg("timeout_s") = 10.0)
      .def("read", [](ShmChannel& c, int reader, double timeout_s) -> py::object {
        std::string out;
        int rc;
        {
          py::gil_scoped_release rel;
          rc = c.read(reader, out, timeout_s);
        }
        if (rc != 0) return py::none();
        return py::bytes(out);
      }, py::arg("reader"), py::arg("timeout_s") = 10.0)
      .def("read_into", [](ShmChannel& c, int reader, uintptr_t p, size_t cap, double timeout_s) {
        py::gil_scoped_release rel;
        return c.read_into(reader, reinterpret_cast<void*>(p), cap, timeout_s);
      }, py::arg("reader"), py::arg("ptr"), py::arg("capacity"), py::arg("timeout_s") = 10.0)
      .def("close", &ShmChannel::close)
      .def_static("unlink", &ShmChannel::unlink);

  // ---- EPLB policy
  m.def("eplb_rebalance", &eplb_rebalance, py::arg("load"), py::arg("num_devices"), py::arg("slots_per_device"),
        "load: [layers][experts] -> (placement [layers][devices*slots], replica_count [layers][experts])");
  m.def("eplb_should_update", &eplb_should_update, py::arg("old_load"), py::arg("new_load"), py::arg("threshold"));

  // ---- suffix-tree drafter
  py::class_<SuffixCache>(m, "SuffixCache")
      .def(py::init<int, int>(), py::arg("max_depth") = 64, py::arg("max_sequences") = 4096)
      .def("append", &SuffixCache::append)
      .def("evict", &SuffixCache::evict)
      .def("speculate", &SuffixCache::speculate, py::arg("seq_id"), py::arg("context"), py::arg("max_tokens"),
           py::arg("min_match") = 2)
      .def("speculate_scored", &SuffixCache::speculate_scored, py::arg("context"), py::arg("max_spec_tokens"),
           py::arg("max_spec_factor") = 1.0f, py::arg("max_spec_offset") = 0.0f, py::arg("min_token_prob") = 0.1f)
      .def_property_readonly("num_nodes", &SuffixCache::num_nodes);
}
