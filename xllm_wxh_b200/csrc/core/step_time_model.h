// Step-time model used by the latency-aware scheduling policies.
//
// Same role as the reference's TimePredictor (xllm/core/scheduler/profile/time_predictor.cpp) as seen by its
// schedulers through ProfileManager::predict_step_time / get_constant_overhead (profile_manager.h:31-100):
//
//   prefill_ms(n tokens after kv cached tokens) = a1 * n + a2 * n * (kv + n / 2)      (+ a0 once per step)
//   decode_ms(one token against kv cached tokens) = b1 + b2 * kv                      (+ b0 once per step)
//
// The coefficients come from the start-up profiler (least-squares fit over timed synthetic steps).  With all
// coefficients zero every prediction is zero and latency budgets never bind.
#pragma once
#include <algorithm>

namespace xl {

struct StepTimeModel {
  double a0 = 0, a1 = 0, a2 = 0;  // prefill
  double b0 = 0, b1 = 0, b2 = 0;  // decode

  bool fitted() const { return a1 > 0 || a2 > 0 || b1 > 0 || b2 > 0 || a0 > 0 || b0 > 0; }
  double constant_overhead() const { return std::max(a0, b0); }
  // cost of handling tokens [kv, upto) of one sequence in a step, without the per-step constant
  double prefill_ms(int upto, int kv) const {
    const double n = std::max(0, upto - kv);
    return a1 * n + a2 * n * (kv + n / 2.0);
  }
  double decode_ms(int kv) const { return b1 + b2 * kv; }

  // Largest `upto` in [kv, num_tokens] with prefill_ms(upto, kv) <= budget_ms (binary search, as
  // MixScheduler::get_max_chunk, mix_scheduler.cpp:616-655).
  int max_chunk(int num_tokens, int kv, double budget_ms) const {
    if (num_tokens <= kv) return kv;
    if (prefill_ms(num_tokens, kv) <= budget_ms) return num_tokens;
    if (budget_ms <= 0) return kv;
    int lo = kv + 1, hi = num_tokens + 1;  // [lo, hi)
    while (lo < hi) {
      const int mid = lo + (hi - lo) / 2;
      if (prefill_ms(mid, kv) <= budget_ms) lo = mid + 1; else hi = mid;
    }
    return lo - 1;
  }
};

}  // namespace xl
