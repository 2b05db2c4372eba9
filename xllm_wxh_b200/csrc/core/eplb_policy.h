// Expert-parallel load-balancing policy.
//
// Same decisions as the reference policy (xllm/core/framework/eplb/eplb_policy.cpp:40-175):
//   1. a layer is re-planned only when the cosine similarity between its new and its last
//      planned (max-normalised) load vector drops below a threshold;
//   2. redundant slots go to the currently heaviest experts, one at a time, each replica
//      lowering that expert's per-copy weight to w*c/(c+1);
//   3. replicas are placed first, each on the least-loaded device; then the primaries in
//      descending weight on the least-loaded device that still has a free slot.
// Inputs/outputs are plain vectors; slot value = logical expert id.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <numeric>
#include <stdexcept>
#include <utility>
#include <vector>

namespace xl {

inline bool eplb_should_update(const std::vector<double>& old_load, const std::vector<double>& new_load,
                               double threshold) {
  if (old_load.size() != new_load.size()) return true;
  double mo = 1e-6, mn = 1e-6;
  for (double v : old_load) mo = std::max(mo, v + 1e-6);
  for (double v : new_load) mn = std::max(mn, v + 1e-6);
  double dot = 0, no = 0, nn = 0;
  for (size_t i = 0; i < old_load.size(); ++i) {
    double a = old_load[i] / mo, b = new_load[i] / mn;
    dot += a * b;
    no += a * a;
    nn += b * b;
  }
  double cs = dot / (std::max(std::sqrt(no), 1e-8) * std::max(std::sqrt(nn), 1e-8));
  return cs < threshold;
}

// One layer.  Returns placement[num_devices * slots_per_device] (logical expert per physical slot).
inline std::vector<int> eplb_pack_layer(const std::vector<double>& load, int num_devices, int slots_per_device,
                                        std::vector<int>* replicas_out = nullptr) {
  const int E = static_cast<int>(load.size());
  const int total_slots = num_devices * slots_per_device;
  const int redundant = total_slots - E;
  if (redundant < 0) throw std::invalid_argument("eplb: fewer physical slots than experts");
  std::vector<double> w(load);
  std::vector<int> copies(E, 1);
  for (int i = 0; i < redundant; ++i) {
    int mx = static_cast<int>(std::max_element(w.begin(), w.end()) - w.begin());
    w[mx] = w[mx] * copies[mx] / (copies[mx] + 1.0);
    ++copies[mx];
  }
  std::vector<int> placement(total_slots, -1);
  std::vector<double> dev_load(num_devices, 0.0);
  std::vector<int> dev_fill(num_devices, 0);
  auto least_loaded = [&](bool need_free) {
    int best = -1;
    for (int d = 0; d < num_devices; ++d) {
      if (need_free && dev_fill[d] >= slots_per_device) continue;
      if (best < 0 || dev_load[d] < dev_load[best]) best = d;
    }
    return best;
  };
  auto put = [&](int d, int e) {
    placement[d * slots_per_device + dev_fill[d]++] = e;
    dev_load[d] += w[e];
  };
  for (int e = 0; e < E; ++e)
    for (int c = 1; c < copies[e]; ++c) {
      int d = least_loaded(true);
      // a replica next to another copy of the same expert is wasted: prefer another device
      bool dup = false;
      for (int s = 0; s < dev_fill[d]; ++s) dup |= (placement[d * slots_per_device + s] == e);
      if (dup) {
        int alt = -1;
        for (int dd = 0; dd < num_devices; ++dd) {
          if (dev_fill[dd] >= slots_per_device) continue;
          bool has = false;
          for (int s = 0; s < dev_fill[dd]; ++s) has |= (placement[dd * slots_per_device + s] == e);
          if (!has && (alt < 0 || dev_load[dd] < dev_load[alt])) alt = dd;
        }
        if (alt >= 0) d = alt;
      }
      put(d, e);
    }
  std::vector<int> order(E);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return w[a] > w[b]; });
  for (int e : order) {
    int d = least_loaded(true);
    if (d < 0) break;
    put(d, e);
  }
  if (replicas_out) *replicas_out = copies;
  return placement;
}

// All layers: load[layers][experts] -> (placement[layers][slots], replicas[layers][experts])
inline std::pair<std::vector<std::vector<int>>, std::vector<std::vector<int>>> eplb_rebalance(
    const std::vector<std::vector<double>>& load, int num_devices, int slots_per_device) {
  std::vector<std::vector<int>> placement, replicas;
  for (auto& l : load) {
    std::vector<int> rep;
    placement.push_back(eplb_pack_layer(l, num_devices, slots_per_device, &rep));
    replicas.push_back(std::move(rep));
  }
  return {placement, replicas};
}

}  // namespace xl
