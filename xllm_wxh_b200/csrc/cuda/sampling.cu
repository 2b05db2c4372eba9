// Fused sampling over a [rows, vocab] logits matrix: penalties, temperature, top-k, top-p, sampling or argmax,
// log-probabilities and top-N alternatives, one CTA per row.
//
// The reference does this with libtorch ops on CUDA (sort-based top-k/top-p, softmax, multinomial:
// xllm/core/framework/sampling/sampler.cpp:28-132, logits_utils.cpp:61-160) and has fused device samplers only on
// MLU (param.h:796-853).  Here nothing is sorted: the top-k and the top-p cut-offs are found exactly by a
// three-level radix selection (11+11+10 bits of an order-preserving key) over count / probability-mass
// histograms in shared memory, and the token is drawn by inverse-CDF in vocabulary order.
//
// Rows with 0 < top_k <= 256 (the usual serving case) take a shorter way with the same result: the k-th largest of the
// 1024 thread-local maxima of the first pass is a lower bound of the k-th largest logit, so one more pass collects the few
// elements above it into shared memory, and top-k, top-p and the draw are decided among those candidates: two passes
// over the row instead of about ten.
#include "common.cuh"

namespace xl {

constexpr int kSampleThreads = 1024;

template <typename T> __device__ __forceinline__ float ldf(const T* p, size_t i);
template <> __device__ __forceinline__ float ldf<float>(const float* p, size_t i) { return p[i]; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }

__device__ __forceinline__ uint32_t fkey(float x) {   // larger float <=> larger key
  uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float uniform_from_seed(uint32_t lo, uint32_t hi) {   // splitmix64 finaliser -> (0,1)
  uint64_t z = ((uint64_t(hi) << 32) | lo) + 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z = z ^ (z >> 31);
  return (float(uint32_t(z >> 40)) + 0.5f) * (1.0f / 16777216.0f);
}

struct BlockRed {
  float f[32];
  int i[32];
};

__device__ __forceinline__ float block_sum(float v, BlockRed& s) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) s.f[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = (threadIdx.x < (blockDim.x >> 5)) ? s.f[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) {
    t = warp_sum(t);
    if (threadIdx.x == 0) s.f[0] = t;
  }
  __syncthreads();
  return s.f[0];
}

// max value and the smallest index attaining it
__device__ __forceinline__ void block_argmax(float& v, int& idx, BlockRed& s) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, v, o);
    int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) { s.f[threadIdx.x >> 5] = v; s.i[threadIdx.x >> 5] = idx; }
  __syncthreads();
  if (threadIdx.x < 32) {
    float tv = (threadIdx.x < (blockDim.x >> 5)) ? s.f[threadIdx.x] : -INFINITY;
    int ti = (threadIdx.x < (blockDim.x >> 5)) ? s.i[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, tv, o);
      int oi = __shfl_xor_sync(0xffffffffu, ti, o);
      if (ov > tv || (ov == tv && oi < ti)) { tv = ov; ti = oi; }
    }
    if (threadIdx.x == 0) { s.f[0] = tv; s.i[0] = ti; }
  }
  __syncthreads();
  v = s.f[0];
  idx = s.i[0];
}

// In-place penalties on the listed token ids of each row (frequency / presence first, then repetition).
template <typename T>
__global__ void penalty_kernel(T* __restrict__ logits, int V, size_t ld, const int* __restrict__ pen_cu,
                               const int* __restrict__ pen_ids, const int* __restrict__ pen_counts,
                               const float* __restrict__ rep, const float* __restrict__ freq, const float* __restrict__ pres) {
  const int row = blockIdx.x;
  const int a = pen_cu[row], b = pen_cu[row + 1];
  const float rp = rep[row], fp = freq[row], pp = pres[row];
  for (int i = a + threadIdx.x; i < b; i += blockDim.x) {
    const int id = pen_ids[i];
    if (id < 0 || id >= V) continue;
    // high half: how often the token was generated (frequency / presence count generated tokens only, as the
    // reference's count map does, sequence.cpp:147-154,240-242); every listed id takes the repetition penalty
    const float cnt = float((pen_counts[i] >> 16) & 0xFFFF);
    float x = ldf(logits, row * ld + id);
    x -= cnt * fp + (cnt > 0.f ? pp : 0.f);
    x = x < 0.f ? x * rp : x / rp;
    logits[row * ld + id] = T(x);
  }
}

constexpr int kCandCap = 2048;     // candidates the short way keeps in shared memory (more: the general way)
constexpr int kCandMaxK = 256;

struct SampleSmem {
  int cnt[2048];
  float mass[2048];
  uint32_t tl[kSampleThreads];     // thread-local maxima (keys)
  float cand_v[kCandCap];
  int cand_i[kCandCap];
  int cand_n;
  uint32_t cand_thr;
  BlockRed red;
  float seg_mass[32];
  uint32_t sel_key;
  int sel_bin;
  float sel_mass_above;
  int sel_cnt_above;
  int winner_warp;
  float target_in_seg;
  int token;
};

// Visit every element of a row: 16-byte loads (8 bf16 or 4 fp32 per thread and step) when the row allows it.
template <typename T, typename F>
__device__ __forceinline__ void for_each_elem(const T* __restrict__ x, int V, F&& f) {
  constexpr int W = 16 / sizeof(T);
  if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    const int nv = V / W;
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    for (int j = threadIdx.x; j < nv; j += blockDim.x) {
      const uint4 q = xv[j];
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
      if constexpr (sizeof(T) == 2) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          f(__uint_as_float(w[e] << 16), j * 8 + 2 * e);
          f(__uint_as_float(w[e] & 0xFFFF0000u), j * 8 + 2 * e + 1);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) f(__uint_as_float(w[e]), j * 4 + e);
      }
    }
    for (int i = nv * W + threadIdx.x; i < V; i += blockDim.x) f(ldf(x, i), i);
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) f(ldf(x, i), i);
  }
}

// Warp 0 finds, going down from the highest bin, the bin in which the running count reaches `k_left`:
// returns the bin (or -1 when the total stays below) and the count of the bins above it.
__device__ __forceinline__ int cross_bin_by_count(const int* cnt, int nb, int k_left, int* cnt_above) {
  const int lane = threadIdx.x & 31;
  const int chunk = nb / 32;
  const int hi = nb - lane * chunk;              // this lane's bins: [hi - chunk, hi)
  int s = 0;
  for (int b = hi - 1; b >= hi - chunk; --b) s += cnt[b];
  int inc = s;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  const uint32_t crossed = __ballot_sync(0xffffffffu, inc >= k_left);
  if (crossed == 0) return -1;
  const int first = __ffs(crossed) - 1;
  int bin = 0, above = 0;
  if (lane == first) {
    int c = inc - s;
    int b = hi - 1;
    for (; b > hi - chunk; --b) {
      if (c + cnt[b] >= k_left) break;
      c += cnt[b];
    }
    bin = b;
    above = c;
  }
  bin = __shfl_sync(0xffffffffu, bin, first);
  *cnt_above = __shfl_sync(0xffffffffu, above, first);
  return bin;
}

// k-th largest of the blockDim.x keys in sm.tl (1 <= k <= blockDim.x), by radix selection on counts.
__device__ uint32_t kth_largest_of_thread_keys(int k, SampleSmem& sm) {
  uint32_t prefix = 0;
  int k_left = k;
  const int shifts[3] = {21, 10, 0};
  const int bits[3] = {11, 11, 10};
  const uint32_t key = sm.tl[threadIdx.x];
  for (int level = 0; level < 3; ++level) {
    const int nb = 1 << bits[level];
    for (int i = threadIdx.x; i < nb; i += blockDim.x) sm.cnt[i] = 0;
    __syncthreads();
    const uint32_t hi_mask = level == 0 ? 0u : (0xFFFFFFFFu << (shifts[level - 1]));
    if ((key & hi_mask) == prefix) atomicAdd(&sm.cnt[(key >> shifts[level]) & (nb - 1)], 1);
    __syncthreads();
    if (threadIdx.x < 32) {
      int above = 0;
      const int b = cross_bin_by_count(sm.cnt, nb, k_left, &above);
      if (threadIdx.x == 0) { sm.sel_bin = b < 0 ? 0 : b; sm.sel_cnt_above = b < 0 ? 0 : above; }
    }
    __syncthreads();
    prefix |= uint32_t(sm.sel_bin) << shifts[level];
    k_left -= sm.sel_cnt_above;
    __syncthreads();
  }
  return prefix;
}

// Radix selection of a threshold key among the elements with key >= floor_key.
//   by_count: largest key T with  count(key > T) < k        (keeps the k largest, plus ties)
//   by mass : largest key T with  mass(key > T) <= P        (top-p nucleus incl. the crossing token)
// Returns T; *mass_ge receives mass(key >= T).
template <typename T>
__device__ uint32_t radix_select(const T* __restrict__ x, int V, float m, float inv_t, uint32_t floor_key, bool by_count, int k,
                                 float P, SampleSmem& sm, float* mass_ge) {
  uint32_t prefix = 0;
  int k_left = k;
  float p_left = P;
  float mass_above_total = 0.f;
  const int shifts[3] = {21, 10, 0};
  const int bits[3] = {11, 11, 10};
  for (int level = 0; level < 3; ++level) {
    const int nb = 1 << bits[level];
    for (int i = threadIdx.x; i < nb; i += blockDim.x) { sm.cnt[i] = 0; sm.mass[i] = 0.f; }
    __syncthreads();
    const uint32_t hi_mask = level == 0 ? 0u : (0xFFFFFFFFu << (shifts[level - 1]));
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = ldf(x, i);
      const uint32_t key = fkey(v);
      if (key < floor_key || (key & hi_mask) != prefix) continue;
      const int bin = (key >> shifts[level]) & (nb - 1);
      atomicAdd(&sm.cnt[bin], 1);
      atomicAdd(&sm.mass[bin], __expf((v - m) * inv_t));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int c = 0;
      float ms = 0.f;
      int b = nb - 1;
      for (; b >= 0; --b) {
        if (sm.cnt[b] == 0) continue;
        const bool cross = by_count ? (c + sm.cnt[b] >= k_left) : (ms + sm.mass[b] > p_left);
        if (cross) break;
        c += sm.cnt[b];
        ms += sm.mass[b];
      }
      if (b < 0) {            // never crossed: everything is kept; select the smallest populated bin
        c = 0; ms = 0.f;
        int last = 0;
        for (int q = nb - 1; q >= 0; --q) if (sm.cnt[q] > 0) last = q;
        for (int q = nb - 1; q > last; --q) { c += sm.cnt[q]; ms += sm.mass[q]; }
        b = last;
      }
      sm.sel_bin = b;
      sm.sel_cnt_above = c;
      sm.sel_mass_above = ms;
    }
    __syncthreads();
    prefix |= uint32_t(sm.sel_bin) << shifts[level];
    k_left -= sm.sel_cnt_above;
    p_left -= sm.sel_mass_above;
    mass_above_total += sm.sel_mass_above;
    if (level == 2) *mass_ge = mass_above_total + sm.mass[sm.sel_bin];
    __syncthreads();
  }
  return prefix < floor_key ? floor_key : prefix;
}

template <typename T>
__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const T* __restrict__ logits, int V, size_t ld, const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const int* __restrict__ seed_lo, const int* __restrict__ seed_hi,
              int* __restrict__ out_tokens, float* __restrict__ out_logprobs, int n_top, float* __restrict__ top_vals,
              int* __restrict__ top_ids, int short_way) {
  __shared__ SampleSmem sm;
  const int row = blockIdx.x;
  const T* x = logits + size_t(row) * ld;
  const float temp = temperature[row];
  const bool greedy = temp == 0.f;
  const float inv_t = greedy ? 1.f : 1.f / temp;

  // pass 1: max / argmax (the smallest index among equal maxima)
  float mv = -INFINITY;
  int mi = 0x7fffffff;
  for_each_elem(x, V, [&](float v, int i) {
    if (v > mv || (v == mv && i < mi)) { mv = v; mi = i; }
  });
  sm.tl[threadIdx.x] = mi == 0x7fffffff ? 0u : fkey(mv);
  block_argmax(mv, mi, sm.red);
  const float m = mv;
  int token = mi;
  float z_final;   // normaliser of the distribution the token is drawn from
  uint32_t thr = 0;

  bool drawn = false;
  const int k_row = greedy ? 0 : top_k[row];
  if (short_way && !greedy && k_row > 0 && k_row <= kCandMaxK && k_row < V && V >= int(blockDim.x)) {
    // ---- short way: candidates above the k-th largest thread-local maximum
    const uint32_t tau = kth_largest_of_thread_keys(k_row, sm);
    if (threadIdx.x == 0) sm.cand_n = 0;
    __syncthreads();
    for_each_elem(x, V, [&](float v, int i) {
      if (fkey(v) >= tau) {
        const int at = atomicAdd(&sm.cand_n, 1);
        if (at < kCandCap) { sm.cand_v[at] = v; sm.cand_i[at] = i; }
      }
    });
    __syncthreads();
    const int n = sm.cand_n;
    if (n <= kCandCap) {
      // top-k: T = the k-th largest key among the candidates (ties at T stay in)
      if (threadIdx.x == 0) sm.cand_thr = 0u;
      __syncthreads();
      for (int a = threadIdx.x; a < n; a += blockDim.x) {
        const uint32_t ka = fkey(sm.cand_v[a]);
        int gt = 0, eq = 0;
        for (int b = 0; b < n; ++b) {
          const uint32_t kb = fkey(sm.cand_v[b]);
          gt += kb > ka;
          eq += kb == ka;
        }
        if (gt < k_row && k_row <= gt + eq) sm.cand_thr = ka;       // every thread that gets here writes the same key
      }
      __syncthreads();
      uint32_t t_keep = sm.cand_thr;
      float zk = 0.f;
      for (int a = threadIdx.x; a < n; a += blockDim.x)
        if (fkey(sm.cand_v[a]) >= t_keep) zk += __expf((sm.cand_v[a] - m) * inv_t);
      zk = block_sum(zk, sm.red);
      const float pnuc = top_p[row];
      if (pnuc < 1.f) {
        // top-p inside the top-k set: the largest key whose mass(key' >= key) exceeds p * zk is the crossing token
        const float P = pnuc * zk;
        uint32_t best = 0u;
        for (int a = threadIdx.x; a < n; a += blockDim.x) {
          const uint32_t ka = fkey(sm.cand_v[a]);
          if (ka < t_keep) continue;
          float ge = 0.f;
          for (int b = 0; b < n; ++b) {
            const float vb = sm.cand_v[b];
            if (fkey(vb) >= ka) ge += __expf((vb - m) * inv_t);
          }
          if (ge > P && ka > best) best = ka;
        }
        // block maximum of `best` through the argmax helper (keys compared as floats of their rank order)
        __syncthreads();
        sm.cand_thr = 0u;
        __syncthreads();
        if (best) atomicMax(&sm.cand_thr, best);
        __syncthreads();
        if (sm.cand_thr > t_keep) t_keep = sm.cand_thr;
      }
      float zp = 0.f;
      for (int a = threadIdx.x; a < n; a += blockDim.x)
        if (fkey(sm.cand_v[a]) >= t_keep) zp += __expf((sm.cand_v[a] - m) * inv_t);
      zp = block_sum(zp, sm.red);
      // draw in vocabulary order over the kept candidates
      const float target = uniform_from_seed(uint32_t(seed_lo[row]), uint32_t(seed_hi[row])) * zp;
      if (threadIdx.x == 0) { sm.token = -1; sm.sel_bin = -1; }
      __syncthreads();
      for (int a = threadIdx.x; a < n; a += blockDim.x) {
        const float va = sm.cand_v[a];
        if (fkey(va) < t_keep) continue;
        const int ia = sm.cand_i[a];
        float before = 0.f;
        for (int b = 0; b < n; ++b)
          if (sm.cand_i[b] < ia && fkey(sm.cand_v[b]) >= t_keep) before += __expf((sm.cand_v[b] - m) * inv_t);
        if (before <= target && target < before + __expf((va - m) * inv_t)) atomicMax(&sm.token, ia);
        atomicMax(&sm.sel_bin, ia);            // the last kept index: where a target that fell past the end by rounding lands
      }
      __syncthreads();
      token = sm.token >= 0 ? sm.token : sm.sel_bin;
      thr = t_keep;
      z_final = zp;
      drawn = true;
    }
    __syncthreads();
  }

  if (!greedy && !drawn) {
    // pass 2: total mass
    float z = 0.f;
    for_each_elem(x, V, [&](float v, int) { z += __expf((v - m) * inv_t); });
    z = block_sum(z, sm.red);
    const int k = top_k[row];
    const float pnuc = top_p[row];
    float zk = z;
    if (k > 0 && k < V) thr = radix_select(x, V, m, inv_t, 0u, true, k, 0.f, sm, &zk);
    float zp = zk;
    if (pnuc < 1.f) thr = radix_select(x, V, m, inv_t, thr, false, 0, pnuc * zk, sm, &zp);
    // inverse CDF in vocabulary order over the kept set: warp w owns the contiguous segment [w*seg, (w+1)*seg)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seg = (V + 31) / 32;
    const int s0 = warp * seg, s1 = min(V, s0 + seg);
    float ms = 0.f;
    for (int i = s0 + lane; i < s1; i += 32) {
      const float v = ldf(x, i);
      if (fkey(v) >= thr) ms += __expf((v - m) * inv_t);
    }
    ms = warp_sum(ms);
    if (lane == 0) sm.seg_mass[warp] = ms;
    __syncthreads();
    if (threadIdx.x == 0) {
      float tot = 0.f;
      for (int w = 0; w < 32; ++w) tot += sm.seg_mass[w];
      const float u = uniform_from_seed(uint32_t(seed_lo[row]), uint32_t(seed_hi[row]));
      float target = u * tot, acc = 0.f;
      int win = -1;
      for (int w = 0; w < 32; ++w) {
        if (sm.seg_mass[w] > 0.f) {
          win = w;
          if (acc + sm.seg_mass[w] > target) break;
          acc += sm.seg_mass[w];
        }
      }
      if (win >= 0 && acc + sm.seg_mass[win] <= target) acc = fmaxf(0.f, target - sm.seg_mass[win] * 0.5f);   // rounding: stay inside
      sm.winner_warp = win;
      sm.target_in_seg = target - acc;
      sm.seg_mass[0] = tot;
      sm.token = token;
    }
    __syncthreads();
    z_final = sm.seg_mass[0];
    if (warp == sm.winner_warp) {
      float run = 0.f;
      const float target = sm.target_in_seg;
      int found = -1, last_kept = -1;
      for (int base = s0; base < s1 && found < 0; base += 32) {
        const int i = base + lane;
        float pm = 0.f;
        if (i < s1) {
          const float v = ldf(x, i);
          if (fkey(v) >= thr) pm = __expf((v - m) * inv_t);
        }
        float inc = pm;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const float t = __shfl_up_sync(0xffffffffu, inc, o);
          if (lane >= o) inc += t;
        }
        const bool hit = pm > 0.f && (run + inc > target);
        const uint32_t ballot = __ballot_sync(0xffffffffu, hit);
        const uint32_t kept = __ballot_sync(0xffffffffu, pm > 0.f);
        if (kept) last_kept = base + 31 - __clz(kept);
        if (ballot) found = base + __ffs(ballot) - 1;
        run += __shfl_sync(0xffffffffu, inc, 31);
      }
      if (found < 0) found = last_kept;      // target fell past the end by rounding
      if (lane == 0 && found >= 0) sm.token = found;
    }
    __syncthreads();
    token = sm.token;
  } else if (greedy) {
    z_final = 0.f;
    if (out_logprobs || n_top > 0) {
      float z = 0.f;
      for_each_elem(x, V, [&](float v, int) { z += __expf(v - m); });
      z_final = block_sum(z, sm.red);
    }
  }
  if (threadIdx.x == 0) {
    out_tokens[row] = token;
    if (out_logprobs) out_logprobs[row] = (ldf(x, token) - m) * inv_t - __logf(z_final);
  }
  // top-N alternatives: N rounds of "largest key below the previous one" (ties broken by index)
  if (n_top > 0) {
    float prev_v = INFINITY;
    int prev_i = -1;
    const float logz = __logf(z_final);
    for (int n = 0; n < n_top; ++n) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = ldf(x, i);
        const bool below = (v < prev_v) || (v == prev_v && i > prev_i);
        if (below && fkey(v) >= thr && (v > bv || (v == bv && i < bi))) { bv = v; bi = i; }
      }
      block_argmax(bv, bi, sm.red);
      if (threadIdx.x == 0) {
        top_vals[size_t(row) * n_top + n] = (bi == 0x7fffffff) ? -INFINITY : (bv - m) * inv_t - logz;
        top_ids[size_t(row) * n_top + n] = (bi == 0x7fffffff) ? -1 : bi;
      }
      prev_v = bv;
      prev_i = bi;
      __syncthreads();
    }
  }
}

// ---------------------------------------------------------------- vocabulary-parallel sampling: per-shard candidates
// Under tensor parallelism every rank holds a slice of the vocabulary.  The k largest logits of a row (plus ties at the
// k-th) lie among the k largest of each slice, so every rank extracts those candidates from its slice, the ranks exchange
// rows of `W` (value, global id) pairs instead of whole logit rows, and the sampler runs on the merged candidates.  Rows
// with temperature 0 contribute their arg-max.  A row whose candidates (ties included) exceed W, or the shared-memory
// list, raises `*overflow` (the caller then gathers the logits instead).
template <typename T>
__global__ void __launch_bounds__(kSampleThreads)
topk_candidates_kernel(const T* __restrict__ logits, int V, size_t ld, const float* __restrict__ temperature,
                       const int* __restrict__ top_k, int id_offset, int W, float* __restrict__ out_vals, int* __restrict__ out_ids,
                       int* __restrict__ overflow) {
  __shared__ SampleSmem sm;
  const int row = blockIdx.x;
  const T* x = logits + size_t(row) * ld;
  float* ov = out_vals + size_t(row) * W;
  int* oi = out_ids + size_t(row) * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) { ov[i] = -INFINITY; oi[i] = -1; }
  float mv = -INFINITY;
  int mi = 0x7fffffff;
  for_each_elem(x, V, [&](float v, int i) {
    if (v > mv || (v == mv && i < mi)) { mv = v; mi = i; }
  });
  sm.tl[threadIdx.x] = mi == 0x7fffffff ? 0u : fkey(mv);
  block_argmax(mv, mi, sm.red);
  int k = temperature[row] == 0.f ? 1 : top_k[row];
  if (k == 1) {                       // the arg-max (smallest index among equal maxima), as the sampler takes it
    if (threadIdx.x == 0) { ov[0] = mv; oi[0] = mi + id_offset; }
    return;
  }
  if (k <= 0 || k > kCandMaxK || k > W) {
    if (threadIdx.x == 0) atomicExch(overflow, 1);
    return;
  }
  if (k >= V) k = V;
  const uint32_t tau = V >= int(blockDim.x) ? kth_largest_of_thread_keys(min(k, int(blockDim.x)), sm) : 0u;
  if (threadIdx.x == 0) sm.cand_n = 0;
  __syncthreads();
  for_each_elem(x, V, [&](float v, int i) {
    if (fkey(v) >= tau) {
      const int at = atomicAdd(&sm.cand_n, 1);
      if (at < kCandCap) { sm.cand_v[at] = v; sm.cand_i[at] = i; }
    }
  });
  __syncthreads();
  const int n = sm.cand_n;
  if (n > kCandCap) {
    if (threadIdx.x == 0) atomicExch(overflow, 1);
    return;
  }
  if (threadIdx.x == 0) { sm.cand_thr = 0u; sm.sel_cnt_above = 0; }
  __syncthreads();
  for (int a = threadIdx.x; a < n; a += blockDim.x) {
    const uint32_t ka = fkey(sm.cand_v[a]);
    int gt = 0, eq = 0;
    for (int b = 0; b < n; ++b) {
      const uint32_t kb = fkey(sm.cand_v[b]);
      gt += kb > ka;
      eq += kb == ka;
    }
    if (gt < k && k <= gt + eq) sm.cand_thr = ka;
  }
  __syncthreads();
  const uint32_t t_keep = sm.cand_thr;
  // kept candidates go out in index order (rank among the kept by index), so that every rank's row is deterministic
  for (int a = threadIdx.x; a < n; a += blockDim.x) {
    if (fkey(sm.cand_v[a]) < t_keep) continue;
    const int ia = sm.cand_i[a];
    int pos = 0;
    for (int b = 0; b < n; ++b) pos += (fkey(sm.cand_v[b]) >= t_keep) && sm.cand_i[b] < ia;
    if (pos < W) { ov[pos] = sm.cand_v[a]; oi[pos] = ia + id_offset; }
    else atomicExch(overflow, 1);
  }
}

}  // namespace xl

using namespace xl;

// dtype: 0 = fp32 logits, 1 = bf16 logits.  `ld` = row pitch in elements.
XL_API int xl_apply_penalties(void* logits, int dtype, int rows, int V, long ld, const void* pen_cu, const void* pen_ids,
                              const void* pen_counts, const void* rep, const void* freq, const void* pres, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    penalty_kernel<float><<<rows, 256, 0, st>>>(static_cast<float*>(logits), V, size_t(ld), static_cast<const int*>(pen_cu),
                                                static_cast<const int*>(pen_ids), static_cast<const int*>(pen_counts),
                                                static_cast<const float*>(rep), static_cast<const float*>(freq),
                                                static_cast<const float*>(pres));
  else
    penalty_kernel<__nv_bfloat16><<<rows, 256, 0, st>>>(
        static_cast<__nv_bfloat16*>(logits), V, size_t(ld), static_cast<const int*>(pen_cu), static_cast<const int*>(pen_ids),
        static_cast<const int*>(pen_counts), static_cast<const float*>(rep), static_cast<const float*>(freq),
        static_cast<const float*>(pres));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// Per-shard candidates for vocabulary-parallel sampling (see topk_candidates_kernel): out_vals / out_ids [rows, W], ids are
// global (local index + id_offset); `overflow` is a device int the caller zeroes and reads back.
XL_API int xl_topk_candidates(const void* logits, int dtype, int rows, int V, long ld, const void* temperature, const void* top_k,
                              int id_offset, int W, void* out_vals, void* out_ids, void* overflow, void* stream) {
  if (rows <= 0) return 0;
  if (W < 1) return -2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    topk_candidates_kernel<float><<<rows, kSampleThreads, 0, st>>>(
        static_cast<const float*>(logits), V, size_t(ld), static_cast<const float*>(temperature), static_cast<const int*>(top_k),
        id_offset, W, static_cast<float*>(out_vals), static_cast<int*>(out_ids), static_cast<int*>(overflow));
  else
    topk_candidates_kernel<__nv_bfloat16><<<rows, kSampleThreads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(logits), V, size_t(ld), static_cast<const float*>(temperature),
        static_cast<const int*>(top_k), id_offset, W, static_cast<float*>(out_vals), static_cast<int*>(out_ids),
        static_cast<int*>(overflow));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

static int g_sample_short_way = 1;
// Comparison hook: 0 sends every row the general way (radix selection over the whole row), 1 (default) lets rows with
// 0 < top_k <= 256 decide among the candidates above a lower bound of their k-th largest logit.
XL_API void xl_sample_short_way(int on) { g_sample_short_way = on ? 1 : 0; }

XL_API int xl_sample(const void* logits, int dtype, int rows, int V, long ld, const void* temperature, const void* top_k,
                     const void* top_p, const void* seed_lo, const void* seed_hi, void* out_tokens, void* out_logprobs,
                     int n_top, void* top_vals, void* top_ids, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    sample_kernel<float><<<rows, kSampleThreads, 0, st>>>(
        static_cast<const float*>(logits), V, size_t(ld), static_cast<const float*>(temperature),
        static_cast<const int*>(top_k), static_cast<const float*>(top_p), static_cast<const int*>(seed_lo),
        static_cast<const int*>(seed_hi), static_cast<int*>(out_tokens), static_cast<float*>(out_logprobs), n_top,
        static_cast<float*>(top_vals), static_cast<int*>(top_ids), g_sample_short_way);
  else
    sample_kernel<__nv_bfloat16><<<rows, kSampleThreads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(logits), V, size_t(ld), static_cast<const float*>(temperature),
        static_cast<const int*>(top_k), static_cast<const float*>(top_p), static_cast<const int*>(seed_lo),
        static_cast<const int*>(seed_hi), static_cast<int*>(out_tokens), static_cast<float*>(out_logprobs), n_top,
        static_cast<float*>(top_vals), static_cast<int*>(top_ids), g_sample_short_way);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// ---------------------------------------------------------------- speculative decoding: accept / reject
// Validation of k deterministic draft tokens per sequence against the target model's own samples.
// `target` holds the tokens the target sampled at the k+1 validated positions ([B, k+1]); draft j (0-based) is
// accepted iff all earlier drafts were accepted and target[j] == draft[j].  With a draft that proposes one fixed
// token, "the target's sample equals the draft" happens with probability p_target(draft) and, when it does not,
// the target's sample is distributed as the renormalised residual: exactly the rejection-sampling rule
// (reference: framework/sampling/rejection_sampler.cpp:119-198) without needing the draft's probabilities.
// fixed_rate >= 0 replaces the comparison by a seeded coin flip with that acceptance probability
// (reference: RejectionSamplerRateController, XLLM_FIX_SPECULATIVE_ACCEPTANCE_RATE).
// out [B, k+1]: accepted drafts, then the target's token at the first non-accepted position, then -1.
namespace xl {
__global__ void rejection_sample_kernel(const int* __restrict__ target, const int* __restrict__ draft, int* __restrict__ out,
                                        int* __restrict__ num_accepted, int B, int k, float fixed_rate, uint32_t seed_lo,
                                        uint32_t seed_hi) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const int* t = target + size_t(b) * (k + 1);
  const int* d = draft + size_t(b) * k;
  int* o = out + size_t(b) * (k + 1);
  int a = 0;
  for (; a < k; ++a) {
    bool acc;
    if (fixed_rate >= 0.f)
      acc = uniform_from_seed(seed_lo + uint32_t(b) * 2654435761u, seed_hi + uint32_t(a) * 40503u) < fixed_rate;
    else
      acc = t[a] == d[a];
    if (!acc) break;
    o[a] = d[a];
  }
  o[a] = t[a];            // correction (a < k) or bonus token (a == k)
  for (int j = a + 1; j <= k; ++j) o[j] = -1;
  if (num_accepted) num_accepted[b] = a;
}
}  // namespace xl

XL_API int xl_rejection_sample(const void* target, const void* draft, void* out, void* num_accepted, int B, int k, float fixed_rate,
                               unsigned seed_lo, unsigned seed_hi, void* stream) {
  if (B <= 0) return 0;
  xl::rejection_sample_kernel<<<(B + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const int*>(target), static_cast<const int*>(draft), static_cast<int*>(out), static_cast<int*>(num_accepted), B, k,
      fixed_rate, seed_lo, seed_hi);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
