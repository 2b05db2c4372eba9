// Mixture-of-experts support kernels: router (softmax / sigmoid, correction bias, group-limited top-k, renorm,
// routed scaling, per-expert load histogram), expert sort (counting sort of the expanded token list + the 128-row tile
// table the grouped GEMM consumes), row gather ("expand"), and the top-k weighted combine.
//
// Reference semantics: moe_topk_softmax_kernels.cuh:324-611, moe_topk_sigmoid_kernels.cuh:165-383 (CUDA, ungrouped
// only), the MLU op `moe_active_topk` for the group-limited rule (param.h:402-442, layers/mlu/moe_gate.cpp:56-72),
// `moe_gen_idx` / `moe_expand_input` / `moe_combine_result` (param.h:444-537).
#include "common.cuh"

namespace xl {

// ---------------------------------------------------------------- router: one warp per token, E <= 512
template <typename T>
__global__ void moe_router_kernel(const T* __restrict__ logits, const float* __restrict__ bias, float* __restrict__ out_w,
                                  int* __restrict__ out_id, long long* __restrict__ load_hist, int T_tokens, int E, int top_k,
                                  int sigmoid, int renorm, int n_group, int topk_group, float route_scale) {
  constexpr int MAXV = 16;   // values per lane -> E <= 512
  const int lane = threadIdx.x & 31;
  const long t = (blockIdx.x * long(blockDim.x) + threadIdx.x) >> 5;
  if (t >= T_tokens) return;
  const int per = (E + 31) / 32;
  float score[MAXV], sel[MAXV];
  // expert e = j * 32 + lane
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int e = j * 32 + lane;
    float v = -INFINITY;
    if (j < per && e < E) v = float(logits[t * E + e]);
    score[j] = v;
    mx = fmaxf(mx, v);
  }
  if (sigmoid) {
#pragma unroll
    for (int j = 0; j < MAXV; ++j) score[j] = (score[j] == -INFINITY) ? -INFINITY : 1.f / (1.f + __expf(-score[j]));
  } else {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      score[j] = (score[j] == -INFINITY) ? 0.f : __expf(score[j] - mx);
      sum += score[j];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int e = j * 32 + lane;
      score[j] = (j < per && e < E) ? score[j] * inv : -INFINITY;
    }
  }
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int e = j * 32 + lane;
    sel[j] = (j < per && e < E) ? score[j] + (bias ? bias[e] : 0.f) : -INFINITY;
  }
  // ---- group-limited selection: keep the topk_group groups with the largest score
  if (n_group > 1) {
    const int gsize = E / n_group;
    float gscore_mine = -INFINITY;   // lane g (< n_group) ends up holding the score of group g
    for (int g = 0; g < n_group; ++g) {
      // best and second best selection score inside group g
      float b1 = -INFINITY, b2 = -INFINITY;
#pragma unroll
      for (int j = 0; j < MAXV; ++j) {
        const int e = j * 32 + lane;
        if (j < per && e < E && e / gsize == g) {
          const float v = sel[j];
          if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) { b2 = v; }
        }
      }
      // merge (b1, b2) across lanes
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float o1 = __shfl_xor_sync(0xffffffffu, b1, o), o2 = __shfl_xor_sync(0xffffffffu, b2, o);
        const float n1 = fmaxf(b1, o1);
        const float n2 = fmaxf(fminf(b1, o1), fmaxf(b2, o2));
        b1 = n1; b2 = n2;
      }
      const float gs = bias ? (b1 + (b2 == -INFINITY ? 0.f : b2)) : b1;   // noaux_tc: sum of the top-2; else group max
      if (lane == g) gscore_mine = gs;
    }
    // pick topk_group groups (iterative arg-max over lanes 0..n_group-1)
    unsigned keep_mask = 0;
    for (int it = 0; it < topk_group; ++it) {
      float v = (lane < n_group && !((keep_mask >> lane) & 1)) ? gscore_mine : -INFINITY;
      int idx = lane;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
      }
      keep_mask |= 1u << idx;
    }
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int e = j * 32 + lane;
      if (j < per && e < E && !((keep_mask >> (e / gsize)) & 1)) sel[j] = -INFINITY;
    }
  }
  // ---- iterative top-k on the selection scores; weights are the un-biased scores
  float wsum = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  for (int k = 0; k < top_k; ++k) {
    float v = -INFINITY;
    int idx = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int e = j * 32 + lane;
      if (j < per && e < E && (sel[j] > v || (sel[j] == v && e < idx))) { v = sel[j]; idx = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    // owner lane retires the expert and publishes its weight
    float w = 0.f;
    if ((idx & 31) == lane && idx < E) {
      const int j = idx >> 5;
#pragma unroll
      for (int jj = 0; jj < MAXV; ++jj)
        if (jj == j) { w = score[jj]; sel[jj] = -INFINITY; }
    }
    w = __shfl_sync(0xffffffffu, w, idx & 31);
    wsum += w;
    if (lane == k) { my_w = w; my_id = idx; }
  }
  if (lane < top_k) {
    float w = my_w;
    if (renorm) w = w / fmaxf(wsum, 1e-20f);
    out_w[t * top_k + lane] = w * route_scale;
    out_id[t * top_k + lane] = my_id;
    if (load_hist) atomicAdd(reinterpret_cast<unsigned long long*>(load_hist + my_id), 1ull);
  }
}

// ---------------------------------------------------------------- expert sort
// ids [T, k] (global expert ids).  Experts [e0, e0 + E_local) are local; others are dropped.
// Outputs: counts[E_local], offsets[E_local + 1], sorted_src[R] = t * k + slot of the row placed at sorted position r,
// dst_of[T * k] = sorted position (or -1), and the tile table for the grouped GEMM.
__global__ void moe_count_kernel(const int* __restrict__ ids, int n, int e0, int E_local, int* __restrict__ counts) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int e = ids[i] - e0;
    if (e >= 0 && e < E_local) atomicAdd(counts + e, 1);
  }
}

__global__ void moe_scan_tiles_kernel(const int* __restrict__ counts, int E_local, int* __restrict__ offsets,
                                      int* __restrict__ cursor, int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                                      int* __restrict__ tile_row_end, int* __restrict__ num_m_tiles, int max_tiles) {
  // single thread: E_local <= 512, cheap and deterministic
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int off = 0, nt = 0;
  for (int e = 0; e < E_local; ++e) {
    offsets[e] = off;
    cursor[e] = off;
    const int c = counts[e];
    for (int r = 0; r < c && nt < max_tiles; r += 128) {
      tile_expert[nt] = e;
      tile_row0[nt] = off + r;
      tile_row_end[nt] = off + c;
      ++nt;
    }
    off += c;
  }
  offsets[E_local] = off;
  *num_m_tiles = nt;
}

__global__ void moe_scatter_kernel(const int* __restrict__ ids, int n, int e0, int E_local, int* __restrict__ cursor,
                                   int* __restrict__ sorted_src, int* __restrict__ dst_of) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int e = ids[i] - e0;
    int pos = -1;
    if (e >= 0 && e < E_local) {
      pos = atomicAdd(cursor + e, 1);
      sorted_src[pos] = i;
    }
    dst_of[i] = pos;
  }
}

// x_sorted[r, :] = x[sorted_src[r] / k, :] for r < offsets[E_local]
__global__ void moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ sorted_src,
                                       const int* __restrict__ total_rows, __nv_bfloat16* __restrict__ out, int H, int k,
                                       int ldx) {
  const int R = *total_rows;
  const int nvec = H / 8;
  for (int r = blockIdx.x; r < R; r += gridDim.x) {
    const int tok = sorted_src[r] / k;
    const uint4* src = reinterpret_cast<const uint4*>(x + size_t(tok) * ldx);
    uint4* dst = reinterpret_cast<uint4*>(out + size_t(r) * H);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) dst[v] = src[v];
  }
}

// out[t, :] = sum_j w[t, j] * y[dst_of[t * k + j], :]  (+ add[t, :]);  rows with dst_of < 0 contribute nothing
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ dst_of,
                                   const float* __restrict__ w, const __nv_bfloat16* __restrict__ add,
                                   __nv_bfloat16* __restrict__ out, int T_tokens, int H, int k) {
  const int t = blockIdx.x;
  if (t >= T_tokens) return;
  const int nvec = H / 8;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < k; ++j) {
      const int r = dst_of[t * k + j];
      if (r < 0) continue;
      const float wj = w[t * k + j];
      const uint4 a = *reinterpret_cast<const uint4*>(y + size_t(r) * H + v * 8);
      const uint32_t au[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = unpack_bf16x2(au[q]);
        acc[2 * q] += wj * f.x;
        acc[2 * q + 1] += wj * f.y;
      }
    }
    if (add) {
      const uint4 a = *reinterpret_cast<const uint4*>(add + size_t(t) * H + v * 8);
      const uint32_t au[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = unpack_bf16x2(au[q]);
        acc[2 * q] += f.x;
        acc[2 * q + 1] += f.y;
      }
    }
    *reinterpret_cast<uint4*>(out + size_t(t) * H + v * 8) =
        make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
}

}  // namespace xl

using namespace xl;

// dtype: 0 fp32 logits, 1 bf16 logits
XL_API int xl_moe_router(const void* logits, int dtype, const void* bias, void* out_w, void* out_id, void* load_hist, int T,
                         int E, int top_k, int sigmoid, int renorm, int n_group, int topk_group, float route_scale,
                         void* stream) {
  if (T <= 0) return 0;
  if (E > 512 || top_k > 32 || top_k < 1 || n_group > 32 || (n_group > 1 && E % n_group)) return -2;
  const int blocks = (T + 7) / 8;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    moe_router_kernel<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(logits), static_cast<const float*>(bias),
                                                     static_cast<float*>(out_w), static_cast<int*>(out_id),
                                                     static_cast<long long*>(load_hist), T, E, top_k, sigmoid, renorm, n_group,
                                                     topk_group, route_scale);
  else
    moe_router_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(logits), static_cast<const float*>(bias), static_cast<float*>(out_w),
        static_cast<int*>(out_id), static_cast<long long*>(load_hist), T, E, top_k, sigmoid, renorm, n_group, topk_group,
        route_scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// work: int32 scratch of at least 3 * E_local + 3 * max_tiles + 8 words, laid out as
//   counts[E_local] | offsets[E_local + 1] | cursor[E_local] | num_m_tiles[1] | tile_expert | tile_row0 | tile_row_end
XL_API int xl_moe_sort(const void* ids, int n, int e0, int E_local, void* work, int max_tiles, void* sorted_src, void* dst_of,
                       void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int* w = static_cast<int*>(work);
  int* counts = w;
  int* offsets = counts + E_local;
  int* cursor = offsets + E_local + 1;
  int* num_m_tiles = cursor + E_local;
  int* tile_expert = num_m_tiles + 1;
  int* tile_row0 = tile_expert + max_tiles;
  int* tile_row_end = tile_row0 + max_tiles;
  cudaMemsetAsync(counts, 0, sizeof(int) * E_local, st);
  const int blocks = n > 0 ? (n + 255) / 256 : 1;
  moe_count_kernel<<<blocks > 1024 ? 1024 : blocks, 256, 0, st>>>(static_cast<const int*>(ids), n, e0, E_local, counts);
  moe_scan_tiles_kernel<<<1, 32, 0, st>>>(counts, E_local, offsets, cursor, tile_expert, tile_row0, tile_row_end, num_m_tiles,
                                          max_tiles);
  moe_scatter_kernel<<<blocks > 1024 ? 1024 : blocks, 256, 0, st>>>(static_cast<const int*>(ids), n, e0, E_local, cursor,
                                                                    static_cast<int*>(sorted_src), static_cast<int*>(dst_of));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

XL_API int xl_moe_gather_rows(const void* x, const void* sorted_src, const void* total_rows, void* out, int H, int k, int ldx,
                              int max_rows, void* stream) {
  if (max_rows <= 0) return 0;
  if (H % 8) return -2;
  int blocks = max_rows < 148 * 8 ? max_rows : 148 * 8;
  moe_gather_rows_kernel<<<blocks, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const int*>(sorted_src), static_cast<const int*>(total_rows),
      static_cast<__nv_bfloat16*>(out), H, k, ldx);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

XL_API int xl_moe_combine(const void* y, const void* dst_of, const void* w, const void* add, void* out, int T, int H, int k,
                          void* stream) {
  if (T <= 0) return 0;
  if (H % 8) return -2;
  int threads = ((H / 8 + 31) / 32) * 32;
  threads = threads > 256 ? 256 : threads;
  moe_combine_kernel<<<T, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(y), static_cast<const int*>(dst_of), static_cast<const float*>(w),
      static_cast<const __nv_bfloat16*>(add), static_cast<__nv_bfloat16*>(out), T, H, k);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
