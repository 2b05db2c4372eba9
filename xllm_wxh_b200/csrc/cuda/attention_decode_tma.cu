// Split-KV paged GQA decode attention, TMA-fed.
//
// One CTA handles one (sequence, kv head, KV split): a producer warp streams 64-token K and V tiles from the paged
// cache into a 3-stage shared-memory ring with cp.async.bulk.tensor (one box per KV block, or per 64 tokens when the
// block is larger; 128-byte swizzle), completion on mbarriers; four consumer warps each take 16 tokens of every tile,
// compute S = Q K^T and O += P V on the tensor cores from ldmatrix fragments with an online softmax in registers,
// and release the stage.  The `group * q_len` (<= 16) query rows that share the kv head form the M dimension.
// The four partial results are merged through shared memory; with several KV splits the normalised partials and
// their log-sum-exp go to a workspace that a small merge kernel (attention.cu) reduces.
//
// Compared with issuing 16-byte cp.async copies from every lane (the fallback kernel in attention.cu), the copy
// engine removes the per-chunk address arithmetic and block-table lookups from the compute warps, which is what
// bounds a decode kernel whose arithmetic intensity is a few FLOP per byte.
//
// Role: the reference's FlashInfer `batch_decode_with_kv_cache` (xllm/core/kernels/cuda/batch_decode.cpp:26-85).
#include "common.cuh"

namespace xl_dec {
using namespace xl;

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct DecParams {
  const __nv_bfloat16* q;
  __nv_bfloat16* out;
  const int* q_cu;
  const int* kv_lens;
  const int* block_tables;
  int seq_begin, seq_end;
  int max_blocks, block_size, n_q, n_kv, q_stride;
  float scale_log2;
  int window;
  int num_splits;
  float* part_o;
  float* part_lse;
  int num_blocks_total;
  int box_tokens;     // tokens per TMA box: min(block_size, 64)
  int* status;
  const int* dyn_end = nullptr;   // optional device scalar that replaces seq_end (launch sized for a capacity)
  int ws_rows = 0;                // > 0: row capacity of a fixed-size workspace; sequences that do not fit it (or have more
                                  // than 16 query rows x heads per kv head) are skipped and XL_ERR_BOUNDS is recorded
};

constexpr int kStages = 3;
constexpr int kTile = 64;

struct DecBarriers {
  uint64_t full[kStages];
  uint64_t empty[kStages];
};

template <int D>
__global__ void __launch_bounds__(160) decode_attn_tma_kernel(const __grid_constant__ CUtensorMap tmK,
                                                              const __grid_constant__ CUtensorMap tmV, DecParams p) {
  constexpr int HALVES = D / 64;                  // 128-byte column slabs per row
  constexpr int SLAB = kTile * 128;               // bytes of one slab of a 64-token tile
  constexpr int KV_BYTES = HALVES * SLAB;         // K (or V) bytes per stage
  constexpr int STAGE_BYTES = 2 * KV_BYTES;
  constexpr int CH = D / 8;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem;                                          // kStages * STAGE_BYTES, 1024-aligned
  uint8_t* sQ = smem + kStages * STAGE_BYTES;                    // 16 x D bf16, 16-byte-chunk XOR swizzle
  DecBarriers* bars = reinterpret_cast<DecBarriers*>(sQ + 16 * D * 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = p.seq_begin + blockIdx.x;
  const int kvh = blockIdx.y;
  const int split = blockIdx.z;
  const int group = p.n_q / p.n_kv;
  if (seq >= (p.dyn_end ? *p.dyn_end : p.seq_end)) return;
  const int q_start = p.q_cu[seq];
  const int q_len = p.q_cu[seq + 1] - q_start;
  const int kv_len = p.kv_lens[seq];
  if (q_len <= 0) return;
  if (p.ws_rows > 0 && (q_len * group > 16 || (p.num_splits > 1 && q_start + q_len > p.ws_rows))) {
    if (threadIdx.x == 0) atomicExch(p.status, XL_ERR_BOUNDS);
    return;
  }
  const int rows = min(16, q_len * group);
  const int* bt = p.block_tables + size_t(seq) * p.max_blocks;

  const int per_split = ((kv_len + p.num_splits - 1) / p.num_splits + kTile - 1) / kTile * kTile;
  int s_begin = split * per_split;
  const int s_end = min(kv_len, s_begin + per_split);
  if (p.window > 0) s_begin = max(s_begin, (max(0, kv_len - q_len - p.window + 1)) / kTile * kTile);
  const int n_tiles = s_end > s_begin ? (s_end - s_begin + kTile - 1) / kTile : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 4);
    }
    mbar_fence_init();
  }
  // Q rows -> smem (zero beyond `rows`); row m = qtok * group + g
  for (int i = threadIdx.x; i < 16 * CH; i += blockDim.x) {
    const int r = i / CH, c = i % CH;
    const bool ok = r < rows;
    const int qt = ok ? r / group : 0, g = ok ? r % group : 0;
    const __nv_bfloat16* src = p.q + size_t(q_start + qt) * p.q_stride + (kvh * group + g) * D + c * 8;
    cp_async_16(sQ + uint32_t(r) * (D * 2) + (uint32_t(c ^ (r & 7)) << 4), src, ok);
  }
  cp_async_commit();
  cp_async_wait_all();
  __syncthreads();

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int row_a = lane >> 2, row_b = row_a + 8;

  if (warp == 4) {
    // ------------------------------------------------------------ producer
    if (elect_one_sync()) {
      prefetch_tmap(&tmK);
      prefetch_tmap(&tmV);
      const int bt_tok = p.box_tokens;
      int t = 0;
      bool ok = true;
      for (; t < n_tiles; ++t) {
        const int s = t % kStages;
        const uint32_t ph = (t / kStages) & 1;
        if (!mbar_wait(&bars->empty[s], ph ^ 1)) {
          atomicExch(p.status, XL_ERR_WAIT_EMPTY);
          ok = false;
          break;
        }
        const int base = s_begin + t * kTile;
        const int n_tok = min(kTile, s_end - base);
        const int n_boxes = (n_tok + bt_tok - 1) / bt_tok;
        mbar_arrive_expect_tx(&bars->full[s], uint32_t(n_boxes) * bt_tok * 128 * HALVES * 2);
        uint8_t* dK = ring + s * STAGE_BYTES;
        uint8_t* dV = dK + KV_BYTES;
        for (int b = 0; b < n_boxes; ++b) {
          const int tok = base + b * bt_tok;
          int blk = bt[tok / p.block_size];
          if (blk < 0 || blk >= p.num_blocks_total) blk = 0;     // never form an address outside the cache
          const int z = blk * p.block_size + tok % p.block_size;
#pragma unroll
          for (int h = 0; h < HALVES; ++h) {
            tma_load_3d(dK + h * SLAB + b * bt_tok * 128, &tmK, &bars->full[s], h * 64, kvh, z);
            tma_load_3d(dV + h * SLAB + b * bt_tok * 128, &tmV, &bars->full[s], h * 64, kvh, z);
          }
        }
      }
      if (!ok) {   // let the copies already issued land (bounded) before the CTA retires
        const int first = t >= kStages ? t - kStages : 0;
        for (int j = first; j < t; ++j) mbar_wait(&bars->full[j % kStages], (j / kStages) & 1);
      }
    }
  } else {
    // ------------------------------------------------------------ consumers
    uint32_t qf[D / 16][4];
    {
      const int r = (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int c = ks * 2 + (lane >> 4);
        ldsm_x4(smem_u32(sQ + uint32_t(r) * (D * 2) + (uint32_t(c ^ (r & 7)) << 4)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
      }
    }
    const int lim_a = kv_len - q_len + (row_a < rows ? row_a / group : 0);
    const int lim_b = kv_len - q_len + (row_b < rows ? row_b / group : 0);
    const int rk = (lane & 7) + (lane >> 4) * 8;           // K fragment row (token) of this lane
    const int rv = (lane & 7) + ((lane >> 3) & 1) * 8;     // V fragment row (token) of this lane
    for (int t = 0; t < n_tiles; ++t) {
      const int s = t % kStages;
      const uint32_t ph = (t / kStages) & 1;
      if (!mbar_wait(&bars->full[s], ph)) {
        if (lane == 0) atomicExch(p.status, XL_ERR_WAIT_FULL);
        break;
      }
      const int base = s_begin + t * kTile + warp * 16;
      if (base < s_end) {
        const uint8_t* tK = ring + s * STAGE_BYTES + warp * 2048;
        const uint8_t* tV = tK + KV_BYTES;
        float sc[2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          uint32_t b0, b1, b2, b3;
          const int c = (ks & 3) * 2 + ((lane >> 3) & 1);
          ldsm_x4(smem_u32(tK + (ks >> 2) * SLAB + rk * 128 + ((c ^ (rk & 7)) << 4)), b0, b1, b2, b3);
          mma_bf16_16816(sc[0], qf[ks], b0, b1);
          mma_bf16_16816(sc[1], qf[ks], b2, b3);
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 2; ++i) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int tok = base + i * 8 + (lane & 3) * 2 + (e & 1);
            const int lim = (e < 2) ? lim_a : lim_b;
            bool ok = tok <= lim && tok < s_end;
            if (p.window > 0) ok = ok && tok > lim - p.window;
            const float v = ok ? sc[i][e] * p.scale_log2 : -INFINITY;
            sc[i][e] = v;
            mx[e >> 1] = fmaxf(mx[e >> 1], v);
          }
        }
        float alpha[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
          mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
          const float m_new = fmaxf(m_run[h], mx[h]);
          alpha[h] = (m_new == -INFINITY) ? 1.f : exp2f(m_run[h] - m_new);
          m_run[h] = m_new;
        }
        float rs[2] = {0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 2; ++i) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float m = m_run[e >> 1];
            const float pv = (m == -INFINITY) ? 0.f : exp2f(sc[i][e] - m);
            sc[i][e] = pv;
            rs[e >> 1] += pv;
          }
        }
        l_run[0] = l_run[0] * alpha[0] + rs[0];
        l_run[1] = l_run[1] * alpha[1] + rs[1];
        const uint32_t pa[4] = {pack_bf16x2(sc[0][0], sc[0][1]), pack_bf16x2(sc[0][2], sc[0][3]),
                                pack_bf16x2(sc[1][0], sc[1][1]), pack_bf16x2(sc[1][2], sc[1][3])};
        const bool rescale = (alpha[0] != 1.f) || (alpha[1] != 1.f);
#pragma unroll
        for (int dt = 0; dt < D / 16; ++dt) {
          if (rescale) {
            o[2 * dt][0] *= alpha[0]; o[2 * dt][1] *= alpha[0]; o[2 * dt][2] *= alpha[1]; o[2 * dt][3] *= alpha[1];
            o[2 * dt + 1][0] *= alpha[0]; o[2 * dt + 1][1] *= alpha[0]; o[2 * dt + 1][2] *= alpha[1]; o[2 * dt + 1][3] *= alpha[1];
          }
          uint32_t b0, b1, b2, b3;
          const int c = (dt & 3) * 2 + (lane >> 4);
          ldsm_x4_t(smem_u32(tV + (dt >> 2) * SLAB + rv * 128 + ((c ^ (rv & 7)) << 4)), b0, b1, b2, b3);
          mma_bf16_16816(o[2 * dt], pa, b0, b1);
          mma_bf16_16816(o[2 * dt + 1], pa, b2, b3);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->empty[s]);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
  }
  __syncthreads();   // ring no longer needed: reuse it for the merge

  float* sO = reinterpret_cast<float*>(ring);     // [4][16][D]
  float* sM = sO + 4 * 16 * D;                    // [4][16]
  float* sL = sM + 64;
  if (warp < 4) {
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      const int col = i * 8 + (lane & 3) * 2;
      *reinterpret_cast<float2*>(sO + (warp * 16 + row_a) * D + col) = make_float2(o[i][0], o[i][1]);
      *reinterpret_cast<float2*>(sO + (warp * 16 + row_b) * D + col) = make_float2(o[i][2], o[i][3]);
    }
    if ((lane & 3) == 0) {
      sM[warp * 16 + row_a] = m_run[0]; sL[warp * 16 + row_a] = l_run[0];
      sM[warp * 16 + row_b] = m_run[1]; sL[warp * 16 + row_b] = l_run[1];
    }
  }
  __syncthreads();
  if (warp < 4) {
    for (int r = warp; r < rows; r += 4) {
      const float m = fmaxf(fmaxf(sM[r], sM[16 + r]), fmaxf(sM[32 + r], sM[48 + r]));
      float w0 = (sM[r] == -INFINITY) ? 0.f : exp2f(sM[r] - m);
      float w1 = (sM[16 + r] == -INFINITY) ? 0.f : exp2f(sM[16 + r] - m);
      float w2 = (sM[32 + r] == -INFINITY) ? 0.f : exp2f(sM[32 + r] - m);
      float w3 = (sM[48 + r] == -INFINITY) ? 0.f : exp2f(sM[48 + r] - m);
      const float l = w0 * sL[r] + w1 * sL[16 + r] + w2 * sL[32 + r] + w3 * sL[48 + r];
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const int qt = r / group, g = r % group;
      const int hq = kvh * group + g;
      const size_t tok = size_t(q_start + qt);
      for (int c = lane * 2; c < D; c += 64) {
        const float a = w0 * sO[r * D + c] + w1 * sO[(16 + r) * D + c] + w2 * sO[(32 + r) * D + c] + w3 * sO[(48 + r) * D + c];
        const float b = w0 * sO[r * D + c + 1] + w1 * sO[(16 + r) * D + c + 1] + w2 * sO[(32 + r) * D + c + 1] +
                        w3 * sO[(48 + r) * D + c + 1];
        if (p.num_splits == 1) {
          *reinterpret_cast<uint32_t*>(p.out + tok * (size_t(p.n_q) * D) + hq * D + c) = pack_bf16x2(a * inv, b * inv);
        } else {
          float* po = p.part_o + ((tok * p.n_q + hq) * p.num_splits + split) * D;
          *reinterpret_cast<float2*>(po + c) = make_float2(a * inv, b * inv);
        }
      }
      if (p.num_splits > 1 && lane == 0)
        p.part_lse[(tok * p.n_q + hq) * p.num_splits + split] = (l > 0.f) ? m + log2f(l) : -INFINITY;
    }
  }
}

}  // namespace xl_dec

using namespace xl_dec;

// Launches the TMA decode kernel for sequences [seq_begin, seq_end).  Returns -3 when the shape is not covered
// (block size not a multiple of 16, head_dim other than 64/128): the caller then uses the cp.async kernel.
// The split-KV merge (when num_splits > 1) is launched by the caller.
// `dyn_end` (device int pointer, may be null) replaces seq_end at run time; the launch is then sized for
// [seq_begin, seq_end) as a capacity, which lets a captured graph replay with another number of decode sequences.
XL_API int xl_decode_attention_tma_dyn(const void* q, const void* k_cache, const void* v_cache, void* out, const void* q_cu,
                                       const void* kv_lens, const void* block_tables, int seq_begin, int seq_end,
                                       int max_blocks, int block_size, int num_blocks_total, int n_q, int n_kv, int head_dim,
                                       int q_stride, float scale, int window, int num_splits, void* part_o, void* part_lse,
                                       const void* dyn_end, void* stream) {
  if (seq_end <= seq_begin) return 0;
  if (head_dim != 128 && head_dim != 64) return -3;
  if (block_size % 16 != 0 || (block_size > 64 && block_size % 64 != 0) || (block_size < 64 && 64 % block_size != 0)) return -3;
  if (n_q % n_kv || n_q / n_kv > 16) return -3;
  if ((reinterpret_cast<uintptr_t>(k_cache) & 127) || (reinterpret_cast<uintptr_t>(v_cache) & 127)) return -3;
  const int box_tokens = block_size < 64 ? block_size : 64;
  const uint64_t slots = uint64_t(num_blocks_total) * block_size;
  const CUtensorMap* tk = xl_host::tmap_3d(k_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, slots, n_kv, head_dim, box_tokens, 1, 64,
                                           CU_TENSOR_MAP_SWIZZLE_128B);
  const CUtensorMap* tv = xl_host::tmap_3d(v_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, slots, n_kv, head_dim, box_tokens, 1, 64,
                                           CU_TENSOR_MAP_SWIZZLE_128B);
  if (!tk || !tv) return -3;
  DecParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.q_cu = static_cast<const int*>(q_cu);
  p.kv_lens = static_cast<const int*>(kv_lens);
  p.block_tables = static_cast<const int*>(block_tables);
  p.seq_begin = seq_begin; p.seq_end = seq_end;
  p.max_blocks = max_blocks; p.block_size = block_size; p.n_q = n_q; p.n_kv = n_kv; p.q_stride = q_stride;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window;
  p.num_splits = num_splits < 1 ? 1 : num_splits;
  p.part_o = static_cast<float*>(part_o);
  p.part_lse = static_cast<float*>(part_lse);
  p.num_blocks_total = num_blocks_total;
  p.box_tokens = box_tokens;
  p.status = xl_host::status_word();
  p.dyn_end = static_cast<const int*>(dyn_end);
  if (p.num_splits > 1 && (!part_o || !part_lse)) return -2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid(seq_end - seq_begin, n_kv, p.num_splits);
  if (head_dim == 128) {
    const size_t ring = size_t(kStages) * 2 * 2 * kTile * 128;
    const size_t merge = 4 * 16 * 128 * 4 + 128 * 4;
    const size_t smem = (ring > merge ? ring : merge) + 16 * 128 * 2 + sizeof(DecBarriers) + 1024;
    static bool set = false;
    if (!set) { cudaFuncSetAttribute(decode_attn_tma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)); set = true; }
    decode_attn_tma_kernel<128><<<grid, 160, smem, st>>>(*tk, *tv, p);
  } else {
    const size_t ring = size_t(kStages) * 2 * 1 * kTile * 128;
    const size_t merge = 4 * 16 * 64 * 4 + 128 * 4;
    const size_t smem = (ring > merge ? ring : merge) + 16 * 64 * 2 + sizeof(DecBarriers) + 1024;
    static bool set = false;
    if (!set) { cudaFuncSetAttribute(decode_attn_tma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)); set = true; }
    decode_attn_tma_kernel<64><<<grid, 160, smem, st>>>(*tk, *tv, p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

XL_API int xl_decode_attention_tma(const void* q, const void* k_cache, const void* v_cache, void* out, const void* q_cu,
                                   const void* kv_lens, const void* block_tables, int seq_begin, int seq_end, int max_blocks,
                                   int block_size, int num_blocks_total, int n_q, int n_kv, int head_dim, int q_stride,
                                   float scale, int window, int num_splits, void* part_o, void* part_lse, void* stream) {
  return xl_decode_attention_tma_dyn(q, k_cache, v_cache, out, q_cu, kv_lens, block_tables, seq_begin, seq_end, max_blocks,
                                     block_size, num_blocks_total, n_q, n_kv, head_dim, q_stride, scale, window, num_splits,
                                     part_o, part_lse, nullptr, stream);
}

namespace xl_dec {
// merge of split-KV partials (normalised partial outputs weighted by 2^lse): one warp per (token, head)
template <int D>
__global__ void split_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                   __nv_bfloat16* __restrict__ out, const int* __restrict__ q_cu, int seq_begin, int seq_end,
                                   int n_q, int splits, const int* dyn_end = nullptr, int ws_rows = 0, int group = 1,
                                   int* status = nullptr) {
  const int lane = threadIdx.x & 31;
  const long gw = (blockIdx.x * long(blockDim.x) + threadIdx.x) >> 5;
  if (dyn_end) seq_end = *dyn_end;
  if (seq_end <= seq_begin) return;
  const int t0 = q_cu[seq_begin], t1 = q_cu[seq_end];
  const long n = long(t1 - t0) * n_q;
  if (gw >= n) return;
  const size_t tok = size_t(t0) + size_t(gw / n_q);
  const int h = int(gw % n_q);
  if (ws_rows > 0) {
    // fixed-size workspace: a token outside it, or one of a sequence that the attention kernel skipped (more than 16
    // query rows x heads per kv head), has no partial results; leave its output alone and report
    int lo = seq_begin, hi = seq_end;                         // the sequence with q_cu[lo] <= tok < q_cu[lo + 1]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (size_t(q_cu[mid]) <= tok) lo = mid; else hi = mid;
    }
    const int q_len = q_cu[lo + 1] - q_cu[lo];
    if (q_cu[lo + 1] > ws_rows || q_len * group > 16) {
      if (lane == 0 && status) atomicExch(status, XL_ERR_BOUNDS);
      return;
    }
  }
  const float* lse = part_lse + (tok * n_q + h) * splits;
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, lse[s]);
  float acc[D / 32];
#pragma unroll
  for (int i = 0; i < D / 32; ++i) acc[i] = 0.f;
  float den = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float w = (lse[s] == -INFINITY) ? 0.f : exp2f(lse[s] - m);
    den += w;
    const float* po = part_o + ((tok * n_q + h) * splits + s) * D;
#pragma unroll
    for (int i = 0; i < D / 32; ++i) acc[i] += w * po[lane + 32 * i];
  }
  const float inv = den > 0.f ? 1.f / den : 0.f;
#pragma unroll
  for (int i = 0; i < D / 32; ++i) out[tok * (size_t(n_q) * D) + h * D + lane + 32 * i] = __float2bfloat16(acc[i] * inv);
}
}  // namespace xl_dec

// `max_rows` bounds the number of query tokens of sequences [seq_begin, seq_end) (the real count is read on the device).
XL_API int xl_decode_split_merge_dyn(const void* part_o, const void* part_lse, void* out, const void* q_cu, int seq_begin,
                                     int seq_end, int n_q, int head_dim, int splits, long max_rows, const void* dyn_end_v,
                                     void* stream) {
  if (seq_end <= seq_begin || splits <= 1) return 0;
  const int* dyn_end = static_cast<const int*>(dyn_end_v);
  const long warps = max_rows * n_q;
  const int blocks = int((warps + 3) / 4);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (head_dim == 128)
    xl_dec::split_merge_kernel<128><<<blocks, 128, 0, st>>>(static_cast<const float*>(part_o), static_cast<const float*>(part_lse),
                                                            static_cast<__nv_bfloat16*>(out), static_cast<const int*>(q_cu),
                                                            seq_begin, seq_end, n_q, splits, dyn_end);
  else if (head_dim == 64)
    xl_dec::split_merge_kernel<64><<<blocks, 128, 0, st>>>(static_cast<const float*>(part_o), static_cast<const float*>(part_lse),
                                                           static_cast<__nv_bfloat16*>(out), static_cast<const int*>(q_cu),
                                                           seq_begin, seq_end, n_q, splits, dyn_end);
  else
    return -2;
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

XL_API int xl_decode_split_merge(const void* part_o, const void* part_lse, void* out, const void* q_cu, int seq_begin,
                                 int seq_end, int n_q, int head_dim, int splits, long max_rows, void* stream) {
  return xl_decode_split_merge_dyn(part_o, part_lse, out, q_cu, seq_begin, seq_end, n_q, head_dim, splits, max_rows, nullptr, stream);
}

// ============================================================================ allocation-free entry point
// Declared in xllm_kernels.h.  Same kernels as above; the split-KV workspace and the status word live in
// file-scope device arrays instead of caller- or library-allocated memory.
namespace xl_dec {
constexpr size_t kNoAllocScratchBytes = size_t(16) << 20;            // 16 MiB, held by every GPU that loads the library
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];
static __device__ __align__(256) int g_noalloc_status[64];
static void* g_noalloc_scratch_addr[64] = {nullptr};                 // device addresses of the arrays, per device
static void* g_noalloc_status_addr[64] = {nullptr};

static void set_err(char* err, int err_len, const char* msg) {
  if (!err || err_len <= 0) return;
  int i = 0;
  for (; msg[i] && i < err_len - 1; ++i) err[i] = msg[i];
  err[i] = 0;
}
}  // namespace xl_dec

XL_API int xl_decode_attention_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out, const void* q_cu,
                                       const void* kv_lens, const void* block_tables, int n_seqs, int max_rows, int max_blocks,
                                       int block_size, int num_blocks_total, int n_q, int n_kv, int head_dim, int q_stride,
                                       float scale, int num_splits, void* stream, char* err, int err_len) {
  using namespace xl_dec;
  if (n_seqs <= 0) return 0;
  if (head_dim != 128 && head_dim != 64) { set_err(err, err_len, "head_dim must be 64 or 128"); return -3; }
  if (block_size % 16 != 0 || (block_size > 64 && block_size % 64 != 0) || (block_size < 64 && 64 % block_size != 0)) {
    set_err(err, err_len, "block_size must be 16, 32, 64 or a multiple of 64");
    return -3;
  }
  if (n_kv <= 0 || n_q % n_kv || n_q / n_kv > 16) { set_err(err, err_len, "n_q must be a multiple of n_kv, group <= 16"); return -3; }
  if (num_splits < 1) num_splits = 1;
  if (max_rows < n_seqs) max_rows = n_seqs;
  const size_t o_bytes = size_t(max_rows) * n_q * num_splits * head_dim * sizeof(float);
  const size_t lse_bytes = size_t(max_rows) * n_q * num_splits * sizeof(float);
  if (num_splits > 1 && o_bytes + lse_bytes > kNoAllocScratchBytes) {
    set_err(err, err_len, "split-KV workspace (max_rows * n_q * num_splits * (head_dim + 1) * 4 bytes) exceeds the 16 MiB built-in scratch: "
                          "use fewer splits or fewer rows per call");
    return -5;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { set_err(err, err_len, "no current CUDA device"); return -1; }
  if (!g_noalloc_scratch_addr[dev]) {
    // once per device, with that device current: the arrays' names are host-side handles, not device addresses
    void* a = nullptr;
    void* b = nullptr;
    if (cudaGetSymbolAddress(&a, g_noalloc_scratch) != cudaSuccess || cudaGetSymbolAddress(&b, g_noalloc_status) != cudaSuccess ||
        !a || !b) {
      set_err(err, err_len, "cudaGetSymbolAddress failed for the built-in scratch");
      return -1;
    }
    g_noalloc_scratch_addr[dev] = a;
    g_noalloc_status_addr[dev] = b;
  }
  const int box_tokens = block_size < 64 ? block_size : 64;
  CUtensorMap tk, tv;                                              // encoded on the stack: nothing is cached or allocated
  {
    const uint64_t slots = uint64_t(num_blocks_total) * block_size;
    uint64_t dims[3] = {uint64_t(head_dim), uint64_t(n_kv), slots};
    uint64_t strides[2] = {uint64_t(head_dim) * 2, uint64_t(head_dim) * n_kv * 2};
    uint32_t box[3] = {64, 1, uint32_t(box_tokens)};
    if (xl_host::encode_tiled(&tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, k_cache, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B) != CUDA_SUCCESS ||
        xl_host::encode_tiled(&tv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, v_cache, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B) != CUDA_SUCCESS) {
      set_err(err, err_len, "tensor-map encoding failed (cache base must be 16-byte aligned)");
      return -4;
    }
  }
  DecParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.q_cu = static_cast<const int*>(q_cu);
  p.kv_lens = static_cast<const int*>(kv_lens);
  p.block_tables = static_cast<const int*>(block_tables);
  p.seq_begin = 0; p.seq_end = n_seqs;
  p.max_blocks = max_blocks; p.block_size = block_size; p.n_q = n_q; p.n_kv = n_kv; p.q_stride = q_stride;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = -1;
  p.num_splits = num_splits;
  p.part_o = reinterpret_cast<float*>(g_noalloc_scratch_addr[dev]);
  p.part_lse = reinterpret_cast<float*>(static_cast<unsigned char*>(g_noalloc_scratch_addr[dev]) + o_bytes);
  p.num_blocks_total = num_blocks_total;
  p.box_tokens = box_tokens;
  p.status = static_cast<int*>(g_noalloc_status_addr[dev]);
  // rows the built-in workspace has room for with this head count and split count (checked again on the device, where
  // the real q_cu is known)
  p.ws_rows = num_splits > 1 ? int(kNoAllocScratchBytes / (size_t(n_q) * num_splits * (head_dim + 1) * sizeof(float))) : 0x7fffffff;
  if (p.ws_rows > max_rows) p.ws_rows = max_rows;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid(n_seqs, n_kv, num_splits);
  if (head_dim == 128) {
    const size_t ring = size_t(kStages) * 2 * 2 * kTile * 128;
    const size_t smem = ring + 16 * 128 * 2 + sizeof(DecBarriers) + 1024;
    cudaFuncSetAttribute(decode_attn_tma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    decode_attn_tma_kernel<128><<<grid, 160, smem, st>>>(tk, tv, p);
    if (num_splits > 1)
      split_merge_kernel<128><<<int((long(max_rows) * n_q + 3) / 4), 128, 0, st>>>(p.part_o, p.part_lse, p.out, p.q_cu, 0, n_seqs, n_q,
                                                                                  num_splits, nullptr, p.ws_rows, n_q / n_kv, p.status);
  } else {
    const size_t ring = size_t(kStages) * 2 * 1 * kTile * 128;
    const size_t smem = ring + 16 * 64 * 2 + sizeof(DecBarriers) + 1024;
    cudaFuncSetAttribute(decode_attn_tma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    decode_attn_tma_kernel<64><<<grid, 160, smem, st>>>(tk, tv, p);
    if (num_splits > 1)
      split_merge_kernel<64><<<int((long(max_rows) * n_q + 3) / 4), 128, 0, st>>>(p.part_o, p.part_lse, p.out, p.q_cu, 0, n_seqs, n_q,
                                                                                 num_splits, nullptr, p.ws_rows, n_q / n_kv, p.status);
  }
  if (cudaGetLastError() != cudaSuccess) { set_err(err, err_len, "kernel launch failed"); return -1; }
  return 0;
}

// Status of the allocation-free entry point on the current device: 0, or the code that one of its kernels recorded since
// the last call of this function (XL_ERR_WAIT_* = a bounded wait on the TMA ring expired, XL_ERR_BOUNDS = a sequence did
// not fit the built-in workspace or had more than 16 query rows x heads per kv head and was skipped).  Waits for the
// work queued on `stream`, reads the word with one copy and clears it; allocates nothing.  Returns -1 when the entry
// point has not run on this device yet or a CUDA call fails.
XL_API int xl_decode_attention_noalloc_status(void* stream) {
  using namespace xl_dec;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || !g_noalloc_status_addr[dev]) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int v = 0;
  if (cudaMemcpyAsync(&v, g_noalloc_status_addr[dev], sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess) return -1;
  if (cudaStreamSynchronize(st) != cudaSuccess) return -1;
  if (v != 0 && cudaMemsetAsync(g_noalloc_status_addr[dev], 0, sizeof(int), st) != cudaSuccess) return -1;
  return v;
}
