// Multi-head latent attention (DeepSeek-V2/V3) in absorbed form over a paged latent cache.
//
//   cache row (per token)  : [ RMSNorm(latent) (C = 512) | RoPE(k_pe) (R = 64) ]            576 bf16
//   query row (per head)   : [ q_nope . W_kc (C)         | RoPE(q_pe) (R)       ]
//   score = q . cache_row * scale ;  out_latent = softmax(score) . cache_row[:C]            (V = the latent itself)
//
// Reference semantics: layers/mlu/deepseek_v2_attention.cpp:184-240,406-496 and the fused MLU ops `fused_mla_q` /
// `fused_mla_kv` (kernels/param.h:933-1083); the reference has no CUDA implementation of MLA.
//
// Kernels:
//   mla_prepare_kernel : latent RMSNorm + interleaved RoPE(k_pe) + cache write; q_nope copied / q_pe rotated into
//                        head-major buffers [Hh, T, .] (the layout the per-head absorb GEMMs and the attention use).
//   mla_attn_kernel    : one CTA = 16 query rows (16 heads of one token for short q_len, 16 tokens of one head for
//                        prefill chunks) x the whole latent width; 64-token cache tiles double-buffered with cp.async;
//                        S = Q K^T by 8 warps on disjoint token columns, softmax through shared memory, O += P V by 8
//                        warps on disjoint latent columns; tensor cores via ldmatrix + mma.sync m16n8k16.
#include "common.cuh"

namespace xl_mla {
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
__device__ __forceinline__ void ldsm_x2(uint32_t addr, uint32_t& r0, uint32_t& r1) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
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
// 16-byte chunk `chunk` of a row: XOR the low three chunk bits with the row (bank-conflict-free ldmatrix)
__device__ __forceinline__ uint32_t swz_chunk(int row, int chunk) { return uint32_t((chunk & ~7) | ((chunk ^ row) & 7)); }

// ---------------------------------------------------------------- prepare
// grid.x = T, one warp per unit: unit 0 = the token's latent/k_pe, unit 1 + h = query head h.
template <int C, int R, int NOPE>
__global__ void mla_prepare_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kv_a,
                                   const int* __restrict__ positions, const int* __restrict__ slots,
                                   const float* __restrict__ cos_sin, const __nv_bfloat16* __restrict__ kv_norm_w,
                                   __nv_bfloat16* __restrict__ cache, __nv_bfloat16* __restrict__ q_nope_hm,
                                   __nv_bfloat16* __restrict__ q_pe_hm, int T, int Hh, float eps, long cache_slots) {
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const float* cs = cos_sin + size_t(positions[t]) * R;    // cos[0:R/2] | sin[R/2:R]
  for (int unit = warp; unit <= Hh; unit += nwarps) {
    if (unit == 0) {
      const int slot = slots[t];
      const __nv_bfloat16* src = kv_a + size_t(t) * (C + R);
      float v[C / 32];
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < C / 32; ++j) {
        v[j] = __bfloat162float(src[lane + 32 * j]);
        ss += v[j] * v[j];
      }
      ss = warp_sum(ss);
      const float rstd = rsqrtf(ss / float(C) + eps);
      if (slot >= 0 && slot < cache_slots) {
        __nv_bfloat16* dst = cache + size_t(slot) * (C + R);
#pragma unroll
        for (int j = 0; j < C / 32; ++j) {
          const float n = __bfloat162float(__float2bfloat16(v[j] * rstd));
          dst[lane + 32 * j] = __float2bfloat16(n * __bfloat162float(kv_norm_w[lane + 32 * j]));
        }
        for (int i = lane; i < R / 2; i += 32) {
          const float a = __bfloat162float(src[C + 2 * i]), b = __bfloat162float(src[C + 2 * i + 1]);
          const float c = cs[i], s = cs[R / 2 + i];
          dst[C + 2 * i] = __float2bfloat16(a * c - b * s);
          dst[C + 2 * i + 1] = __float2bfloat16(b * c + a * s);
        }
      }
    } else {
      const int h = unit - 1;
      const __nv_bfloat16* src = q + (size_t(t) * Hh + h) * (NOPE + R);
      __nv_bfloat16* dn = q_nope_hm + (size_t(h) * T + t) * NOPE;
      for (int i = lane; i < NOPE / 2; i += 32)
        reinterpret_cast<uint32_t*>(dn)[i] = reinterpret_cast<const uint32_t*>(src)[i];
      __nv_bfloat16* dp = q_pe_hm + (size_t(h) * T + t) * R;
      for (int i = lane; i < R / 2; i += 32) {
        const float a = __bfloat162float(src[NOPE + 2 * i]), b = __bfloat162float(src[NOPE + 2 * i + 1]);
        const float c = cs[i], s = cs[R / 2 + i];
        dp[2 * i] = __float2bfloat16(a * c - b * s);
        dp[2 * i + 1] = __float2bfloat16(b * c + a * s);
      }
    }
  }
}

// ---------------------------------------------------------------- attention
struct MlaParams {
  const __nv_bfloat16* q_lat;   // [Hh, T, C] head-major
  const __nv_bfloat16* q_pe;    // [Hh, T, R]
  const __nv_bfloat16* cache;   // [slots, C + R]
  __nv_bfloat16* out;           // [Hh, T, C] head-major
  const int* q_cu;
  const int* kv_lens;
  const int* block_tables;
  int seq_begin, seq_end, max_blocks, block_size, Hh, T;
  float scale_log2;
  long cache_slots;
};

template <int C, int R>
__global__ void __launch_bounds__(256) mla_attn_kernel(MlaParams p) {
  constexpr int DK = C + R;                 // 576
  constexpr int ROWB = DK * 2;              // bytes per row
  constexpr int CH = DK / 8;                // 72 chunks
  constexpr int BKV = 64;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* sQ = smem;                                   // 16 rows
  uint8_t* sKV = sQ + 16 * ROWB;                        // 2 stages x 64 rows
  float* sS = reinterpret_cast<float*>(sKV + 2 * BKV * ROWB);   // [16][64]
  uint8_t* sP = reinterpret_cast<uint8_t*>(sS + 16 * BKV);      // [16][64] bf16, rows of 128 bytes
  float* sM = reinterpret_cast<float*>(sP + 16 * 128);
  float* sL = sM + 16;
  float* sAlpha = sL + 16;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ---- which (sequence, tile) is this CTA?
  const int head_tiles = p.Hh / 16;
  int tile = blockIdx.x, seq = -1, q_start = 0, q_len = 0;
  for (int s = p.seq_begin; s < p.seq_end; ++s) {
    const int a = p.q_cu[s], b = p.q_cu[s + 1];
    const int n = b - a;
    const int nt = n <= 0 ? 0 : (n <= 4 ? n * head_tiles : ((n + 15) / 16) * p.Hh);
    if (tile < nt) { seq = s; q_start = a; q_len = n; break; }
    tile -= nt;
  }
  if (seq < 0) return;
  const int kv_len = p.kv_lens[seq];
  const bool by_head = q_len <= 4;          // rows = 16 heads of one token; else rows = 16 tokens of one head
  const int qt0 = by_head ? tile / head_tiles : (tile / p.Hh) * 16;
  const int h0 = by_head ? (tile % head_tiles) * 16 : tile % p.Hh;
  auto row_tok = [&](int r) { return by_head ? qt0 : qt0 + r; };
  auto row_head = [&](int r) { return by_head ? h0 + r : h0; };
  auto row_valid = [&](int r) { return by_head ? true : (qt0 + r < q_len); };
  const int last_tok = by_head ? qt0 : min(q_len - 1, qt0 + 15);
  const int kv_end = min(kv_len, kv_len - q_len + last_tok + 1);
  const int n_tiles = (kv_end + BKV - 1) / BKV;
  const int* bt = p.block_tables + size_t(seq) * p.max_blocks;

  // ---- Q rows -> smem
  for (int i = threadIdx.x; i < 16 * CH; i += blockDim.x) {
    const int r = i / CH, c = i % CH;
    const bool ok = row_valid(r);
    const size_t qrow = size_t(row_head(ok ? r : 0)) * p.T + q_start + row_tok(ok ? r : 0);
    const __nv_bfloat16* src = (c < C / 8) ? p.q_lat + qrow * C + c * 8 : p.q_pe + qrow * R + (c - C / 8) * 8;
    cp_async_16(sQ + r * ROWB + (swz_chunk(r, c) << 4), src, ok);
  }
  auto load_kv = [&](int t, int stage) {
    uint8_t* dst = sKV + stage * BKV * ROWB;
    const int base = t * BKV;
    for (int i = threadIdx.x; i < BKV * CH; i += blockDim.x) {
      const int r = i / CH, c = i % CH;
      const int tok = base + r;
      const bool ok = tok < kv_end;
      long slot = 0;
      if (ok) slot = long(bt[tok / p.block_size]) * p.block_size + tok % p.block_size;
      if (slot < 0 || slot >= p.cache_slots) slot = 0;
      cp_async_16(dst + r * ROWB + (swz_chunk(r, c) << 4), p.cache + size_t(slot) * DK + c * 8, ok);
    }
    cp_async_commit();
  };
  if (n_tiles > 0) load_kv(0, 0); else cp_async_commit();
  if (threadIdx.x < 16) { sM[threadIdx.x] = -INFINITY; sL[threadIdx.x] = 0.f; }

  float o[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const int row_a = lane >> 2, row_b = row_a + 8;
  const int lim_a = kv_len - q_len + row_tok(row_a), lim_b = kv_len - q_len + row_tok(row_b);

  for (int t = 0; t < n_tiles; ++t) {
    const int stage = t & 1;
    cp_async_wait_all();
    __syncthreads();                                     // tile t (and Q) landed; everyone is done with tile t-1
    if (t + 1 < n_tiles) load_kv(t + 1, stage ^ 1);
    const uint8_t* tKV = sKV + stage * BKV * ROWB;
    const int base = t * BKV;
    // ---- S: warp w -> tokens [8w, 8w+8)
    {
      float sc[4] = {0.f, 0.f, 0.f, 0.f};
      const int ra = (lane & 7) + ((lane >> 3) & 1) * 8;
      const int rk = warp * 8 + (lane & 7);
#pragma unroll 4
      for (int ks = 0; ks < DK / 16; ++ks) {
        uint32_t a[4], b0, b1;
        ldsm_x4(smem_u32(sQ + ra * ROWB + (swz_chunk(ra, 2 * ks + (lane >> 4)) << 4)), a[0], a[1], a[2], a[3]);
        ldsm_x2(smem_u32(tKV + rk * ROWB + (swz_chunk(rk, 2 * ks + ((lane >> 3) & 1)) << 4)), b0, b1);
        mma_bf16_16816(sc, a, b0, b1);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = warp * 8 + (lane & 3) * 2 + (e & 1);
        const int tok = base + col;
        const int lim = (e < 2) ? lim_a : lim_b;
        const bool ok = tok <= lim && tok < kv_end;
        sS[((e < 2) ? row_a : row_b) * BKV + col] = ok ? sc[e] * p.scale_log2 : -INFINITY;
      }
    }
    __syncthreads();
    // ---- softmax: 16 threads per row, 4 tokens each
    {
      const int r = threadIdx.x >> 4, j = threadIdx.x & 15;
      float v[4];
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 4; ++i) { v[i] = sS[r * BKV + 4 * j + i]; mx = fmaxf(mx, v[i]); }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      const float m_old = sM[r];
      const float m_new = fmaxf(m_old, mx);
      float sum = 0.f;
      float pv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        pv[i] = (m_new == -INFINITY) ? 0.f : exp2f(v[i] - m_new);
        sum += pv[i];
      }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
      // P row r, tokens 4j..4j+3 -> 8 bytes inside chunk j/2
      uint2 packed = make_uint2(pack_bf16x2(pv[0], pv[1]), pack_bf16x2(pv[2], pv[3]));
      *reinterpret_cast<uint2*>(sP + r * 128 + (((j >> 1) ^ (r & 7)) << 4) + (j & 1) * 8) = packed;
      __syncwarp();
      if (j == 0) {
        const float alpha = (m_new == -INFINITY) ? 1.f : exp2f(m_old - m_new);
        sAlpha[r] = alpha;
        sM[r] = m_new;
        sL[r] = sL[r] * alpha + sum;
      }
    }
    __syncthreads();
    // ---- O += P V: warp w -> latent columns [64w, 64w+64)
    {
      const float al_a = sAlpha[row_a], al_b = sAlpha[row_b];
#pragma unroll
      for (int i = 0; i < 8; ++i) { o[i][0] *= al_a; o[i][1] *= al_a; o[i][2] *= al_b; o[i][3] *= al_b; }
      const int ra = (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int kk = 0; kk < BKV / 16; ++kk) {
        uint32_t a[4];
        ldsm_x4(smem_u32(sP + ra * 128 + ((((2 * kk + (lane >> 4)) ^ ra) & 7) << 4)), a[0], a[1], a[2], a[3]);
        const int rv = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
        for (int jn = 0; jn < 4; ++jn) {
          uint32_t b0, b1, b2, b3;
          const int ch = warp * 8 + 2 * jn + (lane >> 4);
          ldsm_x4_t(smem_u32(tKV + rv * ROWB + (swz_chunk(rv, ch) << 4)), b0, b1, b2, b3);
          mma_bf16_16816(o[2 * jn], a, b0, b1);
          mma_bf16_16816(o[2 * jn + 1], a, b2, b3);
        }
      }
    }
  }
  __syncthreads();
  // ---- normalise and store (head-major output)
  const float inv_a = sL[row_a] > 0.f ? 1.f / sL[row_a] : 0.f;
  const float inv_b = sL[row_b] > 0.f ? 1.f / sL[row_b] : 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int col = warp * 64 + i * 8 + (lane & 3) * 2;
    if (row_valid(row_a)) {
      const size_t orow = size_t(row_head(row_a)) * p.T + q_start + row_tok(row_a);
      *reinterpret_cast<uint32_t*>(p.out + orow * C + col) = pack_bf16x2(o[i][0] * inv_a, o[i][1] * inv_a);
    }
    if (row_valid(row_b)) {
      const size_t orow = size_t(row_head(row_b)) * p.T + q_start + row_tok(row_b);
      *reinterpret_cast<uint32_t*>(p.out + orow * C + col) = pack_bf16x2(o[i][2] * inv_b, o[i][3] * inv_b);
    }
  }
}

// ---------------------------------------------------------------- lightning indexer scores (DeepSeek-V3.2)
// score[t, s] = sum_h w[t, h] * relu(q[t, h, :] . key[s, :]) for the keys s <= positions[t] of token t's sequence, read
// through its block table; -inf elsewhere.  One CTA = one token x 64 keys: the token's NH x 128 queries and the 64 x 128
// keys in shared memory, 8 warps on 8 keys each over NH / 16 row tiles (ldmatrix + mma.sync m16n8k16), then the
// weighted ReLU summed over the heads with shuffles.  The reference computes this inside its MLU select kernel
// (masked_indexer_select_paged_kv, layers/mlu/indexer.cpp:536-566); the top-k itself stays with the caller.
struct IndexScoreParams {
  const __nv_bfloat16* q;       // [T, NH, 128]
  const float* w;               // [T, NH], softmax scale folded in
  const __nv_bfloat16* keys;    // [cache_slots, 128]
  const int* block_tables;      // [B, max_blocks]
  const int* token_seq;         // [T] (< 0: a padded row, read as sequence 0)
  const int* positions;         // [T]
  float* scores;                // [T, S]
  int T, S, B, max_blocks, block_size;
  long cache_slots;
};

template <int MT>
__global__ void __launch_bounds__(256) index_score_kernel(IndexScoreParams p) {
  constexpr int NH = MT * 16, ROWB = 256, BK = 64;
  __shared__ __align__(128) uint8_t sQ[NH * ROWB];
  __shared__ __align__(128) uint8_t sK[BK * ROWB];
  __shared__ float sW[NH];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.y, base = blockIdx.x * BK;
  const int pos = p.positions[t];
  float* out = p.scores + size_t(t) * p.S;
  if (base > pos) {                                      // every key of the tile lies after the query
    if (threadIdx.x < BK && base + threadIdx.x < p.S) out[base + threadIdx.x] = -INFINITY;
    return;
  }
  const int seq = min(max(p.token_seq[t], 0), p.B - 1);
  const int* bt = p.block_tables + size_t(seq) * p.max_blocks;
  for (int i = threadIdx.x; i < NH * 16; i += blockDim.x) {
    const int r = i >> 4, c = i & 15;
    cp_async_16(sQ + r * ROWB + (swz_chunk(r, c) << 4), p.q + (size_t(t) * NH + r) * 128 + c * 8, true);
  }
  for (int i = threadIdx.x; i < BK * 16; i += blockDim.x) {
    const int r = i >> 4, c = i & 15;
    const int tok = base + r;
    const int blk = tok / p.block_size;
    const bool ok = tok < p.S && tok <= pos && blk < p.max_blocks;
    long slot = 0;
    if (ok) slot = long(bt[blk]) * p.block_size + tok % p.block_size;
    if (slot < 0 || slot >= p.cache_slots) slot = 0;
    cp_async_16(sK + r * ROWB + (swz_chunk(r, c) << 4), p.keys + size_t(slot) * 128 + c * 8, ok);
  }
  if (threadIdx.x < NH) sW[threadIdx.x] = p.w[size_t(t) * NH + threadIdx.x];
  cp_async_commit();
  cp_async_wait_all();
  __syncthreads();
  float acc[MT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
  const int rk = warp * 8 + (lane & 7);
  const int ra0 = (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    uint32_t b0, b1;
    ldsm_x2(smem_u32(sK + rk * ROWB + (swz_chunk(rk, 2 * ks + ((lane >> 3) & 1)) << 4)), b0, b1);
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      uint32_t a[4];
      const int ra = m * 16 + ra0;
      ldsm_x4(smem_u32(sQ + ra * ROWB + (swz_chunk(ra, 2 * ks + (lane >> 4)) << 4)), a[0], a[1], a[2], a[3]);
      mma_bf16_16816(acc[m], a, b0, b1);
    }
  }
  // accumulator element e: head row (lane >> 2) + 8 * (e >> 1) of tile m, key column (lane & 3) * 2 + (e & 1)
  float part[2] = {0.f, 0.f};
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    const float wa = sW[m * 16 + (lane >> 2)], wb = sW[m * 16 + (lane >> 2) + 8];
    part[0] += fmaxf(acc[m][0], 0.f) * wa + fmaxf(acc[m][2], 0.f) * wb;
    part[1] += fmaxf(acc[m][1], 0.f) * wa + fmaxf(acc[m][3], 0.f) * wb;
  }
#pragma unroll
  for (int off = 4; off < 32; off <<= 1) {
    part[0] += __shfl_xor_sync(0xffffffffu, part[0], off);
    part[1] += __shfl_xor_sync(0xffffffffu, part[1], off);
  }
  if (lane < 4) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int tok = base + warp * 8 + lane * 2 + e;
      if (tok < p.S) out[tok] = tok <= pos ? part[e] : -INFINITY;
    }
  }
}

}  // namespace xl_mla

using namespace xl_mla;

// Scores of the lightning indexer for T query tokens over the first S key positions of their sequences.  Returns -3 for a
// head count other than 16, 32 or 64 or a key width other than 128 (the caller then computes them with tensor operations).
XL_API int xl_index_scores(const void* q, const void* w, const void* keys, const void* block_tables, const void* token_seq,
                           const void* positions, void* scores, int T, int S, int B, int max_blocks, int block_size,
                           long cache_slots, int n_heads, int head_dim, void* stream) {
  if (T <= 0 || S <= 0) return 0;
  if (head_dim != 128 || B <= 0 || T > 65535) return -3;
  IndexScoreParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.w = static_cast<const float*>(w);
  p.keys = static_cast<const __nv_bfloat16*>(keys);
  p.block_tables = static_cast<const int*>(block_tables);
  p.token_seq = static_cast<const int*>(token_seq);
  p.positions = static_cast<const int*>(positions);
  p.scores = static_cast<float*>(scores);
  p.T = T; p.S = S; p.B = B; p.max_blocks = max_blocks; p.block_size = block_size; p.cache_slots = cache_slots;
  const dim3 grid((S + 63) / 64, T);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n_heads == 64) index_score_kernel<4><<<grid, 256, 0, st>>>(p);
  else if (n_heads == 32) index_score_kernel<2><<<grid, 256, 0, st>>>(p);
  else if (n_heads == 16) index_score_kernel<1><<<grid, 256, 0, st>>>(p);
  else return -3;
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

XL_API int xl_mla_prepare(const void* q, const void* kv_a, const void* positions, const void* slots, const void* cos_sin,
                          const void* kv_norm_w, void* cache, void* q_nope_hm, void* q_pe_hm, int T, int Hh, int nope, int rope,
                          int kv_lora, float eps, long cache_slots, void* stream) {
  if (T <= 0) return 0;
  if (!(kv_lora == 512 && rope == 64 && nope == 128)) return -3;
  mla_prepare_kernel<512, 64, 128><<<T, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(kv_a), static_cast<const int*>(positions),
      static_cast<const int*>(slots), static_cast<const float*>(cos_sin), static_cast<const __nv_bfloat16*>(kv_norm_w),
      static_cast<__nv_bfloat16*>(cache), static_cast<__nv_bfloat16*>(q_nope_hm), static_cast<__nv_bfloat16*>(q_pe_hm), T, Hh, eps,
      cache_slots);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// `max_tiles` >= sum over sequences of (q_len <= 4 ? q_len * Hh/16 : ceil(q_len/16) * Hh).
XL_API int xl_mla_attention(const void* q_lat_hm, const void* q_pe_hm, const void* cache, void* out_hm, const void* q_cu,
                            const void* kv_lens, const void* block_tables, int seq_begin, int seq_end, int max_blocks,
                            int block_size, long cache_slots, int Hh, int T, int kv_lora, int rope, float scale, int max_tiles,
                            void* stream) {
  if (seq_end <= seq_begin || max_tiles <= 0) return 0;
  if (!(kv_lora == 512 && rope == 64) || Hh % 16) return -3;
  MlaParams p;
  p.q_lat = static_cast<const __nv_bfloat16*>(q_lat_hm);
  p.q_pe = static_cast<const __nv_bfloat16*>(q_pe_hm);
  p.cache = static_cast<const __nv_bfloat16*>(cache);
  p.out = static_cast<__nv_bfloat16*>(out_hm);
  p.q_cu = static_cast<const int*>(q_cu);
  p.kv_lens = static_cast<const int*>(kv_lens);
  p.block_tables = static_cast<const int*>(block_tables);
  p.seq_begin = seq_begin; p.seq_end = seq_end; p.max_blocks = max_blocks; p.block_size = block_size; p.Hh = Hh; p.T = T;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.cache_slots = cache_slots;
  constexpr int ROWB = 576 * 2;
  const size_t smem = 16 * ROWB + 2 * 64 * ROWB + 16 * 64 * 4 + 16 * 128 + 3 * 16 * 4 + 128;
  static bool set = false;
  if (!set) { cudaFuncSetAttribute(mla_attn_kernel<512, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)); set = true; }
  mla_attn_kernel<512, 64><<<max_tiles, 256, smem, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
