// Paged GQA attention: ragged causal prefill (incl. chunked prefill over cached context) and split-KV decode.
//
// Replaces the FlashInfer batch_prefill / batch_decode modules the reference loads on CUDA
// (xllm/core/layers/cuda/flashinfer_attention.cpp:93-349, kernels/cuda/batch_prefill.cpp:100-160,
// batch_decode.cpp:26-85).  Differences that matter for serving:
//   * no host-side "plan": sequence lengths, block tables and the q-tile -> sequence mapping are read from device
//     memory, so a captured CUDA graph replays with new lengths;
//   * KV layout is the reference's [n_blocks, block_size, n_kv_heads, head_dim] (llm_engine.cpp:573-578).
//
// Both kernels keep the softmax state in registers (online softmax, base-2 exponentials) and feed the tensor
// cores with ldmatrix fragments from 16-byte-chunk XOR-swizzled shared memory filled by cp.async.
#include "common.cuh"

namespace xl {

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc, bool valid) {
  const int sz = valid ? 16 : 0;   // src-size 0 => zero fill
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

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

// byte offset of 16-byte chunk `chunk` of row `row` in a tile whose rows hold D bf16 (D*2 bytes), XOR-swizzled
template <int D>
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
  return uint32_t(row) * (D * 2) + (uint32_t(chunk ^ (row & 7)) << 4);
}

constexpr float kLog2e = 1.4426950408889634f;

struct AttnParams {
  const __nv_bfloat16* q;      // [T, Hq, D], row pitch q_stride elements
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  __nv_bfloat16* out;          // [T, Hq*D]
  const int* q_cu;             // [B+1]
  const int* kv_lens;          // [B]
  const int* block_tables;     // [B, max_blocks]
  int seq_begin, seq_end;      // sequences handled by this launch
  const int* dyn_begin;        // optional device scalars that replace seq_begin / seq_end (CUDA-graph replay:
  const int* dyn_end;          // the launch is sized for the capacity, the real range is read on the device)
  int max_blocks, block_size, n_q, n_kv, q_stride;
  float scale_log2;            // softmax scale * log2(e)
  int window;                  // sliding window (<=0: none)
  // split-KV decode
  int num_splits;
  float* part_o;               // [T, Hq, splits, D]
  float* part_lse;             // [T, Hq, splits]
  int num_blocks_total;
};

// ============================================================================ prefill
// CTA = 4 warps x 16 query rows of one head; KV tiles of 64 tokens, double buffered.
template <int D>
__global__ void __launch_bounds__(128) prefill_attn_kernel(AttnParams p, int total_q_tiles_cap) {
  constexpr int BQ = 64, BKV = 64, CH = D / 8;      // CH = 16-byte chunks per row
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + BQ * D * 2;
  uint8_t* sV = sK + 2 * BKV * D * 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int kvh = head / (p.n_q / p.n_kv);

  // which sequence / q tile is this CTA?  (device-side search keeps the launch independent of the lengths)
  int tile = blockIdx.x, seq = -1, q_start = 0, q_len = 0;
  const int seq_begin = p.dyn_begin ? *p.dyn_begin : p.seq_begin;
  const int seq_end = p.dyn_end ? *p.dyn_end : p.seq_end;
  for (int s = seq_begin; s < seq_end; ++s) {
    const int a = p.q_cu[s], b = p.q_cu[s + 1];
    const int nt = (b - a + BQ - 1) / BQ;
    if (tile < nt) { seq = s; q_start = a; q_len = b - a; break; }
    tile -= nt;
  }
  if (seq < 0) return;
  const int kv_len = p.kv_lens[seq];
  const int q0 = tile * BQ;                       // first query row of this tile within the sequence
  const int rows = min(BQ, q_len - q0);
  const int pos0 = kv_len - q_len + q0;           // absolute position of query row 0 of the tile
  const int* bt = p.block_tables + size_t(seq) * p.max_blocks;
  const int kv_end = min(kv_len, pos0 + rows);    // causal: nothing beyond the last query row's position
  int kv_begin = 0;
  if (p.window > 0) kv_begin = max(0, pos0 - p.window + 1) / BKV * BKV;
  const int n_tiles = (kv_end - kv_begin + BKV - 1) / BKV;

  // ---- Q tile -> smem (rows beyond `rows` are zero filled)
  for (int i = threadIdx.x; i < BQ * CH; i += 128) {
    const int r = i / CH, c = i % CH;
    const bool ok = r < rows;
    const __nv_bfloat16* src = p.q + size_t(q_start + q0 + (ok ? r : 0)) * p.q_stride + head * D + c * 8;
    cp_async_16(sQ + swz<D>(r, c), src, ok);
  }
  cp_async_commit();

  auto load_kv = [&](int t, int stage) {
    const int base = kv_begin + t * BKV;
    uint8_t* dK = sK + stage * BKV * D * 2;
    uint8_t* dV = sV + stage * BKV * D * 2;
    for (int i = threadIdx.x; i < BKV * CH; i += 128) {
      const int r = i / CH, c = i % CH;
      const int tok = base + r;
      const bool ok = tok < kv_end;
      int blk = 0;
      if (ok) blk = bt[tok / p.block_size];
      if (blk < 0 || blk >= p.num_blocks_total) blk = 0;
      const size_t off = ((size_t(blk) * p.block_size + (ok ? tok % p.block_size : 0)) * p.n_kv + kvh) * D + c * 8;
      cp_async_16(dK + swz<D>(r, c), p.k_cache + off, ok);
      cp_async_16(dV + swz<D>(r, c), p.v_cache + off, ok);
    }
    cp_async_commit();
  };

  if (n_tiles > 0) load_kv(0, 0);
  cp_async_wait<0>();
  __syncthreads();

  // ---- Q fragments stay in registers
  uint32_t qf[D / 16][4];
  {
    const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int c = ks * 2 + (lane >> 4);
      ldsm_x4(smem_u32(sQ + swz<D>(r, c)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    }
  }
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int row_a = warp * 16 + (lane >> 2);      // this thread's two rows inside the tile
  const int pos_a = pos0 + row_a, pos_b = pos_a + 8;

  for (int t = 0; t < n_tiles; ++t) {
    const int stage = t & 1;
    if (t + 1 < n_tiles) load_kv(t + 1, stage ^ 1);
    const uint8_t* tK = sK + stage * BKV * D * 2;
    const uint8_t* tV = sV + stage * BKV * D * 2;
    const int base = kv_begin + t * BKV;
    // S = Q K^T  (16 x 64 per warp)
    float s[BKV / 8][4];
#pragma unroll
    for (int i = 0; i < BKV / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
      for (int nt = 0; nt < BKV / 16; ++nt) {
        uint32_t b0, b1, b2, b3;
        const int r = nt * 16 + (lane & 7) + (lane >> 4) * 8;
        const int c = ks * 2 + ((lane >> 3) & 1);
        ldsm_x4(smem_u32(tK + swz<D>(r, c)), b0, b1, b2, b3);
        mma_bf16_16816(s[2 * nt], qf[ks], b0, b1);
        mma_bf16_16816(s[2 * nt + 1], qf[ks], b2, b3);
      }
    }
    // mask + online softmax (two rows per thread)
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < BKV / 8; ++i) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int tok = base + i * 8 + (lane & 3) * 2 + (e & 1);
        const int qpos = (e < 2) ? pos_a : pos_b;
        bool ok = tok <= qpos && tok < kv_end;
        if (p.window > 0) ok = ok && tok > qpos - p.window;
        const float v = ok ? s[i][e] * p.scale_log2 : -INFINITY;
        s[i][e] = v;
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
    for (int i = 0; i < BKV / 8; ++i) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float m = m_run[e >> 1];
        const float pv = (m == -INFINITY) ? 0.f : exp2f(s[i][e] - m);
        s[i][e] = pv;
        rs[e >> 1] += pv;
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * alpha[h] + rs[h];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
      o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < BKV / 16; ++kk) {
      uint32_t pa[4];
      pa[0] = pack_bf16x2(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = pack_bf16x2(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = pack_bf16x2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = pack_bf16x2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int dt = 0; dt < D / 16; ++dt) {
        uint32_t b0, b1, b2, b3;
        const int r = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = dt * 2 + (lane >> 4);
        ldsm_x4_t(smem_u32(tV + swz<D>(r, c)), b0, b1, b2, b3);
        mma_bf16_16816(o[2 * dt], pa, b0, b1);
        mma_bf16_16816(o[2 * dt + 1], pa, b2, b3);
      }
    }
    cp_async_wait<0>();
    __syncthreads();
  }

  // ---- finalize
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  const float inv_a = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f;
  const float inv_b = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
  const int out_ld = p.n_q * D;
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    const int col = head * D + i * 8 + (lane & 3) * 2;
    if (row_a < rows)
      *reinterpret_cast<uint32_t*>(p.out + size_t(q_start + q0 + row_a) * out_ld + col) = pack_bf16x2(o[i][0] * inv_a, o[i][1] * inv_a);
    if (row_a + 8 < rows)
      *reinterpret_cast<uint32_t*>(p.out + size_t(q_start + q0 + row_a + 8) * out_ld + col) = pack_bf16x2(o[i][2] * inv_b, o[i][3] * inv_b);
  }
}

// ============================================================================ decode
// CTA = 4 warps; handles one (sequence, kv head, split).  The `group * q_len` (<= 16) query rows that share the
// kv head form the M dimension of the MMA; each warp walks its own 16-token KV tiles through a private
// cp.async ring, and the four partial results are merged through shared memory.
template <int D, int STAGES>
__global__ void __launch_bounds__(128) decode_attn_kernel(AttnParams p) {
  constexpr int TK = 16, CH = D / 8;
  constexpr int TILE_BYTES = TK * D * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = (p.dyn_begin ? *p.dyn_begin : p.seq_begin) + blockIdx.x;
  const int kvh = blockIdx.y;
  const int split = blockIdx.z;
  const int group = p.n_q / p.n_kv;
  if (seq >= (p.dyn_end ? *p.dyn_end : p.seq_end)) return;
  const int q_start = p.q_cu[seq];
  const int q_len = p.q_cu[seq + 1] - q_start;
  const int kv_len = p.kv_lens[seq];
  if (q_len <= 0) return;
  const int rows = min(16, q_len * group);        // row m = qtok * group + g
  uint8_t* sQ = smem;                              // 16 x D
  uint8_t* sKV = smem + 16 * D * 2 + warp * (STAGES * 2 * TILE_BYTES);
  const int* bt = p.block_tables + size_t(seq) * p.max_blocks;

  // KV range of this split, in 64-token units (16 per warp)
  const int per_split = ((kv_len + p.num_splits - 1) / p.num_splits + 63) / 64 * 64;
  int s_begin = split * per_split;
  int s_end = min(kv_len, s_begin + per_split);
  if (p.window > 0) s_begin = max(s_begin, (max(0, kv_len - q_len - p.window + 1)) / 64 * 64);
  const int n_tiles_total = s_end > s_begin ? (s_end - s_begin + TK - 1) / TK : 0;
  const int my_tiles = n_tiles_total > warp ? (n_tiles_total - warp + 3) / 4 : 0;   // tiles warp, warp+4, ...

  // ---- Q rows -> smem (zero beyond `rows`)
  for (int i = threadIdx.x; i < 16 * CH; i += 128) {
    const int r = i / CH, c = i % CH;
    const bool ok = r < rows;
    const int qt = ok ? r / group : 0, g = ok ? r % group : 0;
    const __nv_bfloat16* src = p.q + size_t(q_start + qt) * p.q_stride + (kvh * group + g) * D + c * 8;
    cp_async_16(sQ + swz<D>(r, c), src, ok);
  }
  cp_async_commit();

  auto load_tile = [&](int j, int stage) {   // j-th tile of this warp
    const int base = s_begin + (warp + 4 * j) * TK;
    uint8_t* dK = sKV + stage * 2 * TILE_BYTES;
    uint8_t* dV = dK + TILE_BYTES;
#pragma unroll
    for (int i = lane; i < TK * CH; i += 32) {
      const int r = i / CH, c = i % CH;
      const int tok = base + r;
      const bool ok = tok < s_end;
      int blk = 0;
      if (ok) blk = bt[tok / p.block_size];
      if (blk < 0 || blk >= p.num_blocks_total) blk = 0;
      const size_t off = ((size_t(blk) * p.block_size + (ok ? tok % p.block_size : 0)) * p.n_kv + kvh) * D + c * 8;
      cp_async_16(dK + swz<D>(r, c), p.k_cache + off, ok);
      cp_async_16(dV + swz<D>(r, c), p.v_cache + off, ok);
    }
  };
#pragma unroll
  for (int j = 0; j < STAGES - 1; ++j) {
    if (j < my_tiles) load_tile(j, j);
    cp_async_commit();
  }
  cp_async_wait<STAGES - 1>();     // the Q group (oldest) has landed
  __syncthreads();

  uint32_t qf[D / 16][4];
  {
    const int r = (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
      ldsm_x4(smem_u32(sQ + swz<D>(r, ks * 2 + (lane >> 4))), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
  }
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int row_a = lane >> 2, row_b = row_a + 8;
  // causal limit per row: query token qt sees positions <= kv_len - q_len + qt
  const int lim_a = kv_len - q_len + (row_a < rows ? row_a / group : 0);
  const int lim_b = kv_len - q_len + (row_b < rows ? row_b / group : 0);

  for (int j = 0; j < my_tiles; ++j) {
    const int stage = j % STAGES;
    if (j + STAGES - 1 < my_tiles) load_tile(j + STAGES - 1, (j + STAGES - 1) % STAGES);
    cp_async_commit();
    cp_async_wait<STAGES - 1>();
    __syncwarp();
    const uint8_t* tK = sKV + stage * 2 * TILE_BYTES;
    const uint8_t* tV = tK + TILE_BYTES;
    const int base = s_begin + (warp + 4 * j) * TK;
    float s[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t b0, b1, b2, b3;
      const int r = (lane & 7) + (lane >> 4) * 8;
      const int c = ks * 2 + ((lane >> 3) & 1);
      ldsm_x4(smem_u32(tK + swz<D>(r, c)), b0, b1, b2, b3);
      mma_bf16_16816(s[0], qf[ks], b0, b1);
      mma_bf16_16816(s[1], qf[ks], b2, b3);
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
        const float v = ok ? s[i][e] * p.scale_log2 : -INFINITY;
        s[i][e] = v;
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
        const float pv = (m == -INFINITY) ? 0.f : exp2f(s[i][e] - m);
        s[i][e] = pv;
        rs[e >> 1] += pv;
      }
    }
    l_run[0] = l_run[0] * alpha[0] + rs[0];
    l_run[1] = l_run[1] * alpha[1] + rs[1];
    uint32_t pa[4] = {pack_bf16x2(s[0][0], s[0][1]), pack_bf16x2(s[0][2], s[0][3]), pack_bf16x2(s[1][0], s[1][1]),
                      pack_bf16x2(s[1][2], s[1][3])};
#pragma unroll
    for (int dt = 0; dt < D / 16; ++dt) {
      o[2 * dt][0] *= alpha[0]; o[2 * dt][1] *= alpha[0]; o[2 * dt][2] *= alpha[1]; o[2 * dt][3] *= alpha[1];
      o[2 * dt + 1][0] *= alpha[0]; o[2 * dt + 1][1] *= alpha[0]; o[2 * dt + 1][2] *= alpha[1]; o[2 * dt + 1][3] *= alpha[1];
      uint32_t b0, b1, b2, b3;
      const int r = (lane & 7) + ((lane >> 3) & 1) * 8;
      const int c = dt * 2 + (lane >> 4);
      ldsm_x4_t(smem_u32(tV + swz<D>(r, c)), b0, b1, b2, b3);
      mma_bf16_16816(o[2 * dt], pa, b0, b1);
      mma_bf16_16816(o[2 * dt + 1], pa, b2, b3);
    }
    __syncwarp();
  }
  cp_async_wait<0>();
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  __syncthreads();   // every warp is done with its ring: reuse the memory for the merge

  // ---- merge the four warps: sO[warp][16][D] fp32, sM/sL[warp][16]
  float* sO = reinterpret_cast<float*>(smem + 16 * D * 2);
  float* sM = sO + 4 * 16 * D;
  float* sL = sM + 64;
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
  __syncthreads();
  for (int r = warp; r < rows; r += 4) {
    float m = fmaxf(fmaxf(sM[r], sM[16 + r]), fmaxf(sM[32 + r], sM[48 + r]));
    float w[4], l = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      w[k] = (sM[k * 16 + r] == -INFINITY) ? 0.f : exp2f(sM[k * 16 + r] - m);
      l += w[k] * sL[k * 16 + r];
    }
    const int qt = r / group, g = r % group;
    const int hq = kvh * group + g;
    const size_t tok = size_t(q_start + qt);
    if (p.num_splits == 1) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      for (int c = lane * 2; c < D; c += 64) {
        float a = 0.f, b = 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          a += w[k] * sO[(k * 16 + r) * D + c];
          b += w[k] * sO[(k * 16 + r) * D + c + 1];
        }
        *reinterpret_cast<uint32_t*>(p.out + tok * (p.n_q * D) + hq * D + c) = pack_bf16x2(a * inv, b * inv);
      }
    } else {
      float* po = p.part_o + ((tok * p.n_q + hq) * p.num_splits + split) * D;
      const float inv = l > 0.f ? 1.f / l : 0.f;    // partials are stored normalised; the merge weighs them by 2^lse
      for (int c = lane * 2; c < D; c += 64) {
        float a = 0.f, b = 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          a += w[k] * sO[(k * 16 + r) * D + c];
          b += w[k] * sO[(k * 16 + r) * D + c + 1];
        }
        *reinterpret_cast<float2*>(po + c) = make_float2(a * inv, b * inv);
      }
      if (lane == 0) {
        // (m, l) packed as log-sum-exp in base 2; -inf when the split saw no token
        p.part_lse[(tok * p.n_q + hq) * p.num_splits + split] = (l > 0.f) ? m + log2f(l) : -INFINITY;
      }
    }
  }
}

// merge of split-KV partials: one warp per (token, head)
template <int D>
__global__ void decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                    __nv_bfloat16* __restrict__ out, const int* __restrict__ q_cu, int seq_begin, int seq_end,
                                    int n_q, int splits, const int* dyn_begin, const int* dyn_end) {
  const int lane = threadIdx.x & 31;
  const long gw = (blockIdx.x * long(blockDim.x) + threadIdx.x) >> 5;
  if (dyn_begin) seq_begin = *dyn_begin;
  if (dyn_end) seq_end = *dyn_end;
  if (seq_end <= seq_begin) return;
  const int t0 = q_cu[seq_begin], t1 = q_cu[seq_end];
  const long n = long(t1 - t0) * n_q;
  if (gw >= n) return;
  const size_t tok = size_t(t0) + size_t(gw / n_q);
  const int h = int(gw % n_q);
  const float* lse = part_lse + (tok * n_q + h) * splits;
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, lse[s]);
  float acc[D / 32];
#pragma unroll
  for (int i = 0; i < D / 32; ++i) acc[i] = 0.f;
  float den = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float w = (lse[s] == -INFINITY) ? 0.f : exp2f(lse[s] - m);   // each normalised partial weighs 2^lse_s
    den += w;
    const float* po = part_o + ((tok * n_q + h) * splits + s) * D;
#pragma unroll
    for (int i = 0; i < D / 32; ++i) acc[i] += w * po[lane + 32 * i];
  }
  const float inv = den > 0.f ? 1.f / den : 0.f;
#pragma unroll
  for (int i = 0; i < D / 32; ++i) out[tok * (size_t(n_q) * D) + h * D + lane + 32 * i] = __float2bfloat16(acc[i] * inv);
}

}  // namespace xl

using namespace xl;

XL_API int xl_prefill_attention_tc(const void* q, const void* k_cache, const void* v_cache, void* out, const void* q_cu,
                                   const void* kv_lens, const void* block_tables, int seq_begin, int seq_end, int max_blocks,
                                   int block_size, int num_blocks_total, int n_q, int n_kv, int head_dim, int q_stride,
                                   int total_q_rows, float scale, int window, int q_tiles_cap, const void* dyn_begin,
                                   const void* dyn_end, void* stream);
static int g_prefill_tc = 1;
// Test / comparison hook: 0 routes prefill to the mma.sync kernel, 1 (default) tries the tcgen05 kernel first.
XL_API void xl_prefill_use_tc(int on) { g_prefill_tc = on; }

// q [T, Hq*D] with row pitch q_stride; out [T, Hq*D] contiguous.  Sequences [seq_begin, seq_end) are handled:
// `decode` != 0 -> every sequence has q_len * group <= 16 and the split-KV kernel is used.
//
// `dyn_begin` / `dyn_end` (device int pointers, may be null) replace seq_begin / seq_end at run time: the launch is then
// sized for [seq_begin, seq_end) as a capacity and CTAs outside the real range exit.  This is what lets a captured
// CUDA graph of a mixed decode + prefill step replay with a different split between the two kinds.
// `total_q_rows` = rows of q (T); 0 = unknown, which keeps prefill on the mma.sync kernel.
XL_API int xl_paged_attention_dyn(const void* q, const void* k_cache, const void* v_cache, void* out, const void* q_cu,
                                  const void* kv_lens, const void* block_tables, int seq_begin, int seq_end, int max_blocks,
                                  int block_size, int num_blocks_total, int n_q, int n_kv, int head_dim, int q_stride,
                                  float scale, int window, int decode, int q_tiles_cap, int num_splits, void* part_o,
                                  void* part_lse, const void* dyn_begin, const void* dyn_end, int total_q_rows, void* stream) {
  if (seq_end <= seq_begin) return 0;
  if (head_dim != 128 && head_dim != 64) return -2;
  if (n_q % n_kv) return -2;
  AttnParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.q_cu = static_cast<const int*>(q_cu);
  p.kv_lens = static_cast<const int*>(kv_lens);
  p.block_tables = static_cast<const int*>(block_tables);
  p.seq_begin = seq_begin; p.seq_end = seq_end;
  p.dyn_begin = static_cast<const int*>(dyn_begin);
  p.dyn_end = static_cast<const int*>(dyn_end);
  p.max_blocks = max_blocks; p.block_size = block_size; p.n_q = n_q; p.n_kv = n_kv; p.q_stride = q_stride;
  p.scale_log2 = scale * kLog2e;
  p.window = window;
  p.num_splits = num_splits < 1 ? 1 : num_splits;
  p.part_o = static_cast<float*>(part_o);
  p.part_lse = static_cast<float*>(part_lse);
  p.num_blocks_total = num_blocks_total;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int nseq = seq_end - seq_begin;
  if (decode) {
    if ((n_q / n_kv) > 16) return -2;
    if (p.num_splits > 1 && (!part_o || !part_lse)) return -2;
    constexpr int STAGES = 3;
    dim3 grid(nseq, n_kv, p.num_splits);
    if (head_dim == 128) {
      const size_t ring = 16 * 128 * 2 + 4 * STAGES * 2 * 16 * 128 * 2;
      const size_t merge = 16 * 128 * 2 + 4 * 16 * 128 * 4 + 128 * 4;
      const size_t smem = ring > merge ? ring : merge;
      static bool set = false;
      if (!set) { cudaFuncSetAttribute(decode_attn_kernel<128, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)); set = true; }
      decode_attn_kernel<128, STAGES><<<grid, 128, smem, st>>>(p);
      if (p.num_splits > 1) {
        // upper bound of rows: every sequence contributes at most 16 / group query tokens
        const long warps = long(nseq) * (16 / (n_q / n_kv)) * n_q;
        decode_merge_kernel<128><<<int((warps + 3) / 4), 128, 0, st>>>(p.part_o, p.part_lse, p.out, p.q_cu, seq_begin, seq_end, n_q, p.num_splits, p.dyn_begin, p.dyn_end);
      }
    } else {
      const size_t ring = 16 * 64 * 2 + 4 * STAGES * 2 * 16 * 64 * 2;
      const size_t merge = 16 * 64 * 2 + 4 * 16 * 64 * 4 + 128 * 4;
      const size_t smem = ring > merge ? ring : merge;
      static bool set = false;
      if (!set) { cudaFuncSetAttribute(decode_attn_kernel<64, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)); set = true; }
      decode_attn_kernel<64, STAGES><<<grid, 128, smem, st>>>(p);
      if (p.num_splits > 1) {
        const long warps = long(nseq) * (16 / (n_q / n_kv)) * n_q;
        decode_merge_kernel<64><<<int((warps + 3) / 4), 128, 0, st>>>(p.part_o, p.part_lse, p.out, p.q_cu, seq_begin, seq_end, n_q, p.num_splits, p.dyn_begin, p.dyn_end);
      }
    }
  } else {
    if (q_tiles_cap <= 0) return 0;
    if (g_prefill_tc && total_q_rows > 0) {   // tcgen05 kernel first; it declines (-3) the shapes it does not cover
      const int rc = xl_prefill_attention_tc(q, k_cache, v_cache, out, q_cu, kv_lens, block_tables, seq_begin, seq_end, max_blocks,
                                             block_size, num_blocks_total, n_q, n_kv, head_dim, q_stride, total_q_rows, scale,
                                             window, q_tiles_cap, dyn_begin, dyn_end, stream);
      if (rc != -3) return rc;
    }
    dim3 grid(q_tiles_cap, n_q);
    if (head_dim == 128) {
      const size_t smem = (64 + 4 * 64) * 128 * 2;
      static bool set = false;
      if (!set) { cudaFuncSetAttribute(prefill_attn_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); set = true; }
      prefill_attn_kernel<128><<<grid, 128, smem, st>>>(p, q_tiles_cap);
    } else {
      const size_t smem = (64 + 4 * 64) * 64 * 2;
      prefill_attn_kernel<64><<<grid, 128, smem, st>>>(p, q_tiles_cap);
    }
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

XL_API int xl_paged_attention(const void* q, const void* k_cache, const void* v_cache, void* out, const void* q_cu,
                              const void* kv_lens, const void* block_tables, int seq_begin, int seq_end, int max_blocks,
                              int block_size, int num_blocks_total, int n_q, int n_kv, int head_dim, int q_stride, float scale,
                              int window, int decode, int q_tiles_cap, int num_splits, void* part_o, void* part_lse,
                              void* stream) {
  return xl_paged_attention_dyn(q, k_cache, v_cache, out, q_cu, kv_lens, block_tables, seq_begin, seq_end, max_blocks, block_size,
                                num_blocks_total, n_q, n_kv, head_dim, q_stride, scale, window, decode, q_tiles_cap, num_splits,
                                part_o, part_lse, nullptr, nullptr, 0, stream);
}
