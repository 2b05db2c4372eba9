// Paged causal prefill attention (ragged and chunked) on the 5th-generation tensor cores.
//
// Replaces the FlashInfer `ragged_run` / `paged_run` prefill calls of the reference
// (xllm/core/kernels/cuda/batch_prefill.cpp:100-160, batch_chunked_prefill.cpp:63-91), which on a B200 run the
// mma.sync (fa2) kernels.
//
// One CTA = (sequence, 128 query rows, NH query heads that share one kv head); NH = 2 when the GQA group is even, so
// that the K / V tiles in shared memory feed two heads and two softmax warp groups keep each SM sub-partition busy:
//   warp 0        : TMA producer - the Q tiles once, then a ring of 64-token K and V tiles fetched box by box from
//                   the paged cache through the block table (cp.async.bulk.tensor, 128-byte swizzle, no cluster
//                   broadcast);
//   warp 1        : MMA issuer   - per head S = Q K^T (tcgen05.mma, M=128, N=64, fp32 in TMEM, two S buffers) and
//                   O += P V (M=128, N=128, V read as an MN-major operand straight from its cache layout);
//   warps 2-5 (+6-9): softmax of head 0 (head 1) - one query row per thread: tcgen05.ld of its S row, causal /
//                   length / window mask, online max and sum in the log2 domain, P written as bf16 into a swizzled
//                   shared-memory tile that the second MMA reads, O rescaled in TMEM only when a row maximum grew
//                   by more than 2^8 (otherwise the stale maximum is kept, which is exact after the final division
//                   by the row sum), final O / l stored as bf16.
// QK^T of tile j+1 is issued before P V of tile j, so the tensor pipe works while the softmax warps are busy.
// Every wait is bounded; on expiry the kernel records a status code and leaves.
#include <string.h>

#include "common.cuh"

namespace xl_pf {
using namespace xl;

constexpr int BQ = 128;          // query rows per CTA (= TMEM lanes)
constexpr int BKV = 64;          // kv tokens per tile
constexpr int D = 128;           // head dimension
template <int NH> struct Cfg {
  static constexpr int kStages = NH == 2 ? 4 : 5;
  static constexpr int kThreads = 64 + 128 * NH;
  static constexpr uint32_t kTmemCols = NH == 2 ? 512 : 256;   // per head: S0, S1 (64 columns each) and O (128)
};
constexpr int Q_BYTES = BQ * D * 2;            // 32 KB: two 64-column slabs of [128][64]
constexpr int Q_SLAB = BQ * 128;               // 16 KB
constexpr int KV_SLAB = BKV * 128;             // 8 KB: [64 tokens][64 columns]
constexpr int K_BYTES = 2 * KV_SLAB;           // 16 KB
constexpr int STAGE_BYTES = 2 * K_BYTES;       // K then V
constexpr int P_BYTES = BQ * BKV * 2;          // 16 KB: [128][64] K-major
constexpr int kMaxStages = 5;

struct Barriers {
  uint64_t q_full;
  uint64_t kv_full[kMaxStages];
  uint64_t kv_empty[kMaxStages];
  uint64_t s_full[2][2];      // [head][buffer]
  uint64_t s_free[2][2];
  uint64_t p_full[2];
  uint64_t pv_done[2];
  uint32_t tmem_base;
  int last_split;             // set for the CTA that arrives last at its tile's split counter
};

struct Params {
  __nv_bfloat16* out;          // [T, Hq*D]
  const int* q_cu;
  const int* kv_lens;
  const int* block_tables;
  int seq_begin, seq_end;
  const int* dyn_begin;
  const int* dyn_end;
  int max_blocks, block_size, box_tokens, n_q, n_kv;
  long num_slots;
  float scale_log2;
  int window;
  int* status;
  // KV split (grid.z > 1): every split writes an unnormalised fp32 partial of its key range, the split that arrives
  // last at the tile's counter merges them
  int splits;                  // upper bound (grid.z); a tile uses fewer when its key range is short
  int min_tiles;               // key tiles a split must at least have to be worth its merge
  int ws_tiles;                // q tiles the workspace has room for (tiles beyond it are not split)
  float* ws_o;                 // [unit][split][D/4][BQ] float4, unit = (q tile, head)
  float2* ws_ml;               // [unit][split][BQ]: (reference maximum in the scaled log2 domain, row sum)
  int* ws_cnt;                 // [q tile][head group] arrival counters, zero between launches
};

// MN-major operand tile stored with the 128-byte swizzle: rows (the K index of the MMA) of 128 bytes holding 64
// consecutive MN elements; 8-row groups `sbo` bytes apart; the next 64 MN elements `lbo` bytes away.
__device__ __forceinline__ uint64_t umma_desc_sw128_mn(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr & 0x3FFFF) >> 4);
  d |= uint64_t(lbo_bytes >> 4) << 16;
  d |= uint64_t(sbo_bytes >> 4) << 32;
  d |= uint64_t(1) << 46;
  d |= uint64_t(2) << 61;
  return d;
}

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int NH>
__global__ void __launch_bounds__(Cfg<NH>::kThreads, 1)
prefill_attn_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const Params p) {
  constexpr int kStages = Cfg<NH>::kStages;
  constexpr uint32_t kTmemCols = Cfg<NH>::kTmemCols;
  // The swizzled tiles need a 1024-byte aligned base, which the declared alignment of the dynamic array provides;
  // a CTA that finds it otherwise reports and leaves.
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) atomicExch(p.status, XL_ERR_BOUNDS);
    return;
  }
  uint8_t* sQ = smem;                               // NH tiles
  uint8_t* sKV = sQ + NH * Q_BYTES;
  uint8_t* sP = sKV + kStages * STAGE_BYTES;        // NH tiles
  Barriers* bars = reinterpret_cast<Barriers*>(sP + NH * P_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head0 = blockIdx.y * NH;                // first query head of this CTA
  const int kvh = head0 / (p.n_q / p.n_kv);

  // which sequence / q tile?  Heavier (later) tiles of a causal prompt are scheduled first.
  int tile = int(gridDim.x) - 1 - int(blockIdx.x), seq = -1, q_start = 0, q_len = 0;
  int tile_ord = 0;                                   // ordinal of the tile among the tiles that carry work
  {
    const int sb = p.dyn_begin ? *p.dyn_begin : p.seq_begin;
    const int se = p.dyn_end ? *p.dyn_end : p.seq_end;
    int total = 0;
    for (int s = sb; s < se; ++s) total += (p.q_cu[s + 1] - p.q_cu[s] + BQ - 1) / BQ;
    tile -= int(gridDim.x) - total;            // the last `total` CTAs of the reversed order carry work
    if (tile < 0) return;
    tile_ord = tile;
    for (int s = sb; s < se; ++s) {
      const int a = p.q_cu[s], b = p.q_cu[s + 1];
      const int nt = (b - a + BQ - 1) / BQ;
      if (tile < nt) { seq = s; q_start = a; q_len = b - a; break; }
      tile -= nt;
    }
  }
  if (seq < 0) return;
  const int kv_len = p.kv_lens[seq];
  const int q0 = tile * BQ;
  const int rows = min(BQ, q_len - q0);
  const int pos0 = kv_len - q_len + q0;               // absolute position of query row 0 of the tile
  const int kv_end = min(kv_len, pos0 + rows);
  int kv_begin = 0;
  if (p.window > 0) kv_begin = max(0, pos0 - p.window + 1) / BKV * BKV;
  const int n_tiles_all = (kv_end - kv_begin + BKV - 1) / BKV;
  // this CTA's share of the key tiles (all of them without a split); short key ranges are left whole
  int n_eff = 1;
  if (p.splits > 1 && tile_ord < p.ws_tiles) n_eff = max(1, min(p.splits, n_tiles_all / p.min_tiles));
  if (int(blockIdx.z) >= n_eff) return;
  const int n_splits = n_eff;
  const int chunk = (n_tiles_all + n_splits - 1) / n_splits;
  const int j_first = int(blockIdx.z) * chunk;
  const int n_tiles = max(0, min(n_tiles_all, j_first + chunk) - j_first);
  kv_begin += j_first * BKV;
  const int* bt = p.block_tables + size_t(seq) * p.max_blocks;
  if (n_tiles > 0) {

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->kv_full[s], 1);
      mbar_init(&bars->kv_empty[s], 1);
    }
    for (int h = 0; h < NH; ++h) {
      for (int b = 0; b < 2; ++b) {
        mbar_init(&bars->s_full[h][b], 1);
        mbar_init(&bars->s_free[h][b], 4);
      }
      mbar_init(&bars->p_full[h], 4);
      mbar_init(&bars->pv_done[h], 1);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;       // head h: S buffers at h*256 + {0, 64}, O at h*256 + 128

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (whole warp: lanes share the boxes)
    if (lane == 0) {
      prefetch_tmap(&tmQ);
      prefetch_tmap(&tmK);
      prefetch_tmap(&tmV);
      mbar_arrive_expect_tx(&bars->q_full, NH * Q_BYTES);
#pragma unroll
      for (int h = 0; h < NH; ++h) {
        tma_load_2d(sQ + h * Q_BYTES, &tmQ, &bars->q_full, (head0 + h) * D, q_start + q0);
        tma_load_2d(sQ + h * Q_BYTES + Q_SLAB, &tmQ, &bars->q_full, (head0 + h) * D + 64, q_start + q0);
      }
    }
    const int boxes = BKV / p.box_tokens;            // boxes per 64-token slab (1, 2 or 4)
    const int per_tile = boxes * 4;                  // x 2 slabs x {K, V}
    const int which = lane / (boxes * 2);            // 0 = K, 1 = V
    const int slab = (lane / boxes) & 1;
    const int bx = lane % boxes;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int st = j % kStages;
      const uint32_t ph = (j / kStages) & 1;
      // the block-table entry is fetched before the stage is waited for
      long slot = 0;
      if (lane < per_tile) {
        const int tok = kv_begin + j * BKV + bx * p.box_tokens;
        int bi = tok / p.block_size;
        bi = bi < p.max_blocks ? bi : p.max_blocks - 1;
        slot = long(bt[bi]) * p.block_size + tok % p.block_size;
        if (slot < 0 || slot + p.box_tokens > p.num_slots) slot = 0;
      }
      if (lane == 0) {
        if (!mbar_wait(&bars->kv_empty[st], ph ^ 1)) {
          atomicExch(p.status, XL_ERR_WAIT_EMPTY);
          ok = false;
        } else {
          mbar_arrive_expect_tx(&bars->kv_full[st], STAGE_BYTES);
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (lane < per_tile) {
        uint8_t* dst = sKV + st * STAGE_BYTES + which * K_BYTES + slab * KV_SLAB + bx * p.box_tokens * 128;
        tma_load_3d(dst, which ? &tmV : &tmK, &bars->kv_full[st], slab * 64, kvh, int(slot));
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one_sync()) {
      const uint32_t idesc_s = umma_idesc_f16(BQ, BKV, 1);
      const uint32_t idesc_o = umma_idesc_f16(BQ, D, 1) | (1u << 16);       // B operand (V) is MN-major
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      bool ok = mbar_wait(&bars->q_full, 0);
      if (!ok) atomicExch(p.status, XL_ERR_WAIT_FULL);
      auto issue_pv = [&](int j) -> bool {
        const uint32_t v_addr = smem_u32(sKV + (j % kStages) * STAGE_BYTES + K_BYTES);
#pragma unroll
        for (int h = 0; h < NH; ++h) {
          if (!mbar_wait(&bars->p_full[h], j & 1)) {
            atomicExch(p.status, XL_ERR_WAIT_TMEM_FULL);
            return false;
          }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < BKV / 16; ++k)
            tc_mma_f16(tmem_base + h * 256 + 128, umma_desc_sw128(p_addr + h * P_BYTES, k * 32),
                       umma_desc_sw128_mn(v_addr + k * 2048, KV_SLAB, 1024), idesc_o, (j | k) != 0);
          tc_commit(&bars->pv_done[h]);
        }
        tc_commit(&bars->kv_empty[j % kStages]);
        return true;
      };
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j % kStages, b = j & 1;
        if (!mbar_wait(&bars->kv_full[st], (j / kStages) & 1)) {
          atomicExch(p.status, XL_ERR_WAIT_FULL);
          ok = false;
          break;
        }
        const uint32_t k_addr = smem_u32(sKV + st * STAGE_BYTES);
#pragma unroll
        for (int h = 0; h < NH; ++h) {
          if (!mbar_wait(&bars->s_free[h][b], ((j >> 1) & 1) ^ 1)) {
            atomicExch(p.status, XL_ERR_WAIT_TMEM_EMPTY);
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < D / 16; ++k)
            tc_mma_f16(tmem_base + h * 256 + b * 64, umma_desc_sw128(q_addr + h * Q_BYTES + (k >> 2) * Q_SLAB, (k & 3) * 32),
                       umma_desc_sw128(k_addr + (k >> 2) * KV_SLAB, (k & 3) * 32), idesc_s, k != 0);
          tc_commit(&bars->s_full[h][b]);
        }
        if (ok && j > 0) ok = issue_pv(j - 1);
      }
      if (ok && n_tiles > 0) issue_pv(n_tiles - 1);
    }
  } else {
    // ------------------------------------------------------------ softmax / correction / epilogue: one row per thread
    const int h = (warp - 2) >> 2;                           // head of this warp group
    const int q = warp & 3;                                  // TMEM lane quarter of this warp
    const int r = q * 32 + lane;                             // row inside the tile
    const uint32_t t_s = tmem_base + h * 256 + (uint32_t(q * 32) << 16);
    const uint32_t t_o = t_s + 128;
    uint8_t* prow = sP + h * P_BYTES + r * 128;
    const int pos = pos0 + r;
    const int hi = min(pos, kv_len - 1);                     // last visible kv index of this row
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const float sc = p.scale_log2;
    float m_ref = -INFINITY, l_run = 0.f;                    // m_ref: reference maximum of the raw scores
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int b = j & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&bars->s_full[h][b], (j >> 1) & 1))) {
        if (lane == 0) atomicExch(p.status, XL_ERR_WAIT_TMEM_FULL);
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t s0[32], s1[32];
      tmem_ld_32x32(t_s + b * 64, s0);
      tmem_ld_32x32(t_s + b * 64 + 32, s1);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->s_free[h][b]);
      const int kv0 = kv_begin + j * BKV;
      const bool need_mask = (kv0 + BKV - 1 > pos0) || (kv0 + BKV > kv_len) || (p.window > 0);
      float v[64];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        v[c] = __uint_as_float(s0[c]);
        v[32 + c] = __uint_as_float(s1[c]);
      }
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const int t = kv0 + c;
          if (t > hi || t < lo) v[c] = -INFINITY;
        }
      }
      // eight independent chains keep the dependent-issue latency off the critical path
      float mx8[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) mx8[i] = v[i];
#pragma unroll
      for (int c = 8; c < 64; ++c) mx8[c & 7] = fmaxf(mx8[c & 7], v[c]);
      const float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])), fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
      // keep the stale reference unless the scaled maximum grew by more than 8 (factor 256): P stays below 2^8
      const bool had = m_ref != -INFINITY;
      const bool grow = (mx - m_ref) * sc > 8.f || (!had && mx != -INFINITY);
      const float m_new = grow ? mx : m_ref;
      const bool rescale = grow && had;
      const float alpha = rescale ? fast_exp2((m_ref - m_new) * sc) : 1.f;
      m_ref = m_new;
      const float mneg = (m_ref == -INFINITY) ? 0.f : -m_ref * sc;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 64; c += 2) {
        const float e0 = fast_exp2(fmaf(v[c], sc, mneg)), e1 = fast_exp2(fmaf(v[c + 1], sc, mneg));
        sum4[(c >> 1) & 3] += e0 + e1;
        pk[c >> 1] = pack_bf16x2(e0, e1);
      }
      l_run = l_run * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
      // P and O are touched only after P V of the previous tile has finished
      if (j > 0 && !__all_sync(0xffffffffu, mbar_wait(&bars->pv_done[h], (j - 1) & 1))) {
        if (lane == 0) atomicExch(p.status, XL_ERR_WAIT_TMEM_EMPTY);
        ok = false;
        break;
      }
      tc_fence_after();
      if (j > 0 && __any_sync(0xffffffffu, rescale)) {
#pragma unroll
        for (int c = 0; c < D; c += 32) {
          uint32_t o[32];
          tmem_ld_32x32(t_o + c, o);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_32x32(t_o + c, o);
        }
        tc_wait_st();
      }
      // P row r -> shared memory, K-major with the 128-byte swizzle (16-byte chunk c of row r at chunk c ^ (r & 7))
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_full[h]);
    }
    if (ok && n_tiles > 0) {
      if (!__all_sync(0xffffffffu, mbar_wait(&bars->pv_done[h], (n_tiles - 1) & 1))) {
        if (lane == 0) atomicExch(p.status, XL_ERR_WAIT_TMEM_EMPTY);
        ok = false;
      }
    }
    if (ok && n_splits > 1) {
      // partial of this key range: O relative to m_ref, with m_ref and the row sum beside it
      tc_fence_after();
      const size_t unit = (size_t(tile_ord) * gridDim.y + blockIdx.y) * NH + h;
      float4* wo = reinterpret_cast<float4*>(p.ws_o) + (unit * p.splits + blockIdx.z) * (D / 4) * BQ;
#pragma unroll
      for (int c = 0; c < D; c += 32) {
        uint32_t o[32];
        tmem_ld_32x32(t_o + c, o);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 8; ++i)
          wo[size_t(c / 4 + i) * BQ + r] = make_float4(__uint_as_float(o[4 * i]), __uint_as_float(o[4 * i + 1]),
                                                       __uint_as_float(o[4 * i + 2]), __uint_as_float(o[4 * i + 3]));
      }
      p.ws_ml[(unit * p.splits + blockIdx.z) * BQ + r] = make_float2(m_ref == -INFINITY ? -INFINITY : m_ref * sc, l_run);
      __threadfence();
    } else if (ok) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* dst = p.out + size_t(q_start + q0 + r) * (size_t(p.n_q) * D) + (head0 + h) * D;
#pragma unroll
      for (int c = 0; c < D; c += 32) {
        uint32_t o[32];
        tmem_ld_32x32(t_o + c, o);
        tc_wait_ld();
        if (r < rows) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e)
              w[e] = pack_bf16x2(__uint_as_float(o[8 * i + 2 * e]) * inv, __uint_as_float(o[8 * i + 2 * e + 1]) * inv);
            *reinterpret_cast<uint4*>(dst + c + 8 * i) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
  }  // n_tiles > 0
  if (n_splits == 1) return;

  // ---------------------------------------------------------------- merge of the key splits by the last arrival
  if (threadIdx.x == 0) {
    __threadfence();
    int* cnt = p.ws_cnt + size_t(tile_ord) * gridDim.y + blockIdx.y;
    const int prev = atomicAdd(cnt, 1);
    bars->last_split = prev == n_splits - 1;
    if (prev == n_splits - 1) *cnt = 0;        // every split has arrived: ready for the next launch
  }
  __syncthreads();
  if (!bars->last_split || warp < 2) return;
  __threadfence();
  {
    const int h = (warp - 2) >> 2;
    const int r = (warp & 3) * 32 + lane;
    const int n_valid = (n_tiles_all + chunk - 1) / chunk;          // splits that had keys to look at
    const size_t unit = (size_t(tile_ord) * gridDim.y + blockIdx.y) * NH + h;
    const float2* ml = p.ws_ml + unit * p.splits * BQ + r;
    float w[8];
    float m_all = -INFINITY;
#pragma unroll
    for (int z = 0; z < 8; ++z) {
      w[z] = 0.f;
      if (z < n_valid) {
        const float2 v = __ldcg(ml + size_t(z) * BQ);
        if (v.y > 0.f) m_all = fmaxf(m_all, v.x);
      }
    }
    float l_all = 0.f;
#pragma unroll
    for (int z = 0; z < 8; ++z) {
      if (z < n_valid) {
        const float2 v = __ldcg(ml + size_t(z) * BQ);
        w[z] = v.y > 0.f ? fast_exp2(v.x - m_all) : 0.f;
        l_all += w[z] * v.y;
      }
    }
    const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
    if (r < rows) {
      const float4* wo = reinterpret_cast<const float4*>(p.ws_o) + unit * p.splits * (D / 4) * BQ + r;
      __nv_bfloat16* dst = p.out + size_t(q_start + q0 + r) * (size_t(p.n_q) * D) + (head0 + h) * D;
      for (int c4 = 0; c4 < D / 4; c4 += 2) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
#pragma unroll
        for (int z = 0; z < 8; ++z) {
          if (z < n_valid && w[z] != 0.f) {
            const float4 x = __ldcg(wo + (size_t(z) * (D / 4) + c4) * BQ), y = __ldcg(wo + (size_t(z) * (D / 4) + c4 + 1) * BQ);
            a.x += w[z] * x.x; a.y += w[z] * x.y; a.z += w[z] * x.z; a.w += w[z] * x.w;
            b.x += w[z] * y.x; b.y += w[z] * y.y; b.z += w[z] * y.z; b.w += w[z] * y.w;
          }
        }
        *reinterpret_cast<uint4*>(dst + c4 * 4) = make_uint4(pack_bf16x2(a.x * inv, a.y * inv), pack_bf16x2(a.z * inv, a.w * inv),
                                                            pack_bf16x2(b.x * inv, b.y * inv), pack_bf16x2(b.z * inv, b.w * inv));
      }
    }
  }
}

// Workspace of the KV split: one allocation per device, made at the first use outside a stream capture.
constexpr size_t kSplitWsBytes = size_t(64) << 20;
constexpr size_t kSplitCntBytes = size_t(1) << 16;
static int g_kv_split = 1;     // 0: never split, 1: automatic, >1: forced number of splits (tests)
static uint8_t* split_workspace(cudaStream_t stream) {
  static uint8_t* ws[64] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  if (!ws[dev]) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &st) != cudaSuccess || st != cudaStreamCaptureStatusNone) return nullptr;
    void* p = nullptr;
    if (cudaMalloc(&p, kSplitWsBytes + kSplitCntBytes) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, kSplitWsBytes + kSplitCntBytes);
    ws[dev] = static_cast<uint8_t*>(p);
  }
  return ws[dev];
}

template <int NH>
static int launch_prefill(const CUtensorMap* tq, const CUtensorMap* tk, const CUtensorMap* tv, const Params& p_in, int q_tiles_cap,
                          int total_q_rows, cudaStream_t stream) {
  const size_t smem = size_t(NH) * (Q_BYTES + P_BYTES) + Cfg<NH>::kStages * STAGE_BYTES + sizeof(Barriers);
  static bool set = false;
  if (!set) {
    cudaFuncSetAttribute(prefill_attn_tc_kernel<NH>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    set = true;
  }
  Params p = p_in;
  // Few query tiles x heads (short prompts against a long context, or a tensor-parallel shard with a handful of heads)
  // leave most SMs idle while the busiest CTA walks its whole key range alone: cut key ranges into up to 8 splits.  The
  // grid only offers the splits; every tile takes as many as its own key range is worth (`min_tiles` key tiles each).
  const int tiles_est = (total_q_rows + BQ - 1) / BQ;                 // q_tiles_cap also counts one spare tile per sequence
  const int ctas = (tiles_est > 0 ? tiles_est : 1) * (p.n_q / NH);
  int splits = 1;
  if (g_kv_split > 1) splits = g_kv_split;
  else if (g_kv_split == 1 && ctas * 2 <= xl_host::sm_count()) splits = xl_host::sm_count() / ctas;
  if (splits > 8) splits = 8;
  p.splits = 1;
  p.min_tiles = g_kv_split > 1 ? 1 : 12;
  p.ws_tiles = 0;
  if (splits > 1) {
    uint8_t* w = split_workspace(stream);
    const size_t per_tile = size_t(p.n_q) * splits * (size_t(BQ) * D * 4 + size_t(BQ) * 8);
    size_t tiles = kSplitWsBytes / per_tile;
    const size_t cnt_cap = kSplitCntBytes / 4 / size_t(p.n_q / NH);
    if (tiles > cnt_cap) tiles = cnt_cap;
    if (w && tiles > 0) {
      p.splits = splits;
      p.ws_tiles = int(tiles < size_t(q_tiles_cap) ? tiles : size_t(q_tiles_cap));
      p.ws_o = reinterpret_cast<float*>(w);
      p.ws_ml = reinterpret_cast<float2*>(w + size_t(p.ws_tiles) * p.n_q * splits * size_t(BQ) * D * 4);
      p.ws_cnt = reinterpret_cast<int*>(w + kSplitWsBytes);
    }
  }
  dim3 grid(q_tiles_cap, p.n_q / NH, p.splits);
  prefill_attn_tc_kernel<NH><<<grid, Cfg<NH>::kThreads, smem, stream>>>(*tq, *tk, *tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace xl_pf

// 0: no KV split, 1: automatic (default), 2..8: that many splits whenever the workspace allows (tests, measurements).
XL_API void xl_prefill_kv_split(int mode) { xl_pf::g_kv_split = mode < 0 ? 1 : (mode > 8 ? 8 : mode); }

// Prefill attention of sequences [seq_begin, seq_end) (or the device-side range, see xl_paged_attention_dyn) with the
// tcgen05 kernel.  q [T, Hq*D] with row pitch q_stride, caches [blocks, block_size, n_kv, D].  `q_tiles_cap` bounds the
// number of 128-row query tiles.  Returns -3 when the shape is not covered (the caller then uses the mma.sync kernel).
XL_API int xl_prefill_attention_tc(const void* q, const void* k_cache, const void* v_cache, void* out, const void* q_cu,
                                   const void* kv_lens, const void* block_tables, int seq_begin, int seq_end, int max_blocks,
                                   int block_size, int num_blocks_total, int n_q, int n_kv, int head_dim, int q_stride,
                                   int total_q_rows, float scale, int window, int q_tiles_cap, const void* dyn_begin,
                                   const void* dyn_end, void* stream) {
  using namespace xl_pf;
  if (head_dim != D) return -3;
  if (block_size % 16 != 0 || (block_size > 64 && block_size % 64 != 0) || (block_size < 64 && 64 % block_size != 0)) return -3;
  if (n_q % n_kv) return -3;
  if ((q_stride % 8) || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return -3;
  if ((reinterpret_cast<uintptr_t>(k_cache) & 127) || (reinterpret_cast<uintptr_t>(v_cache) & 127)) return -3;
  if (q_tiles_cap <= 0 || seq_end <= seq_begin) return 0;
  const int box_tokens = block_size < 64 ? block_size : 64;
  const uint64_t slots = uint64_t(num_blocks_total) * block_size;
  const CUtensorMap* tq = xl_host::tmap_2d(q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, total_q_rows, uint64_t(n_q) * D, q_stride, BQ, 64,
                                           CU_TENSOR_MAP_SWIZZLE_128B);
  const CUtensorMap* tk = xl_host::tmap_3d(k_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, slots, n_kv, D, box_tokens, 1, 64,
                                           CU_TENSOR_MAP_SWIZZLE_128B);
  const CUtensorMap* tv = xl_host::tmap_3d(v_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, slots, n_kv, D, box_tokens, 1, 64,
                                           CU_TENSOR_MAP_SWIZZLE_128B);
  if (!tq || !tk || !tv) return -3;
  Params p;
  memset(&p, 0, sizeof(p));
  p.out = static_cast<__nv_bfloat16*>(out);
  p.q_cu = static_cast<const int*>(q_cu);
  p.kv_lens = static_cast<const int*>(kv_lens);
  p.block_tables = static_cast<const int*>(block_tables);
  p.seq_begin = seq_begin; p.seq_end = seq_end;
  p.dyn_begin = static_cast<const int*>(dyn_begin);
  p.dyn_end = static_cast<const int*>(dyn_end);
  p.max_blocks = max_blocks; p.block_size = block_size; p.box_tokens = box_tokens; p.n_q = n_q; p.n_kv = n_kv;
  p.num_slots = long(slots);
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window;
  p.status = xl_host::status_word();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if ((n_q / n_kv) % 2 == 0) return launch_prefill<2>(tq, tk, tv, p, q_tiles_cap, total_q_rows, st);
  return launch_prefill<1>(tq, tk, tv, p, q_tiles_cap, total_q_rows, st);
}
