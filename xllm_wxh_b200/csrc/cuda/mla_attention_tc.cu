// Multi-head latent attention (absorbed form) over the paged latent cache on the 5th-generation tensor cores.
//
//   cache row (per token) : [ latent (C = 512) | RoPE(k_pe) (R = 64) ]     576 bf16, shared by every head
//   S = Q K^T over all 576 columns;  O = softmax(S) . cache[:, :512]       (the latent is also the value)
//
// Semantics of the reference's MLA layer: layers/mlu/deepseek_v2_attention.cpp:184-240,406-496 (the reference has no
// CUDA kernel for it).  `mla.cu` holds the mma.sync kernel this one replaces wherever the shape allows.
//
// Tile = 128 query rows that share one key range: `tpt = 128 / Hh` consecutive tokens of a sequence x all Hh heads of this
// rank (one token x 128 heads for an unsharded DeepSeek-V3; 8 tokens x 16 heads under TP 8).  The accumulator of a whole
// row (512 fp32) would fill the tensor memory of an SM by itself, so a tile is computed by two CTAs that each own one half
// of the latent columns of O (256 TMEM columns), both computing S (four 64-column partial accumulators that the softmax
// adds up: a product that accumulates into its predecessor's tile has to wait for it, so consecutive products go to
// different tiles):
//   warp 0     : TMA producer.  Q once (nine [128 x 64] slabs, 128-byte swizzle), then a FIFO of [64 tokens x 64 columns]
//                chunks of the cache fetched box by box through the block table: the nine chunks of a key tile for
//                S, and, one tile later, the four chunks of this CTA's latent half again (from L2) for P V;
//   warp 1     : MMA issuer.  S(j+1) = Q K^T (36 tcgen05.mma, M = 128, N = 64) is issued before O += P(j) V(j)
//                (16 tcgen05.mma over four column blocks of O, V read as an MN-major operand straight from the cache
//                layout);
//   warps 2-5  : softmax, one query row per thread (tcgen05.ld of the row of S, causal / length mask, online maximum and
//                sum in the log2 domain with a lazy rescale of O, P as bf16 into a swizzled shared-memory tile).
// Long key ranges of few tiles are cut into splits (grid.z); each split stores an unnormalised fp32 partial and a small
// second kernel merges them.  Every wait is bounded; on expiry the kernel records a status code and leaves.
#include <string.h>

#include "common.cuh"

namespace xl_mla_tc {
using namespace xl;

constexpr int BQ = 128;            // rows per tile (= TMEM lanes)
constexpr int BKV = 64;            // key tokens per tile
constexpr int C = 512, R = 64;
constexpr int NCH = (C + R) / 64;  // 9 column chunks of a cache row
constexpr int HALF = C / 2;        // latent columns of O per CTA
constexpr int VCH = HALF / 64;     // 4 value chunks per CTA
constexpr int Q_SLAB = BQ * 128;   // 16 KB
constexpr int CHUNK = BKV * 128;   // 8 KB
constexpr int kSlots = 8;
constexpr int P_BYTES = BQ * BKV * 2;
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 512;      // O: 0..255; four partial accumulators of S at 256, 320, 384, 448
constexpr int kSParts = 4;               // a tcgen05.mma that accumulates into the tile of its predecessor waits for it (about
                                         // 160 cycles here, against 32 cycles of work at N = 64), so the 36 products of a key
                                         // tile's S go round four accumulators that the softmax adds up
constexpr int kMaxSplits = 16;

struct Barriers {
  uint64_t q_full;
  uint64_t full[kSlots];
  uint64_t empty[kSlots];
  uint64_t s_full;
  uint64_t s_free;
  uint64_t p_full;
  uint64_t pv_done;
  uint32_t tmem_base;
};

struct Params {
  __nv_bfloat16* out;          // [Hh, T, C] head-major
  const int* q_cu;
  const int* kv_lens;
  const int* block_tables;
  int seq_begin, seq_end, max_blocks, block_size, box_tokens, Hh, tpt, T;
  long num_slots;
  float scale_log2;
  int* status;
  int splits;                  // grid.z; a tile uses fewer when its key range is short
  int min_tiles;               // key tiles a split must at least have
  int ws_tiles;                // tiles the workspace has room for (tiles beyond it are not split)
  float* ws_o;                 // [tile][half][split][HALF/4][BQ] float4
  float2* ws_ml;               // [tile][split][BQ]: (reference maximum in the scaled log2 domain, row sum)
  long long* trace;            // diagnosis: clock stamps of CTA 0 ([tile][16]; null: off)
};

struct TileInfo {
  int seq, q_start, q_len, qt0, kv_len, kv_end, n_tiles_all, n_eff;
};

// Which (sequence, token group) is tile `tile`, and how many key splits does it use?
__device__ __forceinline__ bool find_tile(const Params& p, int tile, TileInfo& t) {
  t.seq = -1;
  int left = tile;
  for (int s = p.seq_begin; s < p.seq_end; ++s) {
    const int a = p.q_cu[s], b = p.q_cu[s + 1];
    const int nt = (b - a + p.tpt - 1) / p.tpt;
    if (left < nt) {
      t.seq = s; t.q_start = a; t.q_len = b - a;
      break;
    }
    left -= nt;
  }
  if (t.seq < 0) return false;
  t.qt0 = left * p.tpt;
  t.kv_len = p.kv_lens[t.seq];
  const int last_tok = min(t.q_len - 1, t.qt0 + p.tpt - 1);
  t.kv_end = max(0, min(t.kv_len, t.kv_len - t.q_len + last_tok + 1));
  t.n_tiles_all = (t.kv_end + BKV - 1) / BKV;
  t.n_eff = 1;
  if (p.splits > 1 && tile < p.ws_tiles) t.n_eff = max(1, min(p.splits, t.n_tiles_all / p.min_tiles));
  return true;
}

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

// Column chunk of the cache row that FIFO item `i` (0..8) of a key tile carries for latent half `half`: the chunks only S
// needs come first, the CTA's own latent half last.
__device__ __forceinline__ int qk_chunk(int half, int i) {
  if (i < VCH) return (1 - half) * VCH + i;     // the other latent half
  if (i == VCH) return NCH - 1;                 // rope columns
  return half * VCH + (i - VCH - 1);            // own latent half
}

__global__ void __launch_bounds__(kThreads, 1)
mla_attn_tc_kernel(const __grid_constant__ CUtensorMap tmQl, const __grid_constant__ CUtensorMap tmQp,
                   const __grid_constant__ CUtensorMap tmKV, const Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) atomicExch(p.status, XL_ERR_BOUNDS);
    return;
  }
  uint8_t* sQ = smem;                                  // 9 slabs [128 rows][64 columns]
  uint8_t* sRing = sQ + NCH * Q_SLAB;
  uint8_t* sP = sRing + kSlots * CHUNK;
  Barriers* bars = reinterpret_cast<Barriers*>(sP + P_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = int(blockIdx.x) >> 1, half = int(blockIdx.x) & 1;
  TileInfo ti;
  if (!find_tile(p, tile, ti)) return;
  if (int(blockIdx.z) >= ti.n_eff) return;
  const int per_split = (ti.n_tiles_all + ti.n_eff - 1) / ti.n_eff;
  const int j_first = int(blockIdx.z) * per_split;
  const int n_tiles = max(0, min(ti.n_tiles_all, j_first + per_split) - j_first);
  const int kv_begin = j_first * BKV;
  const int* bt = p.block_tables + size_t(ti.seq) * p.max_blocks;
  const int tpt = p.tpt;
  const int pos_base = ti.kv_len - ti.q_len + ti.qt0;        // position of the tile's first token

  if (n_tiles > 0) {
    if (threadIdx.x == 0) {
      mbar_init(&bars->q_full, 1);
      for (int s = 0; s < kSlots; ++s) {
        mbar_init(&bars->full[s], 1);
        mbar_init(&bars->empty[s], 1);
      }
      mbar_init(&bars->s_full, 1);
      mbar_init(&bars->s_free, 4);
      mbar_init(&bars->p_full, 4);
      mbar_init(&bars->pv_done, 1);
      mbar_fence_init();
    }
    if (warp == 1) {
      tmem_alloc(&bars->tmem_base, kTmemCols);
      tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_base;
    const uint32_t t_o_base = tmem_base, t_s_base = tmem_base + HALF;

    if (warp == 0) {
      // ---------------------------------------------------------- TMA producer
      if (lane == 0) {
        prefetch_tmap(&tmQl);
        prefetch_tmap(&tmQp);
        prefetch_tmap(&tmKV);
        mbar_arrive_expect_tx(&bars->q_full, NCH * Q_SLAB);
        for (int c = 0; c < C / 64; ++c) tma_load_3d(sQ + c * Q_SLAB, &tmQl, &bars->q_full, c * 64, ti.q_start + ti.qt0, 0);
        tma_load_3d(sQ + (NCH - 1) * Q_SLAB, &tmQp, &bars->q_full, 0, ti.q_start + ti.qt0, 0);
      }
      const int boxes = BKV / p.box_tokens;            // 1, 2 or 4 boxes per chunk
      auto slot_of = [&](int j) -> int {               // cache slot of this lane's box of key tile j
        const int tok = kv_begin + j * BKV + (lane % boxes) * p.box_tokens;
        int bi = tok / p.block_size;
        bi = bi < p.max_blocks ? bi : p.max_blocks - 1;
        long slot = long(bt[bi]) * p.block_size + tok % p.block_size;
        if (slot < 0 || slot + p.box_tokens > p.num_slots) slot = 0;
        return int(slot);
      };
      uint32_t n = 0;                                  // FIFO position
      bool ok = true;
      auto push = [&](int chunk, int slot) {
        const int st = int(n % kSlots);
        const uint32_t ph = (n / kSlots) & 1;
        if (lane == 0) {
          if (!mbar_wait(&bars->empty[st], ph ^ 1)) {
            atomicExch(p.status, XL_ERR_WAIT_EMPTY);
            ok = false;
          } else {
            mbar_arrive_expect_tx(&bars->full[st], CHUNK);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (ok && lane < boxes)
          tma_load_2d(sRing + st * CHUNK + lane * p.box_tokens * 128, &tmKV, &bars->full[st], chunk * 64, slot);
        __syncwarp();
        ++n;
      };
      int slot_prev = 0;
      for (int s = 0; s <= n_tiles && ok; ++s) {
        int slot_cur = 0;
        if (s < n_tiles) {
          slot_cur = slot_of(s);
          for (int i = 0; i < NCH && ok; ++i) push(qk_chunk(half, i), slot_cur);
        }
        if (s >= 1)
          for (int cc = 0; cc < VCH && ok; ++cc) push(half * VCH + cc, slot_prev);
        slot_prev = slot_cur;
      }
    } else if (warp == 1) {
      // ---------------------------------------------------------- MMA issuer
      if (elect_one_sync()) {
        const uint32_t idesc_s = umma_idesc_f16(BQ, BKV, 1);
        const uint32_t idesc_o = umma_idesc_f16(BQ, 64, 1) | (1u << 16);      // B operand (V) is MN-major
        const uint32_t idesc_o256 = umma_idesc_f16(BQ, HALF, 1) | (1u << 16);
        const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP), ring = smem_u32(sRing);
        bool ok = mbar_wait(&bars->q_full, 0);
        if (!ok) atomicExch(p.status, XL_ERR_WAIT_FULL);
        uint32_t n = 0;
        auto wait_item = [&]() -> bool {
          if (!mbar_wait(&bars->full[n % kSlots], (n / kSlots) & 1)) {
            atomicExch(p.status, XL_ERR_WAIT_FULL);
            return false;
          }
          tc_fence_after();
          return true;
        };
        const bool tr = p.trace && blockIdx.x == 0 && blockIdx.z == 0;
        for (int s = 0; s <= n_tiles && ok; ++s) {
          if (s < n_tiles) {
            if (tr && s < 64) p.trace[s * 16 + 0] = clock64();
            if (!mbar_wait(&bars->s_free, (s & 1) ^ 1)) {
              atomicExch(p.status, XL_ERR_WAIT_TMEM_EMPTY);
              ok = false;
              break;
            }
            tc_fence_after();
            if (tr && s < 64) p.trace[s * 16 + 1] = clock64();
            for (int i = 0; i < NCH && ok; ++i) {
              ok = wait_item();
              if (!ok) break;
              const uint32_t k_addr = ring + (n % kSlots) * CHUNK;
              const uint32_t qa = q_addr + qk_chunk(half, i) * Q_SLAB;
#pragma unroll
              for (int k = 0; k < kSParts; ++k)           // the four 16-column steps of a chunk: one per partial accumulator
                tc_mma_f16(t_s_base + k * 64, umma_desc_sw128(qa, k * 32), umma_desc_sw128(k_addr, k * 32), idesc_s, i != 0);
              tc_commit(&bars->empty[n % kSlots]);
              ++n;
            }
            if (!ok) break;
            tc_commit(&bars->s_full);
            if (tr && s < 64) p.trace[s * 16 + 2] = clock64();
          }
          if (s >= 1) {
            const int j = s - 1;
            if (!mbar_wait(&bars->p_full, j & 1)) {
              atomicExch(p.status, XL_ERR_WAIT_TMEM_FULL);
              ok = false;
              break;
            }
            tc_fence_after();
            if (tr && j < 64) p.trace[j * 16 + 3] = clock64();
            // the four value chunks feed four different column blocks of O: issued key step by key step, so that
            // consecutive products do not wait for each other
            uint32_t v_addr[VCH];
            for (int cc = 0; cc < VCH && ok; ++cc) {
              ok = wait_item();
              v_addr[cc] = ring + (n % kSlots) * CHUNK;
              ++n;
            }
            if (!ok) break;
            if (v_addr[VCH - 1] == v_addr[0] + (VCH - 1) * CHUNK) {
              // the four chunks sit side by side in the ring: one 256-wide product per 16 keys (a product costs about the
              // same whatever its width)
#pragma unroll
              for (int k = 0; k < BKV / 16; ++k)
                tc_mma_f16(t_o_base, umma_desc_sw128(p_addr, k * 32), umma_desc_sw128_mn(v_addr[0] + k * 2048, CHUNK, 1024), idesc_o256,
                           (j | k) != 0);
            } else {
#pragma unroll
              for (int k = 0; k < BKV / 16; ++k)
#pragma unroll
                for (int cc = 0; cc < VCH; ++cc)
                  tc_mma_f16(t_o_base + cc * 64, umma_desc_sw128(p_addr, k * 32), umma_desc_sw128_mn(v_addr[cc] + k * 2048, CHUNK, 1024),
                             idesc_o, (j | k) != 0);
            }
            for (int cc = 0; cc < VCH; ++cc) tc_commit(&bars->empty[(n - VCH + cc) % kSlots]);
            tc_commit(&bars->pv_done);
            if (tr && j < 64) p.trace[j * 16 + 4] = clock64();
          }
        }
      }
    } else {
      // ---------------------------------------------------------- softmax / correction / epilogue: one row per thread
      const int q = warp & 3;                                  // TMEM lane quarter of this warp
      const int r = q * 32 + lane;                             // row of the tile: head r / tpt, token r % tpt
      const int tok = ti.qt0 + r % tpt;
      const int head = r / tpt;
      const bool row_ok = tok < ti.q_len;
      const uint32_t lane_off = uint32_t(q * 32) << 16;
      const uint32_t t_s = t_s_base + lane_off, t_o = t_o_base + lane_off;
      uint8_t* prow = sP + r * 128;
      const int hi = min(pos_base + r % tpt, ti.kv_len - 1);   // last visible key of this row
      const float sc = p.scale_log2;
      float m_ref = -INFINITY, l_run = 0.f;
      bool ok = true;
      const bool tr = p.trace && blockIdx.x == 0 && blockIdx.z == 0 && threadIdx.x == 64;
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (tr && j < 64) p.trace[j * 16 + 8] = clock64();
        if (!__all_sync(0xffffffffu, mbar_wait(&bars->s_full, j & 1))) {
          if (lane == 0) atomicExch(p.status, XL_ERR_WAIT_TMEM_FULL);
          ok = false;
          break;
        }
        tc_fence_after();
        if (tr && j < 64) p.trace[j * 16 + 9] = clock64();
        float v[64];
#pragma unroll
        for (int hcol = 0; hcol < 64; hcol += 32) {          // S = sum of the four partial accumulators
          uint32_t a0[32], a1[32];
          tmem_ld_32x32(t_s + hcol, a0);
          tmem_ld_32x32(t_s + 64 + hcol, a1);
          tc_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) v[hcol + c] = __uint_as_float(a0[c]) + __uint_as_float(a1[c]);
          tmem_ld_32x32(t_s + 128 + hcol, a0);
          tmem_ld_32x32(t_s + 192 + hcol, a1);
          tc_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) v[hcol + c] += __uint_as_float(a0[c]) + __uint_as_float(a1[c]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->s_free);
        if (tr && j < 64) p.trace[j * 16 + 10] = clock64();
        const int kv0 = kv_begin + j * BKV;
        if (kv0 + BKV - 1 > hi) {
#pragma unroll
          for (int c = 0; c < 64; ++c)
            if (kv0 + c > hi) v[c] = -INFINITY;
        }
        float mx8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) mx8[i] = v[i];
#pragma unroll
        for (int c = 8; c < 64; ++c) mx8[c & 7] = fmaxf(mx8[c & 7], v[c]);
        const float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])), fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
        // the stale reference maximum is kept unless the scaled maximum grew by more than 8 (P stays below 2^8), which
        // is exact after the final division by the row sum
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
        if (tr && j < 64) { p.trace[j * 16 + 11] = clock64(); p.trace[j * 16 + 14] = rescale; }
        // P and O are touched only after P V of the previous tile has finished
        if (j > 0 && !__all_sync(0xffffffffu, mbar_wait(&bars->pv_done, (j - 1) & 1))) {
          if (lane == 0) atomicExch(p.status, XL_ERR_WAIT_TMEM_EMPTY);
          ok = false;
          break;
        }
        tc_fence_after();
        if (tr && j < 64) p.trace[j * 16 + 12] = clock64();
        if (j > 0 && __any_sync(0xffffffffu, rescale)) {
#pragma unroll 1
          for (int c = 0; c < HALF; c += 32) {
            uint32_t o[32];
            tmem_ld_32x32(t_o + c, o);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(t_o + c, o);
          }
          tc_wait_st();
        }
#pragma unroll
        for (int c = 0; c < 8; ++c)
          *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
        fence_proxy_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_full);
        if (tr && j < 64) p.trace[j * 16 + 13] = clock64();
      }
      if (ok && !__all_sync(0xffffffffu, mbar_wait(&bars->pv_done, (n_tiles - 1) & 1))) {
        if (lane == 0) atomicExch(p.status, XL_ERR_WAIT_TMEM_EMPTY);
        ok = false;
      }
      if (ok && ti.n_eff > 1) {
        // partial of this key range: O relative to m_ref, with m_ref and the row sum beside it
        tc_fence_after();
        float4* wo = reinterpret_cast<float4*>(p.ws_o) + ((size_t(tile) * 2 + half) * p.splits + blockIdx.z) * (HALF / 4) * BQ;
#pragma unroll 1
        for (int c = 0; c < HALF; c += 32) {
          uint32_t o[32];
          tmem_ld_32x32(t_o + c, o);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 8; ++i)
            wo[size_t(c / 4 + i) * BQ + r] = make_float4(__uint_as_float(o[4 * i]), __uint_as_float(o[4 * i + 1]),
                                                         __uint_as_float(o[4 * i + 2]), __uint_as_float(o[4 * i + 3]));
        }
        if (half == 0)
          p.ws_ml[(size_t(tile) * p.splits + blockIdx.z) * BQ + r] = make_float2(m_ref == -INFINITY ? -INFINITY : m_ref * sc, l_run);
      } else if (ok) {
        tc_fence_after();
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        __nv_bfloat16* dst = p.out + (size_t(head) * p.T + ti.q_start + tok) * C + half * HALF;
#pragma unroll 1
        for (int c = 0; c < HALF; c += 32) {
          uint32_t o[32];
          tmem_ld_32x32(t_o + c, o);
          tc_wait_ld();
          if (row_ok) {
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
  } else if (ti.n_eff == 1 && warp >= 2) {
    // no visible key at all (empty sequence): zero rows
    const int r = (warp & 3) * 32 + lane;
    const int tok = ti.qt0 + r % tpt;
    if (tok < ti.q_len) {
      uint4* dst = reinterpret_cast<uint4*>(p.out + (size_t(r / tpt) * p.T + ti.q_start + tok) * C + half * HALF);
      for (int i = 0; i < HALF / 8; ++i) dst[i] = make_uint4(0, 0, 0, 0);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Pair kernel: the two CTAs of a tile run as a cluster and split the 576-deep Q K^T between them as well.  CTA 0 owns the
// latent columns 0..255 (Q slabs and cache chunks 0..3), CTA 1 the columns 256..511 and the rope columns (chunks 8, 4..7).
// Each computes the partial S of its columns, hands it to the peer through distributed shared memory and adds the one it
// receives (a + b in both CTAs: the same bits), so both hold S, run the same softmax and keep their own P; P V then uses
// the chunks the CTA already holds.  Per key tile a pair loads the nine chunks once (the single-CTA kernel above: 26
// chunk loads), Q takes 64 / 80 KB instead of 144 KB, and the chunk FIFO has 12 slots.
constexpr int kPairSlots = 12;
constexpr int kPairQSlabs = 5;
constexpr int X_BYTES = BQ * BKV * 4;      // one partial S tile, fp32, stored [16 column quads][128 rows] x 16 bytes

struct PairBarriers {
  uint64_t q_full;
  uint64_t full[kPairSlots];
  uint64_t empty[kPairSlots];
  uint64_t s_full;
  uint64_t s_free;
  uint64_t x_full;        // the peer's partial S has landed in this CTA's exchange buffer (one remote arrival per row)
  uint64_t x_free;        // the peer has read the partial S this CTA sent it (one remote arrival per row)
  uint64_t p_full;
  uint64_t pv_done;
  uint32_t tmem_base;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void st_cluster_v4(uint32_t cluster_addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void fence_cluster() { asm volatile("fence.acq_rel.cluster;" ::: "memory"); }
// Bounded wait whose success makes the peer CTA's writes (ordered before its arrival) visible here.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < (1u << 22); ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, P;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
    if (i > 4096) __nanosleep(128);
  }
  return false;
}

__global__ void __launch_bounds__(kThreads, 1)
mla_attn_pair_kernel(const __grid_constant__ CUtensorMap tmQl, const __grid_constant__ CUtensorMap tmQp,
                     const __grid_constant__ CUtensorMap tmKV, const Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {                     // same answer in both CTAs of the cluster
    if (threadIdx.x == 0) atomicExch(p.status, XL_ERR_BOUNDS);
    return;
  }
  uint8_t* sQ = smem;                                  // 5 slabs [128 rows][64 columns] (CTA 0 uses 4)
  uint8_t* sRing = sQ + kPairQSlabs * Q_SLAB;
  uint8_t* sP = sRing + kPairSlots * CHUNK;
  float4* sX = reinterpret_cast<float4*>(sP + P_BYTES);
  PairBarriers* bars = reinterpret_cast<PairBarriers*>(reinterpret_cast<uint8_t*>(sX) + X_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = int(blockIdx.x) >> 1;
  const int half = int(cluster_ctarank());             // 0: latent 0..255; 1: latent 256..511 + rope
  const uint32_t peer = uint32_t(half ^ 1);
  const int n_per = half == 0 ? VCH : VCH + 1;         // chunks (and Q slabs) of this CTA per key tile
  // FIFO item i of a key tile: column chunk of the cache row, and whether P V reads it too
  auto chunk_of = [&](int i) { return half == 0 ? i : (i == 0 ? NCH - 1 : VCH - 1 + i); };
  auto is_value = [&](int i) { return half == 0 || i > 0; };
  TileInfo ti;
  if (!find_tile(p, tile, ti)) return;
  if (int(blockIdx.z) >= ti.n_eff) return;
  const int per_split = (ti.n_tiles_all + ti.n_eff - 1) / ti.n_eff;
  const int j_first = int(blockIdx.z) * per_split;
  const int n_tiles = max(0, min(ti.n_tiles_all, j_first + per_split) - j_first);
  const int kv_begin = j_first * BKV;
  const int* bt = p.block_tables + size_t(ti.seq) * p.max_blocks;
  const int tpt = p.tpt;
  const int pos_base = ti.kv_len - ti.q_len + ti.qt0;

  if (n_tiles > 0) {
    if (threadIdx.x == 0) {
      mbar_init(&bars->q_full, 1);
      for (int s = 0; s < kPairSlots; ++s) {
        mbar_init(&bars->full[s], 1);
        mbar_init(&bars->empty[s], 1);
      }
      mbar_init(&bars->s_full, 1);
      mbar_init(&bars->s_free, 4);
      mbar_init(&bars->x_full, BQ);
      mbar_init(&bars->x_free, BQ);
      mbar_init(&bars->p_full, 4);
      mbar_init(&bars->pv_done, 1);
      mbar_fence_init();
    }
    if (warp == 1) {
      tmem_alloc(&bars->tmem_base, kTmemCols);
      tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();            // the peer's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_base;
    const uint32_t t_o_base = tmem_base, t_s_base = tmem_base + HALF;

    if (warp == 0) {
      // ---------------------------------------------------------- TMA producer
      if (lane == 0) {
        prefetch_tmap(&tmQl);
        prefetch_tmap(&tmQp);
        prefetch_tmap(&tmKV);
        mbar_arrive_expect_tx(&bars->q_full, n_per * Q_SLAB);
        for (int i = 0; i < n_per; ++i) {
          const int c = chunk_of(i);
          if (c == NCH - 1) tma_load_3d(sQ + i * Q_SLAB, &tmQp, &bars->q_full, 0, ti.q_start + ti.qt0, 0);
          else tma_load_3d(sQ + i * Q_SLAB, &tmQl, &bars->q_full, c * 64, ti.q_start + ti.qt0, 0);
        }
      }
      const int boxes = BKV / p.box_tokens;
      uint32_t n = 0;
      bool ok = true;
      for (int t = 0; t < n_tiles && ok; ++t) {
        const int tok = kv_begin + t * BKV + (lane % boxes) * p.box_tokens;
        int bi = tok / p.block_size;
        bi = bi < p.max_blocks ? bi : p.max_blocks - 1;
        long slot = long(bt[bi]) * p.block_size + tok % p.block_size;
        if (slot < 0 || slot + p.box_tokens > p.num_slots) slot = 0;
        for (int i = 0; i < n_per && ok; ++i) {
          const int st = int(n % kPairSlots);
          const uint32_t ph = (n / kPairSlots) & 1;
          if (lane == 0) {
            if (!mbar_wait(&bars->empty[st], ph ^ 1)) {
              atomicExch(p.status, XL_ERR_WAIT_EMPTY);
              ok = false;
            } else {
              mbar_arrive_expect_tx(&bars->full[st], CHUNK);
            }
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (ok && lane < boxes)
            tma_load_2d(sRing + st * CHUNK + lane * p.box_tokens * 128, &tmKV, &bars->full[st], chunk_of(i) * 64, int(slot));
          __syncwarp();
          ++n;
        }
      }
    } else if (warp == 1) {
      // ---------------------------------------------------------- MMA issuer
      if (elect_one_sync()) {
        const uint32_t idesc_s = umma_idesc_f16(BQ, BKV, 1);
        const uint32_t idesc_o64 = umma_idesc_f16(BQ, 64, 1) | (1u << 16);       // B operand (V) is MN-major
        const uint32_t idesc_o256 = umma_idesc_f16(BQ, HALF, 1) | (1u << 16);
        const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP), ring = smem_u32(sRing);
        bool ok = mbar_wait(&bars->q_full, 0);
        if (!ok) atomicExch(p.status, XL_ERR_WAIT_FULL);
        for (int s = 0; s <= n_tiles && ok; ++s) {
          if (s < n_tiles) {
            if (!mbar_wait(&bars->s_free, (s & 1) ^ 1)) {
              atomicExch(p.status, XL_ERR_WAIT_TMEM_EMPTY);
              ok = false;
              break;
            }
            tc_fence_after();
            for (int i = 0; i < n_per; ++i) {
              const uint32_t n = uint32_t(s) * n_per + i;
              const uint32_t st = n % kPairSlots;
              if (!mbar_wait(&bars->full[st], (n / kPairSlots) & 1)) {
                atomicExch(p.status, XL_ERR_WAIT_FULL);
                ok = false;
                break;
              }
              tc_fence_after();
              const uint32_t k_addr = ring + st * CHUNK, qa = q_addr + i * Q_SLAB;
#pragma unroll
              for (int k = 0; k < kSParts; ++k)
                tc_mma_f16(t_s_base + k * 64, umma_desc_sw128(qa, k * 32), umma_desc_sw128(k_addr, k * 32), idesc_s, i != 0);
              if (!is_value(i)) tc_commit(&bars->empty[st]);        // the value chunks stay until P V has read them
            }
            if (!ok) break;
            tc_commit(&bars->s_full);
          }
          if (s >= 1) {
            const int j = s - 1;
            if (!mbar_wait(&bars->p_full, j & 1)) {
              atomicExch(p.status, XL_ERR_WAIT_TMEM_FULL);
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t n0 = uint32_t(j) * n_per + (n_per - VCH);      // FIFO position of the tile's first value chunk
            const uint32_t st0 = n0 % kPairSlots;
            if (st0 + VCH <= kPairSlots) {
              // the four chunks sit side by side: one 256-wide product per 16 keys
#pragma unroll
              for (int k = 0; k < BKV / 16; ++k)
                tc_mma_f16(t_o_base, umma_desc_sw128(p_addr, k * 32), umma_desc_sw128_mn(ring + st0 * CHUNK + k * 2048, CHUNK, 1024),
                           idesc_o256, (j | k) != 0);
            } else {
#pragma unroll
              for (int k = 0; k < BKV / 16; ++k)
                for (int cc = 0; cc < VCH; ++cc)
                  tc_mma_f16(t_o_base + cc * 64, umma_desc_sw128(p_addr, k * 32),
                             umma_desc_sw128_mn(ring + ((n0 + cc) % kPairSlots) * CHUNK + k * 2048, CHUNK, 1024), idesc_o64, (j | k) != 0);
            }
            for (int cc = 0; cc < VCH; ++cc) tc_commit(&bars->empty[(n0 + cc) % kPairSlots]);
            tc_commit(&bars->pv_done);
          }
        }
      }
    } else {
      // ---------------------------------------------------------- softmax / exchange / correction / epilogue
      const int q = warp & 3;
      const int r = q * 32 + lane;
      const int tok = ti.qt0 + r % tpt;
      const int head = r / tpt;
      const bool row_ok = tok < ti.q_len;
      const uint32_t lane_off = uint32_t(q * 32) << 16;
      const uint32_t t_s = t_s_base + lane_off, t_o = t_o_base + lane_off;
      uint8_t* prow = sP + r * 128;
      const uint32_t peer_x = map_to_cta(smem_u32(sX), peer);
      const uint32_t peer_x_full = map_to_cta(smem_u32(&bars->x_full), peer);
      const uint32_t peer_x_free = map_to_cta(smem_u32(&bars->x_free), peer);
      const int hi = min(pos_base + r % tpt, ti.kv_len - 1);
      const float sc = p.scale_log2;
      float m_ref = -INFINITY, l_run = 0.f;
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (!__all_sync(0xffffffffu, mbar_wait(&bars->s_full, j & 1))) {
          if (lane == 0) atomicExch(p.status, XL_ERR_WAIT_TMEM_FULL);
          ok = false;
          break;
        }
        tc_fence_after();
        float v[64];
#pragma unroll
        for (int hcol = 0; hcol < 64; hcol += 32) {          // S = sum of the four partial accumulators
          uint32_t a0[32], a1[32];
          tmem_ld_32x32(t_s + hcol, a0);
          tmem_ld_32x32(t_s + 64 + hcol, a1);
          tc_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) v[hcol + c] = __uint_as_float(a0[c]) + __uint_as_float(a1[c]);
          tmem_ld_32x32(t_s + 128 + hcol, a0);
          tmem_ld_32x32(t_s + 192 + hcol, a1);
          tc_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) v[hcol + c] += __uint_as_float(a0[c]) + __uint_as_float(a1[c]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->s_free);
        // ---- this CTA's partial goes to the peer (once the peer has read the previous one) ...
        if (j > 0 && !__all_sync(0xffffffffu, mbar_wait_cluster(&bars->x_free, (j - 1) & 1))) {
          if (lane == 0) atomicExch(p.status, XL_ERR_WAIT_PEER);
          ok = false;
          break;
        }
#pragma unroll
        for (int c4 = 0; c4 < 16; ++c4)
          st_cluster_v4(peer_x + uint32_t(c4 * BQ + r) * 16, v[4 * c4], v[4 * c4 + 1], v[4 * c4 + 2], v[4 * c4 + 3]);
        mbar_arrive_cluster(peer_x_full);          // every row releases its own stores (a cluster-wide fence costs far more)
        // ---- ... and the peer's partial is added to it
        if (!__all_sync(0xffffffffu, mbar_wait_cluster(&bars->x_full, j & 1))) {
          if (lane == 0) atomicExch(p.status, XL_ERR_WAIT_PEER);
          ok = false;
          break;
        }
#pragma unroll
        for (int c4 = 0; c4 < 16; ++c4) {
          const float4 x = sX[c4 * BQ + r];
          v[4 * c4] += x.x; v[4 * c4 + 1] += x.y; v[4 * c4 + 2] += x.z; v[4 * c4 + 3] += x.w;
        }
        mbar_arrive_cluster(peer_x_free);
        const int kv0 = kv_begin + j * BKV;
        if (kv0 + BKV - 1 > hi) {
#pragma unroll
          for (int c = 0; c < 64; ++c)
            if (kv0 + c > hi) v[c] = -INFINITY;
        }
        float mx8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) mx8[i] = v[i];
#pragma unroll
        for (int c = 8; c < 64; ++c) mx8[c & 7] = fmaxf(mx8[c & 7], v[c]);
        const float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])), fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
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
        if (j > 0 && !__all_sync(0xffffffffu, mbar_wait(&bars->pv_done, (j - 1) & 1))) {
          if (lane == 0) atomicExch(p.status, XL_ERR_WAIT_TMEM_EMPTY);
          ok = false;
          break;
        }
        tc_fence_after();
        if (j > 0 && __any_sync(0xffffffffu, rescale)) {
#pragma unroll 1
          for (int c = 0; c < HALF; c += 32) {
            uint32_t o[32];
            tmem_ld_32x32(t_o + c, o);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(t_o + c, o);
          }
          tc_wait_st();
        }
#pragma unroll
        for (int c = 0; c < 8; ++c)
          *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
        fence_proxy_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_full);
      }
      if (ok && !__all_sync(0xffffffffu, mbar_wait(&bars->pv_done, (n_tiles - 1) & 1))) {
        if (lane == 0) atomicExch(p.status, XL_ERR_WAIT_TMEM_EMPTY);
        ok = false;
      }
      if (ok && ti.n_eff > 1) {
        tc_fence_after();
        float4* wo = reinterpret_cast<float4*>(p.ws_o) + ((size_t(tile) * 2 + half) * p.splits + blockIdx.z) * (HALF / 4) * BQ;
#pragma unroll 1
        for (int c = 0; c < HALF; c += 32) {
          uint32_t o[32];
          tmem_ld_32x32(t_o + c, o);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 8; ++i)
            wo[size_t(c / 4 + i) * BQ + r] = make_float4(__uint_as_float(o[4 * i]), __uint_as_float(o[4 * i + 1]),
                                                         __uint_as_float(o[4 * i + 2]), __uint_as_float(o[4 * i + 3]));
        }
        if (half == 0)
          p.ws_ml[(size_t(tile) * p.splits + blockIdx.z) * BQ + r] = make_float2(m_ref == -INFINITY ? -INFINITY : m_ref * sc, l_run);
      } else if (ok) {
        tc_fence_after();
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        __nv_bfloat16* dst = p.out + (size_t(head) * p.T + ti.q_start + tok) * C + half * HALF;
#pragma unroll 1
        for (int c = 0; c < HALF; c += 32) {
          uint32_t o[32];
          tmem_ld_32x32(t_o + c, o);
          tc_wait_ld();
          if (row_ok) {
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
    cluster_sync_all();            // no store or arrival of the peer is still on its way into this CTA's shared memory
    if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
  } else if (ti.n_eff == 1 && warp >= 2) {
    const int r = (warp & 3) * 32 + lane;
    const int tok = ti.qt0 + r % tpt;
    if (tok < ti.q_len) {
      uint4* dst = reinterpret_cast<uint4*>(p.out + (size_t(r / tpt) * p.T + ti.q_start + tok) * C + half * HALF);
      for (int i = 0; i < HALF / 8; ++i) dst[i] = make_uint4(0, 0, 0, 0);
    }
  }
}

// Merge of the key splits: grid (tile, half), one row per thread.
__global__ void __launch_bounds__(BQ) mla_merge_kernel(const Params p) {
  const int tile = blockIdx.x, half = blockIdx.y;
  TileInfo ti;
  if (!find_tile(p, tile, ti) || ti.n_eff <= 1) return;
  const int r = threadIdx.x;
  const int tok = ti.qt0 + r % p.tpt;
  if (tok >= ti.q_len) return;
  const int per_split = (ti.n_tiles_all + ti.n_eff - 1) / ti.n_eff;
  const int n_valid = (ti.n_tiles_all + per_split - 1) / per_split;      // splits that had keys to look at
  const float2* ml = p.ws_ml + size_t(tile) * p.splits * BQ + r;
  float w[kMaxSplits];
  float m_all = -INFINITY;
  for (int s = 0; s < n_valid; ++s) m_all = fmaxf(m_all, ml[size_t(s) * BQ].x);
  float l_all = 0.f;
  for (int s = 0; s < n_valid; ++s) {
    const float2 v = ml[size_t(s) * BQ];
    w[s] = (v.x == -INFINITY) ? 0.f : exp2f(v.x - m_all);
    l_all += w[s] * v.y;
  }
  const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
  const float4* wo = reinterpret_cast<const float4*>(p.ws_o) + (size_t(tile) * 2 + half) * p.splits * (HALF / 4) * BQ + r;
  __nv_bfloat16* dst = p.out + (size_t(r / p.tpt) * p.T + ti.q_start + tok) * C + half * HALF;
  for (int c4 = 0; c4 < HALF / 4; c4 += 2) {
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
    for (int s = 0; s < n_valid; ++s) {
      const float4 x = wo[(size_t(s) * (HALF / 4) + c4) * BQ], y = wo[(size_t(s) * (HALF / 4) + c4 + 1) * BQ];
      a.x += w[s] * x.x; a.y += w[s] * x.y; a.z += w[s] * x.z; a.w += w[s] * x.w;
      b.x += w[s] * y.x; b.y += w[s] * y.y; b.z += w[s] * y.z; b.w += w[s] * y.w;
    }
    *reinterpret_cast<uint4*>(dst + c4 * 4) = make_uint4(pack_bf16x2(a.x * inv, a.y * inv), pack_bf16x2(a.z * inv, a.w * inv),
                                                         pack_bf16x2(b.x * inv, b.y * inv), pack_bf16x2(b.z * inv, b.w * inv));
  }
}

constexpr size_t kWsBytes = size_t(96) << 20;
static int g_kv_split = 1;     // 0: never split, 1: automatic, >1: forced number of splits (tests)
static long long* g_trace = nullptr;
static int g_pair = 0;         // 1: the two CTAs of a tile as a cluster that shares the Q K^T work; 0: independent CTAs (measured faster)
static uint8_t* workspace(cudaStream_t stream) {
  static uint8_t* ws[64] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  if (!ws[dev]) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &st) != cudaSuccess || st != cudaStreamCaptureStatusNone) return nullptr;
    void* q = nullptr;
    if (cudaMalloc(&q, kWsBytes) != cudaSuccess) return nullptr;
    ws[dev] = static_cast<uint8_t*>(q);
  }
  return ws[dev];
}

}  // namespace xl_mla_tc

// 0: no key split, 1: automatic (default), 2..16: that many splits whenever the workspace allows (tests, measurements).
XL_API void xl_mla_kv_split(int mode) { xl_mla_tc::g_kv_split = mode < 0 ? 1 : (mode > 16 ? 16 : mode); }

// 0 (default): the two CTAs of a tile work independently; 1: cluster-pair kernel (fewer cache loads, but measured 13 %
// slower on B200: 398 against 347 us for 256 sequences x 1152 keys).
XL_API void xl_mla_pair_mode(int on) { xl_mla_tc::g_pair = on ? 1 : 0; }
// Diagnosis hook: device buffer of 64 x 16 int64 that receives clock stamps of CTA 0 of the next launches of the
// independent kernel, per key tile: [0..4] MMA warp (step start, S free seen, Q K^T issued, P seen, P V issued),
// [8..13] one softmax thread (start, S seen, S read, exponentials done, previous P V seen, P written), [14] rescale flag.
XL_API void xl_mla_set_trace(void* buf) { xl_mla_tc::g_trace = static_cast<long long*>(buf); }

// MLA attention of sequences [seq_begin, seq_end) with the tcgen05 kernel.  q_lat_hm [Hh, T, 512], q_pe_hm [Hh, T, 64] and
// out_hm [Hh, T, 512] head-major, cache [slots, 576].  `max_tiles` >= sum over sequences of ceil(q_len / (128 / Hh)).
// Returns -3 when the shape is not covered (the caller then uses the mma.sync kernel).
XL_API int xl_mla_attention_tc(const void* q_lat_hm, const void* q_pe_hm, const void* cache, void* out_hm, const void* q_cu,
                               const void* kv_lens, const void* block_tables, int seq_begin, int seq_end, int max_blocks,
                               int block_size, long cache_slots, int Hh, int T, int kv_lora, int rope, float scale,
                               int max_tiles, void* stream) {
  using namespace xl_mla_tc;
  if (seq_end <= seq_begin || max_tiles <= 0 || T <= 0) return 0;
  if (!(kv_lora == C && rope == R) || Hh < 1 || Hh > BQ || (BQ % Hh) != 0) return -3;
  if (block_size % 16 != 0 || (block_size > 64 && block_size % 64 != 0) || (block_size < 64 && 64 % block_size != 0)) return -3;
  if ((reinterpret_cast<uintptr_t>(q_lat_hm) & 15) || (reinterpret_cast<uintptr_t>(q_pe_hm) & 15) ||
      (reinterpret_cast<uintptr_t>(cache) & 127) || (reinterpret_cast<uintptr_t>(out_hm) & 15))
    return -3;
  const int tpt = BQ / Hh;
  const int box_tokens = block_size < 64 ? block_size : 64;
  const CUtensorMap* tql = xl_host::tmap_3d(q_lat_hm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Hh, T, C, Hh, tpt, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  const CUtensorMap* tqp = xl_host::tmap_3d(q_pe_hm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Hh, T, R, Hh, tpt, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  const CUtensorMap* tkv = xl_host::tmap_2d(cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, uint64_t(cache_slots), C + R, C + R, box_tokens, 64,
                                            CU_TENSOR_MAP_SWIZZLE_128B);
  if (!tql || !tqp || !tkv) return -3;
  Params p;
  memset(&p, 0, sizeof(p));
  p.out = static_cast<__nv_bfloat16*>(out_hm);
  p.q_cu = static_cast<const int*>(q_cu);
  p.kv_lens = static_cast<const int*>(kv_lens);
  p.block_tables = static_cast<const int*>(block_tables);
  p.seq_begin = seq_begin; p.seq_end = seq_end; p.max_blocks = max_blocks; p.block_size = block_size; p.box_tokens = box_tokens;
  p.Hh = Hh; p.tpt = tpt; p.T = T;
  p.num_slots = cache_slots;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = xl_host::status_word();
  p.trace = g_trace;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // Few tiles (a small decode batch) leave most SMs idle while each CTA walks its whole key range alone: cut the key
  // ranges into splits.  The grid only offers the splits; every tile takes as many as its own key range is worth.
  const int tiles_est = (T + tpt - 1) / tpt;
  const int ctas = 2 * (tiles_est < max_tiles ? tiles_est : max_tiles);
  int splits = 1;
  if (g_kv_split > 1) splits = g_kv_split;
  else if (g_kv_split == 1 && ctas * 2 <= xl_host::sm_count()) splits = xl_host::sm_count() / ctas;
  if (splits > kMaxSplits) splits = kMaxSplits;
  p.splits = 1;
  p.min_tiles = g_kv_split > 1 ? 1 : 4;
  if (splits > 1) {
    uint8_t* w = workspace(st);
    const size_t per_tile = size_t(splits) * (2 * size_t(BQ) * HALF * 4 + size_t(BQ) * 8);
    const size_t tiles = kWsBytes / per_tile;
    if (w && tiles > 0) {
      p.splits = splits;
      p.ws_tiles = int(tiles < size_t(max_tiles) ? tiles : size_t(max_tiles));
      p.ws_o = reinterpret_cast<float*>(w);
      p.ws_ml = reinterpret_cast<float2*>(w + size_t(p.ws_tiles) * 2 * splits * size_t(BQ) * HALF * 4);
    }
  }
  dim3 grid(2 * max_tiles, 1, p.splits);
  if (g_pair) {
    const size_t smem = size_t(kPairQSlabs) * Q_SLAB + size_t(kPairSlots) * CHUNK + P_BYTES + X_BYTES + sizeof(PairBarriers);
    static bool set = false;
    if (!set) {
      if (cudaFuncSetAttribute(mla_attn_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return -3;
      set = true;
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, mla_attn_pair_kernel, *tql, *tqp, *tkv, p) != cudaSuccess) return -1;
  } else {
    const size_t smem = size_t(NCH) * Q_SLAB + size_t(kSlots) * CHUNK + P_BYTES + sizeof(Barriers);
    static bool set = false;
    if (!set) {
      if (cudaFuncSetAttribute(mla_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return -3;
      set = true;
    }
    mla_attn_tc_kernel<<<grid, kThreads, smem, st>>>(*tql, *tqp, *tkv, p);
    if (cudaGetLastError() != cudaSuccess) return -1;
  }
  if (p.splits > 1) {
    mla_merge_kernel<<<dim3(p.ws_tiles, 2), BQ, 0, st>>>(p);
    if (cudaGetLastError() != cudaSuccess) return -1;
  }
  return 0;
}
