// bf16 GEMM with tensor-core pairs:  C[M,N] = A[M,K] * W[N,K]^T, one 256 x BN output tile per pair of CTAs
// (thread-block cluster of 2, `tcgen05.mma.cta_group::2`).
//
// Why pairs: with one CTA per tile every MMA reads its whole 128-row A slice and the whole BN-row W slice from
// shared memory while TMA writes the next stage into the same shared memory, and that traffic, not the tensor
// pipe, bounds the single-CTA kernel (gemm_bf16.cu).  In a pair each CTA stages its own 128 rows of A and only
// HALF of the W tile; the paired MMA reads both halves, so shared-memory traffic per FLOP drops by a third.
//
// Roles per CTA (192 threads), as in the single-CTA kernel:
//   warp 0    : TMA producer.  Loads of both CTAs complete on the LEADER's (cluster rank 0) full barrier; no load
//               carries a cluster broadcast: each CTA fetches exactly the bytes it keeps;
//   warp 1    : allocates / frees TMEM with its peer; in the leader, one elected thread issues the paired MMAs and
//               commits them to the stage barriers of BOTH CTAs and to both epilogues' accumulator barriers;
//   warps 2-5 : epilogue of this CTA's 128 rows (tcgen05.ld, bias / SwiGLU / row push, bf16 stores); the
//               accumulator is double buffered in TMEM, released to the leader through a remote mbarrier arrive.
// With few output tiles and a long K (decode-size batches) the K loop of a tile is split over several pairs (SplitK
// below): all SM pairs stream weights, partial tiles meet in an fp32 workspace and are summed in a fixed order.
// Every wait is bounded; on expiry a status code is recorded and the role leaves its loop.  Both CTAs always reach
// the closing cluster barrier, after which TMEM is freed.
//
// The same kernel serves fp8 (e4m3) operands with per-row activation scales and per-tensor or per-output-channel weight
// scales (template parameter ESIZE = 1): a K block is still 128 bytes per row (128 fp8 values), the MMA is
// `kind::f8f6f4`, the whole K loop accumulates in TMEM and the epilogue multiplies by row scale x column scale.  This is
// the contraction of the reference's sm_100 CUTLASS scaled-mm (xllm/core/kernels/cuda/cutlass_w8a8/c3x/
// scaled_mm_sm100_fp8_dispatch.cuh:148-287), which it uses for w8a8 fp8 linears (layers/common/linear.cpp:134-179).
#include <string.h>

#include "common.cuh"

namespace xl2 {
using namespace xl;

constexpr int kBM = 128;          // rows per CTA (256 per pair)
constexpr int kBK = 64;            // bf16 elements per K block (128 bytes per row; fp8: 128 elements)
constexpr int kUmmaK = 16;         // bf16 elements per MMA (32 bytes; fp8: 32 elements)
constexpr int kMaxStages = 8;
constexpr int kThreads = 192;
constexpr int kOutStageBytes = 4 * 2 * 2048;   // 4 epilogue warps x 2 buffers x (32 rows x 64 bytes)

enum { EPI_NONE = 0, EPI_BIAS = 1, EPI_SWIGLU = 2, EPI_RS_PUSH = 3 };

struct Barriers {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  uint64_t epi_sync;          // split-K: rendez-vous of the four epilogue warps (an mbarrier, so that the wait is bounded)
  int epi_ticket[2];          // split-K: ticket value broadcast to the epilogue warps (alternating slots)
};

// Split-K (few output tiles, long K: decode-size batches): the K loop of one output tile is cut into `splits` ranges that
// different CTA pairs run at the same time (one wave).  Every split stores its fp32 partial tile into its own slab of
// `ws`; after a rendez-vous of the splits each of them sums its share of the tile's columns over all slabs in split order
// (so the result does not depend on timing), applies the epilogue and writes C.  The counters reset themselves.
//
// The same machinery balances the last, partly filled wave of a large problem: output tiles [0, full_tiles) are computed
// whole, `tail_tiles` further tiles are cut into `splits` K ranges each, so that the final round gives every SM pair one
// short unit instead of leaving most pairs idle behind a few whole tiles (80 tiles on 74 pairs: 1 + 1/12 rounds instead
// of 2).  With full_tiles = 0 every tile is split (the decode-size case above).
struct SplitK {
  float* ws;                  // [splits][tail_tiles][2 CTA halves][BN / 4 float4 columns][128 rows] fp32
  int* tickets;               // [tail_tiles * 2][2]: arrivals, finishers (reset by the last finisher)
  int splits;
  int full_tiles, tail_tiles;
};

// fp8 operands: C = (A_q W_q^T) * row[m] * (col ? col[n] : 1) * tensor
struct Scales {
  const float* row;           // [M] activation scale of each row (null: 1)
  const float* col;           // [N] weight scale of each output channel (null: 1)
  float tensor;               // weight scale of the whole tensor
};

struct RsPush {
  __nv_bfloat16* recv[8];
  int* flags[8];
  int* done_counter;
  const int* epoch;
  int tp, rank, shard, shard_cap;
  int local;                // 1: rows stay in this rank's C (peers fetch them); only the completion flags are published
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
// address of `local_smem_addr` in the shared memory of CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load of a pair: the completion bytes are credited to the barrier at cluster address `bar_cluster_addr`
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_mma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_mma_f8_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on the barrier at the same offset in both CTAs of the pair once the MMAs issued so far have completed
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask)
               : "memory");
}

// One 32-column chunk of an output row (fp32 in `v`) -> bias / SwiGLU / row push -> bf16 stores.
template <int EPI>
__device__ __forceinline__ void emit_chunk(float (&v)[32], int row, int n, int width, int M, int N, int ldc,
                                           __nv_bfloat16* __restrict__ C, const __nv_bfloat16* __restrict__ bias,
                                           const RsPush& rs) {
  if (row >= M || n >= N) return;
  if (EPI == EPI_SWIGLU) {
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float g0 = v[2 * j], g1 = v[2 * j + 1], u0 = v[16 + 2 * j], u1 = v[16 + 2 * j + 1];
      o[j] = pack_bf16x2(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1);
    }
    uint4* dst = reinterpret_cast<uint4*>(C + size_t(row) * ldc + (n >> 1));
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
    return;
  }
  if (EPI == EPI_BIAS) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (n + j < N) v[j] += __bfloat162float(__ldg(bias + n + j));
  }
  __nv_bfloat16* dst = C + size_t(row) * ldc + n;
  if (EPI == EPI_RS_PUSH && !rs.local) {
    const int owner = row / rs.shard;
    dst = rs.recv[owner] + (size_t(rs.rank) * rs.shard_cap + (row - owner * rs.shard)) * size_t(ldc) + n;
  }
  if (n + width <= N) {
    uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j * 8 < width)
        d4[j] = make_uint4(pack_bf16x2(v[8 * j], v[8 * j + 1]), pack_bf16x2(v[8 * j + 2], v[8 * j + 3]),
                           pack_bf16x2(v[8 * j + 4], v[8 * j + 5]), pack_bf16x2(v[8 * j + 6], v[8 * j + 7]));
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < width && n + j < N) dst[j] = __float2bfloat16(v[j]);
  }
}

// fp8 operands: the accumulator of row `row`, columns n..n+31, times activation row scale x weight scale
__device__ __forceinline__ void scale_chunk(float (&v)[32], int row, int n, int M, int N, const Scales& sc) {
  const float rsc = (sc.row && row < M ? __ldg(sc.row + row) : 1.f) * sc.tensor;
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] *= rsc * (sc.col && n + j < N ? __ldg(sc.col + n + j) : 1.f);
}

// One whole 32-column chunk of 32 rows (one epilogue warp) -> bias / SwiGLU -> bf16 in shared memory -> one bulk tensor
// store.  `stage` is this warp's buffer for the chunk: rows of 64 bytes (32 bytes with SwiGLU) in the layout of the
// tensor map's swizzle (16-byte pieces XOR-ed with row bits, which also keeps the lanes' writes on distinct banks).
template <int EPI>
__device__ __forceinline__ void store_chunk_tma(float (&v)[32], uint8_t* stage, int lane, int row0, int n, int M, int N,
                                                const CUtensorMap* tmC, const __nv_bfloat16* __restrict__ bias) {
  if (row0 >= M || n >= N) return;                      // warp-uniform
  // the store issued two chunks ago read this buffer: it must be done with it
  if (lane == 0) tma_store_wait_read<1>();
  __syncwarp();
  if (EPI == EPI_SWIGLU) {
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float g0 = v[2 * j], g1 = v[2 * j + 1], u0 = v[16 + 2 * j], u1 = v[16 + 2 * j + 1];
      o[j] = pack_bf16x2(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1);
    }
    const int sw = (lane >> 2) & 1;                     // 32-byte swizzle: piece ^= address bit 7
    *reinterpret_cast<uint4*>(stage + lane * 32 + ((0 ^ sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<uint4*>(stage + lane * 32 + ((1 ^ sw) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
  } else {
    if (EPI == EPI_BIAS) {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (n + j < N) v[j] += __bfloat162float(__ldg(bias + n + j));
    }
    const int sw = (lane >> 1) & 3;                     // 64-byte swizzle: piece ^= address bits 8:7
#pragma unroll
    for (int j = 0; j < 4; ++j)
      *reinterpret_cast<uint4*>(stage + lane * 64 + ((j ^ sw) << 4)) =
          make_uint4(pack_bf16x2(v[8 * j], v[8 * j + 1]), pack_bf16x2(v[8 * j + 2], v[8 * j + 3]),
                     pack_bf16x2(v[8 * j + 4], v[8 * j + 5]), pack_bf16x2(v[8 * j + 6], v[8 * j + 7]));
  }
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
    tma_store_2d(tmC, stage, EPI == EPI_SWIGLU ? (n >> 1) : n, row0);
    tma_store_commit();
  }
}

template <int EPI, int ESIZE>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmC, int tma_out,
                      __nv_bfloat16* __restrict__ C, const __nv_bfloat16* __restrict__ bias, int M, int N, int K, int ldc,
                      int BN, int stages, int* __restrict__ status, const __grid_constant__ RsPush rs,
                      const __grid_constant__ SplitK sk, const __grid_constant__ Scales sc) {
  constexpr int kBKe = 128 / ESIZE;                 // elements per K block
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int a_stage_bytes = kBM * kBK * 2;
  const int b_stage_bytes = (BN / 2) * kBK * 2;     // this CTA's half of the W tile
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + stages * a_stage_bytes;
  // output staging of the epilogue warps: two [32 rows x 64 bytes] boxes each, sent with bulk tensor stores
  uint8_t* smem_out = smem_b + stages * b_stage_bytes;
  Barriers* bars = reinterpret_cast<Barriers*>(smem_out + kOutStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();            // 0 = leader
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int m_tiles = (M + 2 * kBM - 1) / (2 * kBM);
  const int n_tiles = (N + BN - 1) / BN;
  const int mn_tiles = m_tiles * n_tiles;
  const int k_blocks = (K + kBKe - 1) / kBKe;
  const int kb_per_split = (k_blocks + sk.splits - 1) / sk.splits;
  // work units: whole tiles first, then the K ranges of the split tiles (split index outermost: the ranges of one tile
  // run side by side on different pairs)
  const int full_tiles = sk.splits > 1 ? sk.full_tiles : mn_tiles;
  const int tail_tiles = sk.splits > 1 ? sk.tail_tiles : 0;
  // Order of a pair's work: its K range of a split tile first, then its whole tiles.  The rendez-vous and the reduction
  // of the split tiles then run in the epilogue warps while the tensor cores are already busy with the first whole tile,
  // and all ranges of a tile start together at the beginning of the kernel.
  const int split_units = tail_tiles * sk.splits;
  auto work_at = [&](int i) -> int {
    if (pair < split_units) {
      if (i == 0) return full_tiles + pair;
      --i;
    }
    const int w = pair + i * num_pairs;
    return w < full_tiles ? w : -1;
  };
  auto unit_of = [&](int w, int& mn, int& ks, int& kb0, int& kb1) -> bool {
    if (w < full_tiles) {
      mn = w; ks = 0; kb0 = 0; kb1 = k_blocks;
      return false;
    }
    const int u = w - full_tiles;
    mn = full_tiles + u % tail_tiles;
    ks = u / tail_tiles;
    kb0 = ks * kb_per_split;
    kb1 = min(k_blocks, kb0 + kb_per_split);
    return true;
  };
  const uint32_t tmem_cols = (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128 : (2 * BN <= 256) ? 256 : 512;
  const uint32_t acc_stride = tmem_cols / 2;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&bars->full[s], 1);      // leader's producer arms it; the bytes of both CTAs complete it
      mbar_init(&bars->empty[s], 1);     // one paired commit per use
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->tmem_full[a], 1);
      mbar_init(&bars->tmem_empty[a], 8);   // used in the leader only: 4 epilogue warps of each CTA
    }
    mbar_init(&bars->epi_sync, 4);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(&bars->tmem_base, tmem_cols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();      // barriers of both CTAs are initialised before any remote arrive or load completion
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  // Everything above (barriers, tensor memory, the cluster rendez-vous) may run beside the tail of the kernel before this
  // one in the stream; nothing that kernel wrote is read before this point.
  grid_dep_wait();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one_sync()) {
      prefetch_tmap(&tmA);
      prefetch_tmap(&tmB);
      uint32_t it = 0;
      bool ok = true;
      for (int wi = 0, tile; (tile = work_at(wi)) >= 0 && ok; ++wi) {
        int mn, ks, kb_begin, kb_end;
        unit_of(tile, mn, ks, kb_begin, kb_end);
        const int m0 = (mn % m_tiles) * (2 * kBM) + int(cta) * kBM;
        const int n0 = (mn / m_tiles) * BN + int(cta) * (BN / 2);
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const int s = it % stages;
          const uint32_t ph = (it / stages) & 1;
          if (!mbar_wait(&bars->empty[s], ph ^ 1)) {
            atomicExch(status, XL_ERR_WAIT_EMPTY);
            ok = false;
            break;
          }
          if (cta == 0) mbar_arrive_expect_tx(&bars->full[s], 2 * (a_stage_bytes + b_stage_bytes));
          const uint32_t bar = map_to_cta(smem_u32(&bars->full[s]), 0);
          tma_load_2d_pair(smem_a + s * a_stage_bytes, &tmA, bar, kb * kBKe, m0);
          tma_load_2d_pair(smem_b + s * b_stage_bytes, &tmB, bar, kb * kBKe, n0);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (cta == 0 && elect_one_sync()) {
      const uint32_t idesc = ESIZE == 2 ? umma_idesc_f16(2 * kBM, BN, 1) : umma_idesc_e4m3(2 * kBM, BN);
      uint32_t it = 0, local_tile = 0;
      bool ok = true;
      for (int wi = 0, tile; (tile = work_at(wi)) >= 0 && ok; ++wi, ++local_tile) {
        const uint32_t acc = local_tile & 1;
        const uint32_t acc_ph = (local_tile >> 1) & 1;
        if (!mbar_wait(&bars->tmem_empty[acc], acc_ph ^ 1)) {
          atomicExch(status, XL_ERR_WAIT_TMEM_EMPTY);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * acc_stride;
        int mn, ks, kb_begin, kb_end;
        unit_of(tile, mn, ks, kb_begin, kb_end);
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const int s = it % stages;
          const uint32_t ph = (it / stages) & 1;
          if (!mbar_wait(&bars->full[s], ph)) {
            atomicExch(status, XL_ERR_WAIT_FULL);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem_a + s * a_stage_bytes);
          const uint32_t b_addr = smem_u32(smem_b + s * b_stage_bytes);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {          // four MMAs of 32 bytes of K each
            if (ESIZE == 2)
              tc_mma_f16_pair(d_tmem, umma_desc_sw128(a_addr, k * kUmmaK * 2), umma_desc_sw128(b_addr, k * kUmmaK * 2), idesc,
                              ((kb - kb_begin) | k) != 0);
            else
              tc_mma_f8_pair(d_tmem, umma_desc_sw128(a_addr, k * kUmmaK * 2), umma_desc_sw128(b_addr, k * kUmmaK * 2), idesc,
                             ((kb - kb_begin) | k) != 0);
          }
          tc_commit_pair(&bars->empty[s]);
        }
        if (ok) tc_commit_pair(&bars->tmem_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue of this CTA's 128 rows
    const int q = warp & 3;
    uint32_t local_tile = 0;
    bool ok = true;
    const int epi_tid = (warp - 2) * 32 + lane;            // 0..127 over the four epilogue warps
    uint32_t epi_phase = 0;
    uint32_t store_seq = 0;                                // bulk tensor stores issued by this warp (buffer = parity)
    for (int wi = 0, tile; (tile = work_at(wi)) >= 0 && ok; ++wi, ++local_tile) {
      int mn, ks, kb_begin_u, kb_end_u;
      const bool split = unit_of(tile, mn, ks, kb_begin_u, kb_end_u);
      const int tmn = mn - full_tiles;                       // index among the split tiles
      const int m0 = (mn % m_tiles) * (2 * kBM) + int(cta) * kBM;
      const int n0 = (mn / m_tiles) * BN;
      const uint32_t acc = local_tile & 1;
      const uint32_t acc_ph = (local_tile >> 1) & 1;
      if (!mbar_wait(&bars->tmem_full[acc], acc_ph)) {
        if (lane == 0) atomicExch(status, XL_ERR_WAIT_TMEM_FULL);
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t t_row = tmem_base + acc * acc_stride + (uint32_t(q * 32) << 16);
      // The accumulator leaves TMEM in 32-column chunks, one chunk ahead: the load of chunk c+1 is in flight while
      // chunk c is converted and stored.  Whole chunks of a whole tile go through shared memory and leave as bulk
      // tensor stores ([32 rows x 32 columns] boxes: full 64-byte row segments instead of 16 bytes per lane and row).
      auto ld_chunk = [&](int c, uint32_t (&r)[32]) {
        if (c + 32 <= BN) {
          tmem_ld_32x32(t_row + c, r);
        } else {
          tmem_ld_32x16_lo(t_row + c, r);
        }
      };
      auto put_chunk = [&](int c, uint32_t (&r)[32]) {
        const int width = (c + 32 <= BN) ? 32 : 16;
        const int n = n0 + c;
        if (split) {
          // fp32 partial of this K range -> this split's slab of the (tile, CTA half).  Slab layout: float4 number
          // (chunk * 8 + j) of all 128 rows side by side, so that a warp stores (and later loads) 512 contiguous bytes.
          float4* slab = reinterpret_cast<float4*>(sk.ws) + (size_t(ks * tail_tiles + tmn) * 2 + cta) * (size_t(kBM) * ((BN + 31) / 32) * 8);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            __stcg(slab + size_t((c >> 5) * 8 + j) * kBM + (q * 32 + lane),
                   width == 32 || j < 4 ? make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                      __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]))
                                        : make_float4(0.f, 0.f, 0.f, 0.f));
          return;
        }
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (width == 32 || j < 16) ? __uint_as_float(r[j]) : 0.f;
        if (ESIZE == 1) scale_chunk(v, row, n, M, N, sc);
        if (tma_out && width == 32) {
          store_chunk_tma<EPI>(v, smem_out + q * 4096 + (store_seq & 1) * 2048, lane, m0 + q * 32, n, M, N, &tmC, bias);
          ++store_seq;
        } else {
          emit_chunk<EPI>(v, row, n, width, M, N, ldc, C, bias, rs);
        }
      };
      {
        uint32_t r0[32], r1[32];
        ld_chunk(0, r0);
        for (int c = 0; c < BN; c += 64) {
          tc_wait_ld();
          if (c + 32 < BN) ld_chunk(c + 32, r1);
          put_chunk(c, r0);
          if (c + 32 < BN) {
            tc_wait_ld();
            if (c + 64 < BN) ld_chunk(c + 64, r0);
            put_chunk(c + 32, r1);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&bars->tmem_empty[acc]), 0));
      if (split) {
        // Rendez-vous of the splits of this (tile, CTA half): all of them are resident at the same time (the split units
        // are the last unit of their pairs, and the grid is one wave of pairs).  Afterwards every split reduces and
        // emits its share of the tile's 32-column chunks, reading the slabs of all splits in split order.
        int* arrive = sk.tickets + (tmn * 2 + int(cta)) * 2;
        auto epi_rendezvous = [&]() -> bool {
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->epi_sync);
          const bool done = mbar_wait(&bars->epi_sync, epi_phase & 1);
          ++epi_phase;
          return done;
        };
        __threadfence();
        bool good = epi_rendezvous();                          // all four warps have stored their partial rows
        if (good && epi_tid == 0) {
          atomicAdd(arrive, 1);
          int seen = 0;
          for (int i = 0; i < (1 << 22); ++i) {
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(arrive) : "memory");
            if (seen >= sk.splits) break;
            if (i > 64) __nanosleep(64);
          }
          bars->epi_ticket[local_tile & 1] = seen;
        }
        good = epi_rendezvous() && good;
        if (!good || bars->epi_ticket[local_tile & 1] < sk.splits) {
          if (lane == 0) atomicExch(status, XL_ERR_WAIT_PEER);
          ok = false;
          break;
        }
        __threadfence();
        const int chunks = (BN + 31) / 32;
        const int c_begin = ks * chunks / sk.splits, c_end = (ks + 1) * chunks / sk.splits;
        for (int ci = c_begin; ci < c_end; ++ci) {
          const int c = ci * 32;
          const int width = (c + 32 <= BN) ? 32 : 16;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.f;
          for (int sp = 0; sp < sk.splits; ++sp) {             // fixed order: the sum does not depend on timing
            const float4* slab = reinterpret_cast<const float4*>(sk.ws) + (size_t(sp * tail_tiles + tmn) * 2 + cta) * (size_t(kBM) * ((BN + 31) / 32) * 8);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 t = __ldcg(slab + size_t(ci * 8 + j) * kBM + (q * 32 + lane));
              v[4 * j] += t.x; v[4 * j + 1] += t.y; v[4 * j + 2] += t.z; v[4 * j + 3] += t.w;
            }
          }
          if (ESIZE == 1) scale_chunk(v, row, n0 + c, M, N, sc);
          emit_chunk<EPI>(v, row, n0 + c, width, M, N, ldc, C, bias, rs);
        }
        if (!epi_rendezvous()) { ok = false; break; }          // this split is done reading the slabs
        if (epi_tid == 0) {
          const int prev = atomicAdd(arrive + 1, 1);
          if (prev == sk.splits - 1) { arrive[0] = 0; arrive[1] = 0; }    // the last split resets the tile's counters
        }
      }
    }
    if (tma_out && lane == 0) {
      // this warp's bulk stores are complete (written, not only read) before the CTA reports or exits
      tma_store_wait<0>();
      asm volatile("fence.proxy.async.global;" ::: "memory");
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // both epilogues are done with TMEM; no arrive or load of the pair is in flight
  if (warp == 1) tmem_dealloc_pair(tmem_base, tmem_cols);
  if (EPI == EPI_RS_PUSH && threadIdx.x == 0) {
    if (rs.local) __threadfence(); else __threadfence_system();   // this CTA's stores are ordered before the count
    const int prev = atomicAdd(rs.done_counter, 1);
    if (prev == int(gridDim.x) - 1) {
      *rs.done_counter = 0;
      __threadfence_system();
      const int e = *rs.epoch + 1;
      // one system-scope fence (above), then relaxed stores: a release store per peer would pay one NVLink round trip each
      for (int r = 0; r < rs.tp; ++r)
        asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(rs.flags[r] + rs.rank), "r"(e) : "memory");
    }
  }
}

// Plan for the last, partly filled wave: `tiles` output tiles on `pairs` SM pairs leave tiles % pairs tiles for the final
// round; when those are few they are cut along K into `splits` ranges so that (nearly) every pair gets one short unit.
// Returns the number of splits (1: leave the tail whole) and the cost of the final round in tile times.
// Measured on M = 1279: worth it from K = 2048 on (the hidden part needs a main loop of some length beside it) and for
// tiles at least 160 wide (narrow tiles re-read A too often to be a good base for it).
static int plan_tail(long tiles, int pairs, int k_blocks, int bn, double* cost) {
  const long rem = tiles % pairs;
  *cost = rem ? 1.0 : 0.0;
  if (tiles < pairs || rem == 0 || rem * 2 > pairs || k_blocks < 32 || bn < 160) return 1;
  int splits = int(pairs / rem);
  if (splits > k_blocks / 4) splits = k_blocks / 4;       // at least four K blocks per range
  if (splits > 16) splits = 16;
  if (splits < 2) return 1;
  const int per = (k_blocks + splits - 1) / splits;
  splits = (k_blocks + per - 1) / per;                    // no empty range
  // a range costs its K blocks plus what is not hidden of the slab store, the rendez-vous and the reduction (they run
  // beside the first whole tile's main loop)
  const double c = double(per + 6) / double(k_blocks);
  if (splits < 2 || c > 0.8) return 1;
  *cost = c;
  return splits;
}

// Tile width for pairs: fill whole waves of SM pairs, prefer wide tiles.  Returns the score through *score.
static int pick_bn_pair(int M, int N, int K, int pairs, int epi, double* score_out, bool allow_tail) {
  const int m_tiles = (M + 2 * kBM - 1) / (2 * kBM);
  const int k_blocks = (K + kBK - 1) / kBK;
  const int step = 32;
  int best = 128;
  double best_score = -1;
  for (int bn = 64; bn <= 256; bn += step) {
    const int n_tiles = (N + bn - 1) / bn;
    const long tiles = long(m_tiles) * n_tiles;
    double last = 1.0;
    if (allow_tail) plan_tail(tiles, pairs, k_blocks, bn, &last);
    const double rounds = double(tiles / pairs) + ((tiles % pairs) ? last : 0.0);
    const double useful = double(N) / double(n_tiles * bn) * double(M) / double(m_tiles * 2 * kBM);
    const double util = double(tiles) / (rounds * pairs);
    const double shape = 0.5 + 0.5 * double(bn) / 256.0;
    const double score = util * useful * shape;
    if (score > best_score + 1e-9) {
      best_score = score;
      best = bn;
    }
  }
  if (score_out) *score_out = best_score;
  return best;
}

static int g_force_bn = 0;
static int g_tma_out = 1;           // 0: the epilogue stores straight from registers (comparison hook)
static int g_pdl = 1;               // 1: launched with programmatic stream serialization (the prologue may run beside the
                                    // tail of a predecessor that releases its dependents early); 0: plain launch
static int g_splitk = 1;            // 0: never split K; 1: split when the output has too few tiles to fill the SM pairs

// Split-K workspace: one allocation per device, made at the first use outside a stream capture (fp32 slabs + tickets).
constexpr size_t kWsBytes = size_t(96) << 20;
constexpr size_t kTicketBytes = size_t(1) << 16;
static uint8_t* splitk_workspace(cudaStream_t stream) {
  static uint8_t* ws[64] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  if (!ws[dev]) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &st) != cudaSuccess || st != cudaStreamCaptureStatusNone) return nullptr;
    void* p = nullptr;
    if (cudaMalloc(&p, kWsBytes + kTicketBytes) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, kWsBytes + kTicketBytes);
    ws[dev] = static_cast<uint8_t*>(p);
  }
  return ws[dev];
}

template <int EPI, int ESIZE = 2>
static int launch_pair(const void* A, const void* W, void* C, const void* bias, int M, int N, int K, int lda, int ldw, int ldc,
                       cudaStream_t stream, const RsPush* rs_in, const Scales* sc_in = nullptr) {
  constexpr int kBKe = 128 / ESIZE;
  const int sms = xl_host::sm_count();
  const int pairs = sms / 2;
  double score = 0;
  const bool pushes_rows = EPI == EPI_RS_PUSH && !(rs_in && rs_in->local);
  const bool may_split = g_splitk && !pushes_rows;
  int BN = g_force_bn > 0 ? g_force_bn : pick_bn_pair(M, N, K * ESIZE / 2, pairs, EPI, &score, may_split);
  const int m_tiles = (M + 2 * kBM - 1) / (2 * kBM);
  const int k_blocks = (K + kBKe - 1) / kBKe;
  SplitK sk;
  sk.ws = nullptr; sk.tickets = nullptr; sk.splits = 1; sk.full_tiles = 0; sk.tail_tiles = 0;
  auto arm = [&](int splits, int full, int tail, int bn) -> bool {
    const size_t slab = size_t(tail) * (2 * kBM) * size_t((bn + 31) / 32 * 32) * sizeof(float);
    if (splits < 2 || slab * splits > kWsBytes || size_t(tail) * 4 * sizeof(int) > kTicketBytes) return false;
    uint8_t* w = splitk_workspace(stream);
    if (!w) return false;
    sk.ws = reinterpret_cast<float*>(w);
    sk.tickets = reinterpret_cast<int*>(w + kWsBytes);
    sk.splits = splits; sk.full_tiles = full; sk.tail_tiles = tail;
    return true;
  };
  if (may_split && k_blocks >= 16) {
    // (a) Few, long tiles (decode-size batches against a wide K): cut the K loop of every tile so that every SM pair
    //     streams weights.
    const int bn_s = g_force_bn > 0 ? g_force_bn : (N >= 256 ? 256 : BN);
    const int tiles_s = m_tiles * ((N + bn_s - 1) / bn_s);
    if (tiles_s * 2 <= pairs) {
      int splits = pairs / tiles_s;
      if (splits > k_blocks / 8) splits = k_blocks / 8;
      if (splits > 8) splits = 8;
      const size_t slab = size_t(tiles_s) * (2 * kBM) * size_t((bn_s + 31) / 32 * 32) * sizeof(float);
      while (splits > 1 && slab * splits > kWsBytes) --splits;
      if (splits > 1) {
        const int per = (k_blocks + splits - 1) / splits;
        splits = (k_blocks + per - 1) / per;              // no empty split
        if (splits < 4 && k_blocks < 128) splits = 1;     // measured: a 2- or 3-way split of a short K does not pay for its rendez-vous
        if (arm(splits, 0, tiles_s, bn_s)) BN = bn_s;
      }
    } else {
      // (b) A last wave with few tiles: cut only those.
      const long tiles = long(m_tiles) * ((N + BN - 1) / BN);
      double cost = 1.0;
      const int splits = plan_tail(tiles, pairs, k_blocks, BN, &cost);
      const int tail = int(tiles % pairs);
      if (splits > 1) arm(splits, int(tiles) - tail, tail, BN);
    }
  }
  const int stage_bytes = kBM * kBK * 2 + (BN / 2) * kBK * 2;
  int stages = (200 * 1024) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) return -3;
  const size_t smem = size_t(stages) * stage_bytes + kOutStageBytes + sizeof(Barriers) + 1024;
  const CUtensorMapDataType in_dt = ESIZE == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const CUtensorMap* ta = xl_host::tmap_2d(A, in_dt, ESIZE, M, K, lda, kBM, kBKe, CU_TENSOR_MAP_SWIZZLE_128B);
  const CUtensorMap* tb = xl_host::tmap_2d(W, in_dt, ESIZE, N, K, ldw, BN / 2, kBKe, CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ta || !tb) return -4;
  Scales sc;
  sc.row = sc.col = nullptr; sc.tensor = 1.f;
  if (sc_in) sc = *sc_in;
  // Output through bulk tensor stores when C can be described by a tensor map (16-byte aligned base and pitch) and
  // the rows stay in C (the row-push epilogue addresses other ranks' buffers per row).
  const CUtensorMap* tc = nullptr;
  if (g_tma_out && !pushes_rows && (reinterpret_cast<uintptr_t>(C) & 15) == 0 && (size_t(ldc) * 2) % 16 == 0) {
    if (EPI == EPI_SWIGLU)
      tc = xl_host::tmap_2d(C, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, N / 2, ldc, 32, 16, CU_TENSOR_MAP_SWIZZLE_32B);
    else
      tc = xl_host::tmap_2d(C, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, N, ldc, 32, 32, CU_TENSOR_MAP_SWIZZLE_64B);
  }
  RsPush rs;
  memset(&rs, 0, sizeof(rs));
  if (rs_in) rs = *rs_in;
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(gemm_bf16_pair_kernel<EPI, ESIZE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    attr_set = true;
  }
  const int n_tiles = (N + BN - 1) / BN;
  const int units = sk.splits > 1 ? sk.full_tiles + sk.tail_tiles * sk.splits : m_tiles * n_tiles;
  const int grid = 2 * max(1, min(units, pairs));
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_pdl ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_bf16_pair_kernel<EPI, ESIZE>, *ta, *tb, tc ? *tc : *ta, tc ? 1 : 0,
                                     reinterpret_cast<__nv_bfloat16*>(C),
                                     reinterpret_cast<const __nv_bfloat16*>(bias), M, N, K, ldc, BN, stages,
                                     xl_host::status_word(), rs, sk, sc);
  return e == cudaSuccess ? 0 : -1;
}

}  // namespace xl2

// Entry points used by gemm_bf16.cu's dispatch.  `epi`: 0 none, 1 bias, 2 SwiGLU (interleaved W), 3 row push (TP).
// `score` (may be null) receives the wave-fill score of the chosen tile width, comparable with the single-CTA one.
extern "C" int xl_gemm_bf16_pair_launch(int epi, const void* A, const void* W, void* C, const void* bias, int M, int N, int K,
                                        int lda, int ldw, int ldc, void* stream, const void* rs) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const xl2::RsPush* r = static_cast<const xl2::RsPush*>(rs);
  switch (epi) {
    case 0: return xl2::launch_pair<xl2::EPI_NONE>(A, W, C, bias, M, N, K, lda, ldw, ldc, st, nullptr);
    case 1: return xl2::launch_pair<xl2::EPI_BIAS>(A, W, C, bias, M, N, K, lda, ldw, ldc, st, nullptr);
    case 2: return xl2::launch_pair<xl2::EPI_SWIGLU>(A, W, C, bias, M, N, K, lda, ldw, ldc, st, nullptr);
    case 3: return xl2::launch_pair<xl2::EPI_RS_PUSH>(A, W, C, bias, M, N, K, lda, ldw, ldc, st, r);
  }
  return -2;
}
extern "C" double xl_gemm_bf16_pair_score(int epi, int M, int N, int K, int may_split) {
  double s = 0;
  xl2::pick_bn_pair(M, N, K, xl_host::sm_count() / 2, epi, &s, may_split && xl2::g_splitk);
  return s;
}
XL_API void xl_gemm_pair_force_bn(int bn) { xl2::g_force_bn = bn; }
// Test / comparison hook: 0 never split the K loop, 1 (default) split it when the output has too few tiles.
XL_API void xl_gemm_pair_splitk(int on) { xl2::g_splitk = on; }
// Test / comparison hook: 1 (default) whole output chunks leave through shared memory and bulk tensor stores.
XL_API void xl_gemm_pair_tma_out(int on) { xl2::g_tma_out = on; }
// Comparison hook: 0 launches the pair GEMM without the programmatic-serialization attribute.
XL_API void xl_gemm_pair_pdl(int on) { xl2::g_pdl = on ? 1 : 0; }

// fp8 (e4m3) operands with per-row activation scales and per-tensor / per-output-channel weight scales:
//   C[M,N] (bf16) = (A_q[M,K] W_q[N,K]^T) * row_scale[m] * tensor_scale * (col_scale ? col_scale[n] : 1)  (+ bias[n])
// `epi`: 0 none, 1 bias, 2 SwiGLU over interleaved gate / up rows (col_scale, when given, in the same interleaved order).
// lda / ldw in elements (bytes).  K must be a multiple of 16 (TMA pitch rule).
XL_API int xl_gemm_fp8_scaled(int epi, const void* A, const void* W, void* C, const void* bias, const void* row_scale,
                              const void* col_scale, float tensor_scale, int M, int N, int K, int lda, int ldw, int ldc,
                              void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (lda % 16) || (ldw % 16)) return -2;
  xl2::Scales sc;
  sc.row = static_cast<const float*>(row_scale);
  sc.col = static_cast<const float*>(col_scale);
  sc.tensor = tensor_scale;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (epi) {
    case 0: return xl2::launch_pair<xl2::EPI_NONE, 1>(A, W, C, nullptr, M, N, K, lda, ldw, ldc, st, nullptr, &sc);
    case 1: return xl2::launch_pair<xl2::EPI_BIAS, 1>(A, W, C, bias, M, N, K, lda, ldw, ldc, st, nullptr, &sc);
    case 2: return xl2::launch_pair<xl2::EPI_SWIGLU, 1>(A, W, C, nullptr, M, N, K, lda, ldw, ldc, st, nullptr, &sc);
  }
  return -2;
}
