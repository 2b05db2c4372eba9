// bf16 GEMM on the 5th-generation tensor cores:  C[M,N] = A[M,K] * W[N,K]^T (+ bias), fp32 accumulate.
//
// Replaces the reference's cuBLAS call (xllm/core/kernels/cuda/matmul.cpp:20-24 -> F::linear) for every
// dense projection (qkv, o, gate_up, down, lm_head, router).
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0   : TMA producer  - cp.async.bulk.tensor loads of a 128 x 64 A tile and a BN x 64 W tile per
//              k-block into a ring of shared-memory stages (128-byte swizzle), completion on mbarriers;
//   warp 1   : MMA issuer    - one elected thread issues tcgen05.mma (M=128, N=BN, K=16) four times per
//              k-block, accumulating in TMEM; tcgen05.commit releases the smem stage / publishes the tile;
//   warps 2-5: epilogue      - tcgen05.ld of the fp32 accumulator (double-buffered in TMEM so that the
//              next tile's mainloop overlaps), optional bias / SwiGLU, bf16 pack, 16-byte global stores.
// BN (tile width) is a run-time multiple of 16 in [32, 256], chosen per problem so that the tile count
// fills whole waves of SMs.
#include <string.h>

#include "common.cuh"

namespace xl {

constexpr int kBM = 128;
constexpr int kBK = 64;          // 64 bf16 = 128 bytes = one swizzle row
constexpr int kUmmaK = 16;
constexpr int kMaxStages = 8;
constexpr int kGemmThreads = 192;

struct GemmSmemBarriers {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

enum { EPI_NONE = 0, EPI_BIAS = 1, EPI_SWIGLU = 2, EPI_RS_PUSH = 3 };

// EPI_RS_PUSH (tensor-parallel row-parallel linear): this rank's partial tile is not stored locally; each row is
// pushed over NVLink straight from the epilogue registers into the receive buffer of the rank that owns the row
// (rows are owned in contiguous shards of `shard` rows).  When the last CTA of the kernel has finished, it
// publishes "partials of this rank have landed" to every owner with a system-scope release store.
struct RsPush {
  __nv_bfloat16* recv[8];   // recv[r] = base of rank r's receive buffer  [tp][shard_cap][N]
  int* flags[8];            // flags[r] = rank r's arrival flags           [tp]
  int* done_counter;        // local
  const int* epoch;         // local, bumped by the reduce kernel that follows
  int tp, rank, shard, shard_cap;
  int local;                // 1: rows stay in this rank's C (peers fetch them); only the completion flags are published
};

// Grouped (MoE expert) mode: A rows are sorted by expert; a device-side tile table maps every 128-row tile to its
// expert (selects the weight slab: W is [E * N, K]), its first row and the end of its expert's row range.
struct Grouped {
  const int* tile_expert;
  const int* tile_row0;
  const int* tile_row_end;
  const int* num_m_tiles;   // device scalar
  int enabled;
  // output placement: C row = row - expert * c_rows_per_expert, C column offset = expert * c_col_stride
  // (both 0 for the plain "sorted rows in, sorted rows out" case)
  int c_rows_per_expert;
  int c_col_stride;
};

// EPI_SWIGLU: W rows are interleaved in groups of 16 (16 gate rows, then the 16 matching up rows), so
// every 32-column accumulator chunk holds both halves; the output has N/2 columns.
template <int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 __nv_bfloat16* __restrict__ C, const __nv_bfloat16* __restrict__ bias, int M, int N, int K, int ldc,
                 int BN, int stages, int* __restrict__ status, const __grid_constant__ RsPush rs,
                 const __grid_constant__ Grouped grp) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int a_stage_bytes = kBM * kBK * 2;
  const int b_stage_bytes = BN * kBK * 2;
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + stages * a_stage_bytes;
  GemmSmemBarriers* bars = reinterpret_cast<GemmSmemBarriers*>(smem_b + stages * b_stage_bytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tiles = grp.enabled ? *grp.num_m_tiles : (M + kBM - 1) / kBM;
  const int n_tiles = (N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  const int k_blocks = (K + kBK - 1) / kBK;
  const uint32_t tmem_cols = (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128 : (2 * BN <= 256) ? 256 : 512;
  const uint32_t acc_stride = tmem_cols / 2;   // column offset of the second accumulator

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->tmem_full[a], 1);
      mbar_init(&bars->tmem_empty[a], 4);
    }
    bars->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one_sync()) {
      prefetch_tmap(&tmA);
      prefetch_tmap(&tmB);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int mt = tile % m_tiles;
        const int m0 = grp.enabled ? grp.tile_row0[mt] : mt * kBM;
        const int n0 = (tile / m_tiles) * BN;
        const int w_row = n0 + (grp.enabled ? grp.tile_expert[mt] * N : 0);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % stages;
          const uint32_t ph = (it / stages) & 1;
          if (!mbar_wait(&bars->empty[s], ph ^ 1)) {
            atomicExch(status, XL_ERR_WAIT_EMPTY);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&bars->full[s], a_stage_bytes + b_stage_bytes);
          tma_load_2d(smem_a + s * a_stage_bytes, &tmA, &bars->full[s], kb * kBK, m0);
          tma_load_2d(smem_b + s * b_stage_bytes, &tmB, &bars->full[s], kb * kBK, w_row);
        }
      }
      if (!ok) {
        // give the copies already issued a bounded time to land before the CTA retires
        const uint32_t first = it >= uint32_t(stages) ? it - stages : 0;
        for (uint32_t j = first; j < it; ++j) mbar_wait(&bars->full[j % stages], (j / stages) & 1);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one_sync()) {
      const uint32_t idesc = umma_idesc_f16(kBM, BN, 1);
      uint32_t it = 0, local_tile = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
        const uint32_t acc = local_tile & 1;
        const uint32_t acc_ph = (local_tile >> 1) & 1;
        if (!mbar_wait(&bars->tmem_empty[acc], acc_ph ^ 1)) {
          atomicExch(status, XL_ERR_WAIT_TMEM_EMPTY);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * acc_stride;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
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
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            tc_mma_f16(d_tmem, umma_desc_sw128(a_addr, k * kUmmaK * 2), umma_desc_sw128(b_addr, k * kUmmaK * 2), idesc,
                       (kb | k) != 0);
          }
          tc_commit(&bars->empty[s]);   // stage reusable once these MMAs have read it
        }
        if (ok) tc_commit(&bars->tmem_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps, one TMEM lane quarter each)
    const int q = warp & 3;
    uint32_t local_tile = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
      const int mt = tile % m_tiles;
      const int m0 = grp.enabled ? grp.tile_row0[mt] : mt * kBM;
      const int row_lim = grp.enabled ? grp.tile_row_end[mt] : M;
      const int n0 = (tile / m_tiles) * BN;
      const int c_row_off = grp.enabled ? grp.tile_expert[mt] * grp.c_rows_per_expert : 0;
      const int c_col_off = grp.enabled ? grp.tile_expert[mt] * grp.c_col_stride : 0;
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
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        if (c + 32 <= BN) {
          tmem_ld_32x32(t_row + c, r);
        } else {  // BN is a multiple of 16: last half chunk
          uint32_t h[16];
          tmem_ld_32x16(t_row + c, h);
#pragma unroll
          for (int j = 0; j < 16; ++j) { r[j] = h[j]; r[16 + j] = 0; }
        }
        tc_wait_ld();
        const int width = (c + 32 <= BN) ? 32 : 16;
        const int n = n0 + c;
        if (EPI == EPI_SWIGLU) {
          // columns [0,16) gate, [16,32) up of output columns (n/2 .. n/2+16)
          if (row < row_lim && n < N) {
            uint32_t o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float g0 = __uint_as_float(r[2 * j]), g1 = __uint_as_float(r[2 * j + 1]);
              float u0 = __uint_as_float(r[16 + 2 * j]), u1 = __uint_as_float(r[16 + 2 * j + 1]);
              float a0 = g0 / (1.f + __expf(-g0)) * u0;
              float a1 = g1 / (1.f + __expf(-g1)) * u1;
              o[j] = pack_bf16x2(a0, a1);
            }
            uint4* dst = reinterpret_cast<uint4*>(C + size_t(row - c_row_off) * ldc + c_col_off + (n >> 1));
            dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
            dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
          }
        } else {
          if (row < row_lim && n < N) {
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
            if (EPI == EPI_BIAS) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n + j < N) v[j] += __bfloat162float(__ldg(bias + n + j));
            }
            __nv_bfloat16* dst = C + size_t(row - c_row_off) * ldc + c_col_off + n;
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
              for (int j = 0; j < width && n + j < N; ++j) dst[j] = __float2bfloat16(v[j]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->tmem_empty[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, tmem_cols);
  if (EPI == EPI_RS_PUSH && threadIdx.x == 0) {
    if (rs.local) __threadfence(); else __threadfence_system();   // this CTA's stores are ordered before the count
    const int prev = atomicAdd(rs.done_counter, 1);
    if (prev == int(gridDim.x) - 1) {                    // last CTA of this rank
      *rs.done_counter = 0;
      __threadfence_system();
      const int e = *rs.epoch + 1;
      // one system-scope fence (above), then relaxed stores: a release store per peer would pay one NVLink round trip each
      for (int r = 0; r < rs.tp; ++r)
        asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(rs.flags[r] + rs.rank), "r"(e) : "memory");
    }
  }
}

static int g_force_bn = 0;
static int g_mode = 0;      // 0: choose per problem, 1: single-CTA tiles only, 2: CTA-pair tiles whenever possible

}  // namespace xl
// CTA-pair kernel (gemm_bf16_2cta.cu)
extern "C" int xl_gemm_bf16_pair_launch(int epi, const void* A, const void* W, void* C, const void* bias, int M, int N, int K,
                                        int lda, int ldw, int ldc, void* stream, const void* rs);
extern "C" double xl_gemm_bf16_pair_score(int epi, int M, int N, int K, int may_split);
namespace xl {

static double g_last_score = 0;

// Tile width: fill whole waves of SMs, prefer wide tiles (less A re-read per FLOP).
static int pick_bn(int M, int N, int sms, int epi) {
  if (g_force_bn > 0) return g_force_bn;
  const int m_tiles = (M + kBM - 1) / kBM;
  const int step = (epi == EPI_SWIGLU) ? 32 : 16;
  int best = 128;
  double best_score = -1;
  for (int bn = 32; bn <= 256; bn += step) {
    const int n_tiles = (N + bn - 1) / bn;
    const long tiles = long(m_tiles) * n_tiles;
    const long rounds = (tiles + sms - 1) / sms;
    const double useful = double(N) / double(n_tiles * bn);          // padding waste in the last tile column
    const double util = double(tiles) / double(rounds * sms);
    const double shape = 0.5 + 0.5 * double(bn) / 256.0;             // wider tiles move fewer bytes per FLOP
    const double score = util * useful * shape;
    if (score > best_score + 1e-9) {
      best_score = score;
      best = bn;
    }
  }
  g_last_score = best_score;
  return best;
}

template <int EPI>
static int launch(const void* A, const void* W, void* C, const void* bias, int M, int N, int K, int lda, int ldw, int ldc,
                  cudaStream_t stream, const RsPush* rs_in = nullptr, const Grouped* grp_in = nullptr, int num_experts = 1,
                  int max_m_tiles = 0) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldw % 8) || (ldc % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15) ||
      ((EPI != EPI_RS_PUSH || (rs_in && rs_in->local)) && (reinterpret_cast<uintptr_t>(C) & 15)))
    return -2;  // TMA and 16-byte stores need 16-byte aligned rows
  if (EPI == EPI_SWIGLU && (N % 32)) return -2;
  const int sms = xl_host::sm_count();
  const int BN = pick_bn(M, N, sms, EPI);
  if (!grp_in && g_mode != 1 && (M > kBM || K >= 2048) && g_force_bn == 0) {
    // A pair of CTAs per 256-row tile moves a third less shared-memory traffic per FLOP; it wins unless its coarser
    // tiles fill the SMs much worse than single-CTA tiles do.
    const double pair_score = xl_gemm_bf16_pair_score(EPI, M, N, K, !(EPI == EPI_RS_PUSH && !(rs_in && rs_in->local)));
    // (small batches against a long K also go to the pair kernel: it splits the K loop over the SM pairs)
    if (g_mode == 2 || M <= kBM || pair_score * 1.2 >= g_last_score) {
      RsPush rs_copy;
      memset(&rs_copy, 0, sizeof(rs_copy));
      if (rs_in) rs_copy = *rs_in;
      return xl_gemm_bf16_pair_launch(EPI, A, W, C, bias, M, N, K, lda, ldw, ldc, stream, rs_in ? &rs_copy : nullptr);
    }
  }
  const int stage_bytes = kBM * kBK * 2 + BN * kBK * 2;
  int stages = (200 * 1024) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) return -3;
  const size_t smem = size_t(stages) * stage_bytes + sizeof(GemmSmemBarriers) + 1024;
  const CUtensorMap* ta = xl_host::tmap_2d(A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, kBM, kBK, CU_TENSOR_MAP_SWIZZLE_128B);
  const CUtensorMap* tb = xl_host::tmap_2d(W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, uint64_t(N) * num_experts, K, ldw, BN, kBK,
                                           CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ta || !tb) return -4;
  static bool attr_set[4] = {false, false, false, false};
  RsPush rs;
  memset(&rs, 0, sizeof(rs));
  if (rs_in) rs = *rs_in;
  Grouped grp;
  memset(&grp, 0, sizeof(grp));
  if (grp_in) grp = *grp_in;
  if (!attr_set[EPI]) {
    cudaFuncSetAttribute(gemm_bf16_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    attr_set[EPI] = true;
  }
  const int m_tiles = grp_in ? max_m_tiles : (M + kBM - 1) / kBM, n_tiles = (N + BN - 1) / BN;
  const int grid = max(1, min(m_tiles * n_tiles, sms));
  gemm_bf16_kernel<EPI><<<grid, kGemmThreads, smem, stream>>>(*ta, *tb, reinterpret_cast<__nv_bfloat16*>(C),
                                                            reinterpret_cast<const __nv_bfloat16*>(bias), M, N, K, ldc, BN,
                                                            stages, xl_host::status_word(), rs, grp);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace xl

// C[M,N] = A[M,K] W[N,K]^T (+bias[N]).  Leading dimensions in elements.  Returns 0 on success.
XL_API int xl_gemm_bf16(const void* A, const void* W, void* C, const void* bias, int M, int N, int K, int lda, int ldw, int ldc,
                        void* stream) {
  if (bias) return xl::launch<xl::EPI_BIAS>(A, W, C, bias, M, N, K, lda, ldw, ldc, static_cast<cudaStream_t>(stream));
  return xl::launch<xl::EPI_NONE>(A, W, C, nullptr, M, N, K, lda, ldw, ldc, static_cast<cudaStream_t>(stream));
}

// out[M, N/2] = silu(gate) * up, with W rows interleaved in groups of 16 (see `xl_interleave_gate_up`).
XL_API int xl_gemm_bf16_swiglu(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldw, int ldc,
                               void* stream) {
  return xl::launch<xl::EPI_SWIGLU>(A, W, C, nullptr, M, N, K, lda, ldw, ldc, static_cast<cudaStream_t>(stream));
}

// Grouped GEMM over expert-sorted rows: C[r, :] = A[r, :] * W[expert(r)]^T for the rows listed in the tile table
// (`tile_*` arrays and `num_m_tiles` live on the device; `max_m_tiles` bounds them for the launch).
// swiglu != 0: W holds interleaved gate/up rows and C has N/2 columns.
XL_API int xl_grouped_gemm_bf16(const void* A, const void* W, void* C, int M_cap, int N, int K, int lda, int ldc, int num_experts,
                                const void* tile_expert, const void* tile_row0, const void* tile_row_end,
                                const void* num_m_tiles, int max_m_tiles, int swiglu, int c_rows_per_expert, int c_col_stride,
                                void* stream) {
  xl::Grouped g;
  g.c_rows_per_expert = c_rows_per_expert;
  g.c_col_stride = c_col_stride;
  g.tile_expert = static_cast<const int*>(tile_expert);
  g.tile_row0 = static_cast<const int*>(tile_row0);
  g.tile_row_end = static_cast<const int*>(tile_row_end);
  g.num_m_tiles = static_cast<const int*>(num_m_tiles);
  g.enabled = 1;
  if (max_m_tiles <= 0) return 0;
  if (swiglu)
    return xl::launch<xl::EPI_SWIGLU>(A, W, C, nullptr, M_cap, N, K, lda, K, ldc, static_cast<cudaStream_t>(stream), nullptr, &g,
                                      num_experts, max_m_tiles);
  return xl::launch<xl::EPI_NONE>(A, W, C, nullptr, M_cap, N, K, lda, K, ldc, static_cast<cudaStream_t>(stream), nullptr, &g,
                                  num_experts, max_m_tiles);
}

// Row-parallel GEMM whose output rows are pushed to their owner ranks (see RsPush).  `recv` / `flags` hold `tp`
// peer pointers each (this rank's own included).  N doubles as the row pitch of the receive buffers.
XL_API int xl_gemm_bf16_rs_push(const void* A, const void* W, int M, int N, int K, int lda, int ldw, void* const* recv,
                                void* const* flags, void* done_counter, const void* epoch, int tp, int rank, int shard,
                                int shard_cap, void* stream) {
  if (tp < 1 || tp > 8 || shard <= 0 || shard > shard_cap || (long(shard) * tp < M)) return -2;
  xl::RsPush rs;
  memset(&rs, 0, sizeof(rs));
  for (int r = 0; r < tp; ++r) {
    rs.recv[r] = static_cast<__nv_bfloat16*>(recv[r]);
    rs.flags[r] = static_cast<int*>(flags[r]);
    if (reinterpret_cast<uintptr_t>(recv[r]) & 15) return -2;
  }
  rs.done_counter = static_cast<int*>(done_counter);
  rs.epoch = static_cast<const int*>(epoch);
  rs.tp = tp; rs.rank = rank; rs.shard = shard; rs.shard_cap = shard_cap;
  return xl::launch<xl::EPI_RS_PUSH>(A, W, nullptr, nullptr, M, N, K, lda, ldw, N, static_cast<cudaStream_t>(stream), &rs);
}

// Row-parallel GEMM whose partial result stays in this rank's buffer C [M, N] (a buffer that the peers have mapped);
// when the last CTA has finished, "partials of this rank are complete" is published to every rank's flag word with a
// system-scope release store.  The reduce kernel of each owner then fetches the rows it owns from all ranks.
XL_API int xl_gemm_bf16_publish(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldw, int ldc,
                                void* const* flags, void* done_counter, const void* epoch, int tp, int rank, void* stream) {
  if (tp < 1 || tp > 8) return -2;
  xl::RsPush rs;
  memset(&rs, 0, sizeof(rs));
  for (int r = 0; r < tp; ++r) rs.flags[r] = static_cast<int*>(flags[r]);
  rs.done_counter = static_cast<int*>(done_counter);
  rs.epoch = static_cast<const int*>(epoch);
  rs.tp = tp; rs.rank = rank; rs.shard = M > 0 ? M : 1; rs.shard_cap = rs.shard; rs.local = 1;
  return xl::launch<xl::EPI_RS_PUSH>(A, W, C, nullptr, M, N, K, lda, ldw, ldc, static_cast<cudaStream_t>(stream), &rs);
}

// Test / tuning hook: force the tile width (0 = automatic).
XL_API void xl_gemm_force_bn(int bn) { xl::g_force_bn = bn; }
// Test / tuning hook: 0 choose per problem, 1 single-CTA tiles only, 2 CTA-pair tiles whenever M > 128.
XL_API void xl_gemm_set_mode(int mode) { xl::g_mode = mode; }
