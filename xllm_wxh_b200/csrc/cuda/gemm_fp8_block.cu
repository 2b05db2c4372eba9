// Block-scaled fp8 (e4m3) GEMM on tcgen05:  C[M,N] (bf16) = dequant(A) * dequant(W)^T
//   A  : e4m3 [M, K] with one fp32 scale per row per 128 columns      (sa [M, K/128], "1x128" activation scales)
//   W  : e4m3 [N, K] with one fp32 scale per 128x128 block            (sw [ceil(N/128), K/128], HF `weight_scale_inv`)
//
// The reference serves fp8 only with per-tensor / per-token scales through CUTLASS
// (xllm/core/kernels/cuda/cutlass_w8a8/c3x/scaled_mm_sm100_fp8_dispatch.cuh) and parses, but cannot run, 128x128
// block-scaled checkpoints (hf_model_loader.cpp:377-381).  Here each 128-wide k-block is multiplied on the tensor
// cores into a fresh TMEM buffer (tcgen05.mma kind::f8f6f4, fp32 accumulate, two buffers alternating), and the epilogue
// warps promote it into fp32 registers with the product of the two scales while the next k-block is being multiplied.
//
// Same warp roles and TMA / mbarrier ring as gemm_bf16.cu (BLOCK_K = 128 fp8 = one 128-byte swizzle row).
// Optional grouped mode (MoE experts): rows sorted by expert, device-side tile table, W = [E * N, K], sw = [E, N/128, K/128].
#include <string.h>

#include "common.cuh"

namespace xl_f8 {
using namespace xl;

constexpr int kBM = 128;
constexpr int kBN = 128;
constexpr int kBK = 128;         // fp8 elements = 128 bytes
constexpr int kStages = 6;       // 6 x (16 KB + 16 KB)
constexpr int kThreads = 192;

struct Bars {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
};

struct Grouped {
  const int* tile_expert;
  const int* tile_row0;
  const int* tile_row_end;
  const int* num_m_tiles;
  int enabled;
};

__global__ void __launch_bounds__(kThreads, 1)
gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      __nv_bfloat16* __restrict__ C, const float* __restrict__ sa, const float* __restrict__ sw, int M, int N,
                      int K, int ldc, int* __restrict__ status, const __grid_constant__ Grouped grp) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int A_BYTES = kBM * kBK, B_BYTES = kBN * kBK;
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages * A_BYTES;
  Bars* bars = reinterpret_cast<Bars*>(smem_b + kStages * B_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = grp.enabled ? *grp.num_m_tiles : (M + kBM - 1) / kBM;
  const int n_tiles = (N + kBN - 1) / kBN;
  const int num_tiles = m_tiles * n_tiles;
  const int k_blocks = (K + kBK - 1) / kBK;
  const int n_blocks_w = (N + 127) / 128;
  constexpr uint32_t tmem_cols = 2 * kBN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&bars->full[s], 1); mbar_init(&bars->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&bars->tmem_full[a], 1); mbar_init(&bars->tmem_empty[a], 4); }
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bars->tmem_base, tmem_cols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    if (elect_one_sync()) {
      prefetch_tmap(&tmA);
      prefetch_tmap(&tmB);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int mt = tile % m_tiles;
        const int m0 = grp.enabled ? grp.tile_row0[mt] : mt * kBM;
        const int n0 = (tile / m_tiles) * kBN;
        const int w_row = n0 + (grp.enabled ? grp.tile_expert[mt] * N : 0);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          if (!mbar_wait(&bars->empty[s], ((it / kStages) & 1) ^ 1)) { atomicExch(status, XL_ERR_WAIT_EMPTY); ok = false; break; }
          mbar_arrive_expect_tx(&bars->full[s], A_BYTES + B_BYTES);
          tma_load_2d(smem_a + s * A_BYTES, &tmA, &bars->full[s], kb * kBK, m0);
          tma_load_2d(smem_b + s * B_BYTES, &tmB, &bars->full[s], kb * kBK, w_row);
        }
      }
      if (!ok) {
        const uint32_t first = it >= uint32_t(kStages) ? it - kStages : 0;
        for (uint32_t j = first; j < it; ++j) mbar_wait(&bars->full[j % kStages], (j / kStages) & 1);
      }
    }
  } else if (warp == 1) {
    if (elect_one_sync()) {
      const uint32_t idesc = umma_idesc_e4m3(kBM, kBN);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < k_blocks && ok; ++kb, ++it) {
          const uint32_t buf = it & 1;
          if (!mbar_wait(&bars->tmem_empty[buf], ((it >> 1) & 1) ^ 1)) { atomicExch(status, XL_ERR_WAIT_TMEM_EMPTY); ok = false; break; }
          const int s = it % kStages;
          if (!mbar_wait(&bars->full[s], (it / kStages) & 1)) { atomicExch(status, XL_ERR_WAIT_FULL); ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem_a + s * A_BYTES), b_addr = smem_u32(smem_b + s * B_BYTES);
          const uint32_t d_tmem = tmem_base + buf * kBN;
#pragma unroll
          for (int k = 0; k < 4; ++k)       // 4 x (K = 32 fp8 = 32 bytes)
            tc_mma_f8f6f4(d_tmem, umma_desc_sw128(a_addr, k * 32), umma_desc_sw128(b_addr, k * 32), idesc, k != 0);
          tc_commit(&bars->empty[s]);
          tc_commit(&bars->tmem_full[buf]);
        }
      }
    }
  } else {
    const int q = warp & 3;
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int mt = tile % m_tiles;
      const int m0 = grp.enabled ? grp.tile_row0[mt] : mt * kBM;
      const int row_lim = grp.enabled ? grp.tile_row_end[mt] : M;
      const int n0 = (tile / m_tiles) * kBN;
      const int expert = grp.enabled ? grp.tile_expert[mt] : 0;
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < row_lim;
      const float* sa_row = sa + size_t(row_ok ? row : 0) * k_blocks;
      const float* sw_row = sw + (size_t(expert) * n_blocks_w + n0 / 128) * k_blocks;
      float acc[kBN];
#pragma unroll
      for (int j = 0; j < kBN; ++j) acc[j] = 0.f;
      for (int kb = 0; kb < k_blocks; ++kb, ++it) {
        const uint32_t buf = it & 1;
        const float scale = row_ok ? sa_row[kb] * sw_row[kb] : 0.f;
        if (!mbar_wait(&bars->tmem_full[buf], (it >> 1) & 1)) {
          if (lane == 0) atomicExch(status, XL_ERR_WAIT_TMEM_FULL);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t t_row = tmem_base + buf * kBN + (uint32_t(q * 32) << 16);
#pragma unroll
        for (int c = 0; c < kBN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c, r);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[c + j] = fmaf(__uint_as_float(r[j]), scale, acc[c + j]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->tmem_empty[buf]);
      }
      if (ok && row_ok) {
#pragma unroll
        for (int c = 0; c < kBN; c += 8) {
          const int n = n0 + c;
          if (n + 8 <= N) {
            *reinterpret_cast<uint4*>(C + size_t(row) * ldc + n) =
                make_uint4(pack_bf16x2(acc[c], acc[c + 1]), pack_bf16x2(acc[c + 2], acc[c + 3]), pack_bf16x2(acc[c + 4], acc[c + 5]),
                           pack_bf16x2(acc[c + 6], acc[c + 7]));
          } else {
            for (int j = 0; j < 8 && n + j < N; ++j) C[size_t(row) * ldc + n + j] = __float2bfloat16(acc[c + j]);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, tmem_cols);
}

// ---------------------------------------------------------------- activation quantisation (1 x 128 groups)
// One warp per (row, 128-column group): amax -> scale = amax / 448 -> e4m3.  `GATED`: the input row holds
// [gate | up] halves and the quantised value is silu(gate) * up (SwiGLU fused with the quantisation).
template <bool GATED>
__global__ void quant_act_kernel(const __nv_bfloat16* __restrict__ x, __nv_fp8_e4m3* __restrict__ q, float* __restrict__ scales,
                                 int T, int K, int ldx, const int* __restrict__ rows_dev) {
  const int lane = threadIdx.x & 31;
  const int groups = K / 128;
  const long n = long(rows_dev ? *rows_dev : T) * groups;
  for (long w = (blockIdx.x * long(blockDim.x) + threadIdx.x) >> 5; w < n; w += (long(gridDim.x) * blockDim.x) >> 5) {
    const int t = int(w / groups), g = int(w % groups);
    const __nv_bfloat16* src = x + size_t(t) * ldx + g * 128 + lane * 4;
    float v[4];
    {
      const uint2 a = *reinterpret_cast<const uint2*>(src);
      const float2 f0 = unpack_bf16x2(a.x), f1 = unpack_bf16x2(a.y);
      v[0] = f0.x; v[1] = f0.y; v[2] = f1.x; v[3] = f1.y;
    }
    if (GATED) {
      const uint2 b = *reinterpret_cast<const uint2*>(src + K);
      const float2 u0 = unpack_bf16x2(b.x), u1 = unpack_bf16x2(b.y);
      const float u[4] = {u0.x, u0.y, u1.x, u1.y};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float a = v[j] / (1.f + __expf(-v[j])) * u[j];
        v[j] = __bfloat162float(__float2bfloat16(a));      // the un-fused path rounds the activation to bf16 first
      }
    }
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    amax = fmaxf(warp_max(amax), 1e-10f);
    const float scale = amax / 448.f;
    const float inv = 1.f / scale;
    __nv_fp8_e4m3 o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = __nv_fp8_e4m3(fminf(fmaxf(v[j] * inv, -448.f), 448.f));
    *reinterpret_cast<uint32_t*>(q + size_t(t) * K + g * 128 + lane * 4) = *reinterpret_cast<uint32_t*>(o);
    if (lane == 0) scales[size_t(t) * groups + g] = scale;
  }
}

}  // namespace xl_f8

using namespace xl_f8;

// x bf16 [T, K] (row pitch ldx) -> q e4m3 [T, K], scales fp32 [T, K/128].  gated != 0: x is [T, 2K] = [gate | up].
// `rows_dev` (optional device int) overrides T with a count known only on the device.
XL_API int xl_quant_act_1x128(const void* x, void* q, void* scales, int T, int K, int ldx, int gated, const void* rows_dev,
                              void* stream) {
  if (T <= 0) return 0;
  if (K % 128 || ldx % 4) return -2;
  long warps = long(T) * (K / 128);
  int blocks = int((warps + 7) / 8);
  if (blocks > 148 * 16) blocks = 148 * 16;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (gated)
    quant_act_kernel<true><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_fp8_e4m3*>(q),
                                                   static_cast<float*>(scales), T, K, ldx, static_cast<const int*>(rows_dev));
  else
    quant_act_kernel<false><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_fp8_e4m3*>(q),
                                                    static_cast<float*>(scales), T, K, ldx, static_cast<const int*>(rows_dev));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

static int launch_fp8(const void* A, const void* W, void* C, const void* sa, const void* sw, int M, int N, int K, int ldc,
                      const Grouped* g, int num_experts, int max_m_tiles, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 128 || ldc % 8 || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15)) return -2;
  const CUtensorMap* ta = xl_host::tmap_2d(A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, K, kBM, kBK, CU_TENSOR_MAP_SWIZZLE_128B);
  const CUtensorMap* tb = xl_host::tmap_2d(W, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, uint64_t(N) * num_experts, K, K, kBN, kBK,
                                           CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ta || !tb) return -4;
  Grouped grp;
  memset(&grp, 0, sizeof(grp));
  if (g) grp = *g;
  const size_t smem = size_t(kStages) * (kBM * kBK + kBN * kBK) + sizeof(Bars) + 1024;
  static bool set = false;
  if (!set) { cudaFuncSetAttribute(gemm_fp8_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)); set = true; }
  const int sms = xl_host::sm_count();
  const int m_tiles = g ? max_m_tiles : (M + kBM - 1) / kBM;
  const int n_tiles = (N + kBN - 1) / kBN;
  int grid = m_tiles * n_tiles;
  if (grid > sms) grid = sms;
  if (grid < 1) grid = 1;
  gemm_fp8_block_kernel<<<grid, kThreads, smem, st>>>(*ta, *tb, static_cast<__nv_bfloat16*>(C), static_cast<const float*>(sa),
                                                      static_cast<const float*>(sw), M, N, K, ldc, xl_host::status_word(), grp);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

XL_API int xl_gemm_fp8_block(const void* A, const void* W, void* C, const void* sa, const void* sw, int M, int N, int K, int ldc,
                             void* stream) {
  return launch_fp8(A, W, C, sa, sw, M, N, K, ldc, nullptr, 1, 0, static_cast<cudaStream_t>(stream));
}

XL_API int xl_grouped_gemm_fp8_block(const void* A, const void* W, void* C, const void* sa, const void* sw, int M_cap, int N, int K,
                                     int ldc, int num_experts, const void* tile_expert, const void* tile_row0,
                                     const void* tile_row_end, const void* num_m_tiles, int max_m_tiles, void* stream) {
  if (max_m_tiles <= 0) return 0;
  Grouped g;
  g.tile_expert = static_cast<const int*>(tile_expert);
  g.tile_row0 = static_cast<const int*>(tile_row0);
  g.tile_row_end = static_cast<const int*>(tile_row_end);
  g.num_m_tiles = static_cast<const int*>(num_m_tiles);
  g.enabled = 1;
  return launch_fp8(A, W, C, sa, sw, M_cap, N, K, ldc, &g, num_experts, max_m_tiles, static_cast<cudaStream_t>(stream));
}
