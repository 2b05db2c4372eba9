// Tensor-parallel fused collectives over NVLink peer memory (plain P2P loads/stores, system-scope flags).
//
// The reference finishes every row-parallel linear with an NCCL all-reduce, then runs a separate residual-add +
// RMSNorm kernel (xllm/core/layers/common/linear.cpp:822-825, qwen2_decoder_layer.cpp:99-100).  Here the chain is
//   GEMM (partials pushed to row owners from the epilogue, gemm_bf16.cu EPI_RS_PUSH)
//   -> this kernel: wait for the partials of all ranks, sum them in fp32, add the residual shard, RMSNorm,
//      and store the normalised rows into EVERY rank's activation buffer (all-gather by peer stores),
//      then wait until all ranks have delivered their rows.
// Each rank keeps only its own shard of the residual stream.
//
// Every wait is bounded (~2 s); on expiry the kernel records XL_ERR_WAIT_PEER in the status word and returns.
#include <string.h>

#include "common.cuh"

namespace xl {

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Wait until *p >= want.  Bounded by wall time; returns false on expiry.
__device__ __forceinline__ bool wait_flag_ge(const int* p, int want, unsigned long long limit_ns) {
  if (ld_acquire_sys(p) >= want) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
    for (int i = 0; i < 64; ++i) {
      if (ld_acquire_sys(p) >= want) return true;
      __nanosleep(40);
    }
    if (globaltimer_ns() - t0 > limit_ns) return false;
  }
}

struct TpReduceParams {
  const __nv_bfloat16* recv;      // local receive buffer [tp][shard_cap][H]
  const __nv_bfloat16* residual;  // local residual shard [shard][H]
  __nv_bfloat16* residual_out;    // local [shard][H]
  const __nv_bfloat16* norm_w;    // [H]
  __nv_bfloat16* gathered[8];     // every rank's activation buffer [T][H]
  int* flags_in;                  // local: partial-arrival flags [tp]   (written by the GEMMs of all ranks)
  int* gather_flags[8];           // every rank's gather-arrival flags [tp]
  int* gather_flags_local;        // == gather_flags[rank]
  int* done_counter;              // local
  int* epoch;                     // local, incremented at the end
  int* status;
  int tp, rank, shard, shard_cap, rows_here, H;
  float eps;
  unsigned long long limit_ns;
};

__global__ void __launch_bounds__(512) tp_reduce_norm_gather_kernel(const __grid_constant__ TpReduceParams p) {
  extern __shared__ float row_cache[];
  __shared__ float red[32];
  __shared__ int s_ok;
  const int want = *p.epoch + 1;
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int r = 0; r < p.tp && ok; ++r)
      if (!wait_flag_ge(p.flags_in + r, want, p.limit_ns)) ok = 0;
    if (!ok) atomicExch(p.status, XL_ERR_WAIT_PEER);
    s_ok = ok;
  }
  __syncthreads();
  const bool ok = s_ok != 0;
  const int H = p.H, nvec = H / 8;
  if (ok) {
    for (int row = blockIdx.x; row < p.rows_here; row += gridDim.x) {
      float ss = 0.f;
      for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
        float f[8];
        {
          uint4 a = *reinterpret_cast<const uint4*>(p.residual + size_t(row) * H + v * 8);
          uint32_t au[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) { float2 t = unpack_bf16x2(au[j]); f[2 * j] = t.x; f[2 * j + 1] = t.y; }
        }
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int r = 0; r < p.tp; ++r) {
          uint4 a = *reinterpret_cast<const uint4*>(p.recv + (size_t(r) * p.shard_cap + row) * H + v * 8);
          uint32_t au[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) { float2 t = unpack_bf16x2(au[j]); acc[2 * j] += t.x; acc[2 * j + 1] += t.y; }
        }
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          // y = bf16(sum of partials); residual' = bf16(y + residual): the same roundings as all-reduce + add
          float y0 = __bfloat162float(__float2bfloat16(acc[2 * j])), y1 = __bfloat162float(__float2bfloat16(acc[2 * j + 1]));
          o[j] = pack_bf16x2(y0 + f[2 * j], y1 + f[2 * j + 1]);
          float2 t = unpack_bf16x2(o[j]);
          f[2 * j] = t.x; f[2 * j + 1] = t.y;
        }
        *reinterpret_cast<uint4*>(p.residual_out + size_t(row) * H + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
#pragma unroll
        for (int j = 0; j < 8; ++j) { ss += f[j] * f[j]; row_cache[v * 8 + j] = f[j]; }
      }
      ss = warp_sum(ss);
      __syncthreads();
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
      __syncthreads();
      if (threadIdx.x < 32) {
        float t = threadIdx.x < (blockDim.x + 31) / 32 ? red[threadIdx.x] : 0.f;
        t = warp_sum(t);
        if (threadIdx.x == 0) red[0] = rsqrtf(t / float(H) + p.eps);
      }
      __syncthreads();
      const float rstd = red[0];
      const size_t grow = size_t(p.rank) * p.shard + row;      // global row index
      for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
        uint4 wv = *reinterpret_cast<const uint4*>(p.norm_w + v * 8);
        uint32_t wu[4] = {wv.x, wv.y, wv.z, wv.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 ww = unpack_bf16x2(wu[j]);
          float n0 = __bfloat162float(__float2bfloat16(row_cache[v * 8 + 2 * j] * rstd));
          float n1 = __bfloat162float(__float2bfloat16(row_cache[v * 8 + 2 * j + 1] * rstd));
          o[j] = pack_bf16x2(n0 * ww.x, n1 * ww.y);
        }
        const uint4 ov = make_uint4(o[0], o[1], o[2], o[3]);
        for (int r = 0; r < p.tp; ++r) {
          const int dst = (p.rank + r) % p.tp;                  // start with the local copy, spread peers
          *reinterpret_cast<uint4*>(p.gathered[dst] + grow * H + v * 8) = ov;
        }
      }
      __syncthreads();
    }
  }
  // ---- publish "rows of this rank are in place", then wait for everybody else's rows
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const int prev = atomicAdd(p.done_counter, 1);
    if (prev == int(gridDim.x) - 1) {
      *p.done_counter = 0;
      __threadfence_system();
      for (int r = 0; r < p.tp; ++r) st_release_sys(p.gather_flags[r] + p.rank, want);
      bool all = ok;
      for (int r = 0; r < p.tp && all; ++r)
        if (!wait_flag_ge(p.gather_flags_local + r, want, p.limit_ns)) all = false;
      if (!all) atomicExch(p.status, XL_ERR_WAIT_PEER);
      *p.epoch = want;
      __threadfence_system();
    }
  }
}

}  // namespace xl

using namespace xl;

// ---------------------------------------------------------------- host: allocation + IPC plumbing
XL_API void* xl_dev_malloc(long bytes) {
  void* p = nullptr;
  if (cudaMalloc(&p, size_t(bytes)) != cudaSuccess) return nullptr;
  cudaMemset(p, 0, size_t(bytes));
  return p;
}
XL_API int xl_dev_free(void* p) { return cudaFree(p) == cudaSuccess ? 0 : -1; }
XL_API int xl_ipc_get_handle(void* p, void* out64) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) return -1;
  memcpy(out64, &h, sizeof(h));
  return int(sizeof(h));
}
XL_API void* xl_ipc_open_handle(const void* in64) {
  cudaIpcMemHandle_t h;
  memcpy(&h, in64, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return nullptr;
  return p;
}
XL_API int xl_ipc_close_handle(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? 0 : -1; }

XL_API int xl_tp_reduce_norm_gather(const void* recv, const void* residual, void* residual_out, const void* norm_w,
                                    void* const* gathered, void* flags_in, void* const* gather_flags, void* done_counter,
                                    void* epoch, int tp, int rank, int shard, int shard_cap, int rows_here, int H, float eps,
                                    double timeout_s, void* stream) {
  if (tp < 1 || tp > 8 || H % 8) return -2;
  TpReduceParams p;
  memset(&p, 0, sizeof(p));
  p.recv = static_cast<const __nv_bfloat16*>(recv);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.residual_out = static_cast<__nv_bfloat16*>(residual_out);
  p.norm_w = static_cast<const __nv_bfloat16*>(norm_w);
  for (int r = 0; r < tp; ++r) {
    p.gathered[r] = static_cast<__nv_bfloat16*>(gathered[r]);
    p.gather_flags[r] = static_cast<int*>(gather_flags[r]);
  }
  p.gather_flags_local = static_cast<int*>(gather_flags[rank]);
  p.flags_in = static_cast<int*>(flags_in);
  p.done_counter = static_cast<int*>(done_counter);
  p.epoch = static_cast<int*>(epoch);
  p.status = xl_host::status_word();
  p.tp = tp; p.rank = rank; p.shard = shard; p.shard_cap = shard_cap; p.rows_here = rows_here; p.H = H; p.eps = eps;
  p.limit_ns = (unsigned long long)(timeout_s * 1e9);
  int grid = rows_here < 1 ? 1 : rows_here;
  const int sms = xl_host::sm_count();
  if (grid > 2 * sms) grid = 2 * sms;
  int threads = ((H / 8 + 31) / 32) * 32;
  threads = threads > 512 ? 512 : (threads < 32 ? 32 : threads);
  tp_reduce_norm_gather_kernel<<<grid, threads, H * sizeof(float), static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
