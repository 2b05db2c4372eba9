// Expert-parallel token dispatch and combine over NVLink peer memory (plain P2P stores, system-scope flags).
//
// Role of the reference's DeepEP-style all-to-all (xllm/core/layers/common/deep_ep.cpp, layers/mlu/fused_moe_all2all.cpp:
// 111-252; vendor ops moe_all2all_dispatch / combine, param.h:539-663), which exists only for MLU; on CUDA the
// reference has no MoE path at all.  Protocol per MoE layer (R ranks, every rank is source and destination):
//
//   dispatch_send : one warp per (token, slot).  The row is written straight into the destination rank's receive
//                   buffer, region [source rank], at a position taken from a local cursor; a (local expert, return
//                   slot) record goes next to it.  The last CTA publishes per-destination row counts and an epoch
//                   flag (st.release.sys).
//   recv_prepare  : the destination waits for all R flags and flattens the R regions into one id list (-1 = empty),
//                   which the ordinary expert sort / grouped GEMM path consumes.
//   return_send   : every expert output row is stored into the source rank's return slot [token * k + slot];
//                   the last CTA publishes the return flags.
//   combine_wait  : the source waits for all return flags; the top-k weighted sum then reads purely local memory.
//
// All waits are bounded; on expiry XL_ERR_WAIT_PEER is recorded in the status word and the kernel returns.
#include <string.h>

#include "common.cuh"

namespace xl {

__device__ __forceinline__ void ep_st_relaxed(int* p, int v) {
  asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ep_ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void ep_st_release(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ep_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool ep_wait_ge(const int* p, int want, unsigned long long limit_ns) {
  if (ep_ld_acquire(p) >= want) return true;
  const unsigned long long t0 = ep_timer_ns();
  for (;;) {
    for (int i = 0; i < 64; ++i) {
      if (ep_ld_acquire(p) >= want) return true;
      __nanosleep(40);
    }
    if (ep_timer_ns() - t0 > limit_ns) return false;
  }
}

struct EpPeers {
  __nv_bfloat16* recv_x[8];   // [R][cap][H] on every rank
  int2* recv_meta[8];         // [R][cap]
  int* recv_count[8];         // [R]
  int* disp_flags[8];         // [R]
  __nv_bfloat16* ret_y[8];    // [slots_cap][H]
  int* ret_flags[8];          // [R]
};

struct EpLocal {
  int* send_cursor;           // [R]
  int* done_counter;          // [4]
  int* epoch;                 // [1]
  int* status;
  int R, rank, cap, H, E_local;
  unsigned long long limit_ns;
};

__global__ void ep_dispatch_send_kernel(const __grid_constant__ EpPeers peers, const __grid_constant__ EpLocal loc,
                                        const __nv_bfloat16* __restrict__ x, const int* __restrict__ ids, int T, int k, int ldx) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const long n = long(T) * k;
  const int nvec = loc.H / 8;
  for (long pair = blockIdx.x * long(warps_per_block) + (threadIdx.x >> 5); pair < n; pair += long(gridDim.x) * warps_per_block) {
    const int id = ids[pair];
    int d = id / loc.E_local;
    if (id < 0 || d >= loc.R) continue;     // invalid id: drop (the combine treats a missing return as zero)
    const int le = id - d * loc.E_local;
    int pos = 0;
    if (lane == 0) pos = atomicAdd(loc.send_cursor + d, 1);
    pos = __shfl_sync(0xffffffffu, pos, 0);
    if (pos >= loc.cap) {                   // capacity exceeded: recorded, row dropped
      if (lane == 0) atomicExch(loc.status, XL_ERR_BOUNDS);
      continue;
    }
    const size_t row = size_t(loc.rank) * loc.cap + pos;
    const uint4* src = reinterpret_cast<const uint4*>(x + size_t(pair / k) * ldx);
    uint4* dst = reinterpret_cast<uint4*>(peers.recv_x[d] + row * loc.H);
    for (int v = lane; v < nvec; v += 32) dst[v] = src[v];
    if (lane == 0) peers.recv_meta[d][row] = make_int2(le, int(pair));
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const int prev = atomicAdd(loc.done_counter + 0, 1);
    if (prev == int(gridDim.x) - 1) {
      loc.done_counter[0] = 0;
      __threadfence_system();
      const int e = *loc.epoch + 1;
      for (int d = 0; d < loc.R; ++d) {
        int c = loc.send_cursor[d];
        if (c > loc.cap) c = loc.cap;
        peers.recv_count[d][loc.rank] = c;
        loc.send_cursor[d] = 0;
      }
      __threadfence_system();
      // one fence (above), then relaxed flag stores that travel concurrently: a release store per peer costs a round trip each
      for (int d = 0; d < loc.R; ++d) ep_st_relaxed(peers.disp_flags[d] + loc.rank, e);
    }
  }
}

// ids_flat[s * cap + pos] = local expert of the row, or -1 where the region is empty
__global__ void ep_recv_prepare_kernel(const __grid_constant__ EpLocal loc, const int2* __restrict__ recv_meta,
                                       const int* __restrict__ recv_count, const int* __restrict__ disp_flags,
                                       int* __restrict__ ids_flat) {
  __shared__ int s_ok;
  const int want = *loc.epoch + 1;
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int s = 0; s < loc.R && ok; ++s)
      if (!ep_wait_ge(disp_flags + s, want, loc.limit_ns)) ok = 0;
    if (!ok) atomicExch(loc.status, XL_ERR_WAIT_PEER);
    s_ok = ok;
  }
  __syncthreads();
  const long n = long(loc.R) * loc.cap;
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < n; i += long(gridDim.x) * blockDim.x) {
    const int s = int(i / loc.cap), pos = int(i % loc.cap);
    ids_flat[i] = (s_ok && pos < recv_count[s]) ? recv_meta[i].x : -1;
  }
}

// y rows (sorted by expert) go back to the return slot of the rank they came from
__global__ void ep_return_send_kernel(const __grid_constant__ EpPeers peers, const __grid_constant__ EpLocal loc,
                                      const __nv_bfloat16* __restrict__ y, const int* __restrict__ sorted_src,
                                      const int* __restrict__ total_rows, const int2* __restrict__ recv_meta) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int R_rows = *total_rows;
  const int nvec = loc.H / 8;
  for (int r = blockIdx.x * warps_per_block + (threadIdx.x >> 5); r < R_rows; r += gridDim.x * warps_per_block) {
    const int flat = sorted_src[r];
    const int src_rank = flat / loc.cap;
    const int slot = recv_meta[flat].y;
    const uint4* src = reinterpret_cast<const uint4*>(y + size_t(r) * loc.H);
    uint4* dst = reinterpret_cast<uint4*>(peers.ret_y[src_rank] + size_t(slot) * loc.H);
    for (int v = lane; v < nvec; v += 32) dst[v] = src[v];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const int prev = atomicAdd(loc.done_counter + 1, 1);
    if (prev == int(gridDim.x) - 1) {
      loc.done_counter[1] = 0;
      __threadfence_system();
      const int e = *loc.epoch + 1;
      for (int s = 0; s < loc.R; ++s) ep_st_relaxed(peers.ret_flags[s] + loc.rank, e);
    }
  }
}

// waits for all return flags, then bumps the epoch (single CTA); the weighted sum follows as an ordinary kernel
__global__ void ep_combine_wait_kernel(const __grid_constant__ EpLocal loc, const int* __restrict__ ret_flags) {
  if (threadIdx.x == 0) {
    const int want = *loc.epoch + 1;
    bool ok = true;
    for (int s = 0; s < loc.R && ok; ++s)
      if (!ep_wait_ge(ret_flags + s, want, loc.limit_ns)) ok = false;
    if (!ok) atomicExch(loc.status, XL_ERR_WAIT_PEER);
    *loc.epoch = want;
    __threadfence_system();
  }
}

}  // namespace xl

using namespace xl;

static void fill(EpPeers& p, EpLocal& l, void* const* recv_x, void* const* recv_meta, void* const* recv_count,
                 void* const* disp_flags, void* const* ret_y, void* const* ret_flags, void* send_cursor, void* done_counter,
                 void* epoch, int R, int rank, int cap, int H, int E_local, double timeout_s) {
  memset(&p, 0, sizeof(p));
  memset(&l, 0, sizeof(l));
  for (int r = 0; r < R; ++r) {
    p.recv_x[r] = static_cast<__nv_bfloat16*>(recv_x[r]);
    p.recv_meta[r] = static_cast<int2*>(recv_meta[r]);
    p.recv_count[r] = static_cast<int*>(recv_count[r]);
    p.disp_flags[r] = static_cast<int*>(disp_flags[r]);
    p.ret_y[r] = static_cast<__nv_bfloat16*>(ret_y[r]);
    p.ret_flags[r] = static_cast<int*>(ret_flags[r]);
  }
  l.send_cursor = static_cast<int*>(send_cursor);
  l.done_counter = static_cast<int*>(done_counter);
  l.epoch = static_cast<int*>(epoch);
  l.status = xl_host::status_word();
  l.R = R; l.rank = rank; l.cap = cap; l.H = H; l.E_local = E_local;
  l.limit_ns = (unsigned long long)(timeout_s * 1e9);
}

// One call = the whole send side of a layer's dispatch.
XL_API int xl_ep_dispatch_send(void* const* recv_x, void* const* recv_meta, void* const* recv_count, void* const* disp_flags,
                               void* const* ret_y, void* const* ret_flags, void* send_cursor, void* done_counter, void* epoch,
                               int R, int rank, int cap, int H, int E_local, double timeout_s, const void* x, const void* ids,
                               int T, int k, int ldx, void* stream) {
  if (R < 1 || R > 8 || H % 8) return -2;
  EpPeers p; EpLocal l;
  fill(p, l, recv_x, recv_meta, recv_count, disp_flags, ret_y, ret_flags, send_cursor, done_counter, epoch, R, rank, cap, H,
       E_local, timeout_s);
  long pairs = long(T) * k;
  int blocks = int((pairs + 7) / 8);
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 4) blocks = 148 * 4;
  ep_dispatch_send_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(p, l, static_cast<const __nv_bfloat16*>(x),
                                                                                static_cast<const int*>(ids), T, k, ldx);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

XL_API int xl_ep_recv_prepare(const void* recv_meta_local, const void* recv_count_local, const void* disp_flags_local,
                              void* epoch, int R, int rank, int cap, double timeout_s, void* ids_flat, void* stream) {
  EpLocal l;
  memset(&l, 0, sizeof(l));
  l.epoch = static_cast<int*>(epoch);
  l.status = xl_host::status_word();
  l.R = R; l.rank = rank; l.cap = cap;
  l.limit_ns = (unsigned long long)(timeout_s * 1e9);
  long n = long(R) * cap;
  int blocks = int((n + 255) / 256);
  if (blocks > 148 * 4) blocks = 148 * 4;
  ep_recv_prepare_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      l, static_cast<const int2*>(recv_meta_local), static_cast<const int*>(recv_count_local),
      static_cast<const int*>(disp_flags_local), static_cast<int*>(ids_flat));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

XL_API int xl_ep_return_send(void* const* recv_x, void* const* recv_meta, void* const* recv_count, void* const* disp_flags,
                             void* const* ret_y, void* const* ret_flags, void* send_cursor, void* done_counter, void* epoch, int R,
                             int rank, int cap, int H, int E_local, double timeout_s, const void* y, const void* sorted_src,
                             const void* total_rows, const void* recv_meta_local, int max_rows, void* stream) {
  if (R < 1 || R > 8 || H % 8) return -2;
  EpPeers p; EpLocal l;
  fill(p, l, recv_x, recv_meta, recv_count, disp_flags, ret_y, ret_flags, send_cursor, done_counter, epoch, R, rank, cap, H,
       E_local, timeout_s);
  int blocks = (max_rows + 7) / 8;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 4) blocks = 148 * 4;
  ep_return_send_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      p, l, static_cast<const __nv_bfloat16*>(y), static_cast<const int*>(sorted_src), static_cast<const int*>(total_rows),
      static_cast<const int2*>(recv_meta_local));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

XL_API int xl_ep_combine_wait(const void* ret_flags_local, void* epoch, int R, double timeout_s, void* stream) {
  EpLocal l;
  memset(&l, 0, sizeof(l));
  l.epoch = static_cast<int*>(epoch);
  l.status = xl_host::status_word();
  l.R = R;
  l.limit_ns = (unsigned long long)(timeout_s * 1e9);
  ep_combine_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(l, static_cast<const int*>(ret_flags_local));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
