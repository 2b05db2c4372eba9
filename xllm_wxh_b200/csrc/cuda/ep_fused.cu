// Expert-parallel token dispatch and combine over NVLink peer memory (plain P2P stores, system-scope flags).
//
// Role of the reference's DeepEP-style all-to-all (xllm/core/layers/common/deep_ep.cpp:80-303,
// layers/mlu/fused_moe_all2all.cpp:111-252; vendor ops moe_all2all_gen_send_layout / dispatch / combine,
// kernels/param.h:539-663; capacity rule layers/mlu/fused_moe.cpp:97-106), which exists only for MLU; on CUDA the
// reference has no MoE path at all.  Per MoE layer (R ranks, every rank is source and destination) three kernels of this
// file run around the two grouped GEMMs:
//
//   ep_dispatch   one cooperative kernel:
//                 (1) count this rank's (token, slot) pairs per (destination, local expert);
//                 (2) exchange the count tables of all ranks (R x E_local ints each, written into every peer) and wait for
//                     them: every rank can now compute the whole layout.  A destination keeps its rows EXPERT-MAJOR and
//                     dense: expert e's rows start at the sum of the totals of experts < e, and inside an expert the rows
//                     of source 0 come first, then source 1, ...  So the sender knows where each of its rows goes, and
//                     the destination knows its tile table (128-row tiles per expert) before any row has arrived;
//                 (3) send: one warp per pair stores the row straight into its place in the destination's receive buffer,
//                     either as bf16 or quantised on the way to e4m3 with one scale per 128 columns (half the NVLink
//                     bytes; the layout of the block-scaled grouped GEMM), plus a (source rank, return slot) record;
//                 (4) the last CTA publishes "my rows are in place" to every rank and waits until all sources have said
//                     so: when the kernel ends, the grouped GEMM can read the receive buffer.  No sort, no gather.
//   ep_return     every expert output row is stored into the return slot [token * k + slot] of the rank it came from;
//                 the last CTA publishes the return flags.
//   ep_combine    waits for all return flags, then the top-k weighted sum (+ shared-expert / residual term) reads local
//                 memory only.
//
// All waits are bounded; on expiry XL_ERR_WAIT_PEER is recorded in the status word and the kernel carries on without
// touching what it waited for.
#include <cooperative_groups.h>
#include <string.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace xl {

__device__ __forceinline__ void ep_st_relaxed(int* p, int v) {
  asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ep_ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ep_ld_relaxed(const int* p) {
  int v;
  asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
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

constexpr int kEpMaxRanks = 8;
constexpr int kEpMaxTable = 1024;        // R * E_local count-table entries per rank

struct EpPeers {
  uint8_t* recv_x[kEpMaxRanks];      // [rows_cap][H] bf16, or [rows_cap][H] e4m3
  float* recv_scale[kEpMaxRanks];    // [rows_cap][H / 128] (fp8 rows)
  int2* recv_meta[kEpMaxRanks];      // [rows_cap] (source rank, return slot)
  int* counts_all[kEpMaxRanks];      // [2 parities][R sources][R * E_local]: count tables of every rank
  int* count_flags[kEpMaxRanks];     // [R]
  int* data_flags[kEpMaxRanks];      // [R]
  __nv_bfloat16* ret_y[kEpMaxRanks]; // [slots_cap][H]
  int* ret_flags[kEpMaxRanks];       // [R]
};

struct EpLocal {
  int* hist;                  // [R * E_local] this rank's pair counts (zero between calls)
  int* base;                  // [R * E_local] first row of (me -> d, e) in d's receive buffer
  int* fill;                  // [R * E_local] rows already placed
  int* abort_flag;            // [1] phase 2 gave up: phase 3 sends nothing
  int* done_counter;          // [4]
  int* epoch;                 // [1]
  int* status;
  // receive side of this rank, written by phase 2: the grouped GEMMs' tile table
  int* total_rows;            // [1]
  int* num_m_tiles;           // [1]
  int* tile_expert;           // [max_tiles]
  int* tile_row0;
  int* tile_row_end;
  int max_tiles;
  int R, rank, rows_cap, H, E_local, fp8;
  unsigned long long limit_ns;
};

__device__ __forceinline__ uint32_t ep_pack_e4m3x4(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return uint32_t(lo) | (uint32_t(hi) << 16);
}

__global__ void __launch_bounds__(256) ep_dispatch_kernel(const __grid_constant__ EpPeers peers, const __grid_constant__ EpLocal loc,
                                                          const __nv_bfloat16* __restrict__ x, const int* __restrict__ ids, int T,
                                                          int k, int ldx) {
  cg::grid_group grid = cg::this_grid();
  __shared__ int s_tot[kEpMaxTable];       // total rows of (destination, expert) over all sources
  __shared__ int s_below[kEpMaxTable];     // rows of sources before this rank
  __shared__ int s_ok;
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const long n = long(T) * k;
  const int RE = loc.R * loc.E_local;
  const int want = *loc.epoch + 1;
  const int parity = want & 1;

  // ---- (1) count
  for (long pair = blockIdx.x * long(blockDim.x) + threadIdx.x; pair < n; pair += long(gridDim.x) * blockDim.x) {
    const int id = ids[pair];
    if (id >= 0 && id < RE) atomicAdd(loc.hist + id, 1);       // id = destination * E_local + local expert
  }
  grid.sync();

  // ---- (2) exchange the count tables, compute the layout (block 0)
  if (blockIdx.x == 0) {
    for (int i = threadIdx.x; i < RE; i += blockDim.x) {
      const int c = loc.hist[i];
      for (int p = 0; p < loc.R; ++p) peers.counts_all[p][(size_t(parity) * loc.R + loc.rank) * RE + i] = c;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      for (int p = 0; p < loc.R; ++p) ep_st_relaxed(peers.count_flags[p] + loc.rank, want);
      int ok = 1;
      for (int s = 0; s < loc.R && ok; ++s)
        if (!ep_wait_ge(peers.count_flags[loc.rank] + s, want, loc.limit_ns)) ok = 0;
      if (!ok) atomicExch(loc.status, XL_ERR_WAIT_PEER);
      s_ok = ok;
      *loc.abort_flag = !ok;
    }
    __syncthreads();
    if (s_ok) {
      const int* all = peers.counts_all[loc.rank] + size_t(parity) * loc.R * RE;      // [source][destination * E_local + e]
      for (int i = threadIdx.x; i < RE; i += blockDim.x) {
        int tot = 0, below = 0;
        for (int s = 0; s < loc.R; ++s) {
          const int c = ep_ld_relaxed(all + size_t(s) * RE + i);
          tot += c;
          if (s < loc.rank) below += c;
        }
        s_tot[i] = tot;
        s_below[i] = below;
      }
      __syncthreads();
      for (int i = threadIdx.x; i < RE; i += blockDim.x) {
        const int d = i / loc.E_local, e = i - d * loc.E_local;
        int off = 0;
        for (int q = 0; q < e; ++q) off += s_tot[d * loc.E_local + q];                 // experts before e at destination d
        loc.base[i] = off + s_below[i];
        loc.fill[i] = 0;
      }
      if (threadIdx.x == 0) {
        // this rank's own receive side: rows per expert -> 128-row tiles
        int row = 0, nt = 0;
        for (int e = 0; e < loc.E_local; ++e) {
          const int cnt = s_tot[loc.rank * loc.E_local + e];
          const int end = min(row + cnt, loc.rows_cap);
          for (int r0 = row; r0 < end && nt < loc.max_tiles; r0 += 128) {
            loc.tile_expert[nt] = e;
            loc.tile_row0[nt] = r0;
            loc.tile_row_end[nt] = end;
            ++nt;
          }
          row += cnt;
        }
        if (row > loc.rows_cap) atomicExch(loc.status, XL_ERR_BOUNDS);
        *loc.total_rows = min(row, loc.rows_cap);
        *loc.num_m_tiles = nt;
      }
    }
    __threadfence();
  }
  grid.sync();

  // ---- (3) send
  const bool go = *loc.abort_flag == 0;
  const int H = loc.H;
  if (go) {
    for (long pair = blockIdx.x * long(warps_per_block) + (threadIdx.x >> 5); pair < n; pair += long(gridDim.x) * warps_per_block) {
      const int id = ids[pair];
      if (id < 0 || id >= RE) continue;      // invalid id: no row travels, the combine skips the slot
      const int d = id / loc.E_local;
      int pos = 0;
      if (lane == 0) pos = loc.base[id] + atomicAdd(loc.fill + id, 1);
      pos = __shfl_sync(0xffffffffu, pos, 0);
      // rows_cap is the same on every rank; the destination clamps its table the same way
      if (pos >= loc.rows_cap) {
        if (lane == 0) atomicExch(loc.status, XL_ERR_BOUNDS);
        continue;
      }
      const __nv_bfloat16* src = x + size_t(pair / k) * ldx;
      if (!loc.fp8) {
        const uint4* s4 = reinterpret_cast<const uint4*>(src);
        uint4* dst = reinterpret_cast<uint4*>(peers.recv_x[d] + size_t(pos) * H * 2);
        for (int v = lane; v < H / 8; v += 32) dst[v] = s4[v];
      } else {
        // 16 consecutive values per lane and pass: a 128-column block is 8 lanes
        uint8_t* dst = peers.recv_x[d] + size_t(pos) * H;
        float* dsc = peers.recv_scale[d] + size_t(pos) * (H / 128);
        for (int c_base = 0; c_base < H; c_base += 512) {         // every lane takes part in the shuffles of every pass
          const int c0 = c_base + lane * 16;
          const bool in = c0 < H;
          uint4 a = make_uint4(0, 0, 0, 0), b = a;
          if (in) {
            a = *reinterpret_cast<const uint4*>(src + c0);
            b = *reinterpret_cast<const uint4*>(src + c0 + 8);
          }
          const uint32_t u[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
          float f[16];
          float amax = 0.f;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float2 t = unpack_bf16x2(u[j]);
            f[2 * j] = t.x; f[2 * j + 1] = t.y;
            amax = fmaxf(amax, fmaxf(fabsf(t.x), fabsf(t.y)));
          }
          amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
          amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
          amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
          const float sc = fmaxf(amax, 1e-10f) / 448.f;
          const float inv = 1.f / sc;
          if (in) {
            *reinterpret_cast<uint4*>(dst + c0) = make_uint4(ep_pack_e4m3x4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv),
                                                            ep_pack_e4m3x4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv),
                                                            ep_pack_e4m3x4(f[8] * inv, f[9] * inv, f[10] * inv, f[11] * inv),
                                                            ep_pack_e4m3x4(f[12] * inv, f[13] * inv, f[14] * inv, f[15] * inv));
            if ((lane & 7) == 0) dsc[c0 / 128] = sc;
          }
        }
      }
      if (lane == 0) peers.recv_meta[d][pos] = make_int2(loc.rank, int(pair));
    }
  }
  // ---- (4) publish, then wait for every source
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const int prev = atomicAdd(loc.done_counter + 0, 1);
    if (prev == int(gridDim.x) - 1) {
      loc.done_counter[0] = 0;
      __threadfence_system();
      for (int p = 0; p < loc.R; ++p) ep_st_relaxed(peers.data_flags[p] + loc.rank, want);
      bool ok = go;
      for (int s = 0; s < loc.R && ok; ++s)
        if (!ep_wait_ge(peers.data_flags[loc.rank] + s, want, loc.limit_ns)) ok = false;
      if (!ok) atomicExch(loc.status, XL_ERR_WAIT_PEER);
      for (int i = 0; i < RE; ++i) loc.hist[i] = 0;          // ready for the next call
      __threadfence();
    }
  }
}

// y rows (expert-major, as received) go back to the return slot of the rank they came from
__global__ void ep_return_kernel(const __grid_constant__ EpPeers peers, const __grid_constant__ EpLocal loc,
                                 const __nv_bfloat16* __restrict__ y, int ldy) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int rows = *loc.total_rows;
  const int nvec = loc.H / 8;
  const int want = *loc.epoch + 1;
  for (int r = blockIdx.x * warps_per_block + (threadIdx.x >> 5); r < rows; r += gridDim.x * warps_per_block) {
    const int2 m = peers.recv_meta[loc.rank][r];
    if (m.x < 0 || m.x >= loc.R || m.y < 0) continue;
    const uint4* src = reinterpret_cast<const uint4*>(y + size_t(r) * ldy);
    uint4* dst = reinterpret_cast<uint4*>(peers.ret_y[m.x] + size_t(m.y) * loc.H);
    for (int v = lane; v < nvec; v += 32) dst[v] = src[v];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const int prev = atomicAdd(loc.done_counter + 1, 1);
    if (prev == int(gridDim.x) - 1) {
      loc.done_counter[1] = 0;
      __threadfence_system();
      for (int s = 0; s < loc.R; ++s) ep_st_relaxed(peers.ret_flags[s] + loc.rank, want);
    }
  }
}

// out[t] = sum_j w[t, j] * ret_y[t * k + j] (+ add[t]); waits for the return flags of all ranks first
__global__ void __launch_bounds__(256) ep_combine_kernel(const __grid_constant__ EpLocal loc, const int* __restrict__ ret_flags,
                                                         const __nv_bfloat16* __restrict__ ret_y, const int* __restrict__ ids,
                                                         const float* __restrict__ w, const __nv_bfloat16* __restrict__ add,
                                                         __nv_bfloat16* __restrict__ out, int T, int k) {
  __shared__ int s_ok;
  const int want = *loc.epoch + 1;
  const int RE = loc.R * loc.E_local;
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int s = 0; s < loc.R && ok; ++s)
      if (!ep_wait_ge(ret_flags + s, want, loc.limit_ns)) ok = 0;
    if (!ok) atomicExch(loc.status, XL_ERR_WAIT_PEER);
    s_ok = ok;
  }
  __syncthreads();
  const int H = loc.H, nvec = H / 8;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (s_ok) {
        for (int j = 0; j < k; ++j) {
          const int id = ids[t * k + j];
          if (id < 0 || id >= RE) continue;
          const float wj = w[t * k + j];
          const uint4 a = *reinterpret_cast<const uint4*>(ret_y + (size_t(t) * k + j) * H + v * 8);
          const uint32_t au[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 f = unpack_bf16x2(au[q]);
            acc[2 * q] += wj * f.x;
            acc[2 * q + 1] += wj * f.y;
          }
        }
      }
      if (add) {
        const uint4 a = *reinterpret_cast<const uint4*>(add + size_t(t) * H + v * 8);
        const uint32_t au[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = unpack_bf16x2(au[q]);
          acc[2 * q] += f.x;
          acc[2 * q + 1] += f.y;
        }
      }
      *reinterpret_cast<uint4*>(out + size_t(t) * H + v * 8) =
          make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(loc.done_counter + 2, 1);
    if (prev == int(gridDim.x) - 1) {          // every CTA has read the epoch and the flags: the layer's exchange is over
      loc.done_counter[2] = 0;
      *loc.epoch = want;
      __threadfence();
    }
  }
}

}  // namespace xl

using namespace xl;

// Pointers of one expert-parallel group, as the host passes them: per-rank arrays first, then this rank's scratch.
struct XlEpArgs {
  void* const* recv_x; void* const* recv_scale; void* const* recv_meta; void* const* counts_all; void* const* count_flags;
  void* const* data_flags; void* const* ret_y; void* const* ret_flags;
  void* hist; void* base; void* fill; void* abort_flag; void* done_counter; void* epoch;
  void* total_rows; void* num_m_tiles; void* tile_expert; void* tile_row0; void* tile_row_end;
  int max_tiles, R, rank, rows_cap, H, E_local, fp8;
  double timeout_s;
};

static int ep_fill(const XlEpArgs* a, EpPeers& p, EpLocal& l) {
  if (!a || a->R < 1 || a->R > kEpMaxRanks || a->H % 128 || a->R * a->E_local > kEpMaxTable) return -2;
  memset(&p, 0, sizeof(p));
  memset(&l, 0, sizeof(l));
  for (int r = 0; r < a->R; ++r) {
    p.recv_x[r] = static_cast<uint8_t*>(a->recv_x[r]);
    p.recv_scale[r] = a->recv_scale ? static_cast<float*>(a->recv_scale[r]) : nullptr;
    p.recv_meta[r] = static_cast<int2*>(a->recv_meta[r]);
    p.counts_all[r] = static_cast<int*>(a->counts_all[r]);
    p.count_flags[r] = static_cast<int*>(a->count_flags[r]);
    p.data_flags[r] = static_cast<int*>(a->data_flags[r]);
    p.ret_y[r] = static_cast<__nv_bfloat16*>(a->ret_y[r]);
    p.ret_flags[r] = static_cast<int*>(a->ret_flags[r]);
  }
  l.hist = static_cast<int*>(a->hist); l.base = static_cast<int*>(a->base); l.fill = static_cast<int*>(a->fill);
  l.abort_flag = static_cast<int*>(a->abort_flag);
  l.done_counter = static_cast<int*>(a->done_counter);
  l.epoch = static_cast<int*>(a->epoch);
  l.status = xl_host::status_word();
  l.total_rows = static_cast<int*>(a->total_rows); l.num_m_tiles = static_cast<int*>(a->num_m_tiles);
  l.tile_expert = static_cast<int*>(a->tile_expert); l.tile_row0 = static_cast<int*>(a->tile_row0);
  l.tile_row_end = static_cast<int*>(a->tile_row_end);
  l.max_tiles = a->max_tiles;
  l.R = a->R; l.rank = a->rank; l.rows_cap = a->rows_cap; l.H = a->H; l.E_local = a->E_local; l.fp8 = a->fp8;
  if (l.fp8 && !a->recv_scale) return -2;
  l.limit_ns = (unsigned long long)(a->timeout_s * 1e9);
  return 0;
}

// Dispatch of one layer: x [T, H] bf16 (row pitch ldx), ids [T, k] = destination rank * E_local + local expert (< 0: none).
XL_API int xl_ep_dispatch(const XlEpArgs* args, const void* x, const void* ids, int T, int k, int ldx, void* stream) {
  EpPeers p; EpLocal l;
  const int rc = ep_fill(args, p, l);
  if (rc) return rc;
  if (ldx % 8) return -2;
  // one resident wave (the kernel synchronises its grid): two CTAs of 256 threads per SM
  static int max_blocks_per_sm = 0;
  if (!max_blocks_per_sm) {
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&max_blocks_per_sm, ep_dispatch_kernel, 256, 0) != cudaSuccess || max_blocks_per_sm < 1)
      max_blocks_per_sm = 1;
  }
  int blocks = xl_host::sm_count() * (max_blocks_per_sm < 2 ? max_blocks_per_sm : 2);
  const long pairs = long(T) * k;
  const int need = int((pairs + 7) / 8);
  if (need < blocks) blocks = need < 1 ? 1 : need;
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  const int* ip = static_cast<const int*>(ids);
  void* kargs[] = {&p, &l, &xp, &ip, &T, &k, &ldx};
  const cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(ep_dispatch_kernel), dim3(blocks), dim3(256), kargs, 0,
                                                    static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : -1;
}

// Return of one layer: y [rows, H] bf16 (row pitch ldy) in the expert-major order of the receive buffer.
XL_API int xl_ep_return(const XlEpArgs* args, const void* y, int ldy, int max_rows, void* stream) {
  EpPeers p; EpLocal l;
  const int rc = ep_fill(args, p, l);
  if (rc) return rc;
  int blocks = (max_rows + 7) / 8;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 4) blocks = 148 * 4;
  ep_return_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(p, l, static_cast<const __nv_bfloat16*>(y), ldy);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// Combine of one layer into out [T, H]: waits for every rank's return, then out[t] = sum_j w[t, j] * returned row (+ add[t]).
XL_API int xl_ep_combine(const XlEpArgs* args, const void* ids, const void* w, const void* add, void* out, int T, int k,
                         void* stream) {
  EpPeers p; EpLocal l;
  const int rc = ep_fill(args, p, l);
  if (rc) return rc;
  int blocks = T < 1 ? 1 : T;
  if (blocks > 148 * 8) blocks = 148 * 8;
  ep_combine_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      l, p.ret_flags[l.rank], p.ret_y[l.rank], static_cast<const int*>(ids), static_cast<const float*>(w),
      static_cast<const __nv_bfloat16*>(add), static_cast<__nv_bfloat16*>(out), T, k);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
