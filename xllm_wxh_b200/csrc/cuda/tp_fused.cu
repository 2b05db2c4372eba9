// Tensor-parallel fused collectives over NVLink peer memory (plain P2P loads/stores, system-scope flags).
//
// The reference finishes every row-parallel linear with an NCCL all-reduce, then runs a separate residual-add +
// RMSNorm kernel (xllm/core/layers/common/linear.cpp:822-825, qwen2_decoder_layer.cpp:99-100).  Here the chain is
//   GEMM whose last CTA publishes "partials of this rank are complete" to every rank (gemm_bf16.cu EPI_RS_PUSH).
//     pull mode (default): the partial result stays in the producing rank's buffer, which every peer has mapped;
//     push mode          : the epilogue stores each row into the owner's receive buffer (16-byte stores per lane,
//                          which NVLink carries poorly; kept for comparison);
//   -> this kernel: wait for the flags of all ranks, fetch (pull mode: coalesced 16-byte peer loads, one row of 8 KB
//      per CTA pass) and sum the partials of the rows this rank owns in fp32, add the residual shard, RMSNorm,
//      and store the normalised rows into EVERY rank's activation buffer (all-gather by coalesced peer stores),
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
// 16-byte load that bypasses L1 (the data was written by another GPU or by an earlier kernel through L2)
__device__ __forceinline__ uint4 ld_nc_v4(const __nv_bfloat16* p) {
  uint4 v;
  asm volatile("ld.global.relaxed.sys.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
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
  const __nv_bfloat16* recv;      // push mode: local receive buffer [tp][shard_cap][H]
  const __nv_bfloat16* partial[8];// pull mode (recv == nullptr): every rank's partial result [T][H] (peer mapped)
  const __nv_bfloat16* residual;  // local residual shard [shard][H]
  __nv_bfloat16* residual_out;    // local [shard][H]
  const __nv_bfloat16* norm_w;    // [H]
  __nv_bfloat16* gathered[8];     // every rank's activation buffer [T][H]
  int* flags_in;                  // local: partial-completion flags [tp]   (written by the GEMMs of all ranks)
  int* gather_cnt[8];             // every rank's arrival counters [2][8]: [epoch parity][source rank]
  int* gather_cnt_local;          // == gather_cnt[rank]
  int* done_counter;              // local
  int* epoch;                     // local, incremented at the end
  int* status;
  int tp, rank, shard, shard_cap, rows_here, H, total_rows, grid_cap;
  float eps;
  unsigned long long limit_ns;
  unsigned long long* trace;      // optional [8]: globaltimer stamps of the phases (diagnosis; null in normal use)
};

__device__ __forceinline__ void red_relaxed_sys_add(int* p, int v) {
  asm volatile("red.relaxed.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// release pattern for several peers at once: one fence, then relaxed updates that travel concurrently
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

// CTAs launched by rank `s` for its `rows` owned rows (same formula as the host launcher)
__device__ __forceinline__ int reduce_grid_of(int rows, int grid_cap) {
  const int g = rows < 1 ? 1 : rows;
  return g < grid_cap ? g : grid_cap;
}

// One CTA pass = one row (H <= 8 * blockDim) or one half of a row; the partials of the NEXT pass are requested
// before the current one is reduced, so the NVLink round trip overlaps the arithmetic and the stores.
template <int NR>
__global__ void __launch_bounds__(512, NR == 2 ? 2 : 1) tp_reduce_norm_gather_kernel(const __grid_constant__ TpReduceParams p) {
  // The GEMM that follows in the stream may set itself up (barriers, tensor memory) while this kernel still runs; it reads
  // what this kernel writes only behind its own grid-dependency wait.
  grid_dep_launch();
  extern __shared__ float row_cache[];
  __shared__ float red[32];
  __shared__ int s_ok;
  const int want = *p.epoch + 1;
  const int parity = want & 1;
  if (p.trace && threadIdx.x == 0) atomicMin(p.trace + 0, globaltimer_ns());
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int r = 0; r < NR && ok; ++r)
      if (!wait_flag_ge(p.flags_in + r, want, p.limit_ns)) ok = 0;
    if (!ok) atomicExch(p.status, XL_ERR_WAIT_PEER);
    s_ok = ok;
    if (p.trace) atomicMax(p.trace + 1, globaltimer_ns());
  }
  __syncthreads();
  const bool ok = s_ok != 0;
  const int H = p.H, nvec = H / 8;
  const int parts = (nvec + int(blockDim.x) - 1) / int(blockDim.x);     // passes per row

  auto fetch = [&](int row, int part, uint4 (&a)[NR], uint4& res) {
    const int v = part * int(blockDim.x) + int(threadIdx.x);
    if (v >= nvec) return;
    res = *reinterpret_cast<const uint4*>(p.residual + size_t(row) * H + v * 8);
    if (p.recv) {
#pragma unroll
      for (int r = 0; r < NR; ++r) a[r] = *reinterpret_cast<const uint4*>(p.recv + (size_t(r) * p.shard_cap + row) * H + v * 8);
    } else {
      const size_t off = (size_t(p.rank) * p.shard + row) * H + v * 8;
#pragma unroll
      for (int r = 0; r < NR; ++r) a[r] = ld_nc_v4(p.partial[r] + off);
    }
  };

  if (ok) {
    int row = blockIdx.x, part = 0;
    bool have = row < p.rows_here;
    uint4 cur[NR], cres = make_uint4(0, 0, 0, 0);
    if (have) fetch(row, part, cur, cres);
    float ss = 0.f;
    while (have) {
      int nrow = row, npart = part + 1;
      if (npart == parts) { npart = 0; nrow += gridDim.x; }
      const bool nhave = nrow < p.rows_here;
      uint4 nxt[NR], nres = make_uint4(0, 0, 0, 0);
      if (nhave) fetch(nrow, npart, nxt, nres);

      const int v = part * int(blockDim.x) + int(threadIdx.x);
      if (v < nvec) {
        float f[8], acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        {
          uint32_t au[4] = {cres.x, cres.y, cres.z, cres.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) { float2 t = unpack_bf16x2(au[j]); f[2 * j] = t.x; f[2 * j + 1] = t.y; }
        }
        // summed in rank order: every rank computes the same bits for the same row
#pragma unroll
        for (int r = 0; r < NR; ++r) {
          uint32_t au[4] = {cur[r].x, cur[r].y, cur[r].z, cur[r].w};
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
      if (part == parts - 1) {
        ss = warp_sum(ss);
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
        for (int w = threadIdx.x; w < nvec; w += blockDim.x) {
          uint4 wv = *reinterpret_cast<const uint4*>(p.norm_w + w * 8);
          uint32_t wu[4] = {wv.x, wv.y, wv.z, wv.w};
          uint32_t o[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 ww = unpack_bf16x2(wu[j]);
            float n0 = __bfloat162float(__float2bfloat16(row_cache[w * 8 + 2 * j] * rstd));
            float n1 = __bfloat162float(__float2bfloat16(row_cache[w * 8 + 2 * j + 1] * rstd));
            o[j] = pack_bf16x2(n0 * ww.x, n1 * ww.y);
          }
          const uint4 ov = make_uint4(o[0], o[1], o[2], o[3]);
#pragma unroll
          for (int r = 0; r < NR; ++r) {
            const int dst = (p.rank + r) % NR;                  // start with the local copy, spread peers
            *reinterpret_cast<uint4*>(p.gathered[dst] + grow * H + w * 8) = ov;
          }
        }
        ss = 0.f;
        __syncthreads();     // row_cache and red are reused by the next row
      }
#pragma unroll
      for (int r = 0; r < NR; ++r) cur[r] = nxt[r];
      cres = nres;
      row = nrow; part = npart; have = nhave;
    }
  }
  // ---- tell every rank "the rows of this CTA are in place" (release: ordered after the CTA's peer stores).  Only the
  //      CTA that reports last on this rank then waits until the CTAs of all ranks have reported: a wait in every CTA
  //      would need the whole grid resident at once, which a grid larger than one wave is not.  The counters of the
  //      two epoch parities alternate, so the reset below cannot collide with a rank that is already one step ahead.
  __syncthreads();
  if (threadIdx.x == 0) {
    if (p.trace) atomicMax(p.trace + 2, globaltimer_ns());
    fence_acq_rel_sys();
#pragma unroll
    for (int r = 0; r < NR; ++r) red_relaxed_sys_add(p.gather_cnt[(p.rank + r) % NR] + parity * 8 + p.rank, 1);
    if (p.trace) atomicMax(p.trace + 3, globaltimer_ns());
    const int prev = atomicAdd(p.done_counter, 1);
    if (prev == int(gridDim.x) - 1) {
      bool all = ok;
      for (int r = 0; r < NR && all; ++r) {
        const int rows_r = max(0, min(p.shard, p.total_rows - r * p.shard));
        if (!wait_flag_ge(p.gather_cnt_local + parity * 8 + r, reduce_grid_of(rows_r, p.grid_cap), p.limit_ns)) all = false;
      }
      if (!all) atomicExch(p.status, XL_ERR_WAIT_PEER);
      if (p.trace) p.trace[4] = globaltimer_ns();
      *p.done_counter = 0;
      for (int r = 0; r < NR; ++r) p.gather_cnt_local[parity * 8 + r] = 0;
      *p.epoch = want;
      __threadfence();
      if (p.trace) p.trace[5] = globaltimer_ns();
    }
  }
}


// ---------------------------------------------------------------- bulk-copy variant of the pull kernel
// Same protocol and arithmetic as tp_reduce_norm_gather_kernel in pull mode, but the rows travel as bulk asynchronous
// copies (`cp.async.bulk`, 1-D TMA): a producer thread requests the NR partial rows and the residual row of the next
// passes into a ring of shared-memory stages (one mbarrier per stage), the other threads reduce out of shared memory,
// and the normalised row leaves as one bulk store per destination rank.  Whole rows per request keep the NVLink
// packets large and many rows in flight per SM; no load carries a cluster broadcast.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}

constexpr int kBulkThreads = 256;

template <int NR>
__global__ void __launch_bounds__(kBulkThreads, NR <= 4 ? 2 : 1) tp_pull_bulk_kernel(const __grid_constant__ TpReduceParams p, int stages) {
  // The GEMM that follows in the stream may set itself up (barriers, tensor memory) while this kernel still runs; it reads
  // what this kernel writes only behind its own grid-dependency wait.
  grid_dep_launch();
  extern __shared__ __align__(128) uint8_t bsm[];
  __shared__ float red[32];
  __shared__ int s_ok;
  __shared__ uint64_t full[8];
  const int H = p.H, row_bytes = H * 2, nvec = H / 8;
  const int stage_bytes = (NR + 1) * row_bytes;            // NR partial rows + the residual row
  uint8_t* out_buf = bsm + stages * stage_bytes;           // two normalised rows (double buffered for the bulk stores)
  const int want = *p.epoch + 1;
  const int parity = want & 1;
  const int tid = threadIdx.x;
  if (p.trace && tid == 0) atomicMin(p.trace + 0, globaltimer_ns());
  if (tid == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    mbar_fence_init();
    int ok = 1;
    for (int r = 0; r < NR && ok; ++r)
      if (!wait_flag_ge(p.flags_in + r, want, p.limit_ns)) ok = 0;
    if (!ok) atomicExch(p.status, XL_ERR_WAIT_PEER);
    s_ok = ok;
    if (p.trace) atomicMax(p.trace + 1, globaltimer_ns());
  }
  __syncthreads();
  bool ok = s_ok != 0;
  const int my_rows = ok && int(blockIdx.x) < p.rows_here ? (p.rows_here - 1 - int(blockIdx.x)) / int(gridDim.x) + 1 : 0;

  auto request = [&](int i) {          // producer thread: fetch pass i into its stage
    const int s = i % stages;
    const int row = int(blockIdx.x) + i * int(gridDim.x);
    uint8_t* st = bsm + s * stage_bytes;
    mbar_arrive_expect_tx(&full[s], uint32_t(stage_bytes));
    const size_t off = (size_t(p.rank) * p.shard + row) * H;
#pragma unroll
    for (int r = 0; r < NR; ++r) bulk_load(st + r * row_bytes, p.partial[r] + off, uint32_t(row_bytes), &full[s]);
    bulk_load(st + NR * row_bytes, p.residual + size_t(row) * H, uint32_t(row_bytes), &full[s]);
  };
  if (tid == 0)
    for (int i = 0; i < my_rows && i < stages; ++i) request(i);

  for (int i = 0; i < my_rows && ok; ++i) {
    const int s = i % stages;
    const int row = int(blockIdx.x) + i * int(gridDim.x);
    if (!mbar_wait(&full[s], (i / stages) & 1)) {
      if (tid == 0) atomicExch(p.status, XL_ERR_WAIT_FULL);
      ok = false;
      break;
    }
    const uint8_t* st = bsm + s * stage_bytes;
    float ss = 0.f;
    float fcache[4][8];                 // this thread's elements of the row (H <= 8192: at most 4 vectors of 8)
    int nv = 0;
    for (int v = tid; v < nvec; v += kBulkThreads, ++nv) {
      float f[8], acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      {
        const uint4 a = *reinterpret_cast<const uint4*>(st + NR * row_bytes + v * 16);
        uint32_t au[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { float2 t = unpack_bf16x2(au[j]); f[2 * j] = t.x; f[2 * j + 1] = t.y; }
      }
#pragma unroll
      for (int r = 0; r < NR; ++r) {      // rank order: the same bits on every rank
        const uint4 a = *reinterpret_cast<const uint4*>(st + r * row_bytes + v * 16);
        uint32_t au[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { float2 t = unpack_bf16x2(au[j]); acc[2 * j] += t.x; acc[2 * j + 1] += t.y; }
      }
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float y0 = __bfloat162float(__float2bfloat16(acc[2 * j])), y1 = __bfloat162float(__float2bfloat16(acc[2 * j + 1]));
        o[j] = pack_bf16x2(y0 + f[2 * j], y1 + f[2 * j + 1]);
        float2 t = unpack_bf16x2(o[j]);
        f[2 * j] = t.x; f[2 * j + 1] = t.y;
      }
      *reinterpret_cast<uint4*>(p.residual_out + size_t(row) * H + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
#pragma unroll
      for (int j = 0; j < 8; ++j) { ss += f[j] * f[j]; fcache[nv][j] = f[j]; }
    }
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();                     // every thread has read the stage: it can be refilled
    if (tid == 0) {
      if (i + stages < my_rows) request(i + stages);
      // the out buffer used two rows ago must have been read by its bulk stores
      asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
    }
    if (tid < 32) {
      float t = tid < kBulkThreads / 32 ? red[tid] : 0.f;
      t = warp_sum(t);
      if (tid == 0) red[0] = rsqrtf(t / float(H) + p.eps);
    }
    __syncthreads();
    const float rstd = red[0];
    uint8_t* ob = out_buf + (i & 1) * row_bytes;
    nv = 0;
    for (int v = tid; v < nvec; v += kBulkThreads, ++nv) {
      const uint4 wv = *reinterpret_cast<const uint4*>(p.norm_w + v * 8);
      uint32_t wu[4] = {wv.x, wv.y, wv.z, wv.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 ww = unpack_bf16x2(wu[j]);
        float n0 = __bfloat162float(__float2bfloat16(fcache[nv][2 * j] * rstd));
        float n1 = __bfloat162float(__float2bfloat16(fcache[nv][2 * j + 1] * rstd));
        o[j] = pack_bf16x2(n0 * ww.x, n1 * ww.y);
      }
      *reinterpret_cast<uint4*>(ob + v * 16) = make_uint4(o[0], o[1], o[2], o[3]);
    }
    fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) {
      const size_t grow = size_t(p.rank) * p.shard + row;
#pragma unroll
      for (int r = 0; r < NR; ++r) bulk_store(p.gathered[(p.rank + r) % NR] + grow * H, ob, uint32_t(row_bytes));
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
  }
  // ---- all bulk stores of this CTA are complete before its arrival is published
  __syncthreads();
  if (tid == 0) {
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    asm volatile("fence.proxy.async.global;" ::: "memory");      // bulk (async proxy) writes before the release below
    if (p.trace) atomicMax(p.trace + 2, globaltimer_ns());
    fence_acq_rel_sys();
#pragma unroll
    for (int r = 0; r < NR; ++r) red_relaxed_sys_add(p.gather_cnt[(p.rank + r) % NR] + parity * 8 + p.rank, 1);
    if (p.trace) atomicMax(p.trace + 3, globaltimer_ns());
    const int prev = atomicAdd(p.done_counter, 1);
    if (prev == int(gridDim.x) - 1) {
      bool all = s_ok != 0;
      for (int r = 0; r < NR && all; ++r) {
        const int rows_r = max(0, min(p.shard, p.total_rows - r * p.shard));
        if (!wait_flag_ge(p.gather_cnt_local + parity * 8 + r, reduce_grid_of(rows_r, p.grid_cap), p.limit_ns)) all = false;
      }
      if (!all) atomicExch(p.status, XL_ERR_WAIT_PEER);
      if (p.trace) p.trace[4] = globaltimer_ns();
      *p.done_counter = 0;
      for (int r = 0; r < NR; ++r) p.gather_cnt_local[parity * 8 + r] = 0;
      *p.epoch = want;
      __threadfence();
      if (p.trace) p.trace[5] = globaltimer_ns();
    }
  }
}


// ---------------------------------------------------------------- NVLS variant: the reduction runs inside the NVSwitch
// `mc_partial` and `mc_gathered` are multicast addresses (one NVLink multicast object bound to the same-size buffer of
// every rank).  The owner of a row issues ONE `multimem.ld_reduce` per 16 bytes: the switch fetches the partial rows of
// all ranks, adds them in fp32 and returns the bf16 sum, so (N-1)/N of the reduce-scatter traffic never enters this
// GPU; the normalised row leaves as ONE `multimem.st` per 16 bytes, which the switch replicates into every rank's
// activation buffer, so this GPU sends each row once instead of N-1 times.  Flags stay on plain peer addresses with the
// same protocol as the kernels above (epoch-valued GEMM flags in, per-CTA arrivals out, last CTA waits and resets).
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const __nv_bfloat16* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_v4(__nv_bfloat16* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

struct TpNvlsParams {
  const __nv_bfloat16* mc_partial;   // multicast view of the partial GEMM results [T][H]
  __nv_bfloat16* mc_gathered;        // multicast view of the activation buffers   [T][H]
  const __nv_bfloat16* local_in;     // rows of this rank that need no reduction [shard][H] (kernels without REDUCE_IN)
  __nv_bfloat16* local_out;          // normalised rows kept on this rank [shard][H] (kernels without GATHER_OUT)
  const __nv_bfloat16* residual;     // local residual shard [shard][H]
  __nv_bfloat16* residual_out;
  const __nv_bfloat16* norm_w;
  int* flags_in;                     // local: epoch of every rank's finished GEMM [tp]
  int* gather_cnt[8];                // every rank's arrival counters [2][8]
  int* gather_cnt_local;
  int* done_counter;
  int* epoch;
  int* status;
  int tp, rank, shard, rows_here, H, total_rows, grid_cap, rows_per_cta;
  float eps;
  unsigned long long limit_ns;
  unsigned long long* trace;
};

// CTAs that a rank with `rows` owned rows launches (the same formula on the host)
__host__ __device__ __forceinline__ int nvls_grid_of(int rows, int rows_per_cta, int grid_cap) {
  const int g = rows < 1 ? 1 : (rows + rows_per_cta - 1) / rows_per_cta;
  return g < grid_cap ? g : grid_cap;
}

constexpr int kNvlsThreads = 256;

// VPT = 16-byte vectors per thread and row (H <= 2048 * VPT).  Small CTAs, several per SM: every row of a shard of a
// few hundred rows has its own resident CTA, so the switch round trips of all rows overlap.
//
// The two halves of the step can also run apart (tensor-parallel attention around a row-sharded MLP):
//   REDUCE_IN && !GATHER_OUT : reduce-scatter + residual + RMSNorm, the normalised rows stay on their owner;
//   !REDUCE_IN && GATHER_OUT : rows computed by their owner + residual + RMSNorm, all-gathered to every rank.
template <int NR, int VPT, bool REDUCE_IN, bool GATHER_OUT>
__global__ void __launch_bounds__(kNvlsThreads, VPT <= 2 ? 4 : 2) tp_nvls_reduce_norm_gather_kernel(const __grid_constant__ TpNvlsParams p) {
  // The GEMM that follows in the stream may set itself up (barriers, tensor memory) while this kernel still runs; it reads
  // what this kernel writes only behind its own grid-dependency wait.
  grid_dep_launch();
  __shared__ float red[32];
  __shared__ int s_ok;
  const int tid = threadIdx.x;
  const int want = *p.epoch + 1;
  const int parity = want & 1;
  const int H = p.H, nvec = H / 8;
  if (p.trace && tid == 0) atomicMin(p.trace + 0, globaltimer_ns());
  if (tid == 0) {
    int ok = 1;
    if (REDUCE_IN)
      for (int r = 0; r < NR && ok; ++r)
        if (!wait_flag_ge(p.flags_in + r, want, p.limit_ns)) ok = 0;
    if (!ok) atomicExch(p.status, XL_ERR_WAIT_PEER);
    s_ok = ok;
    if (p.trace) atomicMax(p.trace + 1, globaltimer_ns());
  }
  __syncthreads();
  const bool ok = s_ok != 0;

  auto fetch = [&](int row, uint4 (&a)[VPT]) {
    const size_t grow = size_t(p.rank) * p.shard + row;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = tid + i * kNvlsThreads;
      if (v < nvec)
        a[i] = REDUCE_IN ? multimem_ld_reduce_bf16x8(p.mc_partial + grow * H + v * 8)
                         : *reinterpret_cast<const uint4*>(p.local_in + size_t(row) * H + v * 8);
    }
  };

  if (ok) {
    // Two rows ahead: while row i is normalised and leaves through `multimem.st` (traffic INTO every GPU), the
    // `multimem.ld_reduce` of rows i+1 and i+2 are in flight (traffic OUT of every GPU): both link directions stay busy.
    // A CTA therefore takes several rows (the grid is a fraction of the shard's rows).
    const int stride = int(gridDim.x);
    int row = blockIdx.x;
    uint4 cur[VPT], nx1[VPT];
    if (row < p.rows_here) fetch(row, cur);
    if (row + stride < p.rows_here) fetch(row + stride, nx1);
    while (row < p.rows_here) {
      uint4 nx2[VPT];
      if (row + 2 * stride < p.rows_here) fetch(row + 2 * stride, nx2);
      float f[VPT][8];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = tid + i * kNvlsThreads;
        if (v < nvec) {
          const uint4 rv = *reinterpret_cast<const uint4*>(p.residual + size_t(row) * H + v * 8);
          const uint32_t yu[4] = {cur[i].x, cur[i].y, cur[i].z, cur[i].w};
          const uint32_t ru[4] = {rv.x, rv.y, rv.z, rv.w};
          uint32_t o[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            // y = bf16(sum of partials) comes from the switch; residual' = bf16(y + residual), as all-reduce + add
            const float2 y = unpack_bf16x2(yu[j]), r = unpack_bf16x2(ru[j]);
            o[j] = pack_bf16x2(y.x + r.x, y.y + r.y);
            const float2 t = unpack_bf16x2(o[j]);
            f[i][2 * j] = t.x; f[i][2 * j + 1] = t.y;
            ss += t.x * t.x + t.y * t.y;
          }
          *reinterpret_cast<uint4*>(p.residual_out + size_t(row) * H + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
      ss = warp_sum(ss);
      if ((tid & 31) == 0) red[tid >> 5] = ss;
      __syncthreads();
      if (tid < 32) {
        float t = tid < kNvlsThreads / 32 ? red[tid] : 0.f;
        t = warp_sum(t);
        if (tid == 0) red[0] = rsqrtf(t / float(H) + p.eps);
      }
      __syncthreads();
      const float rstd = red[0];
      const size_t grow = size_t(p.rank) * p.shard + row;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = tid + i * kNvlsThreads;
        if (v < nvec) {
          const uint4 wv = *reinterpret_cast<const uint4*>(p.norm_w + v * 8);
          const uint32_t wu[4] = {wv.x, wv.y, wv.z, wv.w};
          uint32_t o[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 ww = unpack_bf16x2(wu[j]);
            const float n0 = __bfloat162float(__float2bfloat16(f[i][2 * j] * rstd));
            const float n1 = __bfloat162float(__float2bfloat16(f[i][2 * j + 1] * rstd));
            o[j] = pack_bf16x2(n0 * ww.x, n1 * ww.y);
          }
          if (GATHER_OUT) multimem_st_v4(p.mc_gathered + grow * H + v * 8, make_uint4(o[0], o[1], o[2], o[3]));
          else *reinterpret_cast<uint4*>(p.local_out + size_t(row) * H + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
      __syncthreads();                   // red[] is reused by the next row
#pragma unroll
      for (int i = 0; i < VPT; ++i) { cur[i] = nx1[i]; nx1[i] = nx2[i]; }
      row += stride;
    }
  }
  // ---- arrival: this CTA's multicast stores are ordered before the counters that every rank's last CTA waits on
  __syncthreads();
  if (tid == 0) {
    if (p.trace) atomicMax(p.trace + 2, globaltimer_ns());
    if (GATHER_OUT) {
      fence_acq_rel_sys();
#pragma unroll
      for (int r = 0; r < NR; ++r) red_relaxed_sys_add(p.gather_cnt[(p.rank + r) % NR] + parity * 8 + p.rank, 1);
    } else {
      __threadfence();
    }
    if (p.trace) atomicMax(p.trace + 3, globaltimer_ns());
    const int prev = atomicAdd(p.done_counter, 1);
    if (prev == int(gridDim.x) - 1) {
      bool all = ok;
      if (GATHER_OUT) {
        for (int r = 0; r < NR && all; ++r) {
          const int rows_r = max(0, min(p.shard, p.total_rows - r * p.shard));
          if (!wait_flag_ge(p.gather_cnt_local + parity * 8 + r, nvls_grid_of(rows_r, p.rows_per_cta, p.grid_cap), p.limit_ns)) all = false;
        }
        if (!all) atomicExch(p.status, XL_ERR_WAIT_PEER);
      }
      if (p.trace) p.trace[4] = globaltimer_ns();
      *p.done_counter = 0;
      if (GATHER_OUT)
        for (int r = 0; r < NR; ++r) p.gather_cnt_local[parity * 8 + r] = 0;
      *p.epoch = want;
      __threadfence();
      if (p.trace) p.trace[5] = globaltimer_ns();
    }
  }
}

// Partial results that some other kernel produced (an fp8 GEMM, the routed experts of a MoE layer) enter the fused
// reduction here: the rows are copied into this rank's peer-visible partial buffer and, when the last CTA has finished,
// this rank's epoch goes to every rank's flag word, exactly as the row-parallel GEMM's epilogue does.
struct TpPublishParams {
  const uint4* src;       // [rows][ld16] 16-byte words
  uint4* dst;             // [rows][row16]
  long ld16;
  int rows, row16;
  int* flags[8];
  int* done_counter;
  const int* epoch;
  int tp, rank;
};

__global__ void __launch_bounds__(256) tp_publish_rows_kernel(const __grid_constant__ TpPublishParams p) {
  const long total = long(p.rows) * p.row16;
  for (long i = long(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
    const long r = i / p.row16;
    const int c = int(i - r * p.row16);
    p.dst[i] = __ldg(p.src + r * p.ld16 + c);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int prev = atomicAdd(p.done_counter, 1);
    if (prev == int(gridDim.x) - 1) {
      *p.done_counter = 0;
      __threadfence_system();
      const int e = *p.epoch + 1;
      for (int r = 0; r < p.tp; ++r)
        asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p.flags[r] + p.rank), "r"(e) : "memory");
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

static unsigned long long* g_trace = nullptr;
// Diagnosis hook: device buffer of 8 uint64 that receives globaltimer stamps of the next reduce kernels
// ([0] first CTA start (min; preset to a large value), [1] flags seen, [2] rows done, [3] arrivals sent, [4] all arrived, [5] reset).
XL_API void xl_tp_set_trace(void* buf) { g_trace = static_cast<unsigned long long*>(buf); }

static int g_nvls_rows_per_cta = 4;
// Tuning hook: rows that one CTA of the NVLS reduce kernel takes in turn (1 = one resident CTA per row).
XL_API void xl_tp_nvls_rows_per_cta(int n) { g_nvls_rows_per_cta = n < 1 ? 1 : n; }

static int g_bulk = 1;
// Comparison hook: 1 (default) the pull path uses the bulk-copy kernel, 0 the per-thread load / store kernel.
XL_API void xl_tp_use_bulk(int on) { g_bulk = on; }

static int launch_reduce(const void* recv, void* const* partials, const void* residual, void* residual_out, const void* norm_w,
                         void* const* gathered, void* flags_in, void* const* gather_cnt, void* done_counter, void* epoch, int tp,
                         int rank, int shard, int shard_cap, int rows_here, int total_rows, int H, float eps, double timeout_s,
                         void* stream) {
  if ((tp != 2 && tp != 4 && tp != 8) || H % 8 || H > 8 * 1024) return -2;
  if (!recv && !partials) return -2;
  TpReduceParams p;
  memset(&p, 0, sizeof(p));
  p.recv = static_cast<const __nv_bfloat16*>(recv);
  if (!recv)
    for (int r = 0; r < tp; ++r) p.partial[r] = static_cast<const __nv_bfloat16*>(partials[r]);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.residual_out = static_cast<__nv_bfloat16*>(residual_out);
  p.norm_w = static_cast<const __nv_bfloat16*>(norm_w);
  for (int r = 0; r < tp; ++r) {
    p.gathered[r] = static_cast<__nv_bfloat16*>(gathered[r]);
    p.gather_cnt[r] = static_cast<int*>(gather_cnt[r]);
  }
  p.gather_cnt_local = static_cast<int*>(gather_cnt[rank]);
  p.flags_in = static_cast<int*>(flags_in);
  p.done_counter = static_cast<int*>(done_counter);
  p.epoch = static_cast<int*>(epoch);
  p.status = xl_host::status_word();
  p.tp = tp; p.rank = rank; p.shard = shard; p.shard_cap = shard_cap; p.rows_here = rows_here; p.H = H; p.eps = eps;
  p.total_rows = total_rows;
  // one wave: every CTA must be resident at once (a CTA ends with a release that waits for its peer stores, and a second
  // wave would start only after that); two CTAs of 512 threads fit on an SM for two ranks, one for more
  p.grid_cap = (tp == 2 ? 2 : 1) * xl_host::sm_count();
  p.limit_ns = (unsigned long long)(timeout_s * 1e9);
  p.trace = g_trace;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!recv && g_bulk && H % 64 == 0 && H <= 8192) {
    // bulk-copy kernel, one resident wave: two CTAs per SM up to four ranks (two or three stages each), one CTA per SM
    // with as many stages as fit for eight ranks
    const int per_sm = tp <= 4 ? 2 : 1;
    p.grid_cap = per_sm * xl_host::sm_count();
    int grid = rows_here < 1 ? 1 : rows_here;
    if (grid > p.grid_cap) grid = p.grid_cap;
    const int row_bytes = H * 2, stage_bytes = (tp + 1) * row_bytes;
    int stages = ((per_sm == 2 ? 108 : 200) * 1024 - 2 * row_bytes) / stage_bytes;
    if (stages > 8) stages = 8;
    if (stages >= 2) {
      const size_t smem = size_t(stages) * stage_bytes + 2 * row_bytes;
      static bool set[3] = {false, false, false};
      const int idx = tp == 2 ? 0 : (tp == 4 ? 1 : 2);
      if (!set[idx]) {
        if (tp == 2) cudaFuncSetAttribute(tp_pull_bulk_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        else if (tp == 4) cudaFuncSetAttribute(tp_pull_bulk_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        else cudaFuncSetAttribute(tp_pull_bulk_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        set[idx] = true;
      }
      if (tp == 2) tp_pull_bulk_kernel<2><<<grid, kBulkThreads, smem, st>>>(p, stages);
      else if (tp == 4) tp_pull_bulk_kernel<4><<<grid, kBulkThreads, smem, st>>>(p, stages);
      else tp_pull_bulk_kernel<8><<<grid, kBulkThreads, smem, st>>>(p, stages);
      return cudaGetLastError() == cudaSuccess ? 0 : -1;
    }
  }
  int grid = rows_here < 1 ? 1 : rows_here;
  if (grid > p.grid_cap) grid = p.grid_cap;
  int threads = ((H / 8 + 31) / 32) * 32;
  threads = threads > 512 ? 512 : (threads < 32 ? 32 : threads);
  const size_t smem = H * sizeof(float);
  if (tp == 2) tp_reduce_norm_gather_kernel<2><<<grid, threads, smem, st>>>(p);
  else if (tp == 4) tp_reduce_norm_gather_kernel<4><<<grid, threads, smem, st>>>(p);
  else tp_reduce_norm_gather_kernel<8><<<grid, threads, smem, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// Push variant: the GEMMs of all ranks have stored their partial rows into this rank's `recv` buffer.
XL_API int xl_tp_reduce_norm_gather(const void* recv, const void* residual, void* residual_out, const void* norm_w,
                                    void* const* gathered, void* flags_in, void* const* gather_cnt, void* done_counter,
                                    void* epoch, int tp, int rank, int shard, int shard_cap, int rows_here, int total_rows, int H,
                                    float eps, double timeout_s, void* stream) {
  if (!recv) return -2;
  return launch_reduce(recv, nullptr, residual, residual_out, norm_w, gathered, flags_in, gather_cnt, done_counter, epoch, tp, rank,
                       shard, shard_cap, rows_here, total_rows, H, eps, timeout_s, stream);
}

// Pull variant: `partials` holds `tp` pointers to every rank's partial GEMM result [T][H] (this rank's own included);
// the owner fetches the rows it owns from all of them with coalesced peer loads.
XL_API int xl_tp_pull_reduce_norm_gather(void* const* partials, const void* residual, void* residual_out, const void* norm_w,
                                         void* const* gathered, void* flags_in, void* const* gather_cnt, void* done_counter,
                                         void* epoch, int tp, int rank, int shard, int rows_here, int total_rows, int H, float eps,
                                         double timeout_s, void* stream) {
  return launch_reduce(nullptr, partials, residual, residual_out, norm_w, gathered, flags_in, gather_cnt, done_counter, epoch, tp,
                       rank, shard, shard, rows_here, total_rows, H, eps, timeout_s, stream);
}

// NVLS variant: `mc_partial` / `mc_gathered` are the multicast addresses of the partial-result and activation buffers
// (same offsets on every rank); the flags use the peer-mapped plain addresses as in the pull variant.
// `reduce_in` = 0: the rows come from `local_in` [rows_here][H] instead of the switch reduction (`mc_partial`, `flags_in`
// unused); `gather_out` = 0: the normalised rows go to `local_out` [rows_here][H] instead of every rank's activation
// buffer (`mc_gathered`, `gather_cnt` unused).  Each combination keeps its own `done_counter` / `epoch` words.
static int launch_nvls(const void* mc_partial, const void* local_in, const void* residual, void* residual_out, const void* norm_w,
                       void* mc_gathered, void* local_out, void* flags_in, void* const* gather_cnt, void* done_counter,
                       void* epoch, int tp, int rank, int shard, int rows_here, int total_rows, int H, float eps,
                       double timeout_s, void* stream) {
  const bool reduce_in = mc_partial != nullptr, gather_out = mc_gathered != nullptr;
  if ((tp != 2 && tp != 4 && tp != 8) || H % 8 || H > 8 * kNvlsThreads * 4) return -2;
  if ((!reduce_in && !local_in) || (!gather_out && !local_out) || (!reduce_in && !gather_out)) return -2;
  TpNvlsParams p;
  memset(&p, 0, sizeof(p));
  p.mc_partial = static_cast<const __nv_bfloat16*>(mc_partial);
  p.mc_gathered = static_cast<__nv_bfloat16*>(mc_gathered);
  p.local_in = static_cast<const __nv_bfloat16*>(local_in);
  p.local_out = static_cast<__nv_bfloat16*>(local_out);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.residual_out = static_cast<__nv_bfloat16*>(residual_out);
  p.norm_w = static_cast<const __nv_bfloat16*>(norm_w);
  if (gather_out) {
    for (int r = 0; r < tp; ++r) p.gather_cnt[r] = static_cast<int*>(gather_cnt[r]);
    p.gather_cnt_local = static_cast<int*>(gather_cnt[rank]);
  }
  p.flags_in = static_cast<int*>(flags_in);
  p.done_counter = static_cast<int*>(done_counter);
  p.epoch = static_cast<int*>(epoch);
  p.status = xl_host::status_word();
  p.tp = tp; p.rank = rank; p.shard = shard; p.rows_here = rows_here; p.H = H; p.eps = eps; p.total_rows = total_rows;
  const int vpt = (H / 8 + kNvlsThreads - 1) / kNvlsThreads;      // 1..4
  p.grid_cap = (vpt <= 2 ? 4 : 2) * xl_host::sm_count();
  p.limit_ns = (unsigned long long)(timeout_s * 1e9);
  p.trace = g_trace;
  // several rows per CTA so that loads and stores of different rows overlap (see the kernel)
  p.rows_per_cta = g_nvls_rows_per_cta;
  const int grid = nvls_grid_of(rows_here, p.rows_per_cta, p.grid_cap);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define XL_NVLS_LAUNCH(NR, VPT)                                                                                 \
  do {                                                                                                          \
    if (reduce_in && gather_out) tp_nvls_reduce_norm_gather_kernel<NR, VPT, true, true><<<grid, kNvlsThreads, 0, st>>>(p);   \
    else if (reduce_in) tp_nvls_reduce_norm_gather_kernel<NR, VPT, true, false><<<grid, kNvlsThreads, 0, st>>>(p);           \
    else tp_nvls_reduce_norm_gather_kernel<NR, VPT, false, true><<<grid, kNvlsThreads, 0, st>>>(p);                          \
  } while (0)
#define XL_NVLS_BY_VPT(NR) \
  do { if (vpt <= 1) XL_NVLS_LAUNCH(NR, 1); else if (vpt == 2) XL_NVLS_LAUNCH(NR, 2); else XL_NVLS_LAUNCH(NR, 4); } while (0)
  if (tp == 2) XL_NVLS_BY_VPT(2);
  else if (tp == 4) XL_NVLS_BY_VPT(4);
  else XL_NVLS_BY_VPT(8);
#undef XL_NVLS_BY_VPT
#undef XL_NVLS_LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

XL_API int xl_tp_nvls_reduce_norm_gather(const void* mc_partial, const void* residual, void* residual_out, const void* norm_w,
                                         void* mc_gathered, void* flags_in, void* const* gather_cnt, void* done_counter,
                                         void* epoch, int tp, int rank, int shard, int rows_here, int total_rows, int H, float eps,
                                         double timeout_s, void* stream) {
  if (!mc_partial || !mc_gathered) return -2;
  return launch_nvls(mc_partial, nullptr, residual, residual_out, norm_w, mc_gathered, nullptr, flags_in, gather_cnt, done_counter,
                     epoch, tp, rank, shard, rows_here, total_rows, H, eps, timeout_s, stream);
}

// Reduce-scatter half alone: sum of the partial results of the rows this rank owns (in the switch) + residual + RMSNorm;
// the normalised rows stay here (`local_out` [rows_here][H]).
XL_API int xl_tp_nvls_reduce_norm(const void* mc_partial, const void* residual, void* residual_out, const void* norm_w,
                                  void* local_out, void* flags_in, void* done_counter, void* epoch, int tp, int rank, int shard,
                                  int rows_here, int total_rows, int H, float eps, double timeout_s, void* stream) {
  if (!mc_partial || !local_out) return -2;
  return launch_nvls(mc_partial, nullptr, residual, residual_out, norm_w, nullptr, local_out, flags_in, nullptr, done_counter, epoch,
                     tp, rank, shard, rows_here, total_rows, H, eps, timeout_s, stream);
}

// All-gather half alone: rows computed by their owner (`local_in` [rows_here][H]) + residual + RMSNorm, written to every
// rank's activation buffer through the multicast address.
XL_API int xl_tp_nvls_norm_gather(const void* local_in, const void* residual, void* residual_out, const void* norm_w,
                                  void* mc_gathered, void* const* gather_cnt, void* done_counter, void* epoch, int tp, int rank,
                                  int shard, int rows_here, int total_rows, int H, float eps, double timeout_s, void* stream) {
  if (!local_in || !mc_gathered) return -2;
  return launch_nvls(nullptr, local_in, residual, residual_out, norm_w, mc_gathered, nullptr, nullptr, gather_cnt, done_counter,
                     epoch, tp, rank, shard, rows_here, total_rows, H, eps, timeout_s, stream);
}

// Copy `rows` x H bf16 partial results (row pitch `ld` elements) into this rank's partial buffer and publish them to the
// `tp` ranks' flag words; the reduce entry points above then treat them like the output of the publishing GEMM.
XL_API int xl_tp_publish_rows(const void* src, int ld, void* partial, int rows, int H, void* const* flags, void* done_counter,
                              const void* epoch, int tp, int rank, void* stream) {
  if (tp < 1 || tp > 8 || (H & 7) || (ld & 7) || (reinterpret_cast<uintptr_t>(src) & 15) ||
      (reinterpret_cast<uintptr_t>(partial) & 15))
    return -2;
  TpPublishParams p;
  memset(&p, 0, sizeof(p));
  p.src = static_cast<const uint4*>(src);
  p.dst = static_cast<uint4*>(partial);
  p.ld16 = ld / 8;
  p.rows = rows;
  p.row16 = H / 8;
  for (int r = 0; r < tp; ++r) p.flags[r] = static_cast<int*>(flags[r]);
  p.done_counter = static_cast<int*>(done_counter);
  p.epoch = static_cast<const int*>(epoch);
  p.tp = tp;
  p.rank = rank;
  const long total = long(rows) * p.row16;
  int grid = int((total + 256 * 4 - 1) / (256 * 4));
  if (grid < 1) grid = 1;
  if (grid > 296) grid = 296;
  tp_publish_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
