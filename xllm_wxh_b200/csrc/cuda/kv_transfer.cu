// Paged-KV block push from a prefill instance to a decode instance over NVLink peer memory.
//
// The reference moves KV between prefill and decode instances only on Ascend NPUs (LlmDataDist / Mooncake:
// xllm/core/framework/kv_cache/kv_cache_transfer.cpp, llm_worker_impl.cpp:98-113; compiled under USE_NPU only).  Here
// the prefill rank copies whole cache blocks with 16-byte peer stores into the block ids the decode instance reserved:
//   grid.y = cache tensor (layer x {K, V} or the single MLA latent tensor), grid.x = CTAs striding over (pair, chunk);
//   when the last CTA of a tensor has finished, it publishes `ready[tensor] = epoch` to the decode GPU with a
//   system-scope release store, so the consumer may start on the first layers while later ones are still in flight.
#include <string.h>

#include "common.cuh"

namespace xl {

struct KvPushParams {
  const uint8_t* const* src;     // [n_tensors] local cache bases (device array of pointers)
  uint8_t* const* dst;           // [n_tensors] peer cache bases
  const int2* pairs;             // [n_pairs] (src block, dst block)
  int* done_counters;            // [n_tensors] local
  int* ready_flags;              // [n_tensors] on the peer (may be null)
  const long* block_bytes;       // [n_tensors]
  long src_blocks, dst_blocks;   // bounds
  int n_pairs, epoch;
  int* status;
};

__global__ void kv_push_kernel(const KvPushParams p) {
  const int tensor = blockIdx.y;
  const long bb = p.block_bytes[tensor];
  const long vec_per_block = bb / 16;
  const long total = long(p.n_pairs) * vec_per_block;
  const uint8_t* s = p.src[tensor];
  uint8_t* d = p.dst[tensor];
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
    const int pair = int(i / vec_per_block);
    const long v = i % vec_per_block;
    const int2 pr = p.pairs[pair];
    if (pr.x < 0 || pr.x >= p.src_blocks || pr.y < 0 || pr.y >= p.dst_blocks) {   // never form an out-of-range address
      atomicExch(p.status, XL_ERR_BOUNDS);
      continue;
    }
    const uint4 val = *reinterpret_cast<const uint4*>(s + size_t(pr.x) * bb + v * 16);
    *reinterpret_cast<uint4*>(d + size_t(pr.y) * bb + v * 16) = val;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const int prev = atomicAdd(p.done_counters + tensor, 1);
    if (prev == int(gridDim.x) - 1) {
      p.done_counters[tensor] = 0;
      __threadfence_system();
      if (p.ready_flags) asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p.ready_flags + tensor), "r"(p.epoch) : "memory");
    }
  }
}

}  // namespace xl

XL_API int xl_kv_push(const void* src_ptrs, const void* dst_ptrs, const void* pairs, void* done_counters, void* ready_flags,
                      const void* block_bytes, long src_blocks, long dst_blocks, int n_tensors, int n_pairs, int epoch,
                      void* stream) {
  if (n_pairs <= 0 || n_tensors <= 0) return 0;
  xl::KvPushParams p;
  p.src = static_cast<const uint8_t* const*>(src_ptrs);
  p.dst = static_cast<uint8_t* const*>(dst_ptrs);
  p.pairs = static_cast<const int2*>(pairs);
  p.done_counters = static_cast<int*>(done_counters);
  p.ready_flags = static_cast<int*>(ready_flags);
  p.block_bytes = static_cast<const long*>(block_bytes);
  p.src_blocks = src_blocks; p.dst_blocks = dst_blocks;
  p.n_pairs = n_pairs; p.epoch = epoch;
  p.status = xl_host::status_word();
  int gx = n_pairs * 4;
  if (gx > 148 * 2) gx = 148 * 2;
  if (gx < 1) gx = 1;
  dim3 grid(gx, n_tensors);
  xl::kv_push_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
