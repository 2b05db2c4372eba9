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

// Pack whole cache blocks into / out of a block-major staging area (host tier of the prefix cache).
// The paged cache keeps one tensor per layer and K / V ([blocks, block, heads, dim] each), so one logical block is
// n_tensors separate pieces; the host tier stores a block as one contiguous record (piece of tensor t at tensor_off[t]),
// which makes every host<->device transfer a single large copy for the copy engines.
//   to_cache == 0: packed[slot] <- cache pieces of `block`      (before a device->host copy)
//   to_cache == 1: cache pieces of `block` <- packed[slot]      (after a host->device copy)
struct KvPackParams {
  uint8_t* const* cache;       // [n_tensors] cache bases (device array of pointers)
  const long* block_bytes;     // [n_tensors]
  const long* tensor_off;      // [n_tensors]
  const int2* pairs;           // [n_pairs] (cache block, staging slot)
  uint8_t* packed;             // [slots][stride]
  long stride, cache_blocks, slots;
  int n_pairs, to_cache;
  int* status;
};

__global__ void kv_pack_kernel(const KvPackParams p) {
  const int tensor = blockIdx.y;
  const long bb = p.block_bytes[tensor];
  const long off = p.tensor_off[tensor];
  const long vec_per_block = bb / 16;
  const long total = long(p.n_pairs) * vec_per_block;
  uint8_t* c = p.cache[tensor];
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
    const int pair = int(i / vec_per_block);
    const long v = i % vec_per_block;
    const int2 pr = p.pairs[pair];
    if (pr.x < 0 || pr.x >= p.cache_blocks || pr.y < 0 || pr.y >= p.slots) {   // never form an out-of-range address
      atomicExch(p.status, XL_ERR_BOUNDS);
      continue;
    }
    uint4* in_cache = reinterpret_cast<uint4*>(c + size_t(pr.x) * bb + v * 16);
    uint4* in_pack = reinterpret_cast<uint4*>(p.packed + size_t(pr.y) * p.stride + off + v * 16);
    if (p.to_cache) *in_cache = *in_pack; else *in_pack = *in_cache;
  }
}

}  // namespace xl

XL_API int xl_kv_pack(const void* cache_ptrs, const void* block_bytes, const void* tensor_off, const void* pairs, void* packed,
                      long stride, long cache_blocks, long slots, int n_tensors, int n_pairs, int to_cache, void* stream) {
  if (n_pairs <= 0 || n_tensors <= 0) return 0;
  if (stride % 16 != 0 || (reinterpret_cast<uintptr_t>(packed) & 15) != 0) return -2;
  xl::KvPackParams p;
  p.cache = static_cast<uint8_t* const*>(const_cast<void*>(cache_ptrs));
  p.block_bytes = static_cast<const long*>(block_bytes);
  p.tensor_off = static_cast<const long*>(tensor_off);
  p.pairs = static_cast<const int2*>(pairs);
  p.packed = static_cast<uint8_t*>(packed);
  p.stride = stride; p.cache_blocks = cache_blocks; p.slots = slots;
  p.n_pairs = n_pairs; p.to_cache = to_cache;
  p.status = xl_host::status_word();
  int gx = n_pairs * 2;   // a side-stream kernel: leave most SMs to the step that runs beside it
  if (gx > 32) gx = 32;
  dim3 grid(gx, n_tensors);
  xl::kv_pack_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

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

// Weight pull of a waking instance: one device-to-device copy from a CUDA-IPC mapped tensor of an awake instance (the
// copy engines move it over NVLink when the source lives on another GPU).  One call per tensor.
XL_API int xl_copy_d2d(void* dst, const void* src, long bytes, void* stream) {
  if (bytes <= 0) return 0;
  if (!dst || !src) return -2;
  return cudaMemcpyAsync(dst, src, size_t(bytes), cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)) == cudaSuccess ? 0 : -1;
}
