// Host-side helpers shared by the kernel launchers: tensor-map cache, device queries, status word.
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace xl_host {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

CUresult encode_tiled(CUtensorMap* map, CUtensorMapDataType dt, uint32_t rank, const void* base, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = get_encode();
  if (!fn) return CUDA_ERROR_NOT_SUPPORTED;
  cuuint32_t elem_strides[5] = {1, 1, 1, 1, 1};
  return fn(map, dt, rank, const_cast<void*>(base), reinterpret_cast<const cuuint64_t*>(dims),
            reinterpret_cast<const cuuint64_t*>(strides_bytes), reinterpret_cast<const cuuint32_t*>(box), elem_strides,
            CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}

struct Key {
  const void* base;
  uint64_t rows, cols, ld;
  uint32_t br, bc;
  int dt, swz;
  bool operator==(const Key& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && br == o.br && bc == o.bc && dt == o.dt &&
           swz == o.swz;
  }
};
struct KeyHash {
  size_t operator()(const Key& k) const {
    uint64_t h = reinterpret_cast<uint64_t>(k.base) * 0x9e3779b97f4a7c15ULL;
    h ^= (k.rows * 0xbf58476d1ce4e5b9ULL) ^ (k.cols * 0x94d049bb133111ebULL) ^ (k.ld << 7) ^ (uint64_t(k.br) << 40) ^
         (uint64_t(k.bc) << 20) ^ uint64_t(k.dt * 31 + k.swz);
    return static_cast<size_t>(h ^ (h >> 29));
  }
};

const CUtensorMap* tmap_2d(const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t ld,
                           uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swz) {
  static std::mutex mu;
  static std::unordered_map<Key, CUtensorMap*, KeyHash> cache;
  Key k{base, rows, cols, ld, box_rows, box_cols, int(dt), int(swz)};
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(k);
  if (it != cache.end()) return it->second;
  if (cache.size() > 8192) {  // bounded: maps are cheap to rebuild
    for (auto& kv : cache) delete kv.second;
    cache.clear();
  }
  CUtensorMap* m = new CUtensorMap;
  uint64_t dims[2] = {cols, rows};
  uint64_t strides[1] = {ld * uint64_t(elem_bytes)};
  uint32_t box[2] = {box_cols, box_rows};
  CUresult r = encode_tiled(m, dt, 2, base, dims, strides, box, swz);
  if (r != CUDA_SUCCESS) {
    delete m;
    return nullptr;
  }
  cache.emplace(k, m);
  return m;
}

// cached 3-D map of a [d2, d1, d0] row-major tensor (d0 innermost, contiguous), box = [b2, b1, b0]
const CUtensorMap* tmap_3d(const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t d2, uint64_t d1, uint64_t d0,
                           uint32_t b2, uint32_t b1, uint32_t b0, CUtensorMapSwizzle swz) {
  static std::mutex mu;
  static std::unordered_map<Key, CUtensorMap*, KeyHash> cache;
  Key k{base, d2, d1 * 1000003ULL + b1, d0, b2, b0, int(dt), int(swz)};
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(k);
  if (it != cache.end()) return it->second;
  if (cache.size() > 4096) {
    for (auto& kv : cache) delete kv.second;
    cache.clear();
  }
  CUtensorMap* m = new CUtensorMap;
  uint64_t dims[3] = {d0, d1, d2};
  uint64_t strides[2] = {d0 * uint64_t(elem_bytes), d0 * d1 * uint64_t(elem_bytes)};
  uint32_t box[3] = {b0, b1, b2};
  CUresult r = encode_tiled(m, dt, 3, base, dims, strides, box, swz);
  if (r != CUDA_SUCCESS) {
    delete m;
    return nullptr;
  }
  cache.emplace(k, m);
  return m;
}

int sm_count() {
  static int n[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (n[dev] == 0) cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
  return n[dev];
}

int* status_word() {
  static int* w[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  std::lock_guard<std::mutex> g(mu);
  if (!w[dev]) {
    cudaMalloc(&w[dev], 256);
    cudaMemset(w[dev], 0, 256);
  }
  return w[dev];
}

}  // namespace xl_host

// Reads and clears the device status word (0 = every bounded wait completed).  Synchronises the device.
XL_API int xl_read_status() {
  int* w = xl_host::status_word();
  int v = 0;
  cudaDeviceSynchronize();
  cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost);
  if (v != 0) cudaMemset(w, 0, sizeof(int));
  return v;
}

XL_API int xl_sm_count() { return xl_host::sm_count(); }
