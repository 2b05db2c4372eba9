// 128-bit seeded hash used for prefix-cache block keys.
//
// The reference chains XXH3-128 (seed 1024) over the int32 token bytes of each
// full block: key_i = H(key_{i-1} || tokens_i)  (xllm/core/framework/prefix_cache/
// prefix_cache.cpp:31-58).  The same chaining is kept here; the mixing function is
// MurmurHash3 x64/128 (public domain algorithm by Austin Appleby), written out
// below, because the keys never leave this process.
#pragma once
#include <cstdint>
#include <cstring>
#include <functional>

namespace xl {

struct Hash128 {
  uint64_t lo = 0, hi = 0;
  bool operator==(const Hash128& o) const { return lo == o.lo && hi == o.hi; }
  bool operator!=(const Hash128& o) const { return !(*this == o); }
};

struct Hash128Hasher {
  size_t operator()(const Hash128& h) const { return static_cast<size_t>(h.lo ^ (h.hi * 0x9e3779b97f4a7c15ULL)); }
};

namespace detail {
inline uint64_t rotl64(uint64_t x, int r) { return (x << r) | (x >> (64 - r)); }
inline uint64_t fmix64(uint64_t k) {
  k ^= k >> 33; k *= 0xff51afd7ed558ccdULL;
  k ^= k >> 33; k *= 0xc4ceb9fe1a85ec53ULL;
  k ^= k >> 33; return k;
}
}  // namespace detail

inline Hash128 hash128(const void* key, size_t len, uint64_t seed) {
  using namespace detail;
  const uint8_t* data = static_cast<const uint8_t*>(key);
  const size_t nblocks = len / 16;
  uint64_t h1 = seed, h2 = seed;
  const uint64_t c1 = 0x87c37b91114253d5ULL, c2 = 0x4cf5ad432745937fULL;
  for (size_t i = 0; i < nblocks; ++i) {
    uint64_t k1, k2;
    std::memcpy(&k1, data + i * 16, 8);
    std::memcpy(&k2, data + i * 16 + 8, 8);
    k1 *= c1; k1 = rotl64(k1, 31); k1 *= c2; h1 ^= k1;
    h1 = rotl64(h1, 27); h1 += h2; h1 = h1 * 5 + 0x52dce729;
    k2 *= c2; k2 = rotl64(k2, 33); k2 *= c1; h2 ^= k2;
    h2 = rotl64(h2, 31); h2 += h1; h2 = h2 * 5 + 0x38495ab5;
  }
  const uint8_t* tail = data + nblocks * 16;
  uint64_t k1 = 0, k2 = 0;
  switch (len & 15) {
    case 15: k2 ^= uint64_t(tail[14]) << 48; [[fallthrough]];
    case 14: k2 ^= uint64_t(tail[13]) << 40; [[fallthrough]];
    case 13: k2 ^= uint64_t(tail[12]) << 32; [[fallthrough]];
    case 12: k2 ^= uint64_t(tail[11]) << 24; [[fallthrough]];
    case 11: k2 ^= uint64_t(tail[10]) << 16; [[fallthrough]];
    case 10: k2 ^= uint64_t(tail[9]) << 8; [[fallthrough]];
    case 9:  k2 ^= uint64_t(tail[8]);
             k2 *= c2; k2 = rotl64(k2, 33); k2 *= c1; h2 ^= k2; [[fallthrough]];
    case 8:  k1 ^= uint64_t(tail[7]) << 56; [[fallthrough]];
    case 7:  k1 ^= uint64_t(tail[6]) << 48; [[fallthrough]];
    case 6:  k1 ^= uint64_t(tail[5]) << 40; [[fallthrough]];
    case 5:  k1 ^= uint64_t(tail[4]) << 32; [[fallthrough]];
    case 4:  k1 ^= uint64_t(tail[3]) << 24; [[fallthrough]];
    case 3:  k1 ^= uint64_t(tail[2]) << 16; [[fallthrough]];
    case 2:  k1 ^= uint64_t(tail[1]) << 8; [[fallthrough]];
    case 1:  k1 ^= uint64_t(tail[0]);
             k1 *= c1; k1 = rotl64(k1, 31); k1 *= c2; h1 ^= k1;
  }
  h1 ^= len; h2 ^= len;
  h1 += h2; h2 += h1;
  h1 = fmix64(h1); h2 = fmix64(h2);
  h1 += h2; h2 += h1;
  return Hash128{h1, h2};
}

// key_i = H(prev_key (16 B) || int32 tokens of block i)
inline Hash128 chain_block_hash(const Hash128* prev, const int32_t* tokens, int n, uint64_t seed) {
  // small stack buffer: blocks are at most a few hundred tokens
  uint8_t stackbuf[16 + 4 * 512];
  uint8_t* buf = stackbuf;
  size_t need = 16 + size_t(n) * 4;
  bool heap = need > sizeof(stackbuf);
  if (heap) buf = new uint8_t[need];
  size_t off = 0;
  if (prev) { std::memcpy(buf, prev, 16); off = 16; }
  std::memcpy(buf + off, tokens, size_t(n) * 4);
  Hash128 h = hash128(buf, off + size_t(n) * 4, seed);
  if (heap) delete[] buf;
  return h;
}

}  // namespace xl
