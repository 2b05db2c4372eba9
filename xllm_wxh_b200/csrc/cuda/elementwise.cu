// Memory-bound fused ops: RMSNorm, residual-add + RMSNorm, SwiGLU, embedding gather,
// per-head q/k RMSNorm + RoPE + paged KV-cache write.
//
// Math follows the reference kernels: norm.cu:42-172 (`cast(x*rstd)*w`, residual updated with the sum),
// activation.cu:46-99 (silu in fp32), fused_qknorm_rope.cu:75-280 (one warp per (token, head): RMSNorm over the
// head, then neox RoPE from a [cos|sin] fp32 cache), reshape_paged_cache.cu:23-59 (scatter by slot id).
#include "common.cuh"

namespace xl {

// ---------------------------------------------------------------- RMSNorm (+ residual add)
// One CTA per row.  The summed row is kept in shared memory as fp32 between the two passes.
template <bool ADD>
__global__ void rms_norm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual_in,
                                const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out,
                                __nv_bfloat16* __restrict__ residual_out, int H, int ldx, float eps) {
  extern __shared__ float row_cache[];
  __shared__ float red[32];
  const int row = blockIdx.x;
  const __nv_bfloat16* xr = x + size_t(row) * ldx;
  const int nvec = H / 8;
  float ss = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    uint4 a = *reinterpret_cast<const uint4*>(xr + v * 8);
    uint32_t au[4] = {a.x, a.y, a.z, a.w};
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = unpack_bf16x2(au[j]);
      f[2 * j] = t.x;
      f[2 * j + 1] = t.y;
    }
    if (ADD) {
      uint4 b = *reinterpret_cast<const uint4*>(residual_in + size_t(row) * H + v * 8);
      uint32_t bu[4] = {b.x, b.y, b.z, b.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 t = unpack_bf16x2(bu[j]);
        o[j] = pack_bf16x2(f[2 * j] + t.x, f[2 * j + 1] + t.y);   // the sum is rounded to bf16 first, like the reference
        float2 r = unpack_bf16x2(o[j]);
        f[2 * j] = r.x;
        f[2 * j + 1] = r.y;
      }
      *reinterpret_cast<uint4*>(residual_out + size_t(row) * H + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      ss += f[j] * f[j];
      row_cache[v * 8 + j] = f[j];
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x + 31) / 32 ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) red[0] = rsqrtf(t / float(H) + eps);
  }
  __syncthreads();
  const float rstd = red[0];
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    uint4 wv = *reinterpret_cast<const uint4*>(w + v * 8);
    uint32_t wu[4] = {wv.x, wv.y, wv.z, wv.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 ww = unpack_bf16x2(wu[j]);
      float n0 = __bfloat162float(__float2bfloat16(row_cache[v * 8 + 2 * j] * rstd));
      float n1 = __bfloat162float(__float2bfloat16(row_cache[v * 8 + 2 * j + 1] * rstd));
      o[j] = pack_bf16x2(n0 * ww.x, n1 * ww.y);
    }
    *reinterpret_cast<uint4*>(out + size_t(row) * H + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// Register-resident variant for rows of up to VPT * 8 * blockDim elements: every thread owns VPT vectors of 8 elements,
// all loads of a row (x, residual, weight) are issued before the first use, nothing goes through shared memory except
// the two partial sums.  Same arithmetic as above (sum rounded to bf16, normalised value rounded to bf16, then scaled).
template <bool ADD, int VPT>
__global__ void __launch_bounds__(256) rms_norm_reg_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual_in,
                                                           const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out,
                                                           __nv_bfloat16* __restrict__ residual_out, int H, int ldx, float eps) {
  __shared__ float red[8];
  __shared__ float s_rstd;
  const int row = blockIdx.x;
  const int nvec = H / 8;
  const __nv_bfloat16* xr = x + size_t(row) * ldx;
  uint4 a[VPT], b[VPT], wv[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v < nvec) {
      a[i] = *reinterpret_cast<const uint4*>(xr + v * 8);
      if (ADD) b[i] = *reinterpret_cast<const uint4*>(residual_in + size_t(row) * H + v * 8);
      wv[i] = *reinterpret_cast<const uint4*>(w + v * 8);
    }
  }
  float f[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v < nvec) {
      const uint32_t au[4] = {a[i].x, a[i].y, a[i].z, a[i].w};
      const uint32_t bu[4] = {b[i].x, b[i].y, b[i].z, b[i].w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 t = unpack_bf16x2(au[j]);
        if (ADD) {
          const float2 r = unpack_bf16x2(bu[j]);
          o[j] = pack_bf16x2(t.x + r.x, t.y + r.y);
          t = unpack_bf16x2(o[j]);
        }
        f[i][2 * j] = t.x;
        f[i][2 * j + 1] = t.y;
        ss += t.x * t.x + t.y * t.y;
      }
      if (ADD) *reinterpret_cast<uint4*>(residual_out + size_t(row) * H + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) s_rstd = rsqrtf(t / float(H) + eps);
  }
  __syncthreads();
  const float rstd = s_rstd;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v < nvec) {
      const uint32_t wu[4] = {wv[i].x, wv[i].y, wv[i].z, wv[i].w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 ww = unpack_bf16x2(wu[j]);
        const float n0 = __bfloat162float(__float2bfloat16(f[i][2 * j] * rstd));
        const float n1 = __bfloat162float(__float2bfloat16(f[i][2 * j + 1] * rstd));
        o[j] = pack_bf16x2(n0 * ww.x, n1 * ww.y);
      }
      *reinterpret_cast<uint4*>(out + size_t(row) * H + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

template <bool ADD>
static bool launch_rms_norm_reg(const __nv_bfloat16* x, const __nv_bfloat16* res_in, const __nv_bfloat16* w, __nv_bfloat16* out,
                                __nv_bfloat16* res_out, int T, int H, int ldx, float eps, cudaStream_t st) {
  const int nvec = H / 8;
  if (nvec <= 256) rms_norm_reg_kernel<ADD, 1><<<T, 256, 0, st>>>(x, res_in, w, out, res_out, H, ldx, eps);
  else if (nvec <= 512) rms_norm_reg_kernel<ADD, 2><<<T, 256, 0, st>>>(x, res_in, w, out, res_out, H, ldx, eps);
  else if (nvec <= 1024) rms_norm_reg_kernel<ADD, 4><<<T, 256, 0, st>>>(x, res_in, w, out, res_out, H, ldx, eps);
  else return false;
  return true;
}

// ---------------------------------------------------------------- SwiGLU
__global__ void silu_mul_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, int T, int I, int ldx) {
  const int nvec = I / 8;
  const long total = long(T) * nvec;
  for (long idx = blockIdx.x * long(blockDim.x) + threadIdx.x; idx < total; idx += long(gridDim.x) * blockDim.x) {
    const int t = int(idx / nvec), v = int(idx % nvec);
    uint4 g = *reinterpret_cast<const uint4*>(x + size_t(t) * ldx + v * 8);
    uint4 u = *reinterpret_cast<const uint4*>(x + size_t(t) * ldx + I + v * 8);
    uint32_t gu[4] = {g.x, g.y, g.z, g.w}, uu[4] = {u.x, u.y, u.z, u.w}, o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 a = unpack_bf16x2(gu[j]), b = unpack_bf16x2(uu[j]);
      o[j] = pack_bf16x2(a.x / (1.f + __expf(-a.x)) * b.x, a.y / (1.f + __expf(-a.y)) * b.y);
    }
    *reinterpret_cast<uint4*>(out + size_t(t) * I + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ---------------------------------------------------------------- embedding gather
__global__ void embedding_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                 __nv_bfloat16* __restrict__ out, int H, int V) {
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  const uint4* src = reinterpret_cast<const uint4*>(table + size_t(id) * H);
  uint4* dst = reinterpret_cast<uint4*>(out + size_t(t) * H);
  for (int v = threadIdx.x; v < H / 8; v += blockDim.x) dst[v] = src[v];
}

// ---------------------------------------------------------------- q/k RMSNorm + RoPE + KV write
// One warp per (token, head).  Heads [0, n_q) are queries (rotated in place), [n_q, n_q+n_kv) keys (normed, rotated,
// written to the K cache; also rotated in place), [n_q+n_kv, n_q+2 n_kv) values (copied to the V cache).
template <int D, bool NORM>
__global__ void rope_qknorm_kvwrite_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                                           const int* __restrict__ slots, const float* __restrict__ cos_sin,
                                           const __nv_bfloat16* __restrict__ q_w, const __nv_bfloat16* __restrict__ k_w,
                                           __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int T,
                                           int n_q, int n_kv, float eps, long cache_slots) {
  constexpr int P = D / 64;  // elements per lane in each half
  const int heads = n_q + 2 * n_kv;
  const long gw = (blockIdx.x * long(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= long(T) * heads) return;
  const int t = int(gw / heads), h = int(gw % heads);
  __nv_bfloat16* src = qkv + size_t(t) * heads * D + size_t(h) * D;
  const int slot = slots[t];
  if (h >= n_q + n_kv) {  // value head: plain copy into the cache
    if (slot < 0 || slot >= cache_slots) return;
    __nv_bfloat16* dst = v_cache + (size_t(slot) * n_kv + (h - n_q - n_kv)) * D;
    for (int i = lane; i < D / 8; i += 32) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    return;
  }
  const bool is_k = h >= n_q;
  float a[P], b[P];
#pragma unroll
  for (int j = 0; j < P; ++j) {
    a[j] = __bfloat162float(src[lane * P + j]);
    b[j] = __bfloat162float(src[D / 2 + lane * P + j]);
  }
  if (NORM) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < P; ++j) ss += a[j] * a[j] + b[j] * b[j];
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / float(D) + eps);
    const __nv_bfloat16* w = is_k ? k_w : q_w;
#pragma unroll
    for (int j = 0; j < P; ++j) {
      a[j] = __bfloat162float(__float2bfloat16(a[j] * rstd)) * __bfloat162float(w[lane * P + j]);
      b[j] = __bfloat162float(__float2bfloat16(b[j] * rstd)) * __bfloat162float(w[D / 2 + lane * P + j]);
      a[j] = __bfloat162float(__float2bfloat16(a[j]));
      b[j] = __bfloat162float(__float2bfloat16(b[j]));
    }
  }
  const float* cs = cos_sin + size_t(positions[t]) * D;
  __nv_bfloat16 ra[P], rb[P];
#pragma unroll
  for (int j = 0; j < P; ++j) {
    const float c = cs[lane * P + j], s = cs[D / 2 + lane * P + j];
    ra[j] = __float2bfloat16(a[j] * c - b[j] * s);
    rb[j] = __float2bfloat16(b[j] * c + a[j] * s);
  }
#pragma unroll
  for (int j = 0; j < P; ++j) {
    src[lane * P + j] = ra[j];
    src[D / 2 + lane * P + j] = rb[j];
  }
  if (is_k && slot >= 0 && slot < cache_slots) {
    __nv_bfloat16* dst = k_cache + (size_t(slot) * n_kv + (h - n_q)) * D;
#pragma unroll
    for (int j = 0; j < P; ++j) {
      dst[lane * P + j] = ra[j];
      dst[D / 2 + lane * P + j] = rb[j];
    }
  }
}

// Vectorised variant: D/16 lanes per (token, head), each lane owning 8 consecutive elements of the first half and the
// matching 8 of the second half (two 16-byte loads, two 16-byte stores, 16-byte cache writes).
template <int D, bool NORM>
__global__ void __launch_bounds__(256) rope_qknorm_kvwrite_vec_kernel(
    __nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ slots,
    const float* __restrict__ cos_sin, const __nv_bfloat16* __restrict__ q_w, const __nv_bfloat16* __restrict__ k_w,
    __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int T, int n_q, int n_kv, float eps,
    long cache_slots) {
  constexpr int LPH = D / 16;                       // lanes per head
  const int heads = n_q + 2 * n_kv;
  const long gt = blockIdx.x * long(blockDim.x) + threadIdx.x;
  const long item = gt / LPH;                        // (token, head)
  const int sub = int(gt % LPH);
  const bool active = item < long(T) * heads;
  const int t = active ? int(item / heads) : 0, h = active ? int(item % heads) : 0;
  __nv_bfloat16* src = qkv + size_t(t) * heads * D + size_t(h) * D;
  const int slot = active ? slots[t] : -1;
  const bool slot_ok = slot >= 0 && slot < cache_slots;
  uint4 va = make_uint4(0, 0, 0, 0), vb = va;
  if (active) {
    va = *reinterpret_cast<const uint4*>(src + sub * 8);
    vb = *reinterpret_cast<const uint4*>(src + D / 2 + sub * 8);
  }
  if (active && h >= n_q + n_kv) {                   // value head: plain copy into the cache
    if (slot_ok) {
      __nv_bfloat16* dst = v_cache + (size_t(slot) * n_kv + (h - n_q - n_kv)) * D;
      *reinterpret_cast<uint4*>(dst + sub * 8) = va;
      *reinterpret_cast<uint4*>(dst + D / 2 + sub * 8) = vb;
    }
  }
  const bool rot = active && h < n_q + n_kv;
  const bool is_k = h >= n_q;
  float a[8], b[8];
  {
    uint32_t au[4] = {va.x, va.y, va.z, va.w}, bu[4] = {vb.x, vb.y, vb.z, vb.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 x = unpack_bf16x2(au[j]), y = unpack_bf16x2(bu[j]);
      a[2 * j] = x.x; a[2 * j + 1] = x.y; b[2 * j] = y.x; b[2 * j + 1] = y.y;
    }
  }
  if (NORM) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += a[j] * a[j] + b[j] * b[j];
#pragma unroll
    for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);     // the LPH lanes of a head are adjacent
    const float rstd = rsqrtf(ss / float(D) + eps);
    if (rot) {
      const __nv_bfloat16* w = is_k ? k_w : q_w;
      const uint4 wa = *reinterpret_cast<const uint4*>(w + sub * 8), wb = *reinterpret_cast<const uint4*>(w + D / 2 + sub * 8);
      uint32_t wau[4] = {wa.x, wa.y, wa.z, wa.w}, wbu[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 x = unpack_bf16x2(wau[j]), y = unpack_bf16x2(wbu[j]);
        // the same roundings as the scalar kernel: bf16(x * rstd) * w, then bf16
        a[2 * j] = __bfloat162float(__float2bfloat16(__bfloat162float(__float2bfloat16(a[2 * j] * rstd)) * x.x));
        a[2 * j + 1] = __bfloat162float(__float2bfloat16(__bfloat162float(__float2bfloat16(a[2 * j + 1] * rstd)) * x.y));
        b[2 * j] = __bfloat162float(__float2bfloat16(__bfloat162float(__float2bfloat16(b[2 * j] * rstd)) * y.x));
        b[2 * j + 1] = __bfloat162float(__float2bfloat16(__bfloat162float(__float2bfloat16(b[2 * j + 1] * rstd)) * y.y));
      }
    }
  }
  if (!rot) return;
  const float* cs = cos_sin + size_t(positions[t]) * D;
  float c[8], sn[8];
  *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(cs + sub * 8);
  *reinterpret_cast<float4*>(c + 4) = *reinterpret_cast<const float4*>(cs + sub * 8 + 4);
  *reinterpret_cast<float4*>(sn) = *reinterpret_cast<const float4*>(cs + D / 2 + sub * 8);
  *reinterpret_cast<float4*>(sn + 4) = *reinterpret_cast<const float4*>(cs + D / 2 + sub * 8 + 4);
  uint32_t ra[4], rb[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    ra[j] = pack_bf16x2(a[2 * j] * c[2 * j] - b[2 * j] * sn[2 * j], a[2 * j + 1] * c[2 * j + 1] - b[2 * j + 1] * sn[2 * j + 1]);
    rb[j] = pack_bf16x2(b[2 * j] * c[2 * j] + a[2 * j] * sn[2 * j], b[2 * j + 1] * c[2 * j + 1] + a[2 * j + 1] * sn[2 * j + 1]);
  }
  const uint4 oa = make_uint4(ra[0], ra[1], ra[2], ra[3]), ob = make_uint4(rb[0], rb[1], rb[2], rb[3]);
  *reinterpret_cast<uint4*>(src + sub * 8) = oa;
  *reinterpret_cast<uint4*>(src + D / 2 + sub * 8) = ob;
  if (is_k && slot_ok) {
    __nv_bfloat16* dst = k_cache + (size_t(slot) * n_kv + (h - n_q)) * D;
    *reinterpret_cast<uint4*>(dst + sub * 8) = oa;
    *reinterpret_cast<uint4*>(dst + D / 2 + sub * 8) = ob;
  }
}

}  // namespace xl

using namespace xl;

XL_API int xl_rms_norm(const void* x, const void* w, void* out, int T, int H, int ldx, float eps, void* stream) {
  if (T <= 0) return 0;
  if (H % 8 || ldx % 8) return -2;
  if (launch_rms_norm_reg<false>(static_cast<const __nv_bfloat16*>(x), nullptr, static_cast<const __nv_bfloat16*>(w),
                                 static_cast<__nv_bfloat16*>(out), nullptr, T, H, ldx, eps, static_cast<cudaStream_t>(stream)))
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
  int threads = ((H / 8 + 31) / 32) * 32;
  threads = threads > 1024 ? 1024 : (threads < 32 ? 32 : threads);
  rms_norm_kernel<false><<<T, threads, H * sizeof(float), static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), nullptr, static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(out),
      nullptr, H, ldx, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

XL_API int xl_add_rms_norm(const void* x, const void* residual_in, const void* w, void* out, void* residual_out, int T, int H,
                           int ldx, float eps, void* stream) {
  if (T <= 0) return 0;
  if (H % 8 || ldx % 8) return -2;
  if (launch_rms_norm_reg<true>(static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(residual_in),
                                static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(out),
                                static_cast<__nv_bfloat16*>(residual_out), T, H, ldx, eps, static_cast<cudaStream_t>(stream)))
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
  int threads = ((H / 8 + 31) / 32) * 32;
  threads = threads > 1024 ? 1024 : (threads < 32 ? 32 : threads);
  rms_norm_kernel<true><<<T, threads, H * sizeof(float), static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(residual_in),
      static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(out), static_cast<__nv_bfloat16*>(residual_out), H, ldx,
      eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

XL_API int xl_silu_mul(const void* x, void* out, int T, int I, int ldx, void* stream) {
  if (T <= 0) return 0;
  if (I % 8 || ldx % 8) return -2;
  long total = long(T) * (I / 8);
  int blocks = int((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  silu_mul_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(x),
                                                                        static_cast<__nv_bfloat16*>(out), T, I, ldx);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

XL_API int xl_embedding(const void* ids, const void* table, void* out, int T, int H, int V, void* stream) {
  if (T <= 0) return 0;
  if (H % 8) return -2;
  int threads = H / 8 > 256 ? 256 : ((H / 8 + 31) / 32) * 32;
  embedding_kernel<<<T, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const int*>(ids), static_cast<const __nv_bfloat16*>(table), static_cast<__nv_bfloat16*>(out), H, V);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

XL_API int xl_rope_qknorm_kvwrite(void* qkv, const void* positions, const void* slots, const void* cos_sin, const void* q_w,
                                  const void* k_w, void* k_cache, void* v_cache, int T, int n_q, int n_kv, int head_dim,
                                  float eps, long cache_slots, void* stream) {
  if (T <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // 16-byte accesses need 16-byte aligned rows and caches (always the case for the engine's tensors)
  const bool vec = !((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
                      reinterpret_cast<uintptr_t>(cos_sin) | reinterpret_cast<uintptr_t>(q_w) | reinterpret_cast<uintptr_t>(k_w)) & 15);
  const long items = long(T) * (n_q + 2 * n_kv);
  const int blocks = vec ? int((items * (head_dim / 16) + 255) / 256) : int((items + 7) / 8);
#define LAUNCH(D, NORM)                                                                                                    \
  if (vec)                                                                                                                 \
    rope_qknorm_kvwrite_vec_kernel<D, NORM><<<blocks, 256, 0, st>>>(                                                       \
        static_cast<__nv_bfloat16*>(qkv), static_cast<const int*>(positions), static_cast<const int*>(slots),             \
        static_cast<const float*>(cos_sin), static_cast<const __nv_bfloat16*>(q_w), static_cast<const __nv_bfloat16*>(k_w), \
        static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), T, n_q, n_kv, eps, cache_slots);       \
  else                                                                                                                     \
  rope_qknorm_kvwrite_kernel<D, NORM><<<blocks, 256, 0, st>>>(                                                             \
      static_cast<__nv_bfloat16*>(qkv), static_cast<const int*>(positions), static_cast<const int*>(slots),               \
      static_cast<const float*>(cos_sin), static_cast<const __nv_bfloat16*>(q_w), static_cast<const __nv_bfloat16*>(k_w), \
      static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), T, n_q, n_kv, eps, cache_slots)
  const bool norm = q_w != nullptr;
  if (head_dim == 128) { if (norm) LAUNCH(128, true); else LAUNCH(128, false); }
  else if (head_dim == 64) { if (norm) LAUNCH(64, true); else LAUNCH(64, false); }
  else if (head_dim == 256) { if (norm) LAUNCH(256, true); else LAUNCH(256, false); }
  else return -2;
#undef LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
