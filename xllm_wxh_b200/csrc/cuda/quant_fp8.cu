// Per-token (per-row) dynamic e4m3 quantisation of activations, alone and fused behind RMSNorm.
//
// The reference's w8a8 fp8 linears quantise the activation with one scale per token before its sm_100 CUTLASS
// scaled-mm (xllm/core/layers/common/linear.cpp:134-179; kernels/cuda/fp8_quant.cu:79-105, where the dynamic scale comes
// from a separate torch abs().max() pass) and offer RMSNorm with a static per-tensor fp8 output
// (kernels/cuda/norm.cu:227-393, layers/common/rms_norm.cpp:94-140).  Here one kernel per row does
//   [residual add ->] RMSNorm -> row maximum -> scale = amax / 448 -> e4m3
// with the row held in registers between the two block reductions, so the normalised activation never goes to memory in
// bf16 when the next operation is an fp8 GEMM (xl_gemm_fp8_scaled, which multiplies by the row scale in its epilogue).
#include "common.cuh"

namespace xl {

constexpr float kE4m3Max = 448.f;

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return uint32_t(lo) | (uint32_t(hi) << 16);
}

__device__ __forceinline__ float block_reduce_256(float v, float* red, bool is_max) {
  v = is_max ? warp_max(v) : warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
  t = is_max ? warp_max(t) : warp_sum(t);
  __syncthreads();                      // red[] may be reused by the caller's next reduction
  return t;                             // the block's value in warp 0 (other warps see 0): callers read it in thread 0
}

// NORM: 0 plain quantisation of x, 1 RMSNorm(x) then quantise, 2 RMSNorm(x + residual) then quantise (residual' written).
// VPT: vectors of 8 elements per thread (row length <= VPT * 2048).
template <int NORM, int VPT>
__global__ void __launch_bounds__(256) quant_rows_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual_in,
                                                         const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ q,
                                                         float* __restrict__ scales, __nv_bfloat16* __restrict__ residual_out,
                                                         int H, int ldx, float eps) {
  __shared__ float red[8];
  __shared__ float s_bcast;
  const int row = blockIdx.x;
  const int nvec = H / 8;
  const __nv_bfloat16* xr = x + size_t(row) * ldx;
  float f[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v < nvec) {
      const uint4 a = *reinterpret_cast<const uint4*>(xr + v * 8);
      const uint32_t au[4] = {a.x, a.y, a.z, a.w};
      uint32_t bu[4] = {0, 0, 0, 0};
      if (NORM == 2) {
        const uint4 b = *reinterpret_cast<const uint4*>(residual_in + size_t(row) * H + v * 8);
        bu[0] = b.x; bu[1] = b.y; bu[2] = b.z; bu[3] = b.w;
      }
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 t = unpack_bf16x2(au[j]);
        if (NORM == 2) {
          const float2 r = unpack_bf16x2(bu[j]);
          o[j] = pack_bf16x2(t.x + r.x, t.y + r.y);
          t = unpack_bf16x2(o[j]);
        }
        f[i][2 * j] = t.x;
        f[i][2 * j + 1] = t.y;
        ss += t.x * t.x + t.y * t.y;
      }
      if (NORM == 2) *reinterpret_cast<uint4*>(residual_out + size_t(row) * H + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
  if (NORM != 0) {
    const float tot = block_reduce_256(ss, red, false);
    if (threadIdx.x == 0) s_bcast = rsqrtf(tot / float(H) + eps);
    __syncthreads();
    const float rstd = s_bcast;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * 256;
      if (v < nvec) {
        const uint4 wv = *reinterpret_cast<const uint4*>(w + v * 8);
        const uint32_t wu[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 ww = unpack_bf16x2(wu[j]);
          // the roundings of the bf16 RMSNorm: normalised value, then the product with the weight
          const float n0 = __bfloat162float(__float2bfloat16(f[i][2 * j] * rstd));
          const float n1 = __bfloat162float(__float2bfloat16(f[i][2 * j + 1] * rstd));
          f[i][2 * j] = __bfloat162float(__float2bfloat16(n0 * ww.x));
          f[i][2 * j + 1] = __bfloat162float(__float2bfloat16(n1 * ww.y));
        }
      }
    }
    __syncthreads();
  }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[i][j]));
    }
  }
  const float row_max = block_reduce_256(amax, red, true);
  if (threadIdx.x == 0) {
    const float sc = fmaxf(row_max, 1e-10f) / kE4m3Max;
    s_bcast = sc;
    scales[row] = sc;
  }
  __syncthreads();
  const float inv = 1.f / s_bcast;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v < nvec)
      *reinterpret_cast<uint2*>(q + size_t(row) * H + v * 8) =
          make_uint2(pack_e4m3x4(f[i][0] * inv, f[i][1] * inv, f[i][2] * inv, f[i][3] * inv),
                     pack_e4m3x4(f[i][4] * inv, f[i][5] * inv, f[i][6] * inv, f[i][7] * inv));
  }
}

template <int NORM>
static int launch_quant_rows(const void* x, const void* res_in, const void* w, void* q, void* scales, void* res_out, int T, int H,
                             int ldx, float eps, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 8 || (ldx % 8) || H > 8 * 2048) return -2;
  const int nvec = H / 8;
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto R = static_cast<const __nv_bfloat16*>(res_in);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto Q = static_cast<uint8_t*>(q);
  auto S = static_cast<float*>(scales);
  auto RO = static_cast<__nv_bfloat16*>(res_out);
  if (nvec <= 256) quant_rows_kernel<NORM, 1><<<T, 256, 0, st>>>(X, R, W, Q, S, RO, H, ldx, eps);
  else if (nvec <= 512) quant_rows_kernel<NORM, 2><<<T, 256, 0, st>>>(X, R, W, Q, S, RO, H, ldx, eps);
  else if (nvec <= 1024) quant_rows_kernel<NORM, 4><<<T, 256, 0, st>>>(X, R, W, Q, S, RO, H, ldx, eps);
  else quant_rows_kernel<NORM, 8><<<T, 256, 0, st>>>(X, R, W, Q, S, RO, H, ldx, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace xl

// bf16 [T, H] (row pitch ldx) -> e4m3 [T, H] and one fp32 scale per row (x ~ q * scale).
XL_API int xl_quant_rows_fp8(const void* x, void* q, void* scales, int T, int H, int ldx, void* stream) {
  return xl::launch_quant_rows<0>(x, nullptr, nullptr, q, scales, nullptr, T, H, ldx, 0.f, static_cast<cudaStream_t>(stream));
}
// RMSNorm(x) * w, quantised per row.
XL_API int xl_rms_norm_quant_fp8(const void* x, const void* w, void* q, void* scales, int T, int H, int ldx, float eps, void* stream) {
  return xl::launch_quant_rows<1>(x, nullptr, w, q, scales, nullptr, T, H, ldx, eps, static_cast<cudaStream_t>(stream));
}
// residual' = x + residual (bf16, written to residual_out [T, H]); RMSNorm(residual') * w, quantised per row.
XL_API int xl_add_rms_norm_quant_fp8(const void* x, const void* residual_in, const void* w, void* q, void* scales,
                                     void* residual_out, int T, int H, float eps, void* stream) {
  return xl::launch_quant_rows<2>(x, residual_in, w, q, scales, residual_out, T, H, H, eps, static_cast<cudaStream_t>(stream));
}
