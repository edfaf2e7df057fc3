// Shared device helpers for the TurboQuant B200 kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/turboquant_b200.h"

namespace tq {

constexpr int kCentroidOff = 0;     // centroids at [0, 256) of a codebook block
constexpr int kThresholdOff = 256;  // thresholds at [256, 512)

template <int DT>
__device__ __forceinline__ float load_elem(const void* base, int64_t i) {
  if constexpr (DT == TQ_F32) {
    return reinterpret_cast<const float*>(base)[i];
  } else if constexpr (DT == TQ_F16) {
    return __half2float(reinterpret_cast<const __half*>(base)[i]);
  } else {
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[i]);
  }
}

template <int DT>
__device__ __forceinline__ void store_elem(void* base, int64_t i, float v) {
  if constexpr (DT == TQ_F32) {
    reinterpret_cast<float*>(base)[i] = v;
  } else if constexpr (DT == TQ_F16) {
    reinterpret_cast<__half*>(base)[i] = __float2half_rn(v);
  } else {
    reinterpret_cast<__nv_bfloat16*>(base)[i] = __float2bfloat16_rn(v);
  }
}

// Number of thresholds strictly below y.  thr[] holds levels-1 ascending values
// (unused slots are +inf).  NaN compares false everywhere and lands on 0, which
// is what a first-minimum argmin over an all-NaN row returns.
__device__ __forceinline__ int quantize_scalar(float y, const float* thr, int levels) {
  int lo = 0, hi = levels - 1;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (y > thr[mid]) lo = mid + 1; else hi = mid;
  }
  return lo;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// flat vector number -> element offset of its first coordinate
__device__ __forceinline__ int64_t vec_offset(int64_t n, int64_t H, int64_t S, int64_t sb, int64_t sh, int64_t ss) {
  int64_t s = n % S;
  int64_t t = n / S;
  int64_t h = t % H;
  int64_t b = t / H;
  return b * sb + h * sh + s * ss;
}

__host__ __device__ __forceinline__ int round_up(int v, int m) { return (v + m - 1) / m * m; }

}  // namespace tq
