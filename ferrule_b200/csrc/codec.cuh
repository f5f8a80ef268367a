// Scalar codecs shared by the quantisation kernels and the epilogues that quantise in place:
// UE8M0 scale bytes (2^(b - 127)) and E4M3 values.
#pragma once
#include <cuda_fp8.h>

#include <cstdint>

namespace fb {

__device__ __forceinline__ float e8m0_to_float(uint8_t b) {
  // 2^(b - 127); b = 0 is the subnormal 2^-127
  return b == 0 ? __uint_as_float(1u << 22) : __uint_as_float(static_cast<uint32_t>(b) << 23);
}

// smallest power of two >= x (x > 0) as an E8M0 byte
__device__ __forceinline__ uint8_t e8m0_ceil(float x) {
  const uint32_t bits = __float_as_uint(x);
  int e = static_cast<int>((bits >> 23) & 0xff);
  if (bits & 0x7fffffu) ++e;
  e = max(0, min(254, e));
  return static_cast<uint8_t>(e);
}

__device__ __forceinline__ uint8_t to_e4m3(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

__device__ __forceinline__ float from_e4m3(uint8_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

// 1 x 128 activation block: scale byte for an absolute maximum (floored so that an all-zero block stays finite)
__device__ __forceinline__ uint8_t fp8_block_scale(float amax) { return e8m0_ceil(fmaxf(amax, 1e-4f) / 448.f); }

}  // namespace fb
