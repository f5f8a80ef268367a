// Quantisation / packing kernels (sm_100a), bandwidth-bound, one warp per scale block:
//
//   fb_quant_fp8_rows     bf16 [rows, n] -> e4m3 codes + one UE8M0 scale per 1 x 128 block
//                         (amax floored at 1e-4, scale = 2^ceil(log2(amax / 448)))
//   fb_dequant_fp8_block  e4m3 [out, in] + UE8M0 [ceil(out/128), ceil(in/128)] -> bf16
//   fb_quant_mxfp4_rows   bf16 [rows, n] -> packed e2m1 (low nibble first) + UE8M0 per 32 elements
//   fb_dequant_mxfp4      packed e2m1 + UE8M0/32 -> bf16
//   fb_fp8_qat_rows       in-place quantise -> dequantise with a bf16 write-back (1 x block)
//   fb_hadamard_rows      orthonormal fast Walsh-Hadamard transform of each row (n = power of two <= 1024)
//
// Counterpart of the reference's quantize_kernel family
// (crates/ferrule-backend/native/cuda/implementations/portable/entrypoints.cu:342-448) and its
// E8M0 / E4M3 decoders (:63-66); host codecs with the same rounding live in io/encoding.py.
#include <cuda_fp8.h>

#include "codec.cuh"
#include "common.cuh"
#include "ferrule_b200.h"
#include "launch.cuh"

namespace fb {

// nearest E2M1 code (ties -> even code), magnitudes 0 .5 1 1.5 2 3 4 6
__device__ __forceinline__ uint8_t to_e2m1(float v) {
  const float a = fminf(fabsf(v), 6.f);
  uint8_t c;
  if (a <= 0.25f) c = 0;
  else if (a < 0.75f) c = 1;
  else if (a <= 1.25f) c = 2;
  else if (a < 1.75f) c = 3;
  else if (a <= 2.5f) c = 4;
  else if (a < 3.5f) c = 5;
  else if (a <= 5.f) c = 6;
  else c = 7;
  return v < 0.f ? (c | 8) : c;
}

__device__ __forceinline__ float from_e2m1(uint8_t c) {
  const float mags[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  const float m = mags[c & 7];
  return (c & 8) ? -m : m;
}

// one warp per (row, 128-block): lane handles 4 elements
__global__ void __launch_bounds__(256)
quant_fp8_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q, long long ldq,
                      uint8_t* __restrict__ scale, long long lds, int rows, int n, int writeback_bf16,
                      __nv_bfloat16* __restrict__ xq) {
  pdl_launch_dependents();
  pdl_wait();
  const int blocks_per_row = n / 128;
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= rows * blocks_per_row) return;
  const int r = w / blocks_per_row, b = w - r * blocks_per_row;
  const __nv_bfloat16* src = x + r * ldx + b * 128 + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(&raw);
  float f[4], amax = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    f[j] = __bfloat162float(v[j]);
    amax = fmaxf(amax, fabsf(f[j]));
  }
  amax = fmaxf(warp_max(amax), 1e-4f);
  const uint8_t sb = e8m0_ceil(amax / 448.f);
  const float inv = 1.f / e8m0_to_float(sb);
  uint8_t c[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) c[j] = to_e4m3(f[j] * inv);
  if (q) *reinterpret_cast<uint32_t*>(q + r * ldq + b * 128 + lane * 4) = *reinterpret_cast<uint32_t*>(c);
  if (scale && lane == 0) scale[r * lds + b] = sb;
  if (writeback_bf16) {
    const float s = e8m0_to_float(sb);
    __nv_bfloat16 o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = __float2bfloat16_rn(from_e4m3(c[j]) * s);
    *reinterpret_cast<uint2*>(xq + r * ldx + b * 128 + lane * 4) = *reinterpret_cast<uint2*>(o);
  }
}

__global__ void __launch_bounds__(256)
dequant_fp8_block_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ scale,
                         __nv_bfloat16* __restrict__ out, int rows, int cols, int block) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (i >= static_cast<long long>(rows) * cols) return;
  const int r = static_cast<int>(i / cols), c0 = static_cast<int>(i - static_cast<long long>(r) * cols);
  const int sc = (cols + block - 1) / block;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = c0 + j;
    if (c < cols) {
      const float s = e8m0_to_float(scale[(r / block) * sc + c / block]);
      out[i + j] = __float2bfloat16_rn(from_e4m3(q[i + j]) * s);
    }
  }
}

// one warp per (row, 32-group): lane = element
__global__ void __launch_bounds__(256)
quant_mxfp4_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ packed,
                        uint8_t* __restrict__ scale, int rows, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const int groups = n / 32;
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= rows * groups) return;
  const int r = w / groups, g = w - r * groups;
  const float f = __bfloat162float(x[r * ldx + g * 32 + lane]);
  const float amax = fmaxf(warp_max(fabsf(f)), 1e-12f);
  const uint8_t sb = e8m0_ceil(amax / 6.f);
  const uint8_t code = to_e2m1(f / e8m0_to_float(sb));
  const uint8_t hi = __shfl_down_sync(0xffffffffu, code, 1);
  if ((lane & 1) == 0) packed[static_cast<size_t>(r) * (n / 2) + g * 16 + lane / 2] = code | (hi << 4);
  if (lane == 0) scale[static_cast<size_t>(r) * groups + g] = sb;
}

__global__ void __launch_bounds__(256)
dequant_mxfp4_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scale,
                     __nv_bfloat16* __restrict__ out, int rows, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;   // byte index
  if (i >= static_cast<long long>(rows) * (n / 2)) return;
  const int r = static_cast<int>(i / (n / 2)), b = static_cast<int>(i - static_cast<long long>(r) * (n / 2));
  const float s = e8m0_to_float(scale[static_cast<size_t>(r) * (n / 32) + (2 * b) / 32]);
  const uint8_t v = packed[i];
  __nv_bfloat162 o = __floats2bfloat162_rn(from_e2m1(v & 15) * s, from_e2m1(v >> 4) * s);
  *reinterpret_cast<__nv_bfloat162*>(out + static_cast<size_t>(r) * n + 2 * b) = o;
}

// one CTA per row, n threads/2 butterflies in shared memory
__global__ void __launch_bounds__(512)
hadamard_rows_kernel(__nv_bfloat16* __restrict__ x, long long ldx, int rows, int n, int round_bf16) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float hbuf[];
  const int r = blockIdx.x;
  if (r >= rows) return;
  for (int i = threadIdx.x; i < n; i += blockDim.x) hbuf[i] = __bfloat162float(x[r * ldx + i]);
  __syncthreads();
  for (int h = 1; h < n; h <<= 1) {
    for (int i = threadIdx.x; i < n / 2; i += blockDim.x) {
      const int lo = (i / h) * 2 * h + (i % h);
      const float a = hbuf[lo], b = hbuf[lo + h];
      hbuf[lo] = a + b;
      hbuf[lo + h] = a - b;
    }
    __syncthreads();
  }
  const float s = rsqrtf(static_cast<float>(n));
  for (int i = threadIdx.x; i < n; i += blockDim.x) x[r * ldx + i] = __float2bfloat16_rn(hbuf[i] * s);
}

}  // namespace fb

using namespace fb;

#define FB_CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? FB_OK : FB_ERR_LAUNCH)

extern "C" int fb_quant_fp8_rows(const void* x, long long ldx, void* q, long long ldq, void* scale,
                                 long long lds, int rows, int n, int writeback_bf16, void* stream) {
  if (rows <= 0 || n <= 0 || n % 128 != 0 || (ldx % 4) != 0 || (ldq % 4) != 0) return FB_ERR_SHAPE;
  const long long warps = static_cast<long long>(rows) * (n / 128);
  const int blocks = static_cast<int>((warps + 7) / 8);
  launch_pdl(quant_fp8_rows_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream),
             static_cast<const __nv_bfloat16*>(x), ldx, static_cast<uint8_t*>(q), ldq,
             static_cast<uint8_t*>(scale), lds, rows, n, writeback_bf16,
             static_cast<__nv_bfloat16*>(const_cast<void*>(x)));
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_dequant_fp8_block(const void* q, const void* scale, void* out, int rows, int cols, int block,
                                    void* stream) {
  if (rows <= 0 || cols <= 0 || block <= 0 || cols % 4 != 0) return FB_ERR_SHAPE;
  const long long n = (static_cast<long long>(rows) * cols + 3) / 4;
  launch_pdl(dequant_fp8_block_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0,
             static_cast<cudaStream_t>(stream), static_cast<const uint8_t*>(q),
             static_cast<const uint8_t*>(scale), static_cast<__nv_bfloat16*>(out), rows, cols, block);
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_quant_mxfp4_rows(const void* x, long long ldx, void* packed, void* scale, int rows, int n,
                                   void* stream) {
  if (rows <= 0 || n <= 0 || n % 32 != 0) return FB_ERR_SHAPE;
  const long long warps = static_cast<long long>(rows) * (n / 32);
  launch_pdl(quant_mxfp4_rows_kernel, dim3(static_cast<unsigned>((warps + 7) / 8)), dim3(256), 0,
             static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(x), ldx,
             static_cast<uint8_t*>(packed), static_cast<uint8_t*>(scale), rows, n);
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_dequant_mxfp4(const void* packed, const void* scale, void* out, int rows, int n, void* stream) {
  if (rows <= 0 || n <= 0 || n % 32 != 0) return FB_ERR_SHAPE;
  const long long bytes = static_cast<long long>(rows) * (n / 2);
  launch_pdl(dequant_mxfp4_kernel, dim3(static_cast<unsigned>((bytes + 255) / 256)), dim3(256), 0,
             static_cast<cudaStream_t>(stream), static_cast<const uint8_t*>(packed),
             static_cast<const uint8_t*>(scale), static_cast<__nv_bfloat16*>(out), rows, n);
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_hadamard_rows(void* x, long long ldx, int rows, int n, void* stream) {
  if (rows <= 0 || n < 2 || n > 8192 || (n & (n - 1)) != 0) return FB_ERR_SHAPE;
  const int threads = n / 2 < 512 ? (n / 2 < 32 ? 32 : n / 2) : 512;
  launch_pdl(hadamard_rows_kernel, dim3(rows), dim3(threads), n * sizeof(float), static_cast<cudaStream_t>(stream),
             static_cast<__nv_bfloat16*>(x), ldx, rows, n, 1);
  return FB_CHECK_LAUNCH();
}
