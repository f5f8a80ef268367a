// fb_argmax_noalloc: two-level arg-max whose scratch is a fixed array in the library image, for
// callers that are not allowed to allocate device memory (see no_alloc.h for who they are).
//
// The kernel is a variant of the chunked arg-max of elementwise.cu: grid (chunks, rows); every CTA
// scans one slice of the vocabulary and records its candidate, the CTA that finishes last for a
// row reduces the candidates.  The only difference is where the candidates and the per-row
// counters live.
#include <mutex>

#include "common.cuh"
#include "ferrule_b200.h"
#include "no_alloc.h"

namespace fb {
namespace {

constexpr int kMaxRows = FB_NOALLOC_ARGMAX_MAX_ROWS;
constexpr int kChunks = FB_NOALLOC_ARGMAX_CHUNKS;

struct NoAllocScratch {
  float part_val[kMaxRows * kChunks];
  int part_id[kMaxRows * kChunks];
  unsigned int row_ctr[kMaxRows];
};

// One instance per device that loads this library.  In host code this name is only a handle for
// cudaGetSymbolAddress: it is NOT a device address and must never be passed to a kernel as is.
static __device__ __align__(256) NoAllocScratch g_noalloc_scratch;

__device__ __forceinline__ bool cand_better(float v, int i, float ov, int oi) {
  return v > ov || (v == ov && i < oi);
}

__global__ void __launch_bounds__(256)
argmax_noalloc_kernel(const float* __restrict__ logits, long long ldl, int rows, int vocab, int chunk,
                      NoAllocScratch* __restrict__ scratch, int* __restrict__ out_id,
                      float* __restrict__ out_val) {
  __shared__ float sv[8];
  __shared__ int si[8];
  __shared__ int is_last;
  const int c = blockIdx.x, r = blockIdx.y;
  const float* lr = logits + r * ldl;
  const int lo = c * chunk, hi = min(vocab, lo + chunk);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = lo + threadIdx.x * 4; i < hi; i += blockDim.x * 4) {
    if (i + 3 < hi) {
      const float4 v = *reinterpret_cast<const float4*>(lr + i);
      const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (vv[j] == vv[j] && cand_better(vv[j], i + j, best, bi)) { best = vv[j]; bi = i + j; }
    } else {
      for (int j = i; j < hi; ++j) {
        const float v = lr[j];
        if (v == v && cand_better(v, j, best, bi)) { best = v; bi = j; }
      }
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (cand_better(ov, oi, best, bi)) { best = ov; bi = oi; }
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { sv[w] = best; si[w] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int k = 1; k < (blockDim.x >> 5); ++k)
      if (cand_better(sv[k], si[k], best, bi)) { best = sv[k]; bi = si[k]; }
    scratch->part_val[r * kChunks + c] = best;
    scratch->part_id[r * kChunks + c] = bi;
    __threadfence();
    const unsigned int done = atomicAdd(&scratch->row_ctr[r], 1u);
    is_last = done == static_cast<unsigned int>(kChunks - 1);
  }
  __syncthreads();
  if (!is_last || w != 0) return;
  __threadfence();
  best = -INFINITY;
  bi = 0x7fffffff;
  for (int k = l; k < kChunks; k += 32) {
    const float v = scratch->part_val[r * kChunks + k];
    const int id = scratch->part_id[r * kChunks + k];
    if (cand_better(v, id, best, bi)) { best = v; bi = id; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (cand_better(ov, oi, best, bi)) { best = ov; bi = oi; }
  }
  if (l == 0) {
    out_id[r] = bi == 0x7fffffff ? -1 : bi;
    if (out_val) out_val[r] = best;
  }
}

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
NoAllocScratch* g_scratch_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device, resolved once per device.
int scratch_for_current_device(NoAllocScratch** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FB_ERR_RUNTIME;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) {
      cudaGetLastError();   // leave no sticky error behind for the caller's next CUDA call
      return FB_ERR_RUNTIME;
    }
    g_scratch_ptr[dev] = static_cast<NoAllocScratch*>(p);
  }
  *out = g_scratch_ptr[dev];
  return FB_OK;
}

}  // namespace
}  // namespace fb

extern "C" int fb_argmax_noalloc(const float* logits, long long ldl, int rows, int vocab, int* out_id,
                                 float* out_val, void* stream_) {
  using namespace fb;
  if (logits == nullptr || out_id == nullptr || rows <= 0 || vocab <= 0) return FB_ERR_SHAPE;
  if (rows > kMaxRows) return FB_ERR_LIMIT;   // beyond the built-in scratch: refuse, launch nothing
  if ((ldl % 4) != 0 || (reinterpret_cast<uintptr_t>(logits) & 15)) return FB_ERR_ALIGN;
  NoAllocScratch* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != FB_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  // The scratch keeps whatever the previous call left: the counters must start at zero.
  if (cudaMemsetAsync(scratch->row_ctr, 0, sizeof(unsigned int) * rows, stream) != cudaSuccess)
    return FB_ERR_RUNTIME;
  const int chunk = ((vocab + kChunks - 1) / kChunks + 3) / 4 * 4;
  dim3 grid(kChunks, rows);
  argmax_noalloc_kernel<<<grid, 256, 0, stream>>>(logits, ldl, rows, vocab, chunk, scratch, out_id, out_val);
  return cudaGetLastError() == cudaSuccess ? FB_OK : FB_ERR_LAUNCH;
}
