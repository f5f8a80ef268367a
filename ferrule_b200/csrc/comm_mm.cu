// Two-shot collectives through the NVLink switch (NVLS): reduce-scatter, all-gather and all-reduce of
// [rows, dim] bf16 activations with `multimem.ld_reduce` / `multimem.st`, fused with the per-token reduction of
// the MoE route rows (or fed with a partial that the producing GEMM stored straight into the staging area),
// the residual add and, optionally, the RMSNorm that follows.  See mm_comm.cuh for the protocol.
//
//   fb_mm_collective  one CTA per row:
//     reduce half (mode & 1): [sum this rank's route rows of token t ->] stage  -> signal A
//                             the row's owner: wait A -> ld_reduce + residual -> result on all ranks (or, without
//                             the broadcast half, into this rank's slice of `out`: a reduce-scatter)
//     broadcast half (mode & 2): owner signals B; every rank waits for B and copies the row to `out`
//                             [+ RMSNorm -> norm_out]; without the reduce half the owner broadcasts rows of `src`
//                             (an all-gather)
//
// Rows are owned in contiguous slices of ceil(rows / world).  All CTAs of a launch must be resident together (they
// wait for signals that CTAs of the same launch on other ranks send): rows <= 512.
//
// The reference has no collective (single GPU); its counterpart of the fused reduce is the MoE route reduce of
// crates/ferrule-backend/native/cuda/implementations/portable/entrypoints.cu:1515-1612.
#include "common.cuh"
#include "ferrule_b200.h"
#include "launch.cuh"
#include "mm_comm.cuh"

namespace fb {

__global__ void __launch_bounds__(256)
mm_collective_kernel(const __nv_bfloat16* __restrict__ src, long long lds, int slots, int topk,
                     const int* __restrict__ topk_idx, int e_lo, int e_hi, const __nv_bfloat16* __restrict__ residual,
                     long long ldr, __nv_bfloat16* __restrict__ out, long long ldo, int rows, int dim, int mode,
                     const __nv_bfloat16* __restrict__ norm_w, __nv_bfloat16* __restrict__ norm_out, long long ldn,
                     float eps, MmChannel c, DeviceStatus* st) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int s_ok;
  __shared__ float red[8];
  extern __shared__ float nrow[];          // dim floats when norm_out is set
  const int t = blockIdx.x;
  const int tid = threadIdx.x;
  const uint32_t call = *reinterpret_cast<volatile uint32_t*>(c.priv);
  const uint32_t exp_a = *reinterpret_cast<volatile uint32_t*>(c.priv + 2);
  const uint32_t exp_b = *reinterpret_cast<volatile uint32_t*>(c.priv + 3);
  const uint32_t parity = call & 1u;
  const long long row_off = static_cast<long long>(parity) * c.buf_bytes + static_cast<long long>(t) * dim * 2;
  int lo, hi;
  mm_owned_rows(rows, c.world, c.rank, lo, hi);
  const bool owner = t >= lo && t < hi;
  const bool do_reduce = (mode & 1) != 0, do_bcast = (mode & 2) != 0;
  bool ok = true;

  if (do_reduce) {
    // ---- this rank's partial row -> staging area (skipped when the producer already wrote it there) ----
    if (src != nullptr) {
      __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(c.local + c.stage_off + row_off);
      for (int i = tid * 8; i < dim; i += 256 * 8) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int s = 0; s < slots; ++s) {
          if (s < topk) {
            const int e = topk_idx[t * topk + s];
            if (e < e_lo || e >= e_hi) continue;
          }
          const uint4 v = *reinterpret_cast<const uint4*>(src + (static_cast<long long>(t) * slots + s) * lds + i);
          const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(vp[j]);
        }
        __nv_bfloat16 o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16_rn(acc[j]);
        *reinterpret_cast<uint4*>(stage + i) = *reinterpret_cast<const uint4*>(o);
      }
    }
    __syncthreads();
    if (tid == 0) mm_signal(c, kMmFlagA, 1u);
    // ---- owner: reduce in the switch, add the residual, broadcast or keep ----
    if (owner) {
      if (tid == 0) s_ok = mm_wait(c, kMmFlagA, exp_a + static_cast<uint32_t>(c.world) * rows, st, 0x700) ? 1 : 0;
      __syncthreads();
      ok = s_ok != 0;
      if (ok) {
        const uint8_t* mc_src = c.mc + c.stage_off + row_off;
        for (int i = tid * 8; i < dim; i += 256 * 8) {
          uint4 v = mm_ld_reduce_bf16x8(mc_src + i * 2);
          if (residual != nullptr) {
            const uint4 r = *reinterpret_cast<const uint4*>(residual + (do_bcast ? t : t - lo) * ldr + i);
            __nv_bfloat162* vp = reinterpret_cast<__nv_bfloat162*>(&v);
            const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 a = __bfloat1622float2(vp[j]), b = __bfloat1622float2(rp[j]);
              vp[j] = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
            }
          }
          if (do_bcast) mm_st16(c.mc + c.result_off + row_off + i * 2, v);
          else *reinterpret_cast<uint4*>(out + (t - lo) * ldo + i) = v;       // reduce-scatter: this rank's slice
        }
      }
    }
  } else if (do_bcast && owner) {
    // ---- all-gather: the owner broadcasts its rows of `src` (a [hi - lo, dim] slice) ----
    for (int i = tid * 8; i < dim; i += 256 * 8)
      mm_st16(c.mc + c.result_off + row_off + i * 2, *reinterpret_cast<const uint4*>(src + (t - lo) * lds + i));
  }
  if (do_bcast) {
    __syncthreads();
    if (owner && tid == 0) mm_signal(c, kMmFlagB, 1u);
    if (tid == 0) s_ok = (ok && mm_wait(c, kMmFlagB, exp_b + static_cast<uint32_t>(rows), st, 0x701)) ? 1 : 0;
    __syncthreads();
    if (s_ok) {
      const __nv_bfloat16* res = reinterpret_cast<const __nv_bfloat16*>(c.local + c.result_off + row_off);
      float ss = 0.f;
      for (int i = tid * 8; i < dim; i += 256 * 8) {
        const uint4 v = ll_load_raw(res + i);      // not through L1: the line may hold the row of two calls ago
        *reinterpret_cast<uint4*>(out + t * ldo + i) = v;
        if (norm_out != nullptr) {
          const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float f = __bfloat162float(vp[j]);
            nrow[i + j] = f;
            ss += f * f;
          }
        }
      }
      if (norm_out != nullptr) {
        // same element -> thread mapping and reduction order as add_rmsnorm_kernel: bit-equal to running it after
        ss = warp_sum(ss);
        if ((tid & 31) == 0) red[tid >> 5] = ss;
        __syncthreads();
        float tot = (tid & 31) < 8 ? red[tid & 31] : 0.f;
        tot = warp_sum(tot);
        const float inv = rsqrtf(tot / dim + eps);
        for (int i = tid * 8; i < dim; i += 256 * 8) {
          const uint4 wv = *reinterpret_cast<const uint4*>(norm_w + i);
          const __nv_bfloat16* wp = reinterpret_cast<const __nv_bfloat16*>(&wv);
          __nv_bfloat16 o[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16_rn(nrow[i + j] * inv * __bfloat162float(wp[j]));
          *reinterpret_cast<uint4*>(norm_out + t * ldn + i) = *reinterpret_cast<const uint4*>(o);
        }
      }
    }
  }
  // ---- bookkeeping: the last CTA of the launch advances the call counter and the expected flag totals ----
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const uint32_t done = atomicAdd(c.priv + 1, 1u);
    if (done == gridDim.x - 1) {
      c.priv[1] = 0;
      if (do_reduce) c.priv[2] = exp_a + static_cast<uint32_t>(c.world) * rows;
      if (do_bcast) c.priv[3] = exp_b + static_cast<uint32_t>(rows);
      __threadfence();
      c.priv[0] = call + 1u;
    }
  }
}

}  // namespace fb

using namespace fb;

extern "C" int fb_mm_collective(const void* src, long long lds, int slots, int topk, const int* topk_idx, int e_lo,
                                int e_hi, const void* residual, long long ldr, void* out, long long ldo, int rows,
                                int dim, int mode, const void* norm_w, void* norm_out, long long ldn, float eps,
                                void* local_base, void* mc_base, long long stage_off, long long result_off,
                                long long buf_bytes, void* priv, int rank, int world, unsigned long long wait_ns,
                                void* status, void* stream) {
  if (rows <= 0 || rows > 512 || dim <= 0 || dim % 8 != 0 || mode < 1 || mode > 3 || !out) return FB_ERR_SHAPE;
  if (!local_base || !mc_base || !priv || rank < 0 || rank >= world || world > 8) return FB_ERR_SHAPE;
  if (static_cast<long long>(rows) * dim * 2 > buf_bytes) return FB_ERR_LIMIT;
  if ((mode & 1) && src != nullptr && (slots < 1 || slots < topk)) return FB_ERR_SHAPE;
  if (mode == 2 && !src) return FB_ERR_SHAPE;
  if (norm_out != nullptr && (!(mode & 2) || !norm_w)) return FB_ERR_SHAPE;
  if ((lds % 8) || (ldr % 8) || (ldo % 8) || (ldn % 8) || (stage_off % 16) || (result_off % 16) || (buf_bytes % 16))
    return FB_ERR_ALIGN;
  MmChannel c{static_cast<uint8_t*>(local_base), static_cast<uint8_t*>(mc_base), stage_off, result_off, buf_bytes,
              static_cast<uint32_t*>(priv), rank, world, wait_ns ? wait_ns : 3000000000ull};
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(mm_collective_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536);
    attr = true;
  }
  const size_t smem = norm_out ? static_cast<size_t>(dim) * sizeof(float) : 0;
  launch_pdl(mm_collective_kernel, dim3(rows), dim3(256), smem, static_cast<cudaStream_t>(stream),
             static_cast<const __nv_bfloat16*>(src), lds, slots, topk, topk_idx, e_lo, e_hi,
             static_cast<const __nv_bfloat16*>(residual), ldr, static_cast<__nv_bfloat16*>(out), ldo, rows, dim, mode,
             static_cast<const __nv_bfloat16*>(norm_w), static_cast<__nv_bfloat16*>(norm_out), ldn, eps, c,
             static_cast<DeviceStatus*>(status));
  return cudaGetLastError() == cudaSuccess ? FB_OK : FB_ERR_LAUNCH;
}
