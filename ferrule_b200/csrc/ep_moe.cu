// Expert-parallel MoE over NVLink peer memory (token-sharded ranks, experts sharded by id).
//
//   fb_ep_dispatch        every (token, slot) route: reserve a row in the destination rank's
//                         receive segment for this source, store the activation row and its
//                         {local expert, return row, weight} record there with plain peer stores;
//                         the last CTA publishes the per-destination counts and bumps the
//                         destination's arrival flag          (dispatch all-to-all, push side)
//   fb_ep_collect         destination: wait (bounded) for every source's flag, turn the received
//                         records into a route list (expert id / weight / return address per row;
//                         unused rows = -1) for the route-plan kernel
//   [grouped tcgen05 GEMMs run on the receive buffer; the down projection's scatter epilogue
//    stores each weighted output row into the owning rank's combine buffer and signals]
//   fb_ep_combine_reduce  source: wait for every rank's combine signal, sum a token's top-k rows
//                         in slot order (+ shared-expert row, + residual) -> bf16; optionally
//                         pushes the result into every rank's gather buffer (all-gather) and
//                         signals
//   fb_ep_gather_wait     wait until every rank's gathered rows have landed
//
// Ordering argument (no double buffering needed): a rank can start the next dispatch only after
// its combine-reduce, which needs every peer's combine signal, which a peer sends only after its
// grouped GEMMs have consumed the previous dispatch.  Counters only grow; each kernel keeps its
// own call count in device memory so that graph replays agree across ranks.  Every wait is
// bounded and reports a status instead of hanging.
//
// The reference streams experts on one GPU and has no dispatch; this is the expert-parallel
// counterpart of its prepare/gather + scatter stages
// (crates/ferrule-backend/native/cuda/implementations/cutlass/architectures/sm103/grouped_fp4_moe.cuh:1115-1222).
#include "common.cuh"
#include "ferrule_b200.h"
#include "launch.cuh"

namespace fb {

struct EpParams {
  uint8_t* base[8];          // every rank's symmetric buffer, in this rank's address space
  long long off_recv_x, off_recv_meta, off_recv_cnt, off_comb, off_disp_flag, off_comb_flag, off_gath_flag,
      off_gath_out;
  int rank, world, cap, hidden, topk, experts_local, tcap;
  unsigned long long wait_ns;
  DeviceStatus* st;
};

__device__ __forceinline__ uint32_t* ep_flags(const EpParams& P, int r, long long off) {
  return reinterpret_cast<uint32_t*>(P.base[r] + off);
}

// grid = tokens, 128 threads.  cnt_local [world] and ctr [2] are private to this rank (zeroed once).
__global__ void __launch_bounds__(128)
ep_dispatch_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const int* __restrict__ idx,
                   const float* __restrict__ wts, int tokens, uint32_t* cnt_local, uint32_t* ctr, EpParams P) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int s_pos;
  const int t = blockIdx.x;
  const int E = P.experts_local * P.world;
  for (int s = 0; s < P.topk; ++s) {
    const int e = idx[t * P.topk + s];
    if (e < 0 || e >= E) {
      if (threadIdx.x == 0) report_status(P.st, kStatusBadIndex, 0x900, t, e);
      continue;   // uniform: every thread read the same e
    }
    const int d = e / P.experts_local;
    if (threadIdx.x == 0) s_pos = static_cast<int>(atomicAdd(&cnt_local[d], 1u));
    __syncthreads();
    const int pos = s_pos;
    __syncthreads();
    if (pos >= P.cap) {
      if (threadIdx.x == 0) report_status(P.st, kStatusBadShape, 0x901, d, pos);
      continue;
    }
    const size_t row = static_cast<size_t>(P.rank) * P.cap + pos;
    uint4* dst = reinterpret_cast<uint4*>(P.base[d] + P.off_recv_x + row * P.hidden * 2);
    const uint4* src = reinterpret_cast<const uint4*>(x + t * ldx);
    for (int i = threadIdx.x; i < P.hidden / 8; i += blockDim.x) dst[i] = src[i];
    if (threadIdx.x == 0) {
      int4 m;
      m.x = e - d * P.experts_local;
      m.y = t * P.topk + s;
      m.z = __float_as_int(wts[t * P.topk + s]);
      m.w = 1;
      reinterpret_cast<int4*>(P.base[d] + P.off_recv_meta)[row] = m;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t done = atomicAdd(ctr + 1, 1u);
    if (done == gridDim.x - 1) {
      ctr[1] = 0;
      __threadfence_system();
      for (int d = 0; d < P.world; ++d) {
        const uint32_t c = min(atomicExch(&cnt_local[d], 0u), static_cast<uint32_t>(P.cap));
        reinterpret_cast<volatile uint32_t*>(P.base[d] + P.off_recv_cnt)[P.rank] = c;
      }
      __threadfence_system();
      for (int d = 0; d < P.world; ++d) flag_add_release_sys(ep_flags(P, d, P.off_disp_flag) + P.rank, 1u);
    }
  }
}

// grid = world (one CTA per source), 256 threads.  Writes route arrays of world * cap rows.
__global__ void __launch_bounds__(256)
ep_collect_kernel(uint32_t* ctr, int e_lo, int* __restrict__ r_idx, float* __restrict__ r_w,
                  int* __restrict__ remap_rank, int* __restrict__ remap_row, EpParams P) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int s_cnt;
  const int src = blockIdx.x;
  const uint32_t call = *reinterpret_cast<volatile uint32_t*>(ctr);
  if (threadIdx.x == 0) {
    const bool ok = flag_wait_ge(ep_flags(P, P.rank, P.off_disp_flag) + src, call + 1u, P.wait_ns, P.st, 0x910 + src);
    const uint32_t c = ok ? *reinterpret_cast<volatile uint32_t*>(P.base[P.rank] + P.off_recv_cnt + src * 4) : 0u;
    s_cnt = static_cast<int>(min(c, static_cast<uint32_t>(P.cap)));
  }
  __syncthreads();
  const int cnt = s_cnt;
  const int4* meta = reinterpret_cast<const int4*>(P.base[P.rank] + P.off_recv_meta) + static_cast<size_t>(src) * P.cap;
  for (int i = threadIdx.x; i < P.cap; i += blockDim.x) {
    const int r = src * P.cap + i;
    if (i < cnt) {
      const int4 m = meta[i];
      const bool good = m.x >= 0 && m.x < P.experts_local && m.y >= 0 && m.y < P.tcap * P.topk;
      if (!good) report_status(P.st, kStatusBadIndex, 0x920, r, m.x);
      r_idx[r] = good ? e_lo + m.x : -1;
      r_w[r] = __int_as_float(m.z);
      remap_rank[r] = src;
      remap_row[r] = good ? m.y : 0;
    } else {
      r_idx[r] = -1;
      r_w[r] = 0.f;
      remap_rank[r] = src;
      remap_row[r] = 0;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t done = atomicAdd(ctr + 1, 1u);
    if (done == gridDim.x - 1) {
      ctr[1] = 0;
      __threadfence();
      ctr[0] = call + 1u;
    }
  }
}

// grid = tokens, 256 threads.
__global__ void __launch_bounds__(256)
ep_combine_reduce_kernel(uint32_t* ctr, const __nv_bfloat16* __restrict__ extra, long long lde,
                         const __nv_bfloat16* __restrict__ residual, long long ldr, __nv_bfloat16* __restrict__ out,
                         long long ldo, int tokens, int allgather, int gather_row0, EpParams P) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int s_ok;
  const int t = blockIdx.x;
  const uint32_t call = *reinterpret_cast<volatile uint32_t*>(ctr);
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < P.world) {
    if (!flag_wait_ge(ep_flags(P, P.rank, P.off_comb_flag) + threadIdx.x, call + 1u, P.wait_ns, P.st,
                      0x930 + threadIdx.x))
      s_ok = 0;
  }
  __syncthreads();
  const bool ok = s_ok != 0;
  const __nv_bfloat16* comb = reinterpret_cast<const __nv_bfloat16*>(P.base[P.rank] + P.off_comb);
  for (int i = threadIdx.x * 8; i < P.hidden && ok; i += blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int s = 0; s < P.topk; ++s) {
      const uint4 v = *reinterpret_cast<const uint4*>(comb + (static_cast<size_t>(t) * P.topk + s) * P.hidden + i);
      const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(b[j]);
    }
    if (extra) {
      const uint4 v = *reinterpret_cast<const uint4*>(extra + t * lde + i);
      const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(b[j]);
    }
    if (residual) {
      const uint4 v = *reinterpret_cast<const uint4*>(residual + t * ldr + i);
      const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(b[j]);
    }
    __nv_bfloat16 o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16_rn(acc[j]);
    const uint4 ov = *reinterpret_cast<const uint4*>(o);
    if (out) *reinterpret_cast<uint4*>(out + t * ldo + i) = ov;
    if (allgather) {
      // gathered rows: at this rank's fixed segment, or (gather_row0 >= 0) at the caller's offset, which lets the
      // ranks' slices of a batch land back to back as one [tokens of all ranks, hidden] tensor
      const size_t row = gather_row0 >= 0 ? static_cast<size_t>(gather_row0) + t : static_cast<size_t>(P.rank) * P.tcap + t;
      for (int pr = 0; pr < P.world; ++pr)
        *reinterpret_cast<uint4*>(P.base[pr] + P.off_gath_out + (row * P.hidden + i) * 2) = ov;
    }
  }
  if (allgather) __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t done = atomicAdd(ctr + 1, 1u);
    if (done == gridDim.x - 1) {
      ctr[1] = 0;
      if (allgather) {
        __threadfence_system();
        for (int pr = 0; pr < P.world; ++pr) flag_add_release_sys(ep_flags(P, pr, P.off_gath_flag) + P.rank, 1u);
      }
      __threadfence();
      ctr[0] = call + 1u;
    }
  }
}

__global__ void __launch_bounds__(32)
ep_gather_wait_kernel(uint32_t* ctr, EpParams P) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t call = *reinterpret_cast<volatile uint32_t*>(ctr);
  if (threadIdx.x < P.world)
    flag_wait_ge(ep_flags(P, P.rank, P.off_gath_flag) + threadIdx.x, call + 1u, P.wait_ns, P.st, 0x940 + threadIdx.x);
  __syncwarp();
  if (threadIdx.x == 0) {
    __threadfence();
    ctr[0] = call + 1u;
  }
}

static int fill(const FbEpArgs* a, EpParams* P) {
  if (!a || a->world < 1 || a->world > 8 || a->rank < 0 || a->rank >= a->world) return FB_ERR_SHAPE;
  if (a->hidden <= 0 || a->hidden % 8 != 0 || a->topk <= 0 || a->cap <= 0 || a->experts_local <= 0 || a->tcap <= 0)
    return FB_ERR_SHAPE;
  for (int i = 0; i < a->world; ++i) {
    if (!a->base[i]) return FB_ERR_SHAPE;
    P->base[i] = static_cast<uint8_t*>(a->base[i]);
  }
  P->off_recv_x = a->off_recv_x;
  P->off_recv_meta = a->off_recv_meta;
  P->off_recv_cnt = a->off_recv_cnt;
  P->off_comb = a->off_comb;
  P->off_disp_flag = a->off_disp_flag;
  P->off_comb_flag = a->off_comb_flag;
  P->off_gath_flag = a->off_gath_flag;
  P->off_gath_out = a->off_gath_out;
  P->rank = a->rank;
  P->world = a->world;
  P->cap = a->cap;
  P->hidden = a->hidden;
  P->topk = a->topk;
  P->experts_local = a->experts_local;
  P->tcap = a->tcap;
  P->wait_ns = a->wait_ns ? a->wait_ns : 3000000000ull;
  P->st = static_cast<DeviceStatus*>(a->status);
  return FB_OK;
}

}  // namespace fb

using namespace fb;

#define FB_CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? FB_OK : FB_ERR_LAUNCH)

extern "C" int fb_ep_dispatch(const FbEpArgs* a, const void* x, long long ldx, const int* idx, const float* wts,
                              int tokens, void* cnt_local, void* ctr, void* stream) {
  EpParams P{};
  const int rc = fill(a, &P);
  if (rc != FB_OK) return rc;
  if (tokens <= 0 || tokens > a->tcap || !x || !idx || !wts || !cnt_local || !ctr) return FB_ERR_SHAPE;
  launch_pdl(ep_dispatch_kernel, dim3(tokens), dim3(128), 0, static_cast<cudaStream_t>(stream),
             static_cast<const __nv_bfloat16*>(x), ldx, idx, wts, tokens, static_cast<uint32_t*>(cnt_local),
             static_cast<uint32_t*>(ctr), P);
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_ep_collect(const FbEpArgs* a, void* ctr, int e_lo, int* r_idx, float* r_w, int* remap_rank,
                             int* remap_row, void* stream) {
  EpParams P{};
  const int rc = fill(a, &P);
  if (rc != FB_OK) return rc;
  if (!ctr || !r_idx || !r_w || !remap_rank || !remap_row) return FB_ERR_SHAPE;
  launch_pdl(ep_collect_kernel, dim3(a->world), dim3(256), 0, static_cast<cudaStream_t>(stream),
             static_cast<uint32_t*>(ctr), e_lo, r_idx, r_w, remap_rank, remap_row, P);
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_ep_combine_reduce(const FbEpArgs* a, void* ctr, const void* extra, long long lde,
                                    const void* residual, long long ldr, void* out, long long ldo, int tokens,
                                    int allgather, int gather_row0, void* stream) {
  EpParams P{};
  const int rc = fill(a, &P);
  if (rc != FB_OK) return rc;
  if (!ctr || tokens <= 0 || tokens > a->tcap || (!out && !allgather)) return FB_ERR_SHAPE;
  if (gather_row0 >= 0 && gather_row0 + tokens > a->world * a->tcap) return FB_ERR_SHAPE;
  launch_pdl(ep_combine_reduce_kernel, dim3(tokens), dim3(256), 0, static_cast<cudaStream_t>(stream),
             static_cast<uint32_t*>(ctr), static_cast<const __nv_bfloat16*>(extra), lde,
             static_cast<const __nv_bfloat16*>(residual), ldr, static_cast<__nv_bfloat16*>(out), ldo, tokens,
             allgather, gather_row0, P);
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_ep_gather_wait(const FbEpArgs* a, void* ctr, void* stream) {
  EpParams P{};
  const int rc = fill(a, &P);
  if (rc != FB_OK) return rc;
  if (!ctr) return FB_ERR_SHAPE;
  launch_pdl(ep_gather_wait_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream),
             static_cast<uint32_t*>(ctr), P);
  return FB_CHECK_LAUNCH();
}
