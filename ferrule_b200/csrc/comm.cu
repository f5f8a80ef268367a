// Peer-memory plumbing and the collective kernels that are not GEMM epilogues.
//
//   fb_ipc_*                 symmetric buffers: cudaMalloc + CUDA IPC handles, opened by every
//                            peer rank of the node (NVLink peer access through NVSwitch)
//   fb_moe_reduce_allreduce  per token: fixed-order sum of this rank's route rows (+ shared
//                            expert row) -> push the partial (fp32 or bf16) into every rank's receive
//                            slot as tagged words {value, call tag} with plain peer stores -> poll the
//                            tagged words of all ranks (bounded) -> sum in rank order + residual -> bf16.
//                            No fence and no flag: only the one-way NVLink latency is paid.
//                            With slots = 1 and topk = 0 it is a plain one-shot all-reduce.
//   fb_argmax_allgather      vocabulary-parallel greedy token: every rank pushes its local
//                            (logit, id) per row to all peers, then picks the global winner
//                            (ties -> lower id) identically on every rank.
//   fb_flag_wait_probe       a wait on a flag nobody sets, to exercise the timeout path
//
// Synchronisation: the all-reduce payloads carry their own arrival tag (call counter + 1); the small
// all-gather of arg-max candidates uses arrival counters that only grow.  Payload slots are double
// buffered by the channel's call counter: a peer can be at most one call ahead of this rank, because
// finishing a call needs this rank's pushes.
// Every wait is bounded; on timeout the kernel records a status code and returns.
//
// The reference has no multi-GPU path (its ParallelismPlan is inert:
// crates/ferrule-model/src/support/policies.rs:56-77); these kernels are this build's
// tensor/expert-parallel counterpart of its single-GPU MoE reduce
// (crates/ferrule-backend/native/cuda/implementations/portable/entrypoints.cu:1515-1612).
#include "common.cuh"
#include "ferrule_b200.h"
#include "launch.cuh"

namespace fb {

struct PeerPtrs {
  float* recv[8];
  uint32_t* flags[8];
};

// channel-local bookkeeping (not shared with peers): [0] calls, [1] CTAs done, then seen[]
__device__ __forceinline__ void channel_finish(uint32_t* ctr, uint32_t call) {
  __threadfence();
  const uint32_t done = atomicAdd(ctr + 1, 1u);
  if (done == gridDim.x * gridDim.y - 1) {
    ctr[1] = 0;
    __threadfence();
    ctr[0] = call + 1u;
  }
}

// grid = (rows, channel chunks of 512), 128 threads: one 4-channel group per thread.  More, smaller CTAs keep
// more peer stores in flight than one CTA per row would.
__global__ void __launch_bounds__(128)
moe_reduce_allreduce_kernel(const __nv_bfloat16* __restrict__ route_out, int slots, int topk,
                            const int* __restrict__ topk_idx, int e_lo, int e_hi,
                            const __nv_bfloat16* __restrict__ residual, long long ldr,
                            __nv_bfloat16* __restrict__ out, long long ldo, int rows, int dim,
                            int rank, int world, int rows_cap, PeerPtrs peers, uint32_t* ctr,
                            int payload_bf16, unsigned long long wait_ns, DeviceStatus* st, uint8_t* mc_recv) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 4;      // first of this thread's 4 channels
  const uint32_t call = *reinterpret_cast<volatile uint32_t*>(ctr);
  const uint32_t tag = call + 1u;
  const bool bf16 = payload_bf16 != 0;
  // slot geometry in bytes: [parity][source rank][rows_cap][dim] tagged values, 8 bytes each (4 when bf16)
  const size_t slot_bytes = static_cast<size_t>(rows_cap) * dim * 8;
  const size_t parity_off = static_cast<size_t>(call & 1u) * world * slot_bytes;
  const size_t ch = static_cast<size_t>(t) * dim + i;
  if (i < dim) {
    // ---- this rank's partial of the 4 channels -> every rank's slot for this source ----
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < slots; ++s) {
      if (s < topk) {
        const int e = topk_idx[t * topk + s];
        if (e < e_lo || e >= e_hi) continue;
      }
      const uint2 v = *reinterpret_cast<const uint2*>(route_out + (static_cast<size_t>(t) * slots + s) * dim + i);
      const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[j] += __bfloat162float(vp[j]);
    }
    if (mc_recv != nullptr) {
      ll_push4_mc(mc_recv + parity_off + rank * slot_bytes, ch, acc, tag, bf16);      // the switch replicates it
    } else {
      for (int pr = 0; pr < world; ++pr)
        ll_push4(reinterpret_cast<uint8_t*>(peers.recv[pr]) + parity_off + rank * slot_bytes, ch, acc, tag, bf16);
    }
    // ---- all ranks' partials: poll the tagged words, sum in rank order, add the residual ----
    const uint64_t w0 = globaltimer_ns();
    float sum[4] = {0.f, 0.f, 0.f, 0.f};
    int bad_src = 0;
    if (ll_gather4(reinterpret_cast<const uint8_t*>(peers.recv[rank]) + parity_off, ch, slot_bytes, world, tag,
                   wait_ns, sum, bad_src, bf16)) {
      if (residual) {
        const uint2 v = *reinterpret_cast<const uint2*>(residual + t * ldr + i);
        const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) sum[j] += __bfloat162float(vp[j]);
      }
      __nv_bfloat16 o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = __float2bfloat16_rn(sum[j]);
      *reinterpret_cast<uint2*>(out + t * ldo + i) = *reinterpret_cast<uint2*>(o);
    } else {
      report_status(st, kStatusPeerTimeout, 0x500 + bad_src, static_cast<uint32_t>(t), tag);
    }
    if (threadIdx.x == 0 && st != nullptr) {
      atomicAdd(reinterpret_cast<unsigned long long*>(st) + 2, globaltimer_ns() - w0);
      atomicAdd(reinterpret_cast<unsigned int*>(st) + 6, 1u);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) channel_finish(ctr, call);
}

// one CTA; rows <= 1024.  recv layout: [parity][src][rows_cap][2] floats (value, id)
__global__ void __launch_bounds__(1024)
argmax_allgather_kernel(int* __restrict__ ids, float* __restrict__ vals, int vocab_lo, int rows,
                        int rank, int world, int rows_cap, PeerPtrs peers, uint32_t* ctr,
                        uint32_t* seen, unsigned long long wait_ns, DeviceStatus* st) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t call = *reinterpret_cast<volatile uint32_t*>(ctr);
  const size_t slot_elems = static_cast<size_t>(rows_cap) * 2;
  const size_t base = (static_cast<size_t>(call & 1u) * world) * slot_elems;
  const int r = threadIdx.x;
  if (r < rows) {
    const int id = ids[r];
    const float2 v = make_float2(vals[r], id < 0 ? -1.f : static_cast<float>(id + vocab_lo));
    for (int pr = 0; pr < world; ++pr)
      *reinterpret_cast<float2*>(peers.recv[pr] + base + static_cast<size_t>(rank) * slot_elems + 2 * r) = v;
  }
  __syncthreads();
  if (threadIdx.x < world) flag_add_release_sys(peers.flags[threadIdx.x], 1u);
  __shared__ int ok_s;
  if (threadIdx.x == 0) {
    const uint32_t target = seen[0] + static_cast<uint32_t>(world);
    ok_s = flag_wait_ge(peers.flags[rank], target, wait_ns, st, 0x600) ? 1 : 0;
    seen[0] = target;
  }
  __syncthreads();
  if (ok_s && r < rows) {
    float best = -INFINITY;
    float bid = -1.f;
    for (int src = 0; src < world; ++src) {
      const float2 v = *reinterpret_cast<const float2*>(peers.recv[rank] + base + static_cast<size_t>(src) * slot_elems + 2 * r);
      if (v.y >= 0.f && (v.x > best || (v.x == best && v.y < bid) || bid < 0.f)) { best = v.x; bid = v.y; }
    }
    ids[r] = bid < 0.f ? -1 : static_cast<int>(bid);
    vals[r] = best;
  }
  if (threadIdx.x == 0) channel_finish(ctr, call);
}

__global__ void flag_wait_probe_kernel(const uint32_t* flag, uint32_t target, unsigned long long wait_ns,
                                       DeviceStatus* st, int* result) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0 && blockIdx.x == 0) *result = flag_wait_ge(flag, target, wait_ns, st, 0x700) ? 1 : 0;
}

// Peer-memory latency probe: two ranks bounce a counter through each other's memory `iters` times.
// mine = word in this rank's buffer (the peer writes it), theirs = word in the peer's buffer.
// out_ns[0] = total time seen by this rank.  Every wait is bounded.
__global__ void pingpong_kernel(volatile uint32_t* mine, volatile uint32_t* theirs, int iters, int initiator,
                                unsigned long long limit_ns, unsigned long long* out_ns, DeviceStatus* st) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const uint64_t t0 = globaltimer_ns();
  for (int i = 1; i <= iters; ++i) {
    if (initiator) *theirs = static_cast<uint32_t>(i);
    const uint64_t w0 = globaltimer_ns();
    uint32_t spins = 0;
    while (*mine != static_cast<uint32_t>(i)) {
      if ((++spins & 0x3fu) == 0u && globaltimer_ns() - w0 > limit_ns) {
        report_status(st, kStatusPeerTimeout, 0x710, static_cast<uint32_t>(i), *mine);
        out_ns[0] = 0;
        return;
      }
    }
    if (!initiator) *theirs = static_cast<uint32_t>(i);
  }
  out_ns[0] = globaltimer_ns() - t0;
}

}  // namespace fb

using namespace fb;

extern "C" int fb_ipc_handle_bytes(void) { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }

extern "C" int fb_ipc_alloc(void** ptr, long long bytes, void* handle_out) {
  if (!ptr || bytes <= 0 || !handle_out) return FB_ERR_SHAPE;
  if (cudaMalloc(ptr, static_cast<size_t>(bytes)) != cudaSuccess) return FB_ERR_RUNTIME;
  if (cudaMemset(*ptr, 0, static_cast<size_t>(bytes)) != cudaSuccess) return FB_ERR_RUNTIME;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, *ptr) != cudaSuccess) return FB_ERR_RUNTIME;
  memcpy(handle_out, &h, sizeof(h));
  return cudaDeviceSynchronize() == cudaSuccess ? FB_OK : FB_ERR_RUNTIME;
}

extern "C" int fb_ipc_open(const void* handle, void** ptr) {
  if (!handle || !ptr) return FB_ERR_SHAPE;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  return cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? FB_OK : FB_ERR_RUNTIME;
}

extern "C" int fb_ipc_close(void* ptr) {
  return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? FB_OK : FB_ERR_RUNTIME;
}

extern "C" int fb_ipc_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? FB_OK : FB_ERR_RUNTIME; }

static int fill_peers(PeerPtrs* p, void* const* recv, void* const* flags, int world) {
  if (world < 1 || world > 8) return FB_ERR_SHAPE;
  for (int i = 0; i < world; ++i) {
    if (!recv[i] || !flags[i]) return FB_ERR_SHAPE;
    p->recv[i] = static_cast<float*>(recv[i]);
    p->flags[i] = static_cast<uint32_t*>(flags[i]);
  }
  return FB_OK;
}

extern "C" int fb_moe_reduce_allreduce(const void* route_out, int slots, int topk, const int* topk_idx,
                                       int e_lo, int e_hi, const void* residual, long long ldr,
                                       void* out, long long ldo, int rows, int dim, int rank,
                                       int world, int rows_cap, void* const* peer_recv,
                                       void* const* peer_flags, void* ctr, int payload_bf16,
                                       unsigned long long wait_ns, void* status, void* stream) {
  return fb_moe_reduce_allreduce_mc(route_out, slots, topk, topk_idx, e_lo, e_hi, residual, ldr, out, ldo, rows, dim,
                                    rank, world, rows_cap, peer_recv, peer_flags, ctr, payload_bf16, wait_ns, nullptr,
                                    status, stream);
}

extern "C" int fb_moe_reduce_allreduce_mc(const void* route_out, int slots, int topk, const int* topk_idx,
                                          int e_lo, int e_hi, const void* residual, long long ldr,
                                          void* out, long long ldo, int rows, int dim, int rank,
                                          int world, int rows_cap, void* const* peer_recv,
                                          void* const* peer_flags, void* ctr, int payload_bf16,
                                          unsigned long long wait_ns, void* mc_recv, void* status, void* stream) {
  if (rows <= 0 || rows > rows_cap || dim % 4 != 0 || slots < 1 || slots < topk)
    return FB_ERR_SHAPE;
  if (rank < 0 || rank >= world || !ctr) return FB_ERR_SHAPE;
  PeerPtrs p{};
  const int rc = fill_peers(&p, peer_recv, peer_flags, world);
  if (rc != FB_OK) return rc;
  uint32_t* c = static_cast<uint32_t*>(ctr);
  launch_pdl(moe_reduce_allreduce_kernel, dim3(rows, (dim + 511) / 512), dim3(128), 0, static_cast<cudaStream_t>(stream),
      static_cast<const __nv_bfloat16*>(route_out), slots, topk, topk_idx, e_lo, e_hi,
      static_cast<const __nv_bfloat16*>(residual), ldr, static_cast<__nv_bfloat16*>(out), ldo, rows, dim,
      rank, world, rows_cap, p, c, payload_bf16, wait_ns ? wait_ns : 3000000000ull,
      static_cast<DeviceStatus*>(status), static_cast<uint8_t*>(mc_recv));
  return cudaGetLastError() == cudaSuccess ? FB_OK : FB_ERR_LAUNCH;
}

extern "C" int fb_argmax_allgather(int* ids, float* vals, int vocab_lo, int rows, int rank, int world,
                                   int rows_cap, void* const* peer_recv, void* const* peer_flags,
                                   void* ctr, unsigned long long wait_ns, void* status, void* stream) {
  if (rows <= 0 || rows > 1024 || rows > rows_cap || rank < 0 || rank >= world || !ctr) return FB_ERR_SHAPE;
  PeerPtrs p{};
  const int rc = fill_peers(&p, peer_recv, peer_flags, world);
  if (rc != FB_OK) return rc;
  uint32_t* c = static_cast<uint32_t*>(ctr);
  launch_pdl(argmax_allgather_kernel, dim3(1), dim3(1024), 0, static_cast<cudaStream_t>(stream), 
      ids, vals, vocab_lo, rows, rank, world, rows_cap, p, c, c + 2, wait_ns ? wait_ns : 3000000000ull,
      static_cast<DeviceStatus*>(status));
  return cudaGetLastError() == cudaSuccess ? FB_OK : FB_ERR_LAUNCH;
}

extern "C" int fb_flag_wait_probe(const void* flag, int target, unsigned long long wait_ns, void* status,
                                  int* result, void* stream) {
  launch_pdl(flag_wait_probe_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), 
      static_cast<const uint32_t*>(flag), static_cast<uint32_t>(target), wait_ns,
      static_cast<DeviceStatus*>(status), result);
  return cudaGetLastError() == cudaSuccess ? FB_OK : FB_ERR_LAUNCH;
}

extern "C" int fb_peer_pingpong(void* mine, void* theirs, int iters, int initiator, unsigned long long limit_ns,
                                void* out_ns, void* status, void* stream) {
  if (!mine || !theirs || iters <= 0 || !out_ns) return FB_ERR_SHAPE;
  pingpong_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<volatile uint32_t*>(mine), static_cast<volatile uint32_t*>(theirs), iters, initiator,
      limit_ns ? limit_ns : 2000000000ull, static_cast<unsigned long long*>(out_ns), static_cast<DeviceStatus*>(status));
  return cudaGetLastError() == cudaSuccess ? FB_OK : FB_ERR_LAUNCH;
}
