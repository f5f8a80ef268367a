// Stable-slot expert table on the device (routed experts streamed from host memory).
//
//   fb_expert_table_apply    apply install records {slot, expert, generation, evicted expert} to the
//                            device arrays expert -> slot, slot -> expert, slot -> generation.  Runs on
//                            the compute stream after it has waited for the upload event, so a slot
//                            becomes resolvable exactly when its weights have landed.
//   fb_expert_table_resolve  rewrite the route plan's per-tile expert ids into arena slots (the grouped
//                            GEMM then indexes the arena), count routes whose expert is absent and
//                            list those experts; tiles of absent experts get zero rows.
//
// Counterpart of expert_table_kernel
// (crates/ferrule-backend/native/cuda/implementations/portable/entrypoints.cu:1268-1380) and of the
// host mirror in crates/ferrule-backend/src/cuda/context.rs:1952-2300.
#include "common.cuh"
#include "ferrule_b200.h"
#include "launch.cuh"

namespace fb {

__global__ void expert_table_apply_kernel(int* __restrict__ expert_to_slot, int* __restrict__ slot_expert,
                                          int* __restrict__ slot_gen, const int4* __restrict__ updates, int n,
                                          int n_experts, int n_slots, DeviceStatus* st) {
  pdl_launch_dependents();
  pdl_wait();
  // one thread applies the records in order: a slot may be re-used within one batch of updates
  if (blockIdx.x != 0 || threadIdx.x != 0) return;
  for (int i = 0; i < n; ++i) {
    const int4 u = updates[i];
    if (u.x < 0 || u.x >= n_slots || u.y < 0 || u.y >= n_experts || u.w >= n_experts) {
      report_status(st, kStatusBadIndex, 0xA00, u.x, u.y);
      continue;
    }
    if (u.w >= 0 && expert_to_slot[u.w] == u.x) expert_to_slot[u.w] = -1;
    const int prev = slot_expert[u.x];
    if (prev >= 0 && prev < n_experts && expert_to_slot[prev] == u.x) expert_to_slot[prev] = -1;
    slot_expert[u.x] = u.y;
    slot_gen[u.x] = u.z;
    expert_to_slot[u.y] = u.x;
  }
}

// miss: [0] = number of tiles whose expert is absent, [1 + i] = those experts (first 63)
__global__ void expert_table_resolve_kernel(int* __restrict__ tile_group, int* __restrict__ tile_rows,
                                            const int* __restrict__ num_tiles, int max_tiles,
                                            const int* __restrict__ expert_to_slot, int n_experts,
                                            int* __restrict__ miss) {
  pdl_launch_dependents();
  pdl_wait();
  const int n = min(*num_tiles, max_tiles);
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < n; t += gridDim.x * blockDim.x) {
    const int e = tile_group[t];
    const int slot = (e >= 0 && e < n_experts) ? expert_to_slot[e] : -1;
    if (slot >= 0) {
      tile_group[t] = slot;
    } else {
      const int k = atomicAdd(&miss[0], 1);
      if (k < 63) miss[1 + k] = e;
      tile_group[t] = 0;
      tile_rows[t] = 0;     // the GEMM skips the tile instead of reading an unrelated slot
    }
  }
}

}  // namespace fb

using namespace fb;

#define FB_CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? FB_OK : FB_ERR_LAUNCH)

extern "C" int fb_expert_table_apply(int* expert_to_slot, int* slot_expert, int* slot_gen, const void* updates, int n,
                                     int n_experts, int n_slots, void* status, void* stream) {
  if (n <= 0 || !expert_to_slot || !slot_expert || !slot_gen || !updates) return FB_ERR_SHAPE;
  launch_pdl(expert_table_apply_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), expert_to_slot,
             slot_expert, slot_gen, static_cast<const int4*>(updates), n, n_experts, n_slots,
             static_cast<DeviceStatus*>(status));
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_expert_table_resolve(int* tile_group, int* tile_rows, const int* num_tiles, int max_tiles,
                                       const int* expert_to_slot, int n_experts, int* miss, void* stream) {
  if (!tile_group || !tile_rows || !num_tiles || max_tiles <= 0 || !expert_to_slot || !miss) return FB_ERR_SHAPE;
  launch_pdl(expert_table_resolve_kernel, dim3(1), dim3(256), 0, static_cast<cudaStream_t>(stream), tile_group,
             tile_rows, num_tiles, max_tiles, expert_to_slot, n_experts, miss);
  return FB_CHECK_LAUNCH();
}
