// In-switch (NVLS) collectives: helpers for kernels that reduce and broadcast through an NVLink multicast
// object with `multimem` instructions.
//
// A channel is one symmetric buffer, present at the same offset on every rank and bound to a multicast
// address range:  [ flags | stage x 2 | result x 2 ]
//   stage[p]   every rank writes its own partial rows here (plain local stores)
//   result[p]  the reduced rows, written on all ranks at once by their owner (multimem.st)
//   flags      A: partials written, B: reduced rows broadcast; they only grow, a waiter compares with a running
//              total kept in private memory
// Two-shot all-reduce: write partial -> signal A on all ranks (one multimem.red) -> the owner of a row waits for A,
// loads the row reduced in the switch (multimem.ld_reduce, fp32 accumulation), adds the residual, broadcasts it
// (multimem.st) and signals B -> every rank waits for B and reads the row locally.  Every rank sees the bits its
// owner produced, so replicated computations that follow (routing decisions) agree across ranks; that is why the
// reduction is not done one-shot by every rank for itself.  The owner-only half is a reduce-scatter, the
// broadcast half an all-gather.
//
// p = call parity: a rank can be at most one call ahead of a peer (finishing a call needs every peer's signals of
// that call, and a peer signals a call only after its kernel of the previous call has ended), so two buffers do.
// Every wait is bounded: on expiry the kernel records a status and returns.
#pragma once
#include "common.cuh"

namespace fb {

struct MmChannel {
  uint8_t* local;          // this rank's copy of the symmetric buffer
  uint8_t* mc;             // multicast address of the same buffer
  long long stage_off;     // bytes
  long long result_off;
  long long buf_bytes;     // bytes of one parity of stage / result
  uint32_t* priv;          // private: [0] calls, [1] CTAs done, [2] expected A, [3] expected B
  int rank, world;
  unsigned long long wait_ns;
};

enum { kMmFlagA = 0, kMmFlagB = 16 };   // word offsets inside the flag area (separate 64-byte lines)

__device__ __forceinline__ void mm_signal(const MmChannel& c, int flag_word, uint32_t v) {
  // release at system scope: everything this thread observed (its CTA's stores, through the preceding barrier) is
  // ordered before the flag update on every rank
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(reinterpret_cast<uint32_t*>(c.mc) + flag_word),
               "r"(v)
               : "memory");
}

// wait until the local flag has reached `target` (wrap-safe); false after wait_ns
__device__ __forceinline__ bool mm_wait(const MmChannel& c, int flag_word, uint32_t target, DeviceStatus* st,
                                        uint32_t where) {
  const uint32_t* f = reinterpret_cast<const uint32_t*>(c.local) + flag_word;
  uint32_t v = flag_ld_acquire_sys(f);
  if (static_cast<int32_t>(v - target) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    v = flag_ld_acquire_sys(f);
    if (static_cast<int32_t>(v - target) >= 0) {
      if (st != nullptr) {
        atomicAdd(reinterpret_cast<unsigned long long*>(st) + 2, globaltimer_ns() - t0);
        atomicAdd(reinterpret_cast<unsigned int*>(st) + 6, 1u);
      }
      return true;
    }
    if ((++spins & 0x3fu) == 0u && globaltimer_ns() - t0 > c.wait_ns) {
      report_status(st, kStatusPeerTimeout, where, v, target);
      return false;
    }
  }
}

// 8 bf16 values at `mc_addr` summed over all ranks in the switch (fp32 accumulation)
__device__ __forceinline__ uint4 mm_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}

// 16 bytes stored at the same offset on every rank
__device__ __forceinline__ void mm_st16(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

// rows [lo, hi) owned by `rank` when `rows` rows are split into contiguous, equal slices
__device__ __forceinline__ void mm_owned_rows(int rows, int world, int rank, int& lo, int& hi) {
  const int per = (rows + world - 1) / world;
  lo = min(rows, rank * per);
  hi = min(rows, lo + per);
}

// One warp reduces row `t` (dim channels, multiple of 8) of the staged partials in the switch, adds the residual
// row and broadcasts the bf16 result into every rank's result buffer.
__device__ __forceinline__ void mm_reduce_bcast_row(const MmChannel& c, uint32_t parity, int t, int dim,
                                                    const __nv_bfloat16* residual_row, int lane) {
  const long long row_off = static_cast<long long>(parity) * c.buf_bytes + static_cast<long long>(t) * dim * 2;
  const uint8_t* src = c.mc + c.stage_off + row_off;
  uint8_t* dst = c.mc + c.result_off + row_off;
  for (int i = lane * 8; i < dim; i += 32 * 8) {
    uint4 v = mm_ld_reduce_bf16x8(src + i * 2);
    if (residual_row != nullptr) {
      const uint4 r = *reinterpret_cast<const uint4*>(residual_row + i);
      __nv_bfloat162* vp = reinterpret_cast<__nv_bfloat162*>(&v);
      const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 a = __bfloat1622float2(vp[j]), b = __bfloat1622float2(rp[j]);
        vp[j] = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
      }
    }
    mm_st16(dst + i * 2, v);
  }
}

}  // namespace fb
