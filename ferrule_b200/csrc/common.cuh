// Shared device helpers for the sm_100a kernels: PTX wrappers for mbarrier, TMA
// (cp.async.bulk.tensor, single-CTA destination only), tcgen05 (alloc / mma /
// commit / ld), bounded waits and the device status word.
//
// Every wait in this library is bounded: a waiter that runs out of time records a
// code in the status word, raises the CTA-wide abort flag and returns false; the
// kernel then drains its own copies, frees its TMEM and exits.  Nothing here traps
// or spins without a limit.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fb {

// ---------------------------------------------------------------------------------
// status word (one per library instance, lives in global memory, host-readable)
// ---------------------------------------------------------------------------------
enum StatusCode : uint32_t {
  kStatusOk = 0,
  kStatusMbarTimeout = 1,      // a pipeline mbarrier did not flip in time
  kStatusPeerTimeout = 2,      // a flag written by another rank did not arrive in time
  kStatusBadIndex = 3,         // a page id / row index was out of range (access skipped)
  kStatusBadShape = 4,         // host launcher rejected the shape
};

struct DeviceStatus {
  uint32_t code;      // first failure wins
  uint32_t where;     // kernel-specific site id
  uint32_t detail0;
  uint32_t detail1;
};

__device__ __forceinline__ void report_status(DeviceStatus* st, uint32_t code, uint32_t where,
                                              uint32_t d0 = 0, uint32_t d1 = 0) {
  if (st == nullptr) return;
  if (atomicCAS(&st->code, 0u, code) == 0u) {
    st->where = where;
    st->detail0 = d0;
    st->detail1 = d1;
  }
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() {
  uint32_t l;
  asm volatile("mov.u32 %0, %%laneid;" : "=r"(l));
  return l;
}

// ---------------------------------------------------------------------------------
// programmatic dependent launch: a kernel launched with the programmatic-serialization
// attribute may start while its predecessor in the stream still runs.  `pdl_wait` blocks until
// the predecessor grid has completed and its writes are visible; everything before it must touch
// only memory the predecessor neither reads nor writes (barriers, TMEM, constant weights).
// Without the launch attribute both instructions do nothing.
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.b32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Limit for waits inside one CTA's pipeline (TMA landing, MMA retiring): far above
// any legitimate latency, far below anything a caller would call a hang.
constexpr uint64_t kPipeWaitNs = 2000ull * 1000ull * 1000ull;  // 2 s

// Bounded parity wait.  `abort_flag` is a CTA-shared word: once any role sets it,
// every other wait in the CTA gives up at its next poll.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity,
                                          volatile uint32_t* abort_flag, DeviceStatus* st,
                                          uint32_t where) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0xffu) == 0u) {
      if (*abort_flag != 0u) return false;
      if (globaltimer_ns() - t0 > kPipeWaitNs) {
        *abort_flag = 1u;
        report_status(st, kStatusMbarTimeout, where, parity, blockIdx.x);
        return false;
      }
    }
  }
}

// ---------------------------------------------------------------------------------
// thread-block clusters / distributed shared memory
// ---------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
// All threads of all CTAs of the cluster (hardware barrier, cannot wait on a missing peer:
// CTAs of one cluster are co-scheduled).
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cta address of this CTA -> shared::cluster address of the same offset in CTA `rank`
__device__ __forceinline__ uint32_t mapa_shared(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t cluster_addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t cluster_addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t cluster_addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(cluster_addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_bar_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar_addr)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
      "selp.b32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity,
                                                  volatile uint32_t* abort_flag, DeviceStatus* st,
                                                  uint32_t where) {
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((++spins & 0xffu) == 0u) {
      if (*abort_flag != 0u) return false;
      if (globaltimer_ns() - t0 > kPipeWaitNs) {
        *abort_flag = 1u;
        report_status(st, kStatusMbarTimeout, where, parity, blockIdx.x);
        return false;
      }
    }
  }
}

// ---------------------------------------------------------------------------------
// TMA (tiled bulk tensor copies; destination is always this CTA's own shared memory)
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tmap, uint64_t* bar,
                                            int32_t c0, int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)),
      "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const void* tmap, uint64_t* bar,
                                            int32_t c0, int32_t c1, int32_t c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)),
      "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// L2 eviction policy for data that is read once per step (weights of a decode step): such lines become the
// first candidates for eviction, so the step's reusable lines (activations, routing tables, kernel code) stay
// resident while tens of GB of weights stream through the cache.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}

__device__ __forceinline__ void tma_load_3d_hint(void* smem_dst, const void* tmap, uint64_t* bar, int32_t c0,
                                                 int32_t c1, int32_t c2, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4, %5}], [%2], %6;"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)),
      "r"(c0), "r"(c1), "r"(c2), "l"(policy)
      : "memory");
}

// ---------------------------------------------------------------------------------
// tcgen05 / TMEM
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem] * B[smem], bf16 inputs, fp32 accumulate, one CTA.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], 8-bit float inputs (e4m3/e5m2), fp32 accumulate.
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// All MMAs issued so far by this thread arrive on `bar` once they have retired.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns -> 16 registers per thread.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile laid out by TMA with the
// 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_k128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);  // start address
  d |= static_cast<uint64_t>(1) << 16;                      // leading byte offset (unused, 16 B)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;              // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;                      // descriptor version (Blackwell)
  d |= static_cast<uint64_t>(2) << 61;                      // SWIZZLE_128B
  return d;
}

// Instruction descriptor: fp32 accumulator, both operands K-major, M x N tile.
// fmt: 0 = f16 / e4m3, 1 = bf16 / e5m2 (meaning depends on the mma kind).
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t m, uint32_t n, uint32_t afmt,
                                                  uint32_t bfmt) {
  return (1u << 4) | (afmt << 7) | (bfmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// ---------------------------------------------------------------------------------
// small math helpers
// ---------------------------------------------------------------------------------
__device__ __forceinline__ float bf16_round(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
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

// ---------------------------------------------------------------------------------
// cross-GPU flags (plain peer memory; no multimem)
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void flag_add_release_sys(uint32_t* flag, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(flag), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t flag_ld_acquire_sys(const uint32_t* flag) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
  return v;
}
// Wait until *flag - target is non-negative (wrap-safe), for at most limit_ns.
__device__ __forceinline__ bool flag_wait_ge(const uint32_t* flag, uint32_t target,
                                             uint64_t limit_ns, DeviceStatus* st,
                                             uint32_t where) {
  uint32_t v = flag_ld_acquire_sys(flag);
  if (static_cast<int32_t>(v - target) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    v = flag_ld_acquire_sys(flag);
    if (static_cast<int32_t>(v - target) >= 0) {
      // words 4..6 of the status block: time spent waiting for peers (ns, 64-bit) and number of waits
      if (st != nullptr) {
        atomicAdd(reinterpret_cast<unsigned long long*>(st) + 2, globaltimer_ns() - t0);
        atomicAdd(reinterpret_cast<unsigned int*>(st) + 6, 1u);
      }
      return true;
    }
    if ((++spins & 0x3fu) == 0u) {
      if (globaltimer_ns() - t0 > limit_ns) {
        report_status(st, kStatusPeerTimeout, where, v, target);
        return false;
      }
    }
  }
}

// ---------------------------------------------------------------------------------
// Tagged pushes ("data + flag in one word"): every fp32 travels as the 8-byte pair {bits, tag}, two pairs
// per 16-byte store.  The receiver polls the words themselves until the tag equals the call's tag, so a
// push needs no separate fence / flag round trip: the one-way NVLink latency is all that is paid.  An
// 8-byte aligned pair is written atomically, so a store torn at 8 bytes is still consistent.  Tags are
// the call counter + 1 (never 0: buffers start zeroed); slots are double buffered by call parity.
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void ll_store2(void* dst, float a, float b, uint32_t tag) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(__float_as_uint(a)), "r"(tag),
               "r"(__float_as_uint(b)), "r"(tag)
               : "memory");
}
__device__ __forceinline__ uint4 ll_load_raw(const void* src) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src) : "memory");
  return v;
}
// Poll one 16-byte word until both tags match; false after limit_ns (status recorded by the caller).
__device__ __forceinline__ bool ll_wait2(const void* src, uint32_t tag, uint64_t limit_ns, float& a, float& b) {
  uint4 v = ll_load_raw(src);
  if (v.y != tag || v.w != tag) {
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
      v = ll_load_raw(src);
      if (v.y == tag && v.w == tag) break;
      if ((++spins & 0x3fu) == 0u && globaltimer_ns() - t0 > limit_ns) return false;
    }
  }
  a = __uint_as_float(v.x);
  b = __uint_as_float(v.z);
  return true;
}

// A slot holds `channels` values per row either as fp32 pairs {bits, tag} (8 bytes per channel) or as packed
// bf16 pairs {bf16x2, tag} (4 bytes per channel; halves the NVLink bytes, partials are rounded to bf16).
// Channel offsets are multiples of 4, so 4 channels are two (fp32) or one (bf16) aligned 16-byte words.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ void ll_store_words(void* dst, uint32_t w0, uint32_t w1, uint32_t tag) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(w0), "r"(tag), "r"(w1), "r"(tag)
               : "memory");
}
// base: start of the destination slot (this source's [rows_cap][channels] area); ch: row * channels + channel
__device__ __forceinline__ void ll_push4(void* base, size_t ch, const float (&v)[4], uint32_t tag, bool bf16) {
  if (bf16) {
    ll_store_words(static_cast<uint8_t*>(base) + ch * 4, pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), tag);
  } else {
    uint8_t* d = static_cast<uint8_t*>(base) + ch * 8;
    ll_store_words(d, __float_as_uint(v[0]), __float_as_uint(v[1]), tag);
    ll_store_words(d + 16, __float_as_uint(v[2]), __float_as_uint(v[3]), tag);
  }
}

// The same push through an NVLink multicast address: one store lands in the slot of every rank (the switch
// replicates it), so the pusher issues one store per 16 bytes instead of one per peer.
__device__ __forceinline__ void ll_store_words_mc(void* mc_dst, uint32_t w0, uint32_t w1, uint32_t tag) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_dst), "f"(__uint_as_float(w0)),
               "f"(__uint_as_float(tag)), "f"(__uint_as_float(w1)), "f"(__uint_as_float(tag))
               : "memory");
}
__device__ __forceinline__ void ll_push4_mc(void* mc_base, size_t ch, const float (&v)[4], uint32_t tag, bool bf16) {
  if (bf16) {
    ll_store_words_mc(static_cast<uint8_t*>(mc_base) + ch * 4, pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), tag);
  } else {
    uint8_t* d = static_cast<uint8_t*>(mc_base) + ch * 8;
    ll_store_words_mc(d, __float_as_uint(v[0]), __float_as_uint(v[1]), tag);
    ll_store_words_mc(d + 16, __float_as_uint(v[2]), __float_as_uint(v[3]), tag);
  }
}

// Gather 4 consecutive channels from the slots of `world` (<= 8) source ranks and add them in rank order.
// The loads of all ranks are issued together (one L2 round trip when everything has arrived); words whose
// tag is not the call's yet are re-polled.  first = source 0's slot, ch as in ll_push4, stride = bytes between
// consecutive sources' slots.  Returns false after limit_ns (bad_src = a source that was missing).
__device__ __forceinline__ bool ll_gather4(const void* first, size_t ch, size_t stride, int world, uint32_t tag,
                                           uint64_t limit_ns, float (&acc)[4], int& bad_src, bool bf16) {
  uint4 v[16];
  const uint8_t* p0 = static_cast<const uint8_t*>(first) + ch * (bf16 ? 4 : 8);
#pragma unroll
  for (int s = 0; s < 8; ++s) {
    if (s < world) {
      v[2 * s] = ll_load_raw(p0 + s * stride);
      if (!bf16) v[2 * s + 1] = ll_load_raw(p0 + s * stride + 16);
    }
  }
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while (true) {
    bool all = true;
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      if (s < world) {
        if (v[2 * s].y != tag || v[2 * s].w != tag) {
          v[2 * s] = ll_load_raw(p0 + s * stride);
          all = false;
          bad_src = s;
        }
        if (!bf16 && (v[2 * s + 1].y != tag || v[2 * s + 1].w != tag)) {
          v[2 * s + 1] = ll_load_raw(p0 + s * stride + 16);
          all = false;
          bad_src = s;
        }
      }
    }
    if (all) break;
    if (t0 == 0) t0 = globaltimer_ns();
    if ((++spins & 0x3fu) == 0u && globaltimer_ns() - t0 > limit_ns) return false;
  }
#pragma unroll
  for (int s = 0; s < 8; ++s) {
    if (s < world) {
      if (bf16) {
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v[2 * s].x));
        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v[2 * s].z));
        acc[0] += lo.x; acc[1] += lo.y; acc[2] += hi.x; acc[3] += hi.y;
      } else {
        acc[0] += __uint_as_float(v[2 * s].x);
        acc[1] += __uint_as_float(v[2 * s].z);
        acc[2] += __uint_as_float(v[2 * s + 1].x);
        acc[3] += __uint_as_float(v[2 * s + 1].z);
      }
    }
  }
  return true;
}

}  // namespace fb
