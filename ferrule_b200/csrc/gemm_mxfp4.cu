// MXFP4 x MXFP8 block-scaled weight-stationary GEMM for sm_100a, dense or grouped (routed experts).
//
//   out[row, n] = sum_k  (sx[row, k/32] * X[row, k]) * (sw[g, n, k/32] * W[g, n, k])
//
// Weights: packed e2m1 (two values per byte, low nibble first) [groups, N, K/2] with one UE8M0 scale per row and
// per 32 elements - the layout of the checkpoint's routed experts, so HBM holds half a byte per weight.
// Activations: e4m3 [rows, K] with one UE8M0 scale per 1 x 32 block (fb_quant_mxfp8_rows, or the SwiGLU epilogue of
// this kernel).  The products run on `tcgen05.mma kind::mxf8f6f4.block_scale`: the tensor core multiplies every
// 32-element slice by both scale factors itself and accumulates all of K in fp32 in TMEM, so the epilogue sees
// finished sums.
//
//   * weight tile = UMMA A operand (M = 128 output channels), activation rows = B operand (N = NTOK rows);
//   * TMA brings the packed 4-bit weights in with the 16U4_ALIGN16B tensor-map type, which spreads every 16 values
//     (8 bytes) over a 16-byte slot: a 128-element k-block is one 128-byte swizzle row, as for 8-bit operands;
//   * scale factors travel global -> shared memory -> TMEM: the weight scales are stored pre-arranged
//     (fb_mxfp4_prepare_sf) as one 512-byte block per (128 rows x 128 k) tile, fetched with a bulk copy beside the
//     weight tile and moved to TMEM by `tcgen05.cp.32x128b.warpx4`; the activation scales of a row tile are
//     arranged by the epilogue warps while the previous tile is still being multiplied (two buffers);
//   * every CTA issues its own loads (no cluster multicast), empty tiles of a static plan are skipped, every wait
//     is bounded.
//
// Epilogues: store (bf16 / fp32), SwiGLU (gate | up tiles) with optional re-quantisation of the product to MXFP8
// for the down projection, weighted scatter.
//
// Counterpart of the reference's grouped FP4 expert pipeline: the Mxf8f6f4 mainloops of
// crates/ferrule-backend/native/cuda/implementations/cutlass/architectures/sm103/grouped_fp4_gemm.cuh:52-105, its
// scale-factor layouts (:113-154), the scale re-layout kernel (:304-325, :475-507) and the pipeline order of
// grouped_fp4_moe.cuh:1115-1222 (gate|up -> SwiGLU * weight -> re-quantise -> down -> scatter).
#include <cuda.h>
#include <cuda_fp8.h>
#include <cstdlib>

#include "common.cuh"
#include "ferrule_b200.h"
#include "launch.cuh"

namespace fb {
namespace mx {

constexpr int kTileN = 128;
constexpr int kBlockK = 128;     // elements per k-block = 128 bytes of (padded) shared memory = 4 scale blocks
constexpr int kUmmaK = 32;
constexpr int kThreads = 192;
constexpr int kSfAtom = 512;     // bytes of one scale-factor block: 32 rows x 16 bytes

enum { kOutBf16 = 0, kOutF32 = 1, kOutMxfp8 = 2 };

struct Params {
  int n_out, k, n_tiles, dual_offset, dense_rows, max_tok_tiles, stages;
  const int* tile_group;
  const int* tile_row0;
  const int* tile_rows;
  const int* num_tok_tiles;
  const uint8_t* w_sf;         // prepared weight scales [groups][sf_tiles][k_blocks][512]
  int sf_tiles;                // 128-row scale tiles per group
  const uint8_t* x_scale;      // [rows, k / 32]
  long long ldxs;
  int x_rows_total;
  void* out;
  long long ldo;
  int out_mode;
  uint8_t* out_scale;          // kOutMxfp8: [rows, n_out / 32]
  long long ldos;
  int epilogue;                // 0 store, 1 swiglu, 2 scatter
  const int* dst_row;
  const float* row_scale;
  float act_limit;
  DeviceStatus* status;
  int w_stream;
  int w_tx_bytes;              // bytes one weight-tile load completes on its barrier
  int a_fmt;                   // element format of the weights in the instruction descriptor: 5 = e2m1, 0 = e4m3
  int w_tiled;                 // weights stored tile-major: [groups][128-row tiles][k-blocks][128 rows][64 bytes]
  int sfb_bytes;               // one activation-scale buffer in shared memory
  int sfb_cols;                // TMEM columns of the activation scales of one tile
  int sfb_stride;              // TMEM columns per k-block (4: scale operands start on 4-column boundaries)
  int tmem_cols;
  // static row slots (decode-sized MoE batches) instead of a tile table: group g owns rows [g * slot_rows,
  // (g + 1) * slot_rows), slot_cnt[g] of them are filled, and the slot is walked in slot_rows / NTOK tiles
  const int* slot_cnt;
  int slot_rows;
};

// (group, first row, valid rows) of row tile m
template <int NTOK>
__device__ __forceinline__ void tile_of(const Params& p, int m, int& g, int& row0, int& rows) {
  if (p.slot_rows > 0) {
    const int per = p.slot_rows / NTOK;
    g = m / per;
    const int sub = m - g * per;
    row0 = g * p.slot_rows + sub * NTOK;
    rows = min(max(p.slot_cnt[g] - sub * NTOK, 0), NTOK);
  } else if (p.tile_group != nullptr) {
    g = p.tile_group[m];
    row0 = p.tile_row0[m];
    rows = min(p.tile_rows[m], NTOK);
  } else {
    g = 0;
    row0 = m * NTOK;
    rows = min(NTOK, p.dense_rows - row0);
  }
}

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }

__device__ __forceinline__ uint8_t e8m0_ceil(float x) {
  const uint32_t bits = __float_as_uint(x);
  int e = static_cast<int>((bits >> 23) & 0xff);
  if (bits & 0x7fffffu) ++e;
  e = max(0, min(254, e));
  return static_cast<uint8_t>(e);
}
__device__ __forceinline__ float e8m0_val(uint8_t b) {
  return b == 0 ? __uint_as_float(1u << 22) : __uint_as_float(static_cast<uint32_t>(b) << 23);
}

// D[tmem] (+)= (A * SFA) x (B * SFB); A e2m1, B e4m3, scales UE8M0 in TMEM, K = 32.
__device__ __forceinline__ void umma_mx(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                        uint32_t accumulate, uint32_t tsfa, uint32_t tsfb) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb)
      : "memory");
}

// 32 rows x 16 bytes of shared memory -> 4 TMEM columns, replicated over the four 32-lane quarters.
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint32_t smem_addr) {
  // shared-memory matrix descriptor, no swizzle: 8-row groups of 16-byte rows, 128 bytes apart
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(16 >> 4) << 16;     // leading byte offset (one 16-byte column: unused)
  d |= static_cast<uint64_t>(128 >> 4) << 32;    // stride byte offset between 8-row groups
  d |= static_cast<uint64_t>(1) << 46;
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(d) : "memory");
}

__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// instruction descriptor of the block-scaled kinds: A e2m1 (5), B e4m3 (0), both K-major, UE8M0 scales,
// scale-factor byte ids of A and B (which of the four bytes of a TMEM scale column this K = 32 slice uses)
__device__ __forceinline__ uint32_t mx_idesc(uint32_t n, uint32_t a_sf_id, uint32_t b_sf_id, uint32_t a_fmt) {
  return (b_sf_id << 4) | (a_fmt << 7) | (0u << 10) | ((n >> 3) << 17) | (1u << 23) | ((kTileN >> 4) << 24) |
         (a_sf_id << 29);
}

template <int NTOK, bool DUAL>
struct Cfg {
  static constexpr int kWBytes = kTileN * kBlockK;            // shared-memory bytes of a weight tile (4-bit values in 8-bit slots)
  static constexpr int kXBytes = NTOK * kBlockK;
  static constexpr int kSfaBytes = 1024;                      // one or two 512-byte blocks, padded to the swizzle alignment
  static constexpr int kStageBytes = kWBytes * (DUAL ? 2 : 1) + kXBytes + kSfaBytes;
  static constexpr int kAccCols = NTOK * (DUAL ? 2 : 1);
  static constexpr int kG = (NTOK + 31) / 32;                 // 32-row groups of the activation tile
};

template <int NTOK, bool DUAL>
__global__ void __launch_bounds__(kThreads, 1)
gemm_mxfp4_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                  const Params p) {
  using C = Cfg<NTOK, DUAL>;
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw_mx[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw_mx) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int nstages = p.stages;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + nstages * C::kStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + nstages;
  uint64_t* acc_full = bars + 2 * nstages;
  uint64_t* acc_empty = acc_full + 2;
  uint64_t* sfb_full = acc_empty + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sfb_full + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  uint8_t* sfb_smem = reinterpret_cast<uint8_t*>(bars) + 256;           // two buffers of p.sfb_bytes
  __nv_bfloat16* st_stage = reinterpret_cast<__nv_bfloat16*>(sfb_smem + 2 * p.sfb_bytes);   // two [16][128] bf16 chunks

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < nstages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);
      mbar_init(&sfb_full[a], 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, static_cast<uint32_t>(p.tmem_cols));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // TMEM columns: [two accumulator buffers | weight scales (4 per tile of the pair) | activation scales]
  const uint32_t tmem_sfa = tmem_base + 2 * C::kAccCols;
  const uint32_t tmem_sfb = tmem_sfa + 8;
  pdl_wait();

  const bool grouped = p.tile_group != nullptr || p.slot_rows > 0;
  const int num_tok_tiles = p.slot_rows > 0 ? p.max_tok_tiles
                            : grouped ? min(*p.num_tok_tiles, p.max_tok_tiles) : (p.dense_rows + NTOK - 1) / NTOK;
  const int total = num_tok_tiles * p.n_tiles;
  const int kblocks = p.k / kBlockK;
  const int tile_first = blockIdx.x, tile_stride = gridDim.x;
  auto empty = [&](int t) {
    if (!grouped) return false;
    int g_, r0_, rows_;
    tile_of<NTOK>(p, t / p.n_tiles, g_, r0_, rows_);
    return rows_ <= 0;
  };

  if (warp == 0) {
    // ------------------------------ producer: weights, their scales, activations ------------------------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      long long issued = 0;
      const uint64_t wpol = l2_policy_evict_first();
      const uint32_t tx = static_cast<uint32_t>(p.w_tx_bytes) * (DUAL ? 2 : 1) + C::kXBytes + kSfAtom * (DUAL ? 2 : 1);
      for (int t = tile_first; t < total && ok; t += tile_stride) {
        if (empty(t)) continue;
        const int m = t / p.n_tiles, nt = t - m * p.n_tiles;
        int g, row0, rows_t;
        tile_of<NTOK>(p, m, g, row0, rows_t);
        const uint8_t* sf_g = p.w_sf + (static_cast<size_t>(g) * p.sf_tiles + nt) * kblocks * kSfAtom;
        const uint8_t* sf_u = DUAL ? p.w_sf + (static_cast<size_t>(g) * p.sf_tiles + p.dual_offset / kTileN + nt) * kblocks * kSfAtom
                                   : nullptr;
        for (int kb = 0; kb < kblocks; ++kb) {
          ok = mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag, p.status, 0x900);
          if (!ok) break;
          uint8_t* stage = smem + s * C::kStageBytes;
          uint8_t* sfa = stage + C::kWBytes * (DUAL ? 2 : 1) + C::kXBytes;
          mbar_arrive_expect_tx(&full_bar[s], tx);
          if (p.w_tiled) {
            // tile-major weights: every (128 rows x 128 k) tile is 8 KB of consecutive global memory
            const int t0 = ((g * p.sf_tiles + nt) * kblocks + kb) * kTileN;
            tma_load_3d_hint(stage, &tmap_w, &full_bar[s], 0, t0, 0, wpol);
            if (DUAL)
              tma_load_3d_hint(stage + C::kWBytes, &tmap_w, &full_bar[s], 0,
                               ((g * p.sf_tiles + p.dual_offset / kTileN + nt) * kblocks + kb) * kTileN, 0, wpol);
          } else if (p.w_stream) {
            tma_load_3d_hint(stage, &tmap_w, &full_bar[s], kb * kBlockK, nt * kTileN, g, wpol);
            if (DUAL)
              tma_load_3d_hint(stage + C::kWBytes, &tmap_w, &full_bar[s], kb * kBlockK, p.dual_offset + nt * kTileN, g, wpol);
          } else {
            tma_load_3d(stage, &tmap_w, &full_bar[s], kb * kBlockK, nt * kTileN, g);
            if (DUAL) tma_load_3d(stage + C::kWBytes, &tmap_w, &full_bar[s], kb * kBlockK, p.dual_offset + nt * kTileN, g);
          }
          bulk_g2s(sfa, sf_g + static_cast<size_t>(kb) * kSfAtom, kSfAtom, &full_bar[s]);
          if (DUAL) bulk_g2s(sfa + kSfAtom, sf_u + static_cast<size_t>(kb) * kSfAtom, kSfAtom, &full_bar[s]);
          tma_load_2d(stage + C::kWBytes * (DUAL ? 2 : 1), &tmap_x, &full_bar[s], kb * kBlockK, row0);
          ++issued;
          if (++s == nstages) { s = 0; ph ^= 1u; }
        }
      }
      if (*abort_flag) {
        // copies of this thread may still be in flight: the CTA may not exit under them
        const long long first = issued > nstages ? issued - nstages : 0;
        for (long long i = first; i < issued; ++i) {
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(&full_bar[i % nstages], static_cast<uint32_t>((i / nstages) & 1)) &&
                 globaltimer_ns() - t0 < 2000000ull) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (scale copies + block-scaled MMAs) ------------------------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      long long ti = 0;           // non-empty tiles handled by this CTA: accumulator and scale buffer parity
      bool ok = true;
      for (int t = tile_first; t < total && ok; t += tile_stride) {
        if (empty(t)) continue;
        const int a = static_cast<int>(ti & 1);
        const uint32_t aph = static_cast<uint32_t>((ti >> 1) & 1);
        ok = mbar_wait(&acc_empty[a], aph ^ 1u, abort_flag, p.status, 0x910);
        if (!ok) break;
        ok = mbar_wait(&sfb_full[a], aph, abort_flag, p.status, 0x911);
        if (!ok) break;
        tc_fence_after();
        // activation scales of the whole tile: one copy per 512-byte block (4 TMEM columns each)
        {
          const uint32_t src = smem_u32(sfb_smem + a * p.sfb_bytes);
          for (int c = 0; c < p.sfb_cols; c += 4) tmem_cp_sf(tmem_sfb + c, src + (c / 4) * kSfAtom);
        }
        const uint32_t d0 = tmem_base + a * C::kAccCols;
        for (int kb = 0; kb < kblocks; ++kb) {
          ok = mbar_wait(&full_bar[s], ph, abort_flag, p.status, 0x912);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sw = smem_u32(smem + s * C::kStageBytes);
          const uint32_t sx = sw + C::kWBytes * (DUAL ? 2 : 1);
          const uint32_t ssf = sx + C::kXBytes;
          tmem_cp_sf(tmem_sfa, ssf);
          if (DUAL) tmem_cp_sf(tmem_sfa + 4, ssf + kSfAtom);
          const uint32_t tsfb = tmem_sfb + kb * p.sfb_stride;
#pragma unroll
          for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
            const uint32_t koff = kk * kUmmaK;     // bytes: one 8-bit slot per element in shared memory
            const uint64_t db = umma_desc_k128(sx + koff);
            const uint32_t idesc = mx_idesc(NTOK, kk, kk, static_cast<uint32_t>(p.a_fmt));
            const uint32_t acc = (kb > 0 || kk) ? 1u : 0u;
            umma_mx(d0, umma_desc_k128(sw + koff), db, idesc, acc, tmem_sfa, tsfb);
            if (DUAL) umma_mx(d0 + NTOK, umma_desc_k128(sw + C::kWBytes + koff), db, idesc, acc, tmem_sfa + 4, tsfb);
          }
          umma_commit(&empty_bar[s]);
          if (++s == nstages) { s = 0; ph ^= 1u; }
        }
        if (ok) umma_commit(&acc_full[a]);
        ++ti;
      }
    }
  } else {
    // ------------------------------ epilogue warps (and activation-scale staging) ------------------------------
    const int q = warp & 3;
    const int ch = q * 32 + lane;
    const int epi_tid = (warp - 2) * 32 + lane;
    long long ti = 0;
    bool ok = true;
    uint32_t chunk_ctr = 0;
    // arrange the activation scales of tile `t` for the tensor core: row n = r + 32 g, k-block kb -> TMEM column
    // kb * 4 + g, i.e. byte kb * 512 + r * 16 + g * 4 + (32-element slice) of the buffer
    auto stage_sfb = [&](int t, int buf) {
      const int m = t / p.n_tiles;
      int g_, row0, rows;
      tile_of<NTOK>(p, m, g_, row0, rows);
      uint8_t* dst = sfb_smem + buf * p.sfb_bytes;
      for (int i = epi_tid; i < NTOK * kblocks; i += 128) {
        const int n = i / kblocks, kb = i - n * kblocks;
        uint32_t w = 0x7f7f7f7fu;
        if (n < rows && row0 + n < p.x_rows_total)
          w = *reinterpret_cast<const uint32_t*>(p.x_scale + static_cast<long long>(row0 + n) * p.ldxs + kb * 4);
        const int col = kb * p.sfb_stride + (n >> 5);
        *reinterpret_cast<uint32_t*>(dst + (col >> 2) * kSfAtom + (n & 31) * 16 + (col & 3) * 4) = w;
      }
      fence_proxy_async_smem();               // the copy to TMEM reads through the async proxy
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (epi_tid == 0) mbar_arrive(&sfb_full[buf]);
    };
    // first non-empty tile of this CTA
    int t_next = tile_first;
    while (t_next < total && empty(t_next)) t_next += tile_stride;
    if (t_next < total) stage_sfb(t_next, 0);
    for (int t = t_next; t < total && ok;) {
      int t_after = t + tile_stride;
      while (t_after < total && empty(t_after)) t_after += tile_stride;
      const int a = static_cast<int>(ti & 1);
      const uint32_t aph = static_cast<uint32_t>((ti >> 1) & 1);
      // the other scale buffer belonged to the tile before this one, whose products have been drained
      if (t_after < total) stage_sfb(t_after, a ^ 1);
      const int m = t / p.n_tiles, nt = t - m * p.n_tiles;
      int g_, row0, rows;
      tile_of<NTOK>(p, m, g_, row0, rows);
      const int n = nt * kTileN + ch;
      ok = mbar_wait(&acc_full[a], aph, abort_flag, p.status, 0x920);
      if (!ok) break;
      tc_fence_after();
      const uint32_t tb = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + a * C::kAccCols;
#pragma unroll 1
      for (int c0 = 0; c0 < NTOK; c0 += 16) {
        if (c0 >= rows) break;
        uint32_t v[16], u[16];
        tmem_ld16(tb + c0, v);
        if (DUAL) tmem_ld16(tb + NTOK + c0, u);
        tmem_ld_wait();
        float x[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          x[j] = __uint_as_float(v[j]);
          if (DUAL) {
            float up = __uint_as_float(u[j]);
            if (p.act_limit > 0.f) {
              x[j] = fminf(x[j], p.act_limit);
              up = fminf(fmaxf(up, -p.act_limit), p.act_limit);
            }
            x[j] = silu(x[j]) * up;
          }
          if (p.epilogue == 2 && p.row_scale && c0 + j < rows) x[j] *= p.row_scale[row0 + c0 + j];
        }
        if (p.out_mode == kOutMxfp8) {
          // the 32 lanes of a warp hold 32 consecutive channels of a row: exactly one scale block.  Quantise the
          // bf16-rounded value (the tensor the unfused pipeline would have written) to e4m3 with a UE8M0 scale.
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int r = c0 + j;
            const float xb = bf16_round(x[j]);
            const float amax = fmaxf(warp_max(n < p.n_out ? fabsf(xb) : 0.f), 1e-4f);
            const uint8_t sb = e8m0_ceil(amax / 448.f);
            if (r < rows && n < p.n_out) {
              const long long orow = row0 + r;
              reinterpret_cast<uint8_t*>(p.out)[orow * p.ldo + n] =
                  static_cast<uint8_t>(__nv_cvt_float_to_fp8(xb / e8m0_val(sb), __NV_SATFINITE, __NV_E4M3));
              if (lane == 0) p.out_scale[orow * p.ldos + n / 32] = sb;
            }
          }
        } else if (p.out_mode == kOutF32) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int r = c0 + j;
            if (r < rows && n < p.n_out) {
              long long orow = row0 + r;
              if (p.epilogue == 2 && p.dst_row) orow = p.dst_row[row0 + r];
              if (orow >= 0) reinterpret_cast<float*>(p.out)[orow * p.ldo + n] = x[j];
            }
          }
        } else {
          // bf16 rows leave through a staging tile: 8 threads write each row's 256 bytes
          __nv_bfloat16* sb = st_stage + (chunk_ctr & 1) * (16 * 128);
#pragma unroll
          for (int j = 0; j < 16; ++j) sb[j * 128 + ch] = __float2bfloat16_rn(c0 + j < rows ? x[j] : 0.f);
          asm volatile("bar.sync 1, 128;" ::: "memory");
          {
            const int j = epi_tid >> 3, seg = epi_tid & 7;
            const int r = c0 + j;
            if (r < rows) {
              long long orow = row0 + r;
              if (p.epilogue == 2 && p.dst_row) orow = p.dst_row[row0 + r];
              const int col0 = nt * kTileN + seg * 16;
              if (orow >= 0 && col0 < p.n_out) {
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + orow * p.ldo + col0;
                const uint4* src = reinterpret_cast<const uint4*>(sb + j * 128 + seg * 16);
                reinterpret_cast<uint4*>(dst)[0] = src[0];
                if (col0 + 8 < p.n_out) reinterpret_cast<uint4*>(dst)[1] = src[1];
              }
            }
          }
          ++chunk_ctr;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[a]);
      ++ti;
      t = t_after;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(p.tmem_cols));
  }
}

// ---------------------------------------------------------------------------------
// scale re-layout (once per weight, at load time): linear UE8M0 [groups, rows, k/32] -> one 512-byte block per
// (128 rows, 128 k): byte (r % 32) * 16 + (r / 32) * 4 + slice, rows beyond the weight padded with 0x7f (= 1.0)
// ---------------------------------------------------------------------------------
__global__ void mxfp4_prepare_sf_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, int groups, int rows,
                                        int kblocks, int sf_tiles) {
  const long long total = static_cast<long long>(groups) * sf_tiles * kblocks * kSfAtom;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int b = static_cast<int>(i % kSfAtom);
    const long long blk = i / kSfAtom;
    const int kb = static_cast<int>(blk % kblocks);
    const long long gt = blk / kblocks;
    const int rt = static_cast<int>(gt % sf_tiles), g = static_cast<int>(gt / sf_tiles);
    const int r = b >> 4, gg = (b >> 2) & 3, kk = b & 3;
    const int row = rt * kTileN + gg * 32 + r;
    out[i] = row < rows ? in[(static_cast<long long>(g) * rows + row) * (kblocks * 4) + kb * 4 + kk] : 0x7f;
  }
}

// bf16 [rows, n] -> e4m3 codes + one UE8M0 scale per 1 x 32 block (amax floored at 1e-4, scale = 2^ceil(log2(amax/448)))
__global__ void __launch_bounds__(256)
quant_mxfp8_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q, long long ldq,
                        uint8_t* __restrict__ scale, long long lds, int rows, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const int blocks_per_row = n / 128;
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= rows * blocks_per_row) return;
  const int r = w / blocks_per_row, b = w - r * blocks_per_row;
  const uint2 raw = *reinterpret_cast<const uint2*>(x + r * ldx + b * 128 + lane * 4);
  const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(&raw);
  float f[4], amax = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    f[j] = __bfloat162float(v[j]);
    amax = fmaxf(amax, fabsf(f[j]));
  }
  // 8 lanes share one 32-element block
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
  amax = fmaxf(amax, 1e-4f);
  const uint8_t sb = e8m0_ceil(amax / 448.f);
  const float inv = 1.f / e8m0_val(sb);
  uint8_t c[4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
    c[j] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(f[j] * inv, __NV_SATFINITE, __NV_E4M3));
  *reinterpret_cast<uint32_t*>(q + r * ldq + b * 128 + lane * 4) = *reinterpret_cast<uint32_t*>(c);
  if ((lane & 7) == 0) scale[r * lds + b * 4 + (lane >> 3)] = sb;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encoder() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// dims in elements (4-bit values for the packed type), strides in bytes
static int make_map(CUtensorMap* map, CUtensorMapDataType type, const void* base, uint64_t k, uint64_t rows,
                    uint64_t groups, uint64_t row_stride, uint64_t group_stride, uint32_t box_rows, int rank,
                    int align) {
  EncodeTiledFn fn = encoder();
  if (!fn) return FB_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & (align - 1)) || (row_stride & (align - 1)) || (group_stride & (align - 1)))
    return FB_ERR_ALIGN;
  cuuint64_t dims[3] = {k, rows, groups};
  cuuint64_t strides[2] = {row_stride, group_stride};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(kBlockK), box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, type, rank, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? FB_OK : FB_ERR_DRIVER;
}

template <int NTOK, bool DUAL>
static int launch(const CUtensorMap& mw, const CUtensorMap& mx_, Params p, int max_tiles, cudaStream_t stream) {
  using C = Cfg<NTOK, DUAL>;
  auto kern = gemm_mxfp4_kernel<NTOK, DUAL>;
  constexpr int kLimit = 227 * 1024;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kLimit) != cudaSuccess)
      return FB_ERR_LAUNCH;
    attr = true;
  }
  const int kblocks = p.k / kBlockK;
  // A scale-factor operand of the MMA must start on a 4-column boundary of TMEM (an address in between raises
  // "misaligned address"), so every k-block owns one full 4-column group, whatever the row-tile size.
  p.sfb_stride = 4;
  p.sfb_cols = (kblocks * p.sfb_stride + 3) / 4 * 4;
  p.sfb_bytes = p.sfb_cols / 4 * kSfAtom;
  int cols = 2 * C::kAccCols + 8 + p.sfb_cols;
  int pow2 = 32;
  while (pow2 < cols) pow2 *= 2;
  if (pow2 > 512) return FB_ERR_SHAPE;            // K too long for this row-tile size
  p.tmem_cols = pow2;
  const int fixed = 1024 + 256 + 2 * p.sfb_bytes + 2 * 16 * 128 * 2;
  int stages = (kLimit - fixed) / C::kStageBytes;
  if (stages > 8) stages = 8;
  if (stages < 2) return FB_ERR_SHAPE;
  p.stages = stages;
  const size_t smem = static_cast<size_t>(stages) * C::kStageBytes + fixed;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int ctas = max_tiles < sms ? (max_tiles < 1 ? 1 : max_tiles) : sms;
  launch_pdl(kern, dim3(ctas), dim3(kThreads), smem, stream, mw, mx_, p);
  return cudaGetLastError() == cudaSuccess ? FB_OK : FB_ERR_LAUNCH;
}

}  // namespace mx
}  // namespace fb

using namespace fb;
using namespace fb::mx;

extern "C" int fb_gemm_mxfp4(const FbGemmMxfp4Args* a, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!a || !a->w || !a->x || !a->out || !a->w_sf || !a->x_scale) return FB_ERR_SHAPE;
  if (a->n_out <= 0 || a->k <= 0 || a->k % 128 != 0 || a->groups <= 0 || a->x_rows <= 0) return FB_ERR_SHAPE;
  if (a->epilogue < 0 || a->epilogue > 2 || a->out_mode < 0 || a->out_mode > 2) return FB_ERR_SHAPE;
  const bool dual = a->epilogue == 1;
  if (a->ntok != 16 && a->ntok != 32 && a->ntok != 64 && a->ntok != 128) return FB_ERR_SHAPE;
  if (dual && (a->ntok > 64 || a->dual_offset % 128 != 0)) return FB_ERR_SHAPE;
  if (a->out_mode == kOutMxfp8 && (!a->out_scale || a->epilogue == 2 || a->n_out % 32 != 0)) return FB_ERR_SHAPE;
  const bool slots = a->slot_rows > 0;
  if (slots && (!a->slot_cnt || a->tile_group || a->slot_rows % a->ntok != 0 ||
                static_cast<long long>(a->groups) * a->slot_rows > a->x_rows))
    return FB_ERR_SHAPE;
  const bool grouped = a->tile_group != nullptr || slots;
  if (a->tile_group && (!a->tile_row0 || !a->tile_rows || !a->num_tok_tiles || a->max_tok_tiles <= 0)) return FB_ERR_SHAPE;
  if (!grouped && a->groups != 1) return FB_ERR_SHAPE;
  if (a->out_mode == kOutBf16 && ((a->ldo % 8) != 0 || (reinterpret_cast<uintptr_t>(a->out) & 15) || a->n_out % 8 != 0))
    return FB_ERR_ALIGN;
  if ((a->ldxs % 4) != 0 || (reinterpret_cast<uintptr_t>(a->x_scale) & 3) || (reinterpret_cast<uintptr_t>(a->w_sf) & 15))
    return FB_ERR_ALIGN;
  CUtensorMap mw, mxm;
  // packed 4-bit weights: dimensions count values, strides are bytes (half a byte per value)
  int rc;
  if (a->w_fp8) {
    // e4m3 weights (one byte per value) under the same per-32 scale layout: a plain byte map, no unpacking
    if (a->w_tiled) return FB_ERR_SHAPE;
    rc = make_map(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->w, a->k, a->w_rows_per_group, a->groups,
                  static_cast<uint64_t>(a->ldw_bytes), static_cast<uint64_t>(a->w_group_stride_bytes), kTileN, 3, 16);
  } else if (a->w_tiled) {
    const uint64_t tiles = static_cast<uint64_t>(a->groups) * ((a->w_rows_per_group + kTileN - 1) / kTileN) * (a->k / kBlockK);
    rc = make_map(&mw, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, a->w, kBlockK, tiles * kTileN, 1, kBlockK / 2,
                  tiles * kTileN * (kBlockK / 2), kTileN, 3, 32);
  } else {
    rc = make_map(&mw, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, a->w, a->k, a->w_rows_per_group, a->groups,
                  static_cast<uint64_t>(a->ldw_bytes), static_cast<uint64_t>(a->w_group_stride_bytes), kTileN, 3, 32);
  }
  if (rc != FB_OK) return rc;
  rc = make_map(&mxm, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->x, a->k, a->x_rows, 1, a->ldx, 0, a->ntok, 2, 16);
  if (rc != FB_OK) return rc;
  Params p{};
  p.n_out = a->n_out;
  p.k = a->k;
  p.n_tiles = (a->n_out + kTileN - 1) / kTileN;
  p.dual_offset = a->dual_offset;
  p.dense_rows = a->x_rows;
  p.x_rows_total = a->x_rows;
  p.max_tok_tiles = slots ? a->groups * (a->slot_rows / a->ntok) : a->max_tok_tiles;
  p.slot_cnt = a->slot_cnt;
  p.slot_rows = slots ? a->slot_rows : 0;
  p.tile_group = a->tile_group;
  p.tile_row0 = a->tile_row0;
  p.tile_rows = a->tile_rows;
  p.num_tok_tiles = a->num_tok_tiles;
  p.w_sf = static_cast<const uint8_t*>(a->w_sf);
  p.sf_tiles = (a->w_rows_per_group + kTileN - 1) / kTileN;
  p.x_scale = static_cast<const uint8_t*>(a->x_scale);
  p.ldxs = a->ldxs;
  p.out = a->out;
  p.ldo = a->ldo;
  p.out_mode = a->out_mode;
  p.out_scale = static_cast<uint8_t*>(a->out_scale);
  p.ldos = a->ldos;
  p.epilogue = a->epilogue;
  p.dst_row = a->dst_row;
  p.row_scale = a->row_scale;
  p.act_limit = a->act_limit;
  p.status = static_cast<DeviceStatus*>(a->status);
  {
    static const bool enabled = [] {
      const char* e = getenv("FERRULE_W_EVICT_FIRST");
      return !(e && e[0] == '0');
    }();
    p.w_stream = enabled && (grouped ? a->ntok <= 64 : a->x_rows <= 256);
  }
  // a weight-tile load reports the bytes it read from global memory (half a byte per value) on its barrier, not
  // the bytes it spread over shared memory
  p.w_tx_bytes = a->w_fp8 ? kTileN * kBlockK : kTileN * kBlockK / 2;
  p.a_fmt = a->w_fp8 ? 0 : 5;
  p.w_tiled = a->w_tiled;
  const int tok_tiles = grouped ? p.max_tok_tiles : (a->x_rows + a->ntok - 1) / a->ntok;
  const int max_tiles = tok_tiles * p.n_tiles;
  if (dual) {
    switch (a->ntok) {
      case 16: return launch<16, true>(mw, mxm, p, max_tiles, stream);
      case 32: return launch<32, true>(mw, mxm, p, max_tiles, stream);
      default: return launch<64, true>(mw, mxm, p, max_tiles, stream);
    }
  }
  switch (a->ntok) {
    case 16: return launch<16, false>(mw, mxm, p, max_tiles, stream);
    case 32: return launch<32, false>(mw, mxm, p, max_tiles, stream);
    case 64: return launch<64, false>(mw, mxm, p, max_tiles, stream);
    default: return launch<128, false>(mw, mxm, p, max_tiles, stream);
  }
}

extern "C" int fb_mxfp4_prepare_sf(const void* scale, void* out, int groups, int rows, int k, void* stream) {
  if (!scale || !out || groups <= 0 || rows <= 0 || k <= 0 || k % 128 != 0) return FB_ERR_SHAPE;
  const int kblocks = k / 128, sf_tiles = (rows + kTileN - 1) / kTileN;
  mxfp4_prepare_sf_kernel<<<592, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(scale), static_cast<uint8_t*>(out), groups, rows, kblocks, sf_tiles);
  return cudaGetLastError() == cudaSuccess ? FB_OK : FB_ERR_LAUNCH;
}

extern "C" int fb_quant_mxfp8_rows(const void* x, long long ldx, void* q, long long ldq, void* scale, long long lds,
                                   int rows, int n, void* stream) {
  if (!x || !q || !scale || rows <= 0 || n <= 0 || n % 128 != 0 || (ldx % 4) != 0 || (ldq % 4) != 0) return FB_ERR_SHAPE;
  const long long warps = static_cast<long long>(rows) * (n / 128);
  launch_pdl(quant_mxfp8_rows_kernel, dim3(static_cast<unsigned>((warps * 32 + 255) / 256)), dim3(256), 0,
             static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(x), ldx, static_cast<uint8_t*>(q), ldq,
             static_cast<uint8_t*>(scale), lds, rows, n);
  return cudaGetLastError() == cudaSuccess ? FB_OK : FB_ERR_LAUNCH;
}
