// Weight-stationary ("swap-AB") grouped GEMM for sm_100a.
//
//   out[row, n] = sum_k X[row, k] * W[group(row), n, k]
//
// The weight tile is the UMMA A operand (M = 128 output channels), the activation
// rows are the B operand (UMMA N = NTOK rows, 16..256), so a decode step with a
// handful of rows per expert still fills the 128-lane datapath and streams every
// weight byte exactly once.  Accumulators live in TMEM (double buffered), operands
// arrive by TMA into 128-byte-swizzled shared memory, one thread issues
// tcgen05.mma, four warps drain TMEM and run the fused epilogue:
//
//   kEpiStore   : out[row, n]            = acc                      (bf16 or fp32)
//   kEpiSwiGLU  : out[row, n]            = silu(gate) * up          (two weight tiles per k-block)
//   kEpiScatter : out[dst_row[row], n]   = acc * row_scale[row]     (MoE down projection)
//   kEpiAllReduce: partial tiles are pushed into every rank's receive buffer over
//                 NVLink peer stores, then summed in rank order once all have landed
//                 (one-shot all-reduce fused behind the GEMM, tile by tile).
//
// Counterpart of the reference's row-dot linear and mma.sync projection kernels
// (crates/ferrule-backend/native/cuda/implementations/portable/entrypoints.cu:208-340,
//  .../cutlass/capabilities/fp8_projection.cuh:421-497, bf16_compressor.cuh:223-313) and of
// its CUTLASS grouped expert GEMM (.../architectures/sm103/grouped_fp4_moe.cuh:1115-1222).
#include <cuda.h>
#include <cstdlib>

#include "common.cuh"
#include "ferrule_b200.h"
#include "launch.cuh"

namespace fb {

constexpr int kTileN = 128;   // output channels per tile (UMMA M)
constexpr int kBlockK = 64;   // bf16 elements per k-block = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kGemmThreads = 192;

enum { kEpiStore = 0, kEpiSwiGLU = 1, kEpiScatter = 2, kEpiAllReduce = 3 };

struct GemmParams {
  int n_out;          // output channels per group
  int k;              // reduction length
  int n_tiles;        // ceil(n_out / 128)
  int dual_offset;    // row offset of the "up" block inside a group (SwiGLU mode)
  int dense_rows;     // rows of X when no tile table is given
  int max_tok_tiles;  // capacity of the tile table
  int batched;        // every group multiplies all dense rows (per-head projections)
  int x_group_koff;   // batched: column offset of group g inside an X row = g * x_group_koff
  int out_group_coff; // batched: column offset of group g inside an output row
  int groups;
  int stages;         // pipeline depth actually used (<= GemmCfg::kStages)
  int force_split;    // > 0: use exactly this split-K factor (tests)
  unsigned long long* trace;  // optional: CTA 0 writes globaltimer stamps of its pipeline milestones
  const int* tile_group;
  const int* tile_row0;
  const int* tile_rows;
  const int* num_tok_tiles;  // device scalar
  void* out;
  long long ldo;
  int out_fp32;
  const int* dst_row;
  const float* row_scale;
  float act_limit;  // SwiGLU clamp (0 = none)
  DeviceStatus* status;
  // fused all-reduce
  int rank;
  int world;
  int rows_cap;              // rows per source slot in the receive buffer
  float* peer_recv[8];       // receive buffer of every rank, in this rank's address space
  uint32_t* peer_flags[8];   // per-tile arrival counters of every rank
  uint32_t* local_ctr;       // [0] = calls completed, [1] = CTAs finished this call, [2..] = consumed arrivals per tile
  int ar_bf16;               // kEpiAllReduce: partials travel as bf16 pairs instead of fp32
  uint8_t* mc_recv;          // kEpiAllReduce: multicast address of the receive buffers (one store reaches every rank)
  int w_stream;              // weights are read once by this launch: load them with the L2 evict-first policy
  int stage_store;           // bf16 store / SwiGLU / scatter epilogues of large row tiles: rows leave through a
                             // shared-memory staging tile as 256-byte row segments instead of 2-byte column stores
  const int* remap_rank;     // kEpiScatter, expert-parallel combine: output row -> destination rank ...
  const int* remap_row;      // ... and row in that rank's combine buffer (peer_recv[rank], bf16, pitch ldo)
  const __nv_bfloat16* residual;  // optional, added after the reduction
  long long ldr;
  unsigned long long peer_wait_ns;
};

template <int NTOK, bool DUAL>
struct GemmCfg {
  static constexpr int kWBytes = kTileN * kBlockK * 2;
  static constexpr int kXBytes = NTOK * kBlockK * 2;
  static constexpr int kStageBytes = kWBytes * (DUAL ? 2 : 1) + kXBytes;
  static constexpr int kBudget = 200 * 1024;
  static constexpr int kStagesRaw = kBudget / kStageBytes;
  static constexpr int kStages = kStagesRaw > 10 ? 10 : kStagesRaw;
  static constexpr int kAccCols = NTOK * (DUAL ? 2 : 1);
  static constexpr int kTmemCols = (2 * kAccCols) < 32 ? 32 : (2 * kAccCols);
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
  static_assert(kTmemCols <= 512, "accumulators exceed TMEM");
  static_assert((kTmemCols & (kTmemCols - 1)) == 0, "TMEM columns must be a power of two");
  static_assert(kStages >= 2, "not enough shared memory for a pipeline");
};

struct TileInfo {
  int g, row0, rows, nt;
};

template <int NTOK>
__device__ __forceinline__ TileInfo decode_tile(const GemmParams& p, int t, int tiles_per_group) {
  TileInfo ti;
  const int m = t / p.n_tiles;
  ti.nt = t - m * p.n_tiles;
  if (p.tile_group) {
    ti.g = p.tile_group[m];
    ti.row0 = p.tile_row0[m];
    ti.rows = min(p.tile_rows[m], NTOK);
  } else if (p.batched) {
    ti.g = m / tiles_per_group;
    ti.row0 = (m - ti.g * tiles_per_group) * NTOK;
    ti.rows = min(NTOK, p.dense_rows - ti.row0);
  } else {
    ti.g = 0;
    ti.row0 = m * NTOK;
    ti.rows = min(NTOK, p.dense_rows - ti.row0);
  }
  return ti;
}

// grouped mode: a tile whose expert received no row (static one-tile-per-expert plans, streamed experts that are
// not resident) is skipped by the producer, the MMA issuer and the epilogue alike - no weights are read for it
__device__ __forceinline__ bool tile_empty(const GemmParams& p, int t) {
  return p.tile_group != nullptr && p.tile_rows[t / p.n_tiles] <= 0;
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }

template <int NTOK, bool DUAL, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_swapab_kernel(const __grid_constant__ CUtensorMap tmap_w,
                   const __grid_constant__ CUtensorMap tmap_x, const GemmParams p) {
  using Cfg = GemmCfg<NTOK, DUAL>;
  pdl_launch_dependents();
  const bool tracing = p.trace != nullptr && blockIdx.x == 0;
  if (tracing && threadIdx.x == 0) p.trace[0] = globaltimer_ns();   // kernel entry
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment is required by the 128-byte swizzle atoms.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int nstages = p.stages;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + nstages * Cfg::kStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + nstages;
  uint64_t* acc_full = bars + 2 * nstages;
  uint64_t* acc_empty = acc_full + 2;
  uint64_t* red_bar = acc_empty + 2;  // split-K: peers' partial tiles have landed in `red`
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(red_bar + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  // split-K reduction area (leader CTA only): [peer - 1][accumulator column][128 lanes] fp32
  float* red = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Split-K: the S CTAs of a cluster share one output tile, each reducing a slice of K; the
  // partial accumulators travel to the leader (cluster rank 0) through distributed shared memory.
  const int S = static_cast<int>(cluster_nctarank());
  const int crank = static_cast<int>(cluster_ctarank());
  // all-reduce epilogue: receive-slot geometry in bytes ([parity][source][rows_cap][n_out] tagged values, 8 bytes
  // each) and the [NTOK][128] fp32 staging tile behind the split-K area
  const size_t ar_slot_bytes = static_cast<size_t>(p.rows_cap) * p.n_out * 8;
  // store staging (two [16][128] bf16 chunks) shares the position of the all-reduce staging tile
  __nv_bfloat16* st_stage = reinterpret_cast<__nv_bfloat16*>(
      red + static_cast<size_t>(S > 1 ? S - 1 : 0) * Cfg::kAccCols * 128);
  uint32_t chunk_ctr = 0;
  float* ar_stage = red + static_cast<size_t>(S > 1 ? S - 1 : 0) * Cfg::kAccCols * 128;
  const int tile_first = blockIdx.x / S;
  const int tile_stride = gridDim.x / S;

  if (threadIdx.x == 0) {
    for (int s = 0; s < nstages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);
    }
    mbar_init(red_bar, 128 * (S > 1 ? S - 1 : 1));
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (S > 1) cluster_sync_all();  // the leader's barrier is initialised before any peer arrives on it
  if (tracing && threadIdx.x == 0) p.trace[1] = globaltimer_ns();   // prologue done (barriers, TMEM)
  const uint32_t tmem_base = *tmem_slot;

  // Everything above touched only this CTA's barriers and TMEM.  From here on global memory that
  // the preceding kernel may still be writing is read, so every thread waits for it - except the
  // producer thread of a dense GEMM, which first requests the (constant) weight tiles.
  const bool grouped_mode = p.tile_group != nullptr;
  const bool is_producer = warp == 0 && lane == 0;
  if (!is_producer || grouped_mode) pdl_wait();
  const int tiles_per_group = (p.dense_rows + NTOK - 1) / NTOK;
  const int num_tok_tiles = grouped_mode ? min(*p.num_tok_tiles, p.max_tok_tiles)
                                         : tiles_per_group * (p.batched ? p.groups : 1);
  const int total = num_tok_tiles * p.n_tiles;
  const int kblocks = (p.k + kBlockK - 1) / kBlockK;
  const int kb_begin = static_cast<int>(static_cast<long long>(crank) * kblocks / S);
  const int kb_end = static_cast<int>(static_cast<long long>(crank + 1) * kblocks / S);

  uint32_t call = 0;
  if (EPI == kEpiAllReduce && !is_producer) call = *reinterpret_cast<volatile uint32_t*>(p.local_ctr);
  const size_t ar_parity_off = static_cast<size_t>(call & 1u) * p.world * ar_slot_bytes;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      long long issued = 0;
      const uint64_t wpol = l2_policy_evict_first();
      const bool wstream = p.w_stream != 0;
      auto load_w = [&](void* dst, uint64_t* bar, int c0, int c1, int c2) {
        if (wstream) tma_load_3d_hint(dst, &tmap_w, bar, c0, c1, c2, wpol);
        else tma_load_3d(dst, &tmap_w, bar, c0, c1, c2);
      };
      // Weight tiles do not depend on the preceding kernel: request the first pipeline-full of
      // them before waiting for it, so they stream while that kernel drains.
      int pre = 0;
      if (!grouped_mode) {
        if (tile_first < total) {
          const TileInfo ti = decode_tile<NTOK>(p, tile_first, tiles_per_group);
          const int npre = min(nstages, kb_end - kb_begin);
          for (pre = 0; pre < npre; ++pre) {
            uint8_t* stage = smem + pre * Cfg::kStageBytes;
            const int kb = kb_begin + pre;
            mbar_arrive_expect_tx(&full_bar[pre], Cfg::kStageBytes);
            load_w(stage, &full_bar[pre], kb * kBlockK, ti.nt * kTileN, ti.g);
            if (DUAL) load_w(stage + Cfg::kWBytes, &full_bar[pre], kb * kBlockK, p.dual_offset + ti.nt * kTileN, ti.g);
          }
        }
        pdl_wait();
      }
      if (tracing) p.trace[2] = globaltimer_ns();                     // dependency wait passed
      for (int t = tile_first; t < total && ok; t += tile_stride) {
        if (tile_empty(p, t)) continue;
        const TileInfo ti = decode_tile<NTOK>(p, t, tiles_per_group);
        const int g = ti.g, nt = ti.nt, row0 = ti.row0;
        const int xk0 = p.batched ? g * p.x_group_koff : 0;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          uint8_t* stage = smem + s * Cfg::kStageBytes;
          if (t == tile_first && kb - kb_begin < pre) {
            // barrier armed and weights requested above; only the activation tile is missing
          } else {
            ok = mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag, p.status, 0x100);
            if (!ok) break;
            mbar_arrive_expect_tx(&full_bar[s], Cfg::kStageBytes);
            load_w(stage, &full_bar[s], kb * kBlockK, nt * kTileN, g);
            if (DUAL) load_w(stage + Cfg::kWBytes, &full_bar[s], kb * kBlockK, p.dual_offset + nt * kTileN, g);
          }
          tma_load_2d(stage + Cfg::kWBytes * (DUAL ? 2 : 1), &tmap_x, &full_bar[s],
                      xk0 + kb * kBlockK, row0);
          ++issued;
          if (++s == nstages) { s = 0; ph ^= 1u; }
        }
      }
      // Drain after an abort: copies this thread issued may still be in flight, and the
      // CTA may not exit under them.  Wait (bounded) for the full barrier of each of
      // the last `nstages` issues to complete the phase it was armed for.
      if (*abort_flag) {
        const long long first = issued > nstages ? issued - nstages : 0;
        for (long long i = first; i < issued; ++i) {
          const int si = static_cast<int>(i % nstages);
          const uint32_t pi = static_cast<uint32_t>((i / nstages) & 1);
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(&full_bar[si], pi) && globaltimer_ns() - t0 < 2000000ull) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(kTileN, NTOK, 1, 1);
      int s = 0;
      uint32_t ph = 0;
      int a = 0;
      uint32_t aph = 0;
      bool ok = true;
      for (int t = tile_first; t < total && ok; t += tile_stride) {
        if (tile_empty(p, t)) continue;
        ok = mbar_wait(&acc_empty[a], aph ^ 1u, abort_flag, p.status, 0x200);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d0 = tmem_base + a * Cfg::kAccCols;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          ok = mbar_wait(&full_bar[s], ph, abort_flag, p.status, 0x201);
          if (!ok) break;
          if (tracing && kb == kb_begin) p.trace[3] = globaltimer_ns();  // first stage landed
          tc_fence_after();
          const uint32_t sw = smem_u32(smem + s * Cfg::kStageBytes);
          const uint32_t sx = sw + Cfg::kWBytes * (DUAL ? 2 : 1);
#pragma unroll
          for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
            const uint32_t koff = kk * kUmmaK * 2;
            const uint64_t db = umma_desc_k128(sx + koff);
            const uint32_t acc = (kb > kb_begin || kk) ? 1u : 0u;
            umma_bf16(d0, umma_desc_k128(sw + koff), db, idesc, acc);
            if (DUAL) umma_bf16(d0 + NTOK, umma_desc_k128(sw + Cfg::kWBytes + koff), db, idesc, acc);
          }
          umma_commit(&empty_bar[s]);
          if (++s == nstages) { s = 0; ph ^= 1u; }
        }
        if (ok) umma_commit(&acc_full[a]);
        if (tracing) p.trace[4] = globaltimer_ns();                   // last MMA issued
        a ^= 1;
        if (a == 0) aph ^= 1u;
      }
    }
  } else {
    // ------------------------------ epilogue (4 warps) -------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int ch_in_tile = q * 32 + lane;
    const int epi_tid = (warp - 2) * 32 + lane;
    const bool leader = crank == 0;
    int a = 0;
    uint32_t aph = 0;
    bool ok = true;
    for (int t = tile_first; t < total && ok; t += tile_stride) {
      if (tile_empty(p, t)) continue;
      const TileInfo ti = decode_tile<NTOK>(p, t, tiles_per_group);
      const int row0 = ti.row0, rows = ti.rows;
      const int n = ti.nt * kTileN + ch_in_tile;
      const bool n_ok = n < p.n_out;
      const long long ocol = (p.batched ? static_cast<long long>(ti.g) * p.out_group_coff : 0) + n;
      ok = mbar_wait(&acc_full[a], aph, abort_flag, p.status, 0x300);
      if (!ok) break;
      if (tracing && epi_tid == 0) p.trace[5] = globaltimer_ns();     // accumulator complete
      tc_fence_after();
      const uint32_t tbase = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + a * Cfg::kAccCols;
      if (S > 1 && !leader) {
        // ---- split-K peer: ship the partial accumulator to the leader's shared memory ----
        const uint32_t red_remote =
            mapa_shared(smem_u32(red), 0) +
            (static_cast<uint32_t>((crank - 1) * Cfg::kAccCols) * 128u + static_cast<uint32_t>(ch_in_tile)) * 4u;
#pragma unroll 1
        for (int c0 = 0; c0 < NTOK; c0 += 16) {
          if (c0 >= rows) break;
          uint32_t v[16];
          tmem_ld16(tbase + c0, v);
          uint32_t u[16];
          if (DUAL) tmem_ld16(tbase + NTOK + c0, u);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            st_cluster_f32(red_remote + static_cast<uint32_t>(c0 + j) * 512u, __uint_as_float(v[j]));
            if (DUAL)
              st_cluster_f32(red_remote + static_cast<uint32_t>(NTOK + c0 + j) * 512u, __uint_as_float(u[j]));
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[a]);
        mbar_arrive_remote(mapa_shared(smem_u32(red_bar), 0));
        a ^= 1;
        if (a == 0) aph ^= 1u;
        continue;
      }
      if (S > 1) {
        ok = mbar_wait_cluster(red_bar, 0, abort_flag, p.status, 0x301);
        if (!ok) break;
      }
#pragma unroll 1
      for (int c0 = 0; c0 < NTOK; c0 += 16) {
        if (c0 >= rows) break;  // uniform across the CTA: nothing valid beyond `rows`
        uint32_t v[16];
        tmem_ld16(tbase + c0, v);
        uint32_t u[16];
        if (DUAL) tmem_ld16(tbase + NTOK + c0, u);
        tmem_ld_wait();
        if (S > 1) {
          // fixed summation order: own slice, then peers by cluster rank
          for (int pr = 1; pr < S; ++pr) {
            const float* rp = red + (static_cast<size_t>(pr - 1) * Cfg::kAccCols) * 128 + ch_in_tile;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              v[j] = __float_as_uint(__uint_as_float(v[j]) + rp[static_cast<size_t>(c0 + j) * 128]);
              if (DUAL)
                u[j] = __float_as_uint(__uint_as_float(u[j]) + rp[static_cast<size_t>(NTOK + c0 + j) * 128]);
            }
          }
        }
        if (EPI != kEpiAllReduce && p.stage_store) {
          // Swap-AB leaves a thread with one output channel of 16 rows: written directly that is sixteen 2-byte
          // stores per thread, 64 bytes per warp.  Stage the 16 x 128 chunk in shared memory (two buffers, chunk
          // parity) and let 8 threads write each row's 256 bytes.
          __nv_bfloat16* sb = st_stage + (chunk_ctr & 1) * (16 * 128);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int r = c0 + j;
            float x = 0.f;
            if (r < rows) {
              x = __uint_as_float(v[j]);
              if (EPI == kEpiSwiGLU) {
                float up = __uint_as_float(u[j]);
                if (p.act_limit > 0.f) {
                  x = fminf(x, p.act_limit);
                  up = fminf(fmaxf(up, -p.act_limit), p.act_limit);
                }
                x = silu_f(x) * up;
              }
              if (EPI == kEpiScatter && p.row_scale) x *= p.row_scale[row0 + r];
            }
            sb[j * 128 + ch_in_tile] = __float2bfloat16_rn(x);
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          {
            const int j = epi_tid >> 3, seg = epi_tid & 7;
            const int r = c0 + j;
            if (r < rows) {
              long long orow = row0 + r;
              if (EPI == kEpiScatter && p.dst_row) orow = p.dst_row[row0 + r];
              const int col0 = ti.nt * kTileN + seg * 16;
              if (orow >= 0 && col0 < p.n_out) {
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + orow * p.ldo +
                                     (p.batched ? static_cast<long long>(ti.g) * p.out_group_coff : 0) + col0;
                const uint4* src = reinterpret_cast<const uint4*>(sb + j * 128 + seg * 16);
                reinterpret_cast<uint4*>(dst)[0] = src[0];
                if (col0 + 8 < p.n_out) reinterpret_cast<uint4*>(dst)[1] = src[1];
              }
            }
          }
          ++chunk_ctr;
          continue;
        }
        if (n_ok) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int r = c0 + j;
            if (r < rows) {
              float x = __uint_as_float(v[j]);
              if (EPI == kEpiSwiGLU) {
                float up = __uint_as_float(u[j]);
                if (p.act_limit > 0.f) {
                  x = fminf(x, p.act_limit);
                  up = fminf(fmaxf(up, -p.act_limit), p.act_limit);
                }
                x = silu_f(x) * up;
              }
              long long orow = row0 + r;
              if (EPI == kEpiScatter) {
                if (p.row_scale) x *= p.row_scale[row0 + r];
                orow = p.dst_row ? p.dst_row[row0 + r] : orow;
              }
              if (EPI == kEpiScatter && p.remap_rank != nullptr) {
                // expert-parallel combine: the weighted expert output goes straight into the combine
                // buffer of the rank that owns the token (plain peer stores over NVLink)
                if (orow >= 0) {
                  __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.peer_recv[p.remap_rank[orow]]);
                  dst[static_cast<long long>(p.remap_row[orow]) * p.ldo + ocol] = __float2bfloat16_rn(x);
                }
              } else if (EPI == kEpiAllReduce) {
                ar_stage[r * 128 + ch_in_tile] = x;     // staged row-major, pushed below in 512-byte rows
              } else if (orow >= 0) {
                if (p.out_fp32)
                  reinterpret_cast<float*>(p.out)[orow * p.ldo + ocol] = x;
                else
                  reinterpret_cast<__nv_bfloat16*>(p.out)[orow * p.ldo + ocol] = __float2bfloat16_rn(x);
              }
            }
          }
        }
      }
      // TMEM buffer is free once every warp's loads have completed.
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[a]);
      if (EPI == kEpiAllReduce) {
        // Publish this tile.  The partial sits row-major in shared memory; each epilogue warp pushes whole
        // rows into every rank's receive slot as tagged pairs (value, call tag): 4 channels per lane = two
        // 16-byte stores, 1 KB contiguous per warp, row and peer.  No fence and no flag: receivers poll the tags.
        asm volatile("bar.sync 1, 128;" ::: "memory");
        {
          const int n4 = ti.nt * kTileN + lane * 4;
          const uint32_t tag = call + 1u;
          if (n4 < p.n_out) {
            for (int r = warp - 2; r < rows; r += 4) {
              const float4 val = *reinterpret_cast<const float4*>(ar_stage + r * 128 + lane * 4);
              const float vals[4] = {val.x, val.y, val.z, val.w};
              const size_t ch = static_cast<size_t>(row0 + r) * p.n_out + n4;
              if (p.mc_recv != nullptr) {
                ll_push4_mc(p.mc_recv + ar_parity_off + p.rank * ar_slot_bytes, ch, vals, tag, p.ar_bf16 != 0);
              } else {
                for (int pr = 0; pr < p.world; ++pr)
                  ll_push4(reinterpret_cast<uint8_t*>(p.peer_recv[pr]) + ar_parity_off + p.rank * ar_slot_bytes, ch,
                           vals, tag, p.ar_bf16 != 0);
              }
            }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");    // the staging tile may be overwritten by the next tile
        if (tracing && epi_tid == 0) p.trace[7] = globaltimer_ns();   // partial tile pushed
      }
      a ^= 1;
      if (a == 0) aph ^= 1u;
    }
    if (EPI == kEpiAllReduce) {
      // Second pass, spread over the whole grid (CTAs without a tile of their own help too): a unit is one
      // output row of one tile (128 channels, 4 per lane).  A warp polls the tagged words of its unit from all
      // ranks' slots (arrival = tag of this call), sums in rank order (identical on every rank), adds the
      // residual and writes the row.  With more warps than units every warp pays one L2 round trip.
      const uint32_t tag = call + 1u;
      const int units = p.n_tiles * p.dense_rows;
      const int gwarp = blockIdx.x * 4 + (warp - 2), gwarps = gridDim.x * 4;
      bool waited = false;
      const uint64_t w0 = globaltimer_ns();
      for (int u = gwarp; u < units && ok; u += gwarps) {
        const int nt = u % p.n_tiles;
        const long long orow = u / p.n_tiles;
        const int n4 = nt * kTileN + lane * 4;
        if (n4 >= p.n_out) continue;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        int bad_src = 0;
        if (!ll_gather4(reinterpret_cast<const uint8_t*>(p.peer_recv[p.rank]) + ar_parity_off,
                        static_cast<size_t>(orow) * p.n_out + n4, ar_slot_bytes, p.world, tag, p.peer_wait_ns, acc,
                        bad_src, p.ar_bf16 != 0)) {
          report_status(p.status, kStatusPeerTimeout, 0x400 + bad_src, static_cast<uint32_t>(u), tag);
          ok = false;
          break;
        }
        waited = true;
        if (p.residual) {
          const uint2 rv = *reinterpret_cast<const uint2*>(p.residual + orow * p.ldr + n4);
          const __nv_bfloat16* rb = reinterpret_cast<const __nv_bfloat16*>(&rv);
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[j] += __bfloat162float(rb[j]);
        }
        if (p.out_fp32) {
          *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + orow * p.ldo + n4) =
              make_float4(acc[0], acc[1], acc[2], acc[3]);
        } else {
          __nv_bfloat16 ob[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) ob[j] = __float2bfloat16_rn(acc[j]);
          *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + orow * p.ldo + n4) =
              *reinterpret_cast<const uint2*>(ob);
        }
      }
      if (waited && epi_tid == 0 && p.status != nullptr) {
        atomicAdd(reinterpret_cast<unsigned long long*>(p.status) + 2, globaltimer_ns() - w0);
        atomicAdd(reinterpret_cast<unsigned int*>(p.status) + 6, 1u);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (tracing && threadIdx.x == 0) p.trace[6] = globaltimer_ns();   // epilogue done
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if (EPI == kEpiAllReduce && threadIdx.x == 0) {
    __threadfence();
    const uint32_t done = atomicAdd(p.local_ctr + 1, 1u);
    if (done == gridDim.x - 1) {
      p.local_ctr[1] = 0;
      __threadfence();
      // every CTA of this launch has read the call number already; this thread (the TMA producer) never did
      p.local_ctr[0] = *reinterpret_cast<volatile uint32_t*>(p.local_ctr) + 1u;
    }
  }
  if (EPI == kEpiScatter && p.remap_rank != nullptr) {
    // Each thread fences its own peer stores at system scope, the CTA counts itself in, and the last CTA
    // bumps every rank's flag: this rank's share of the combine is complete.
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t done = atomicAdd(p.local_ctr + 1, 1u);
      if (done == gridDim.x * gridDim.y * gridDim.z - 1) {
        p.local_ctr[1] = 0;
        __threadfence_system();
        for (int pr = 0; pr < p.world; ++pr) flag_add_release_sys(p.peer_flags[pr] + p.rank, 1u);
      }
    }
  }
}

// ---------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// rank-3 bf16 map: dims (k, rows, groups), box (64, box_rows, 1), 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, uint64_t k, uint64_t rows, uint64_t groups,
                    uint64_t row_stride_bytes, uint64_t group_stride_bytes, uint32_t box_rows,
                    int rank) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return FB_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_stride_bytes & 15) ||
      (group_stride_bytes & 15))
    return FB_ERR_ALIGN;
  cuuint64_t dims[3] = {k, rows, groups};
  cuuint64_t strides[2] = {row_stride_bytes, group_stride_bytes};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(kBlockK), box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), dims,
                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FB_OK : FB_ERR_DRIVER;
}

static int g_num_sms = 0;
static int num_sms() {
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

constexpr int kSmemLimit = 227 * 1024;

static bool small_smem_enabled() {
  static const bool on = [] {
    const char* e = getenv("FERRULE_GEMM_SMALL_SMEM");
    return !(e && e[0] == '0');
  }();
  return on;
}
static bool stage_small_enabled() {
  static const bool on = [] {
    const char* e = getenv("FERRULE_GEMM_STAGE_SMALL");
    return !(e && e[0] == '0');
  }();
  return on;
}

// Split-K factor: spread a GEMM with few output tiles over more SMs.  The S CTAs of a cluster
// each take 1/S of the k-blocks of one tile; only used when every tile gets its own cluster.
static int pick_split(int tiles, int kblocks, bool grouped, int acc_cols, int stage_bytes, int extra_bytes) {
  if (grouped) return 1;
  int best = 1;
  for (int s = 2; s <= 4; s *= 2) {  // measured: 8-way costs more in the DSMEM reduction than it saves
    if (tiles * s > num_sms()) break;
    if (kblocks / s < 4) break;
    const int red = (s - 1) * acc_cols * 128 * 4;
    if (kSmemLimit - 2048 - red - extra_bytes < 2 * stage_bytes) break;
    best = s;
  }
  return best;
}

template <int NTOK, bool DUAL, int EPI>
static int launch_cfg(const CUtensorMap& mw, const CUtensorMap& mx, GemmParams p, int max_tiles,
                      bool grouped, cudaStream_t stream) {
  using Cfg = GemmCfg<NTOK, DUAL>;
  auto kern = gemm_swapab_kernel<NTOK, DUAL, EPI>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) !=
        cudaSuccess)
      return FB_ERR_LAUNCH;
    attr_set = true;
  }
  const int kblocks = (p.k + kBlockK - 1) / kBlockK;
  // large row tiles (prefill) write their bf16 output through a staging tile: see the epilogue
  p.stage_store = (EPI != kEpiAllReduce && (NTOK >= 64 || stage_small_enabled()) && !p.out_fp32 && p.remap_rank == nullptr &&
                   p.n_out % 8 == 0 && p.ldo % 8 == 0 && p.out_group_coff % 8 == 0 &&
                   (reinterpret_cast<uintptr_t>(p.out) & 15) == 0) ? 1 : 0;
  // staging areas behind the split-K reduction area: the all-reduce epilogue's [NTOK x 128] fp32 tile, or the
  // two [16 x 128] bf16 chunks of the staged store
  const int extra_bytes = (EPI == kEpiAllReduce ? NTOK * 128 * 4 : 0) + (p.stage_store ? 2 * 16 * 128 * 2 : 0);
  const int split = p.force_split > 0 ? p.force_split
                                      : pick_split(max_tiles, kblocks, grouped, Cfg::kAccCols, Cfg::kStageBytes,
                                                   extra_bytes);
  const int red_bytes = (split > 1 ? (split - 1) * Cfg::kAccCols * 128 * 4 : 0) + extra_bytes;
  int stages = (kSmemLimit - 2048 - red_bytes) / Cfg::kStageBytes;
  if (stages > Cfg::kStages) stages = Cfg::kStages;
  // A dense GEMM whose CTAs each own one tile needs no more stages than its k-blocks: the smaller footprint lets
  // its CTAs become resident beside the preceding kernel's, so that their prologue and weight requests overlap
  // that kernel's tail instead of waiting for its shared memory.
  if (!grouped && max_tiles * split <= num_sms() && small_smem_enabled()) {
    const int kb_per_cta = (kblocks + split - 1) / split;
    if (stages > kb_per_cta) stages = kb_per_cta < 2 ? 2 : kb_per_cta;
  }
  if (stages < 2 || (split > 1 && (max_tiles * split > num_sms() || kblocks < split))) return FB_ERR_SHAPE;
  p.stages = stages;
  const size_t smem = static_cast<size_t>(stages) * Cfg::kStageBytes + 1024 + 256 + red_bytes;
  int clusters = max_tiles < num_sms() ? max_tiles : num_sms();
  if (clusters < 1) clusters = 1;
  // the all-reduce epilogue's second pass runs on every CTA of the grid: fill the GPU even with few tiles
  if (EPI == kEpiAllReduce) clusters = num_sms() / split;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(clusters * split, 1, 1);
  cfg.blockDim = dim3(kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = split;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  if (cudaLaunchKernelEx(&cfg, kern, mw, mx, p) != cudaSuccess) return FB_ERR_LAUNCH;
  return cudaGetLastError() == cudaSuccess ? FB_OK : FB_ERR_LAUNCH;
}

template <bool DUAL, int EPI>
static int launch_ntok(int ntok, const CUtensorMap& mw, const CUtensorMap& mx, const GemmParams& p,
                       int max_tiles, bool grouped, cudaStream_t stream) {
  switch (ntok) {
    case 16: return launch_cfg<16, DUAL, EPI>(mw, mx, p, max_tiles, grouped, stream);
    case 32: return launch_cfg<32, DUAL, EPI>(mw, mx, p, max_tiles, grouped, stream);
    case 64: return launch_cfg<64, DUAL, EPI>(mw, mx, p, max_tiles, grouped, stream);
    case 128: return launch_cfg<128, DUAL, EPI>(mw, mx, p, max_tiles, grouped, stream);
    case 256:
      if constexpr (!DUAL) return launch_cfg<256, DUAL, EPI>(mw, mx, p, max_tiles, grouped, stream);
      return FB_ERR_SHAPE;
    default: return FB_ERR_SHAPE;
  }
}

}  // namespace fb

using namespace fb;

extern "C" int fb_gemm_bf16(const FbGemmArgs* a, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a == nullptr || a->w == nullptr || a->x == nullptr || a->out == nullptr) return FB_ERR_SHAPE;
  if (a->n_out <= 0 || a->k <= 0 || a->groups <= 0 || (a->k % 8) != 0) return FB_ERR_SHAPE;
  if (a->epilogue < 0 || a->epilogue > 3) return FB_ERR_SHAPE;
  const bool dual = a->epilogue == kEpiSwiGLU;
  const int ntok = a->ntok;
  if (ntok != 16 && ntok != 32 && ntok != 64 && ntok != 128 && ntok != 256) return FB_ERR_SHAPE;
  if (dual && ntok > 128) return FB_ERR_SHAPE;
  const bool grouped = a->tile_group != nullptr;
  if (grouped && (!a->tile_row0 || !a->tile_rows || !a->num_tok_tiles || a->max_tok_tiles <= 0))
    return FB_ERR_SHAPE;
  const bool batched = !grouped && a->groups > 1;
  if (batched && (a->epilogue != kEpiStore || a->x_group_koff % 8 != 0)) return FB_ERR_SHAPE;
  if (a->x_rows <= 0) return FB_ERR_SHAPE;

  CUtensorMap mw, mx;
  const uint64_t w_rows = static_cast<uint64_t>(a->w_rows_per_group);
  int rc = make_map(&mw, a->w, a->k, w_rows, a->groups, static_cast<uint64_t>(a->ldw) * 2,
                    static_cast<uint64_t>(a->w_group_stride) * 2, kTileN, 3);
  if (rc != FB_OK) return rc;
  const uint64_t x_cols = batched ? static_cast<uint64_t>(a->x_group_koff) * (a->groups - 1) + a->k : a->k;
  rc = make_map(&mx, a->x, x_cols, a->x_rows, 1, static_cast<uint64_t>(a->ldx) * 2, 0, ntok, 2);
  if (rc != FB_OK) return rc;

  GemmParams p{};
  p.n_out = a->n_out;
  p.k = a->k;
  p.n_tiles = (a->n_out + kTileN - 1) / kTileN;
  p.dual_offset = a->dual_offset;
  p.dense_rows = a->x_rows;
  p.batched = batched ? 1 : 0;
  p.x_group_koff = a->x_group_koff;
  p.out_group_coff = a->out_group_coff;
  p.groups = a->groups;
  p.force_split = a->force_split;
  p.trace = static_cast<unsigned long long*>(a->trace);
  {
    // decode-sized launches read every weight byte once; larger ones re-read weight tiles across row tiles
    static const bool enabled = [] {
      const char* e = getenv("FERRULE_W_EVICT_FIRST");
      return !(e && e[0] == '0');
    }();
    p.w_stream = enabled && (a->tile_group ? ntok <= 64 : a->x_rows <= 256);
  }
  p.max_tok_tiles = a->max_tok_tiles;
  p.tile_group = a->tile_group;
  p.tile_row0 = a->tile_row0;
  p.tile_rows = a->tile_rows;
  p.num_tok_tiles = a->num_tok_tiles;
  p.out = a->out;
  p.ldo = a->ldo;
  p.out_fp32 = a->out_fp32;
  p.dst_row = a->dst_row;
  p.row_scale = a->row_scale;
  p.act_limit = a->act_limit;
  p.status = static_cast<DeviceStatus*>(a->status);
  const int tok_tiles = grouped ? a->max_tok_tiles
                                : ((a->x_rows + ntok - 1) / ntok) * (batched ? a->groups : 1);
  const int max_tiles = tok_tiles * p.n_tiles;

  if (a->epilogue == kEpiAllReduce) {
    if (grouped || a->world < 1 || a->world > 8 || a->rank < 0 || a->rank >= a->world ||
        a->x_rows > a->rows_cap || a->local_ctr == nullptr || a->n_out % 4 != 0)
      return FB_ERR_SHAPE;
    if (max_tiles > a->flag_capacity) return FB_ERR_SHAPE;
    // Every tile's owner CTA waits for its peers' copy of the same tile: all of them
    // must be resident at once on every rank, so the grid may not exceed one wave.
    p.rank = a->rank;
    p.world = a->world;
    p.rows_cap = a->rows_cap;
    for (int i = 0; i < a->world; ++i) {
      if (!a->peer_recv[i] || !a->peer_flags[i]) return FB_ERR_SHAPE;
      p.peer_recv[i] = static_cast<float*>(a->peer_recv[i]);
      p.peer_flags[i] = static_cast<uint32_t*>(a->peer_flags[i]);
    }
    p.local_ctr = static_cast<uint32_t*>(a->local_ctr);
    p.residual = static_cast<const __nv_bfloat16*>(a->residual);
    p.ldr = a->ldr;
    p.ar_bf16 = a->ar_payload_bf16;
    p.mc_recv = static_cast<uint8_t*>(a->mc_recv);
    p.peer_wait_ns = a->peer_wait_ns ? a->peer_wait_ns : 3000000000ull;
    return launch_ntok<false, kEpiAllReduce>(ntok, mw, mx, p, max_tiles, grouped, stream);
  }
  if (dual) return launch_ntok<true, kEpiSwiGLU>(ntok, mw, mx, p, max_tiles, grouped, stream);
  if (a->epilogue == kEpiScatter) {
    if (a->remap_rank != nullptr) {
      if (!a->remap_row || !a->local_ctr || a->world < 1 || a->world > 8 || a->rank < 0 || a->rank >= a->world ||
          a->out_fp32)
        return FB_ERR_SHAPE;
      p.rank = a->rank;
      p.world = a->world;
      p.remap_rank = a->remap_rank;
      p.remap_row = a->remap_row;
      p.local_ctr = static_cast<uint32_t*>(a->local_ctr);
      for (int i = 0; i < a->world; ++i) {
        if (!a->peer_recv[i] || !a->peer_flags[i]) return FB_ERR_SHAPE;
        p.peer_recv[i] = static_cast<float*>(a->peer_recv[i]);
        p.peer_flags[i] = static_cast<uint32_t*>(a->peer_flags[i]);
      }
    }
    return launch_ntok<false, kEpiScatter>(ntok, mw, mx, p, max_tiles, grouped, stream);
  }
  return launch_ntok<false, kEpiStore>(ntok, mw, mx, p, max_tiles, grouped, stream);
}
