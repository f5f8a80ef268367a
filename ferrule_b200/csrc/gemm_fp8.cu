// Block-scaled FP8 (e4m3) weight-stationary GEMM for sm_100a, dense or grouped.
//
//   out[row, n] = sum_kb  sx[row, kb] * sw[g, n/128, kb] * sum_{k in block kb} X[row, k] * W[g, n, k]
//
// Weights: e4m3 [groups, N, K] with one UE8M0 scale per 128 x 128 block; activations: e4m3
// [rows, K] with one UE8M0 scale per 1 x 128 block (fb_quant_fp8_rows).  Same orientation as the
// bf16 kernel (weight tile = UMMA A operand, M = 128; rows = UMMA N), operands by TMA into
// 128-byte-swizzled shared memory (one k-block = 128 fp8 = one swizzle row), `tcgen05.mma
// kind::f8f6f4` (K = 32 per instruction).  Every 128-wide k-block is accumulated on its own into one
// of four TMEM buffers; the epilogue warps drain a buffer while the next k-blocks are multiplied,
// apply the two block scales in fp32 and keep the running sum in registers - the exact scaling
// order of the reference (scale per block, single fp32 accumulation, one rounding at the end).
// Epilogues: store, SwiGLU (gate / up weight tiles), weighted scatter.
//
// `scale_group32`: the weight scales are per row and per 32 elements (MXFP4: e2m1 values, which e4m3
// represents exactly, expanded to one byte each at load time).  Each K = 32 instruction of a k-block then
// writes its own accumulator and the epilogue applies the lane's own group scale.
//
// Counterpart of the reference's FP8 projection kernels
// (crates/ferrule-backend/native/cuda/implementations/cutlass/capabilities/fp8_projection.cuh:421-497,
// shared_ffn.cuh:477-594) and of the FP8 kinds of its row-dot linear (portable/entrypoints.cu:208-284).
#include <cuda.h>
#include <cstdlib>

#include "codec.cuh"
#include "common.cuh"
#include "ferrule_b200.h"
#include "launch.cuh"

namespace fb {
namespace fp8 {

constexpr int kTileN = 128;
constexpr int kBlockK = 128;   // fp8 elements per k-block = 128 bytes = one swizzle row = one scale block
constexpr int kUmmaK = 32;
constexpr int kThreads = 192;
constexpr int kAccBufs = 4;

struct Params {
  int n_out, k, n_tiles, dual_offset, dense_rows, max_tok_tiles, stages;
  int xs_bytes;                // bytes of the activation-scale tile in shared memory (the split-K area follows it)
  const int* tile_group;
  const int* tile_row0;
  const int* tile_rows;
  const int* num_tok_tiles;
  const uint8_t* w_scale;      // [groups, w_scale_rows, k_blocks]
  int w_scale_rows;            // scale rows per group = ceil(weight rows per group / 128)
  int w_rows_total;            // weight rows per group (G32: scales are [groups, rows, k/32])
  const uint8_t* x_scale;      // [rows, ldxs]
  long long ldxs;
  void* out;
  long long ldo;
  int out_fp32;
  int epilogue;                // 0 store, 1 swiglu, 2 scatter
  const int* dst_row;
  const float* row_scale;
  float act_limit;
  DeviceStatus* status;
  int w_stream;              // weights are read once by this launch: L2 evict-first loads
  // static row slots (decode-sized MoE batches): group g owns rows [g * slot_rows, (g + 1) * slot_rows) and
  // slot_cnt[g] of them are filled; the tile table is implied (slot_rows / NTOK tiles per group)
  const int* slot_cnt;
  int slot_rows;
  // quantised output: `out` receives e4m3 codes, out_scale[row * ldos + n / 128] the UE8M0 scale of each
  // 1 x 128 block (what quant_fp8_rows would make of the bf16 output)
  uint8_t* out_scale;
  long long ldos;
  int red_bytes;             // bytes of the split-K area (the amax exchange area follows it)
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

__device__ __forceinline__ float e8m0(uint8_t b) {
  return b == 0 ? __uint_as_float(1u << 22) : __uint_as_float(static_cast<uint32_t>(b) << 23);
}
__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }

template <int NTOK, bool DUAL, bool G32>
struct Cfg {
  static constexpr int kWBytes = kTileN * kBlockK;
  static constexpr int kXBytes = NTOK * kBlockK;
  static constexpr int kStageBytes = kWBytes * (DUAL ? 2 : 1) + kXBytes;
  // G32 (weights scaled per row and per 32 elements, i.e. MXFP4 values held in e4m3 containers): each of the
  // four K = 32 instructions of a k-block gets its own accumulator so the epilogue can scale them apart.
  static constexpr int kSub = G32 ? 4 : 1;
  static constexpr int kRing = G32 ? 2 : kAccBufs;             // k-blocks in flight between MMA and epilogue
  static constexpr int kSubCols = NTOK * (DUAL ? 2 : 1);
  static constexpr int kAccCols = kSubCols * kSub;             // TMEM columns per ring slot
  static constexpr int kTmemCols = kRing * kAccCols < 32 ? 32 : kRing * kAccCols;
  static_assert(kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "TMEM budget");
};

template <int NTOK, bool DUAL, bool G32>
__global__ void __launch_bounds__(kThreads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                const Params p) {
  using C = Cfg<NTOK, DUAL, G32>;
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw8[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw8) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int nstages = p.stages;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + nstages * C::kStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + nstages;
  uint64_t* acc_full = bars + 2 * nstages;
  uint64_t* acc_empty = acc_full + kAccBufs;   // kRing <= kAccBufs slots are used
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + kAccBufs);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  uint8_t* xs_tile = reinterpret_cast<uint8_t*>(bars) + 256;      // [NTOK][k_blocks] activation scales of the tile
  // split-K over a cluster: the S CTAs of a cluster take consecutive slices of the k-blocks of one tile; the
  // peers' scaled fp32 partials travel to the leader (cluster rank 0) through distributed shared memory.
  const int S = static_cast<int>(cluster_nctarank());
  const int crank = static_cast<int>(cluster_ctarank());
  uint64_t* red_bar = reinterpret_cast<uint64_t*>(tmem_slot + 4);
  float* red = reinterpret_cast<float*>(xs_tile + p.xs_bytes);   // leader: [peer - 1][acc column][128 lanes]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < nstages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < kAccBufs; ++a) {
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
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (S > 1) cluster_sync_all();     // the leader's barrier is initialised before any peer arrives on it
  pdl_wait();

  const bool grouped = p.tile_group != nullptr || p.slot_rows > 0;
  const int num_tok_tiles = p.slot_rows > 0 ? p.max_tok_tiles
                            : grouped ? min(*p.num_tok_tiles, p.max_tok_tiles) : (p.dense_rows + NTOK - 1) / NTOK;
  const int total = num_tok_tiles * p.n_tiles;
  const int kblocks = (p.k + kBlockK - 1) / kBlockK;
  const int tile_first = blockIdx.x / S, tile_stride = gridDim.x / S;
  const int kb_begin = static_cast<int>(static_cast<long long>(crank) * kblocks / S);
  const int kb_end = static_cast<int>(static_cast<long long>(crank + 1) * kblocks / S);

  if (warp == 0) {
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      long long issued = 0;
      const uint64_t wpol = l2_policy_evict_first();
      for (int t = tile_first; t < total && ok; t += tile_stride) {
        const int m = t / p.n_tiles, nt = t - m * p.n_tiles;
        int g, row0, rows_t;
        tile_of<NTOK>(p, m, g, row0, rows_t);
        if (rows_t <= 0) continue;          // an expert without rows: its weights are not streamed
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          ok = mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag, p.status, 0x800);
          if (!ok) break;
          uint8_t* stage = smem + s * C::kStageBytes;
          mbar_arrive_expect_tx(&full_bar[s], C::kStageBytes);
          if (p.w_stream) {
            tma_load_3d_hint(stage, &tmap_w, &full_bar[s], kb * kBlockK, nt * kTileN, g, wpol);
            if (DUAL)
              tma_load_3d_hint(stage + C::kWBytes, &tmap_w, &full_bar[s], kb * kBlockK, p.dual_offset + nt * kTileN, g, wpol);
          } else {
            tma_load_3d(stage, &tmap_w, &full_bar[s], kb * kBlockK, nt * kTileN, g);
            if (DUAL) tma_load_3d(stage + C::kWBytes, &tmap_w, &full_bar[s], kb * kBlockK, p.dual_offset + nt * kTileN, g);
          }
          tma_load_2d(stage + C::kWBytes * (DUAL ? 2 : 1), &tmap_x, &full_bar[s], kb * kBlockK, row0);
          ++issued;
          if (++s == nstages) { s = 0; ph ^= 1u; }
        }
      }
      if (*abort_flag) {
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
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(kTileN, NTOK, 0, 0);   // e4m3 x e4m3 -> f32
      int s = 0;
      uint32_t ph = 0;
      long long kbg = 0;    // k-blocks issued by this CTA: selects the TMEM buffer and its phase
      bool ok = true;
      for (int t = tile_first; t < total && ok; t += tile_stride) {
        {
          int g, row0, rows_t;
          tile_of<NTOK>(p, t / p.n_tiles, g, row0, rows_t);
          if (rows_t <= 0) continue;
        }
        for (int kb = kb_begin; kb < kb_end; ++kb, ++kbg) {
          const int a = static_cast<int>(kbg % C::kRing);
          const uint32_t aph = static_cast<uint32_t>((kbg / C::kRing) & 1);
          ok = mbar_wait(&acc_empty[a], aph ^ 1u, abort_flag, p.status, 0x810);
          if (!ok) break;
          ok = mbar_wait(&full_bar[s], ph, abort_flag, p.status, 0x811);
          if (!ok) break;
          tc_fence_after();
          const uint32_t d0 = tmem_base + a * C::kAccCols;
          const uint32_t sw = smem_u32(smem + s * C::kStageBytes);
          const uint32_t sx = sw + C::kWBytes * (DUAL ? 2 : 1);
#pragma unroll
          for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
            const uint32_t koff = kk * kUmmaK;     // bytes (1 byte per element)
            const uint64_t db = umma_desc_k128(sx + koff);
            const uint32_t dk = d0 + (G32 ? kk * C::kSubCols : 0);
            const uint32_t accf = (G32 || kk == 0) ? 0u : 1u;
            umma_f8(dk, umma_desc_k128(sw + koff), db, idesc, accf);
            if (DUAL) umma_f8(dk + NTOK, umma_desc_k128(sw + C::kWBytes + koff), db, idesc, accf);
          }
          umma_commit(&empty_bar[s]);
          umma_commit(&acc_full[a]);
          if (++s == nstages) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else {
    const int q = warp & 3;
    const int ch = q * 32 + lane;
    const int epi_tid = (warp - 2) * 32 + lane;
    long long kbg = 0;
    bool ok = true;
    uint32_t red_phase = 0;
    for (int t = tile_first; t < total && ok; t += tile_stride) {
      const int m = t / p.n_tiles, nt = t - m * p.n_tiles;
      int g, row0, rows;
      tile_of<NTOK>(p, m, g, row0, rows);
      if (rows <= 0) continue;
      const int n = nt * kTileN + ch;
      // activation scales of this tile -> shared memory (rows beyond the tile read as scale 0)
      asm volatile("bar.sync 1, 128;" ::: "memory");
      for (int i = epi_tid; i < NTOK * kblocks; i += 128) {
        const int j = i / kblocks, kb = i - j * kblocks;
        xs_tile[i] = j < rows ? p.x_scale[(row0 + j) * p.ldxs + kb] : 0;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const uint8_t* wsg = p.w_scale + (static_cast<size_t>(g) * p.w_scale_rows + nt) * kblocks;
      const uint8_t* wsu = DUAL ? p.w_scale + (static_cast<size_t>(g) * p.w_scale_rows + p.dual_offset / 128 + nt) * kblocks
                                : nullptr;
      float acc[NTOK];
      float accu[DUAL ? NTOK : 1];
#pragma unroll
      for (int j = 0; j < NTOK; ++j) acc[j] = 0.f;
      if (DUAL) {
#pragma unroll
        for (int j = 0; j < NTOK; ++j) accu[j] = 0.f;
      }
      for (int kb = kb_begin; kb < kb_end; ++kb, ++kbg) {
        const int a = static_cast<int>(kbg % C::kRing);
        const uint32_t aph = static_cast<uint32_t>((kbg / C::kRing) & 1);
        ok = mbar_wait(&acc_full[a], aph, abort_flag, p.status, 0x820);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tb = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + a * C::kAccCols;
        uint32_t g4 = 0, u4 = 0;     // G32: this lane's four group scales of the k-block (one per K = 32 slice)
        if (G32) {
          const size_t srow = static_cast<size_t>(g) * p.w_rows_total + static_cast<size_t>(nt) * kTileN + ch;
          const int sw_cols = kblocks * 4;
          const bool row_ok = nt * kTileN + ch < p.w_rows_total;
          g4 = row_ok ? *reinterpret_cast<const uint32_t*>(p.w_scale + srow * sw_cols + kb * 4) : 0u;
          if (DUAL) {
            const bool rowu_ok = p.dual_offset + nt * kTileN + ch < p.w_rows_total;
            u4 = rowu_ok ? *reinterpret_cast<const uint32_t*>(p.w_scale + (srow + p.dual_offset) * sw_cols + kb * 4) : 0u;
          }
        }
#pragma unroll
        for (int sub = 0; sub < C::kSub; ++sub) {
          const float swg = G32 ? e8m0(static_cast<uint8_t>(g4 >> (8 * sub))) : e8m0(wsg[kb]);
          const float swu = DUAL ? (G32 ? e8m0(static_cast<uint8_t>(u4 >> (8 * sub))) : e8m0(wsu[kb])) : 0.f;
#pragma unroll
          for (int c0 = 0; c0 < NTOK; c0 += 16) {
            uint32_t v[16], u[16];
            tmem_ld16(tb + sub * C::kSubCols + c0, v);
            if (DUAL) tmem_ld16(tb + sub * C::kSubCols + NTOK + c0, u);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float sxj = e8m0(xs_tile[(c0 + j) * kblocks + kb]);
              acc[c0 + j] = fmaf(__uint_as_float(v[j]), swg * sxj, acc[c0 + j]);
              if (DUAL) accu[c0 + j] = fmaf(__uint_as_float(u[j]), swu * sxj, accu[c0 + j]);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[a]);
      }
      if (!ok) break;
      if (S > 1) {
        constexpr int kAcc = NTOK * (DUAL ? 2 : 1);
        if (crank != 0) {
          // ship the scaled partial sums to the leader and move on: only the leader writes output
          const uint32_t remote = mapa_shared(smem_u32(red), 0) +
                                  (static_cast<uint32_t>((crank - 1) * kAcc) * 128u + static_cast<uint32_t>(ch)) * 4u;
#pragma unroll
          for (int j = 0; j < NTOK; ++j) {
            st_cluster_f32(remote + static_cast<uint32_t>(j) * 512u, acc[j]);
            if (DUAL) st_cluster_f32(remote + static_cast<uint32_t>(NTOK + j) * 512u, accu[j]);
          }
          mbar_arrive_remote(mapa_shared(smem_u32(red_bar), 0));
          continue;
        }
        ok = mbar_wait_cluster(red_bar, red_phase, abort_flag, p.status, 0x830);
        red_phase ^= 1u;
        if (!ok) break;
        // fixed summation order: own slice, then peers by cluster rank
        for (int pr = 1; pr < S; ++pr) {
          const float* rp = red + (static_cast<size_t>(pr - 1) * kAcc) * 128 + ch;
#pragma unroll
          for (int j = 0; j < NTOK; ++j) {
            acc[j] += rp[static_cast<size_t>(j) * 128];
            if (DUAL) accu[j] += rp[static_cast<size_t>(NTOK + j) * 128];
          }
        }
      }
      if (p.out_scale != nullptr) {
        // quantised output: the 128 channels of this tile are one scale block of every row.  Values are rounded
        // to bf16 first, so codes and scales equal those of a bf16 store followed by the row quantiser.
        float* am = reinterpret_cast<float*>(xs_tile + p.xs_bytes + p.red_bytes);      // [4 warps][NTOK]
#pragma unroll
        for (int j = 0; j < NTOK; ++j) {
          float x = acc[j];
          if (DUAL) {
            float up = accu[j];
            if (p.act_limit > 0.f) {
              x = fminf(x, p.act_limit);
              up = fminf(fmaxf(up, -p.act_limit), p.act_limit);
            }
            x = silu(x) * up;
          }
          x = (j < rows && n < p.n_out) ? bf16_round(x) : 0.f;
          acc[j] = x;
          const float v = warp_max(fabsf(x));
          if (lane == 0) am[q * NTOK + j] = v;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
        for (int j = 0; j < NTOK; ++j) {
          if (j < rows) {
            const float amax = fmaxf(fmaxf(am[j], am[NTOK + j]), fmaxf(am[2 * NTOK + j], am[3 * NTOK + j]));
            const uint8_t sb = fp8_block_scale(amax);
            const long long orow = row0 + j;
            if (n < p.n_out) reinterpret_cast<uint8_t*>(p.out)[orow * p.ldo + n] = to_e4m3(acc[j] / e8m0_to_float(sb));
            if (ch == 0) p.out_scale[orow * p.ldos + nt] = sb;
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      } else if (n < p.n_out) {
#pragma unroll
        for (int j = 0; j < NTOK; ++j) {
          if (j < rows) {
            float x = acc[j];
            if (DUAL) {
              float up = accu[j];
              if (p.act_limit > 0.f) {
                x = fminf(x, p.act_limit);
                up = fminf(fmaxf(up, -p.act_limit), p.act_limit);
              }
              x = silu(x) * up;
            }
            long long orow = row0 + j;
            if (p.epilogue == 2) {
              if (p.row_scale) x *= p.row_scale[row0 + j];
              if (p.dst_row) orow = p.dst_row[row0 + j];
            }
            if (p.out_fp32) reinterpret_cast<float*>(p.out)[orow * p.ldo + n] = x;
            else reinterpret_cast<__nv_bfloat16*>(p.out)[orow * p.ldo + n] = __float2bfloat16_rn(x);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
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

static int make_map_u8(CUtensorMap* map, const void* base, uint64_t k, uint64_t rows, uint64_t groups,
                       uint64_t row_stride, uint64_t group_stride, uint32_t box_rows, int rank) {
  EncodeTiledFn fn = encoder();
  if (!fn) return FB_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_stride & 15) || (group_stride & 15)) return FB_ERR_ALIGN;
  cuuint64_t dims[3] = {k, rows, groups};
  cuuint64_t strides[2] = {row_stride, group_stride};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(kBlockK), box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, rank, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? FB_OK : FB_ERR_DRIVER;
}

template <int NTOK, bool DUAL, bool G32>
static int launch(const CUtensorMap& mw, const CUtensorMap& mx, Params p, int max_tiles, int kblocks,
                  cudaStream_t stream) {
  using C = Cfg<NTOK, DUAL, G32>;
  auto kern = gemm_fp8_kernel<NTOK, DUAL, G32>;
  constexpr int kLimit = 227 * 1024;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kLimit) != cudaSuccess)
      return FB_ERR_LAUNCH;
    attr = true;
  }
  const int xs_bytes = (NTOK * kblocks + 15) / 16 * 16;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // Split-K over a cluster for dense GEMMs with few tiles (decode-sized projections): every tile gets its own
  // cluster, each CTA keeps at least 4 k-blocks, and the reduction area must leave room for two pipeline stages.
  int split = 1;
  const bool grouped = p.tile_group != nullptr || p.slot_rows > 0;
  constexpr int kAcc = NTOK * (DUAL ? 2 : 1);
  if (!grouped) {
    for (int sp = 2; sp <= 4; sp *= 2) {
      if (max_tiles * sp > sms || kblocks / sp < 4) break;
      if (kLimit - 2048 - xs_bytes - (sp - 1) * kAcc * 512 < 2 * C::kStageBytes) break;
      split = sp;
    }
  }
  const int red_bytes = split > 1 ? (split - 1) * kAcc * 512 : 0;
  int stages = (kLimit - 2048 - xs_bytes - red_bytes - 4 * NTOK * 4) / C::kStageBytes;
  if (stages > 10) stages = 10;
  if (stages < 2) return FB_ERR_SHAPE;
  p.stages = stages;
  p.xs_bytes = xs_bytes;
  p.red_bytes = red_bytes;
  const size_t smem = static_cast<size_t>(stages) * C::kStageBytes + 1024 + 256 + xs_bytes + red_bytes +
                      (p.out_scale ? 4 * NTOK * sizeof(float) : 0);
  int clusters = max_tiles < sms / split ? (max_tiles < 1 ? 1 : max_tiles) : sms / split;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(clusters * split, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr2[2];
  attr2[0].id = cudaLaunchAttributeClusterDimension;
  attr2[0].val.clusterDim.x = split;
  attr2[0].val.clusterDim.y = 1;
  attr2[0].val.clusterDim.z = 1;
  attr2[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr2[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr2;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  if (cudaLaunchKernelEx(&cfg, kern, mw, mx, p) != cudaSuccess) return FB_ERR_LAUNCH;
  return cudaGetLastError() == cudaSuccess ? FB_OK : FB_ERR_LAUNCH;
}

}  // namespace fp8
}  // namespace fb

using namespace fb;
using namespace fb::fp8;

extern "C" int fb_gemm_fp8(const FbGemmFp8Args* a, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!a || !a->w || !a->x || !a->out || !a->w_scale || !a->x_scale) return FB_ERR_SHAPE;
  if (a->n_out <= 0 || a->k <= 0 || a->k % 16 != 0 || a->groups <= 0 || a->x_rows <= 0) return FB_ERR_SHAPE;
  if (a->epilogue < 0 || a->epilogue > 2) return FB_ERR_SHAPE;
  const bool dual = a->epilogue == 1;
  if (a->ntok != 16 && a->ntok != 32 && a->ntok != 64) return FB_ERR_SHAPE;
  if (dual && (a->ntok > 32 || a->dual_offset % 128 != 0)) return FB_ERR_SHAPE;
  const bool slots = a->slot_rows > 0;
  if (slots && (!a->slot_cnt || a->tile_group || a->slot_rows % a->ntok != 0 ||
                static_cast<long long>(a->groups) * a->slot_rows > a->x_rows))
    return FB_ERR_SHAPE;
  if (a->out_scale && (a->epilogue == 2 || a->out_fp32 || a->scale_group32 || a->n_out % 128 != 0)) return FB_ERR_SHAPE;
  const bool grouped = a->tile_group != nullptr || slots;
  if (a->tile_group && (!a->tile_row0 || !a->tile_rows || !a->num_tok_tiles || a->max_tok_tiles <= 0)) return FB_ERR_SHAPE;
  if (!grouped && a->groups != 1) return FB_ERR_SHAPE;
  CUtensorMap mw, mx;
  int rc = make_map_u8(&mw, a->w, a->k, a->w_rows_per_group, a->groups, a->ldw, a->w_group_stride, kTileN, 3);
  if (rc != FB_OK) return rc;
  rc = make_map_u8(&mx, a->x, a->k, a->x_rows, 1, a->ldx, 0, a->ntok, 2);
  if (rc != FB_OK) return rc;
  Params p{};
  p.n_out = a->n_out;
  p.k = a->k;
  p.n_tiles = (a->n_out + kTileN - 1) / kTileN;
  p.dual_offset = a->dual_offset;
  p.dense_rows = a->x_rows;
  p.max_tok_tiles = slots ? a->groups * (a->slot_rows / a->ntok) : a->max_tok_tiles;
  p.slot_cnt = a->slot_cnt;
  p.slot_rows = slots ? a->slot_rows : 0;
  p.out_scale = static_cast<uint8_t*>(a->out_scale);
  p.ldos = a->ldos;
  p.tile_group = a->tile_group;
  p.tile_row0 = a->tile_row0;
  p.tile_rows = a->tile_rows;
  p.num_tok_tiles = a->num_tok_tiles;
  p.w_scale = static_cast<const uint8_t*>(a->w_scale);
  p.w_scale_rows = (a->w_rows_per_group + 127) / 128;
  p.w_rows_total = a->w_rows_per_group;
  p.x_scale = static_cast<const uint8_t*>(a->x_scale);
  p.ldxs = a->ldxs;
  p.out = a->out;
  p.ldo = a->ldo;
  p.out_fp32 = a->out_fp32;
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
  const int kblocks = (a->k + kBlockK - 1) / kBlockK;
  const int tok_tiles = grouped ? p.max_tok_tiles : (a->x_rows + a->ntok - 1) / a->ntok;
  const int max_tiles = tok_tiles * p.n_tiles;
  const bool g32 = a->scale_group32 != 0;
  if (g32 && (a->k % 128 != 0 || a->ntok > 32)) return FB_ERR_SHAPE;
  if (dual) {
    if (g32) return a->ntok == 16 ? launch<16, true, true>(mw, mx, p, max_tiles, kblocks, stream)
                                  : launch<32, true, true>(mw, mx, p, max_tiles, kblocks, stream);
    return a->ntok == 16 ? launch<16, true, false>(mw, mx, p, max_tiles, kblocks, stream)
                         : launch<32, true, false>(mw, mx, p, max_tiles, kblocks, stream);
  }
  if (g32) return a->ntok == 16 ? launch<16, false, true>(mw, mx, p, max_tiles, kblocks, stream)
                                : launch<32, false, true>(mw, mx, p, max_tiles, kblocks, stream);
  switch (a->ntok) {
    case 16: return launch<16, false, false>(mw, mx, p, max_tiles, kblocks, stream);
    case 32: return launch<32, false, false>(mw, mx, p, max_tiles, kblocks, stream);
    default: return launch<64, false, false>(mw, mx, p, max_tiles, kblocks, stream);
  }
}
