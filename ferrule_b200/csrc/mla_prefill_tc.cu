// Prefill attention over the paged latent-KV (MLA, weight-absorbed) cache on the 5th-generation tensor cores.
//
// Work item: one 128-row tile of (query position, head) pairs of ONE sequence - G = 128 / heads consecutive
// query positions times all heads, which is a contiguous 128 x 576 slab of the query matrix - and one half
// (256 of 512 latent features) of the output.  The fp32 output accumulator of a full tile would take all 512
// TMEM columns and leave none for the scores, so two CTAs each keep a 128 x 256 accumulator; both compute the
// scores of the tile (QK^T is repeated, PV is split), and they share nothing.
//
//   TMA producer (warp 0): the query slab once (9 blocks of 128 rows x 64 features, 128-byte swizzle), then per
//     64-token KV tile the 9 feature blocks of the pages that hold it (box = 64 features x min(page, 64) rows,
//     straight from the paged pool, zero-filled past the sequence).
//   MMA issuer (warp 1): S[128 x 64] = Q K^T with both operands K-major from shared memory (36 tcgen05.mma of
//     K = 16), then O[128 x 256] += P V with P read from TMEM as the A operand and the same shared-memory KV
//     tile read as an MN-major B operand (no transposed copy of V exists anywhere).
//   Softmax (warps 2..5, one row per thread): tcgen05.ld of the scores, scale, causal mask, running maximum,
//     exp2, bf16 P written back to TMEM with tcgen05.st.  The accumulator is only rescaled when a row's maximum
//     has grown by more than 2^8 since the reference it was scaled by; the final division uses the sum taken
//     against the same reference, so the result is exact up to rounding.
//
// The KV tile is single-buffered (the query slab and one tile fill shared memory), in two sets with their own
// full / free barriers: the blocks this CTA's PV does not read (the other half's latent blocks and the rope
// block) are free as soon as QK^T has retired, so their reload and the first five ninths of the next tile's
// QK^T overlap this tile's softmax and PV; the score buffer is double-buffered for that.
//
// A row's result depends only on the row and the cache contents - not on which other rows share its tile or
// how a prompt was cut into chunks (KV tiles start at absolute positions 0, 64, ...).
//
// Every wait is bounded (status word, then teardown with TMEM freed); page ids are range-checked and a bad one
// reads zeros instead of faulting.
//
// Counterpart of the reference's tensor-core prefill schedule of hybrid MLA attention
// (crates/ferrule-backend/native/cuda/implementations/cutlass/capabilities/hybrid_mla_attention/schedules/
// bf16_mma.cuh:332-823: 64-token KV tiles, QK / PV on mma.sync).
#include <cuda.h>

#include "common.cuh"
#include "ferrule_b200.h"
#include "launch.cuh"

namespace fb {

constexpr int kTcThreads = 192;
constexpr int kTcM = 128;                 // (position, head) rows per tile
constexpr int kTcKv = 64;                 // tokens per KV tile
constexpr int kTcBlocks = 9;              // 64-feature blocks of a 576-wide row (8 latent + 1 rope)
constexpr int kTcLat = 512;
constexpr int kTcHalf = 256;              // latent features per CTA
constexpr int kTcQBlockBytes = kTcM * 128;
constexpr int kTcKvBlockBytes = kTcKv * 128;
constexpr int kTcSmem = kTcBlocks * (kTcQBlockBytes + kTcKvBlockBytes) + 1024 /*alignment*/ + 256 /*barriers*/;
// TMEM columns: O 0..255, S0 256..319, S1 320..383, P 384..415
constexpr uint32_t kColO = 0, kColS = 256, kColP = 384, kTmemCols = 512;

struct TcParams {
  const int* tiles;          // [n_tiles, 4] = sequence, first query row, query rows (<= G), position of the first
  const int* block_table;    // [num_seqs, max_blocks]
  const float* sink;         // optional [heads], natural-log units
  __nv_bfloat16* out;        // [rows, heads, 512]
  DeviceStatus* status;
  long long ldo;
  long long pool_rows;
  int n_tiles;
  int rows;
  int heads;
  int num_seqs;
  int max_blocks;
  int page_size;
  int box_rows;              // min(page_size, 64)
  float scale_log2;
};

__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// MN-major operand laid out by TMA with the 128-byte swizzle: 64 contiguous elements of the MN dimension per
// 128-byte row, 8 K-rows per 1024-byte group (stride byte offset), the next 64 MN elements `mn_block_bytes` on
// (leading byte offset).
__device__ __forceinline__ uint64_t umma_desc_mn128(uint32_t smem_addr, uint32_t mn_block_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(mn_block_bytes >> 4) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

__global__ void __launch_bounds__(kTcThreads, 1)
mla_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                      const TcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* kv_s = smem + kTcBlocks * kTcQBlockBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(kv_s + kTcBlocks * kTcKvBlockBytes);
  uint64_t* q_full = bars + 0;
  uint64_t* kva_full = bars + 1;
  uint64_t* kvb_full = bars + 2;
  uint64_t* kva_free = bars + 3;
  uint64_t* kvb_free = bars + 4;
  uint64_t* s_full = bars + 5;          // [2]
  uint64_t* p_full = bars + 7;
  uint64_t* o_done = bars + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars + 10);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int half = blockIdx.y;
  const int4 tile = reinterpret_cast<const int4*>(p.tiles)[blockIdx.x];
  const int seq = tile.x, row0 = tile.y, nrows = tile.z, pos0 = tile.w;
  const int H = p.heads, G = kTcM / H;
  if (seq < 0 || seq >= p.num_seqs || row0 < 0 || nrows <= 0 || nrows > G || row0 + nrows > p.rows || pos0 < 0) {
    if (tid == 0) report_status(p.status, kStatusBadIndex, 0xA00, blockIdx.x, seq);
    return;
  }
  const int kv_len = min(pos0 + nrows, p.max_blocks * p.page_size);     // tokens 0 .. kv_len-1 are read
  const int n_kv_tiles = (kv_len + kTcKv - 1) / kTcKv;

  if (tid == 0) {
    mbar_init(q_full, 1);
    mbar_init(kva_full, 1);
    mbar_init(kvb_full, 1);
    mbar_init(kva_free, 1);
    mbar_init(kvb_free, 1);
    mbar_init(s_full + 0, 1);
    mbar_init(s_full + 1, 1);
    mbar_init(p_full, 4);
    mbar_init(o_done, 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_kv);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  pdl_wait();

  // this CTA's PV reads latent blocks [4*half, 4*half+4) ("set B"); the other latent blocks and the rope block
  // ("set A") are only read by QK^T
  const int b_lo = 4 * half, a_lo = 4 * (1 - half);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, kTcBlocks * kTcQBlockBytes);
      for (int b = 0; b < kTcBlocks; ++b) tma_load_2d(q_s + b * kTcQBlockBytes, &map_q, q_full, b * 64, row0 * H);
      const int subs = kTcKv / p.box_rows;
      const long long n_pages = p.pool_rows / p.page_size;
      bool ok = true;
      for (int j = 0; j < n_kv_tiles && ok; ++j) {
        int rowc[8];
        for (int s = 0; s < subs; ++s) {
          const int t0 = j * kTcKv + s * p.box_rows;
          int rc = static_cast<int>(p.pool_rows);              // out of range: the copy fills zeros
          if (t0 < kv_len) {
            const int page = p.block_table[static_cast<long long>(seq) * p.max_blocks + t0 / p.page_size];
            if (page >= 0 && page < n_pages) rc = page * p.page_size + t0 % p.page_size;
            else report_status(p.status, kStatusBadIndex, 0xA01, seq, t0);
          }
          rowc[s] = rc;
        }
        if (j > 0) ok = mbar_wait(kva_free, (j - 1) & 1, abort_flag, p.status, 0xA10);
        if (!ok) break;
        mbar_arrive_expect_tx(kva_full, 5 * kTcKvBlockBytes);
        for (int s = 0; s < subs; ++s) {
          for (int i = 0; i < 5; ++i) {
            const int b = i < 4 ? a_lo + i : 8;
            tma_load_2d(kv_s + b * kTcKvBlockBytes + s * p.box_rows * 128, &map_kv, kva_full, b * 64, rowc[s]);
          }
        }
        if (j > 0) ok = mbar_wait(kvb_free, (j - 1) & 1, abort_flag, p.status, 0xA11);
        if (!ok) break;
        mbar_arrive_expect_tx(kvb_full, 4 * kTcKvBlockBytes);
        for (int s = 0; s < subs; ++s)
          for (int i = 0; i < 4; ++i)
            tma_load_2d(kv_s + (b_lo + i) * kTcKvBlockBytes + s * p.box_rows * 128, &map_kv, kvb_full, (b_lo + i) * 64,
                        rowc[s]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t q_addr = smem_u32(q_s), kv_addr = smem_u32(kv_s);
      constexpr uint32_t idesc_qk = umma_idesc(kTcM, kTcKv, 1, 1);
      constexpr uint32_t idesc_pv = umma_idesc(kTcM, kTcHalf, 1, 1) | (1u << 16);     // B is MN-major
      auto qk_blocks = [&](int j, bool set_b) {
        const uint32_t s_t = tmem + kColS + (j & 1) * kTcKv;
        const int n = set_b ? 4 : 5;
        for (int i = 0; i < n; ++i) {
          const int b = set_b ? b_lo + i : (i < 4 ? a_lo + i : 8);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(s_t, umma_desc_k128(q_addr + b * kTcQBlockBytes + k * 32),
                      umma_desc_k128(kv_addr + b * kTcKvBlockBytes + k * 32), idesc_qk,
                      (set_b || i > 0 || k > 0) ? 1u : 0u);
        }
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, 0xA20);
      if (ok) ok = mbar_wait(kva_full, 0, abort_flag, p.status, 0xA21);
      if (ok) {
        tc_fence_after();
        qk_blocks(0, false);
        ok = mbar_wait(kvb_full, 0, abort_flag, p.status, 0xA22);
      }
      if (ok) {
        tc_fence_after();
        qk_blocks(0, true);
        umma_commit(s_full + 0);
        umma_commit(kva_free);
      }
      for (int j = 0; j < n_kv_tiles && ok; ++j) {
        const bool more = j + 1 < n_kv_tiles;
        if (more) {
          ok = mbar_wait(kva_full, (j + 1) & 1, abort_flag, p.status, 0xA23);
          if (!ok) break;
          tc_fence_after();
          qk_blocks(j + 1, false);                 // runs while the softmax warps work on tile j
        }
        ok = mbar_wait(p_full, j & 1, abort_flag, p.status, 0xA24);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16_ts(tmem + kColO, tmem + kColP + k * 8,
                       umma_desc_mn128(kv_addr + b_lo * kTcKvBlockBytes + k * 2048, kTcKvBlockBytes), idesc_pv,
                       (j > 0 || k > 0) ? 1u : 0u);
        umma_commit(kvb_free);
        if (!more) umma_commit(o_done);
        if (more) {
          ok = mbar_wait(kvb_full, (j + 1) & 1, abort_flag, p.status, 0xA25);
          if (!ok) break;
          tc_fence_after();
          qk_blocks(j + 1, true);
          umma_commit(s_full + ((j + 1) & 1));
          umma_commit(kva_free);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue: one row per thread
    const int quarter = warp & 3;                          // TMEM lanes this warp may touch: 32 * quarter ..
    const int r = quarter * 32 + lane;
    const int g = r / H, head = r - g * H;
    const bool valid = g < nrows;
    const int kvlen_row = valid ? min(pos0 + g + 1, kv_len) : 0;
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
    float m_ref = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv_tiles; ++j) {
      ok = mbar_wait(s_full + (j & 1), (j >> 1) & 1, abort_flag, p.status, 0xA30);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[4][16];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld16(lane_base + kColS + (j & 1) * kTcKv + c * 16, sv[c]);
      tmem_ld_wait();
      float mx = -INFINITY;
      const int tok0 = j * kTcKv;
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float x = __uint_as_float(sv[c][i]) * p.scale_log2;
          x = (tok0 + c * 16 + i < kvlen_row) ? x : -INFINITY;
          sv[c][i] = __float_as_uint(x);
          mx = fmaxf(mx, x);
        }
      const float m_new = fmaxf(m_ref, mx);
      if (j == 0) {
        m_ref = m_new;                                      // nothing accumulated yet
      } else if (__any_sync(0xffffffffu, m_new > m_ref + 8.f)) {
        // rescale this warp's 32 accumulator rows to their current maxima (PV of the previous tile has retired:
        // its commit precedes the one that completed s_full)
        const float f = (m_new == -INFINITY) ? 1.f : exp2f(m_ref - m_new);
        m_ref = m_new;
        l_sum *= f;
#pragma unroll 1
        for (int c = 0; c < kTcHalf / 16; ++c) {
          uint32_t ov[16];
          tmem_ld16(lane_base + kColO + c * 16, ov);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * f);
          tmem_st16(lane_base + kColO + c * 16, ov);
        }
      }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      float add = 0.f;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p0 = exp2f(__uint_as_float(sv[2 * c + (i >> 3)][(2 * i) & 15]) - m_use);
          const float p1 = exp2f(__uint_as_float(sv[2 * c + (i >> 3)][((2 * i) & 15) + 1]) - m_use);
          add += p0 + p1;
          pk[i] = pack_bf16x2(p0, p1);
        }
        tmem_st16(lane_base + kColP + c * 16, pk);
      }
      l_sum += add;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok) {
      ok = mbar_wait(o_done, 0, abort_flag, p.status, 0xA31);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      float l_tot = l_sum;
      if (p.sink != nullptr && valid) {
        const float sk = p.sink[head] * 1.4426950408889634f;
        // the accumulator is scaled by 2^-m_ref: bring the sink term to the same reference
        l_tot += exp2f(sk - ((m_ref == -INFINITY) ? sk : m_ref));
      }
      const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
      __nv_bfloat16* dst = p.out + static_cast<long long>(row0 + g) * p.ldo + static_cast<long long>(head) * kTcLat +
                           half * kTcHalf;
#pragma unroll 1
      for (int c = 0; c < kTcHalf / 16; ++c) {
        uint32_t ov[16];
        tmem_ld16(lane_base + kColO + c * 16, ov);
        tmem_ld_wait();
        if (valid) {
          uint4 w0, w1;
          w0.x = pack_bf16x2(__uint_as_float(ov[0]) * inv, __uint_as_float(ov[1]) * inv);
          w0.y = pack_bf16x2(__uint_as_float(ov[2]) * inv, __uint_as_float(ov[3]) * inv);
          w0.z = pack_bf16x2(__uint_as_float(ov[4]) * inv, __uint_as_float(ov[5]) * inv);
          w0.w = pack_bf16x2(__uint_as_float(ov[6]) * inv, __uint_as_float(ov[7]) * inv);
          w1.x = pack_bf16x2(__uint_as_float(ov[8]) * inv, __uint_as_float(ov[9]) * inv);
          w1.y = pack_bf16x2(__uint_as_float(ov[10]) * inv, __uint_as_float(ov[11]) * inv);
          w1.z = pack_bf16x2(__uint_as_float(ov[12]) * inv, __uint_as_float(ov[13]) * inv);
          w1.w = pack_bf16x2(__uint_as_float(ov[14]) * inv, __uint_as_float(ov[15]) * inv);
          *reinterpret_cast<uint4*>(dst + c * 16) = w0;
          *reinterpret_cast<uint4*>(dst + c * 16 + 8) = w1;
        }
      }
    }
  }
  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------
typedef CUresult (*TcEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static TcEncodeFn tc_encoder() {
  static TcEncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<TcEncodeFn>(ptr);
  }
  return fn;
}

// bf16 [rows, 576] matrix, box 64 features x box_rows rows, 128-byte swizzle, zeros outside
static int tc_map(CUtensorMap* map, const void* base, uint64_t rows, uint32_t box_rows) {
  TcEncodeFn fn = tc_encoder();
  if (!fn) return FB_ERR_DRIVER;
  if (reinterpret_cast<uintptr_t>(base) & 15) return FB_ERR_ALIGN;
  cuuint64_t dims[2] = {576, rows};
  cuuint64_t strides[1] = {576 * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FB_OK : FB_ERR_DRIVER;
}

}  // namespace fb

using namespace fb;

extern "C" int fb_mla_prefill_tc(const FbPrefillAttnArgs* a, void* stream_) {
  if (!a || !a->q || !a->kv || !a->out || !a->tiles || !a->block_table) return FB_ERR_SHAPE;
  if (a->kv_lora != kTcLat || a->rope_dim != 64) return FB_ERR_SHAPE;
  if (a->heads <= 0 || a->heads > kTcM || (kTcM % a->heads) != 0) return FB_ERR_SHAPE;
  if (a->rows <= 0 || a->n_tiles <= 0 || a->num_seqs <= 0 || a->max_blocks <= 0) return FB_ERR_SHAPE;
  if (a->page_size < 8 || (a->page_size & (a->page_size - 1)) != 0) return FB_ERR_SHAPE;
  if (a->ldq != static_cast<long long>(a->heads) * 576) return FB_ERR_SHAPE;      // (row, head) pairs form one matrix
  if ((a->ldo % 8) != 0 || (reinterpret_cast<uintptr_t>(a->out) & 15)) return FB_ERR_ALIGN;
  if (a->pool_rows <= 0 || a->pool_rows > 0x7fffffffLL || (a->pool_rows % a->page_size) != 0) return FB_ERR_SHAPE;
  if (reinterpret_cast<uintptr_t>(a->tiles) & 15) return FB_ERR_ALIGN;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int box_rows = a->page_size < kTcKv ? a->page_size : kTcKv;
  CUtensorMap mq, mkv;
  int rc = tc_map(&mq, a->q, static_cast<uint64_t>(a->rows) * a->heads, kTcM);
  if (rc != FB_OK) return rc;
  rc = tc_map(&mkv, a->kv, static_cast<uint64_t>(a->pool_rows), box_rows);
  if (rc != FB_OK) return rc;
  TcParams p{};
  p.tiles = a->tiles;
  p.block_table = a->block_table;
  p.sink = a->sink;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.status = static_cast<DeviceStatus*>(a->status);
  p.ldo = a->ldo;
  p.pool_rows = a->pool_rows;
  p.n_tiles = a->n_tiles;
  p.rows = a->rows;
  p.heads = a->heads;
  p.num_seqs = a->num_seqs;
  p.max_blocks = a->max_blocks;
  p.page_size = a->page_size;
  p.box_rows = box_rows;
  p.scale_log2 = a->softmax_scale * 1.4426950408889634f;
  if (cudaFuncSetAttribute(mla_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmem) != cudaSuccess)
    return FB_ERR_LAUNCH;
  if (launch_pdl(mla_prefill_tc_kernel, dim3(a->n_tiles, 2), dim3(kTcThreads), kTcSmem, stream, mq, mkv, p) !=
      cudaSuccess)
    return FB_ERR_LAUNCH;
  return FB_OK;
}
