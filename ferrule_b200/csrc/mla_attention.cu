// Paged latent-KV (MLA, weight-absorbed) attention for sm_100a.
//
// All heads of a token share one latent KV row [kv_lora | rope]; a query row per head
// is [q_latent (kv_lora) | q_rope].  score = q . kv_row, value = kv_row[:kv_lora].
//
// A CTA owns one 16-row MMA tile (16 = query rows x heads-per-block of one sequence)
// and one KV split.  KV rows are pulled page by page with bulk async copies
// (cp.async.bulk, one row per copy, completion on an mbarrier) into padded shared
// memory, so one HBM read of a KV row serves every head.  QK^T and PV run on warp-level
// bf16 MMA (m16n8k16): a 16-row tile is below the 64-row minimum of tcgen05, and the
// kernel is bound by the KV stream, not by math.  Online softmax in the log2 domain,
// optional per-head sink logit in the denominator, split-KV partials merged by whichever
// CTA of a (query tile, head block) finishes last (or by a second kernel when no counter is given).  Every page id and slot is range-checked; a bad one masks the row and sets the
// status word instead of faulting.
//
// Counterpart of the reference's explicit-selection sparse MLA attention and hybrid
// proposal attention (crates/ferrule-backend/native/cuda/implementations/cutlass/capabilities/
// hybrid_mla_attention/schedules/bf16_mma.cuh:332-823, hybrid_mla_attention.cuh:521-641) and of
// its CPU sink-softmax reference (crates/ferrule-model/src/attention_backend.rs:47-160).
#include <cstdlib>

#include "common.cuh"
#include "ferrule_b200.h"
#include "launch.cuh"

namespace fb {

constexpr int kAttnThreads = 128;
constexpr int kKvTile = 64;

struct AttnParams {
  const __nv_bfloat16* q;   // [rows, heads, D]
  long long ldq;            // elements between query rows
  const __nv_bfloat16* kv;  // [pool_rows, D]
  long long pool_rows;
  const int* block_table;   // [num_seqs, max_blocks]
  int max_blocks;
  int page_size;
  int num_seqs;
  const int* row_seq;       // [rows]
  const int* row_pos;       // [rows]  (row attends to kv positions 0..row_pos)
  int rows;
  int heads;
  int group_rows;           // query rows per CTA tile (all of one sequence); 16 / group_rows heads per block
  int splits;
  int split_tokens;         // multiple of 64
  float scale_log2;         // softmax scale * log2(e)
  const float* sink;        // optional [heads], natural-log units
  __nv_bfloat16* out;       // [rows, heads, DL]   (splits == 1)
  long long ldo;
  float* part_o;            // [rows, splits, heads, DL] (splits > 1)
  float* part_ml;           // [rows, splits, heads, 2]
  unsigned int* merge_ctr;  // [q groups * head blocks] zeroed once: last split CTA merges in-kernel
  int cluster_merge;        // splits form one thread-block cluster and merge through distributed smem
  const int* selection;     // optional [rows, sel_width] pool rows per query row (-1 = masked); group_rows == 1
  int sel_width;
  DeviceStatus* status;
  int kv_stream;            // decode-sized launch: KV rows are read once, load them with the L2 evict-first policy
  int prefetch_old;         // one query row per sequence (plain decode step): every KV row below the row's own
                            // position was written by an earlier step, so the first tile may be requested before
                            // the dependency wait
  unsigned long long* trace;  // optional: CTA (0,0,0) writes globaltimer stamps of its milestones
};

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, uint32_t bytes,
                                              uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// KV rows of a decode step are read once: evict-first keeps the step's reusable lines in L2
__device__ __forceinline__ void bulk_copy_g2s_stream(void* dst, const void* src, uint32_t bytes, uint64_t* bar,
                                                     uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int DL, int DR>
struct AttnSmem {
  static constexpr int D = DL + DR;
  static constexpr int kRowPad = D + 8;        // bf16 elements; +16 bytes keeps ldmatrix conflict-free
  static constexpr int kPPad = kKvTile + 8;
  static constexpr int kQBytes = 16 * kRowPad * 2;
  static constexpr int kKvBytes = kKvTile * kRowPad * 2;
  static constexpr int kPBytes = 16 * kPPad * 2;
  static constexpr int kRedBytes = 4 * 16 * 4 * 2 + 32 * 4;   // smax, ssum, cluster-merge statistics
  static constexpr int kTotal = kQBytes + kKvBytes + kPBytes + kRedBytes + 64;
};

template <int DL, int DR>
__global__ void __launch_bounds__(kAttnThreads)
mla_attention_kernel(const AttnParams p) {
  pdl_launch_dependents();
  using S = AttnSmem<DL, DR>;
  constexpr int D = S::D;
  constexpr int kRowPad = S::kRowPad;
  constexpr int kDimsPerWarp = DL / 4;
  constexpr int kNT = kDimsPerWarp / 8;  // n-tiles of 8 dims per warp
  static_assert(D % 16 == 0 && DL % 64 == 0, "unsupported head geometry");
  extern __shared__ __align__(128) uint8_t smem_attn[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_attn);
  __nv_bfloat16* KVs = reinterpret_cast<__nv_bfloat16*>(smem_attn + S::kQBytes);
  __nv_bfloat16* Ps = reinterpret_cast<__nv_bfloat16*>(smem_attn + S::kQBytes + S::kKvBytes);
  float* smax = reinterpret_cast<float*>(smem_attn + S::kQBytes + S::kKvBytes + S::kPBytes);
  float* ssum = smax + 64;
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem_attn + S::kQBytes + S::kKvBytes + S::kPBytes +
                                              S::kRedBytes);
  volatile uint32_t* abort_flag = reinterpret_cast<uint32_t*>(bar + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int G = p.group_rows;
  const int Hb = 16 / G;  // heads per block
  const int qgroup = blockIdx.x, split = blockIdx.y, hblock = blockIdx.z;
  const int qrow0 = qgroup * G;
  if (qrow0 >= p.rows) return;
  const bool tracing = p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && tid == 0;
  int stamp = 0;
  if (tracing) p.trace[stamp++] = globaltimer_ns();      // entry (dependency wait passed)

  if (tid == 0) {
    mbar_init(bar, kKvTile);
    *abort_flag = 0;
    fence_barrier_init();
  }
  // ---- before the dependency wait: only memory that no kernel of the running step writes may be read - the
  // batch description (row_seq / row_pos / block_table, written by the copy or kernel that precedes the whole
  // step) and, in a plain decode step, the KV rows of earlier positions.  Their copies for the first tile are
  // requested now, so they stream while the preceding kernel drains. ----
  bool pre_issued = false;
  if (p.prefetch_old) {
    __syncthreads();                       // the barrier is initialised before anything arrives on it
    const int seq0 = p.row_seq[qrow0];
    const int pos0 = p.row_pos[qrow0];
    if (seq0 >= 0 && seq0 < p.num_seqs && tid < kKvTile) {
      const int tok = blockIdx.y * p.split_tokens + tid;
      const int lim = min(min(pos0, p.max_blocks * p.page_size), (blockIdx.y + 1) * p.split_tokens);
      if (tok < lim) {                     // strictly below the row's own position: written by an earlier step
        const int page = p.block_table[static_cast<long long>(seq0) * p.max_blocks + tok / p.page_size];
        const long long slot = static_cast<long long>(page) * p.page_size + tok % p.page_size;
        if (page >= 0 && slot < p.pool_rows) {
          __nv_bfloat16* dst = KVs + tid * kRowPad;
          mbar_arrive_expect_tx(bar, D * 2);
          if (p.kv_stream) bulk_copy_g2s_stream(dst, p.kv + slot * D, D * 2, bar, l2_policy_evict_first());
          else bulk_copy_g2s(dst, p.kv + slot * D, D * 2, bar);
          pre_issued = true;
        }
      }
    }
  }
  pdl_wait();

  if (tracing) p.trace[12] = globaltimer_ns();
  // ---- query tile -> smem (rows beyond the valid set are zero).  The loads are issued first and parked in
  // registers so that their latency overlaps the dependent row -> sequence -> length lookups below ----
  constexpr int kQVecs = (16 * (D / 8) + kAttnThreads - 1) / kAttnThreads;
  uint4 qv[kQVecs];
  {
    const int Hb0 = 16 / p.group_rows;
#pragma unroll
    for (int j = 0; j < kQVecs; ++j) {
      const int i = tid + j * kAttnThreads;
      const int r = i / (D / 8), c = i - r * (D / 8);
      const int qr = blockIdx.x * p.group_rows + r / Hb0, h = blockIdx.z * Hb0 + r % Hb0;
      qv[j] = make_uint4(0, 0, 0, 0);
      if (i < 16 * (D / 8) && qr < p.rows && h < p.heads)
        qv[j] = *reinterpret_cast<const uint4*>(p.q + qr * p.ldq + static_cast<long long>(h) * D + c * 8);
    }
  }
  if (tracing) p.trace[13] = globaltimer_ns();
  const bool by_selection = p.selection != nullptr;
  const int* sel = by_selection ? p.selection + static_cast<long long>(qrow0) * p.sel_width : nullptr;
  int seq = by_selection ? 0 : p.row_seq[qrow0];
  bool seq_ok = by_selection || (seq >= 0 && seq < p.num_seqs);
  if (!seq_ok) {
    if (tid == 0) report_status(p.status, kStatusBadIndex, 0x60, qrow0, seq);
    seq = 0;
  }
  int kv_len_max = 0;
  for (int r = 0; r < G && !by_selection; ++r)
    if (qrow0 + r < p.rows) kv_len_max = max(kv_len_max, p.row_pos[qrow0 + r] + 1);
  if (!seq_ok) kv_len_max = 0;
  kv_len_max = by_selection ? p.sel_width : min(kv_len_max, p.max_blocks * p.page_size);

  if (tracing) p.trace[14] = globaltimer_ns() + (kv_len_max == -12345);
  // per-thread row limits (rows g and g+8 of the tile)
  int kvlen_lo = 0, kvlen_hi = 0;
  {
    const int qr_lo = qrow0 + g / Hb, qr_hi = qrow0 + (g + 8) / Hb;
    if (seq_ok && qr_lo < p.rows && g / Hb < G) kvlen_lo = by_selection ? p.sel_width : p.row_pos[qr_lo] + 1;
    if (seq_ok && qr_hi < p.rows && (g + 8) / Hb < G) kvlen_hi = by_selection ? p.sel_width : p.row_pos[qr_hi] + 1;
  }
  if (tracing) p.trace[15] = globaltimer_ns() + (kvlen_lo + kvlen_hi == -12345);
#pragma unroll
  for (int j = 0; j < kQVecs; ++j) {
    const int i = tid + j * kAttnThreads;
    const int r = i / (D / 8), c = i - r * (D / 8);
    if (i < 16 * (D / 8)) *reinterpret_cast<uint4*>(Qs + r * kRowPad + c * 8) = qv[j];
  }
  __syncthreads();
  if (tracing) p.trace[stamp++] = globaltimer_ns();      // query tile staged

  const int kv_begin = split * p.split_tokens;
  const int kv_end = min(kv_len_max, kv_begin + p.split_tokens);

  float o_acc[kNT][4];
#pragma unroll
  for (int i = 0; i < kNT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

  const uint32_t qs_addr = smem_u32(Qs), kv_addr = smem_u32(KVs), ps_addr = smem_u32(Ps);
  const uint64_t kv_policy = l2_policy_evict_first();
  uint32_t phase = 0;
  bool ok = true;

  for (int tile0 = kv_begin; tile0 < kv_end && ok; tile0 += kKvTile) {
    // ---- load: threads 0..63 fetch one KV row each (rows of the first tile requested before the dependency
    // wait are on their way already) ----
    if (tid < kKvTile && !(pre_issued && tile0 == kv_begin)) {
      const int tok = tile0 + tid;
      __nv_bfloat16* dst = KVs + tid * kRowPad;
      bool issued = false;
      if (tok < kv_end && by_selection) {
        const long long slot = sel[tok];
        if (slot >= 0 && slot < p.pool_rows) {
          mbar_arrive_expect_tx(bar, D * 2);
          if (p.kv_stream) bulk_copy_g2s_stream(dst, p.kv + slot * D, D * 2, bar, kv_policy);
          else bulk_copy_g2s(dst, p.kv + slot * D, D * 2, bar);
          issued = true;
        } else if (slot >= 0) {
          report_status(p.status, kStatusBadIndex, 0x63, qrow0, tok);
        }
      } else if (tok < kv_end) {
        const int page = p.block_table[static_cast<long long>(seq) * p.max_blocks + tok / p.page_size];
        const long long slot = static_cast<long long>(page) * p.page_size + tok % p.page_size;
        if (page >= 0 && slot < p.pool_rows) {
          mbar_arrive_expect_tx(bar, D * 2);
          if (p.kv_stream) bulk_copy_g2s_stream(dst, p.kv + slot * D, D * 2, bar, kv_policy);
          else bulk_copy_g2s(dst, p.kv + slot * D, D * 2, bar);
          issued = true;
        } else {
          report_status(p.status, kStatusBadIndex, 0x61, seq, tok);
        }
      }
      if (!issued) {
        for (int c = 0; c < D / 8; ++c) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0, 0, 0, 0);
        mbar_arrive(bar);
      }
    }
    ok = mbar_wait(bar, phase, abort_flag, p.status, 0x62);
    phase ^= 1u;
    __syncthreads();  // zero-filled rows visible to all
    if (!ok || *abort_flag) { ok = false; break; }
    if (tracing && stamp < 24) p.trace[stamp++] = globaltimer_ns();    // KV tile landed

    // ---- S = Q K^T for this warp's 16 tokens ----
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
    {
      const uint32_t a_base = qs_addr + (((lane & 7) + ((lane >> 3) & 1) * 8) * kRowPad + (lane >> 4) * 8) * 2;
      const uint32_t b_base =
          kv_addr + ((warp * 16 + (lane & 7) + (lane >> 4) * 8) * kRowPad + ((lane >> 3) & 1) * 8) * 2;
#pragma unroll 4
      for (int k0 = 0; k0 < D; k0 += 16) {
        uint32_t a[4], b[4];
        ldsm_x4(a, a_base + k0 * 2);
        ldsm_x4(b, b_base + k0 * 2);
        mma_bf16_16816(s0, a, b[0], b[1]);
        mma_bf16_16816(s1, a, b[2], b[3]);
      }
    }
    if (tracing && stamp < 24) p.trace[stamp++] = globaltimer_ns();    // scores done
    // ---- scale, mask, tile max ----
    const int tok_base = tile0 + warp * 16 + t4 * 2;
    float tmax_lo = -INFINITY, tmax_hi = -INFINITY;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int tok0 = tok_base + j;
      const int tok1 = tok_base + 8 + j;
      // an explicit selection masks its -1 entries (their rows were zero-filled above)
      const bool v0 = !by_selection || (tok0 < p.sel_width && sel[tok0] >= 0);
      const bool v1 = !by_selection || (tok1 < p.sel_width && sel[tok1] >= 0);
      s0[j] = (v0 && tok0 < kvlen_lo) ? s0[j] * p.scale_log2 : -INFINITY;
      s0[2 + j] = (v0 && tok0 < kvlen_hi) ? s0[2 + j] * p.scale_log2 : -INFINITY;
      s1[j] = (v1 && tok1 < kvlen_lo) ? s1[j] * p.scale_log2 : -INFINITY;
      s1[2 + j] = (v1 && tok1 < kvlen_hi) ? s1[2 + j] * p.scale_log2 : -INFINITY;
      tmax_lo = fmaxf(tmax_lo, fmaxf(s0[j], s1[j]));
      tmax_hi = fmaxf(tmax_hi, fmaxf(s0[2 + j], s1[2 + j]));
    }
    tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 1));
    tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 2));
    tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 1));
    tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 2));
    if (t4 == 0) {
      smax[warp * 16 + g] = tmax_lo;
      smax[warp * 16 + g + 8] = tmax_hi;
    }
    __syncthreads();
    float mt_lo = fmaxf(fmaxf(smax[g], smax[16 + g]), fmaxf(smax[32 + g], smax[48 + g]));
    float mt_hi = fmaxf(fmaxf(smax[g + 8], smax[24 + g]), fmaxf(smax[40 + g], smax[56 + g]));
    const float mn_lo = fmaxf(m_lo, mt_lo), mn_hi = fmaxf(m_hi, mt_hi);
    const float sub_lo = mn_lo == -INFINITY ? 0.f : mn_lo, sub_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
    const float alpha_lo = exp2f(m_lo - sub_lo), alpha_hi = exp2f(m_hi - sub_hi);
    m_lo = mn_lo;
    m_hi = mn_hi;
    float p0[4], p1[4];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      p0[j] = exp2f(s0[j] - sub_lo);
      p0[2 + j] = exp2f(s0[2 + j] - sub_hi);
      p1[j] = exp2f(s1[j] - sub_lo);
      p1[2 + j] = exp2f(s1[2 + j] - sub_hi);
    }
    l_lo = l_lo * alpha_lo + p0[0] + p0[1] + p1[0] + p1[1];
    l_hi = l_hi * alpha_hi + p0[2] + p0[3] + p1[2] + p1[3];
    {
      const int col = warp * 16 + t4 * 2;
      *reinterpret_cast<uint32_t*>(Ps + g * S::kPPad + col) = pack_bf16(p0[0], p0[1]);
      *reinterpret_cast<uint32_t*>(Ps + (g + 8) * S::kPPad + col) = pack_bf16(p0[2], p0[3]);
      *reinterpret_cast<uint32_t*>(Ps + g * S::kPPad + col + 8) = pack_bf16(p1[0], p1[1]);
      *reinterpret_cast<uint32_t*>(Ps + (g + 8) * S::kPPad + col + 8) = pack_bf16(p1[2], p1[3]);
    }
#pragma unroll
    for (int i = 0; i < kNT; ++i) {
      o_acc[i][0] *= alpha_lo;
      o_acc[i][1] *= alpha_lo;
      o_acc[i][2] *= alpha_hi;
      o_acc[i][3] *= alpha_hi;
    }
    __syncthreads();
    if (tracing && stamp < 24) p.trace[stamp++] = globaltimer_ns();    // softmax done

    // ---- O += P V for this warp's slice of the latent dims ----
    {
      const uint32_t pa_base = ps_addr + (((lane & 7) + ((lane >> 3) & 1) * 8) * S::kPPad + (lane >> 4) * 8) * 2;
      const uint32_t vb_base =
          kv_addr + (((lane & 7) + ((lane >> 3) & 1) * 8) * kRowPad + warp * kDimsPerWarp + (lane >> 4) * 8) * 2;
#pragma unroll
      for (int kk = 0; kk < kKvTile / 16; ++kk) {
        uint32_t a[4];
        ldsm_x4(a, pa_base + kk * 16 * 2);
#pragma unroll
        for (int nt = 0; nt < kNT; nt += 2) {
          uint32_t b[4];
          ldsm_x4_t(b, vb_base + (kk * 16 * kRowPad + nt * 8) * 2);
          mma_bf16_16816(o_acc[nt], a, b[0], b[1]);
          mma_bf16_16816(o_acc[nt + 1], a, b[2], b[3]);
        }
      }
    }
    __syncthreads();  // KV tile and P are free for the next iteration
    if (tracing && stamp < 24) p.trace[stamp++] = globaltimer_ns();    // PV done
  }
  if (tracing) { stamp = 24; p.trace[stamp++] = globaltimer_ns(); }  // tile loop left

  // ---- combine the per-warp partial row sums ----
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  if (t4 == 0) {
    ssum[warp * 16 + g] = l_lo;
    ssum[warp * 16 + g + 8] = l_hi;
  }
  __syncthreads();
  l_lo = ssum[g] + ssum[16 + g] + ssum[32 + g] + ssum[48 + g];
  l_hi = ssum[g + 8] + ssum[24 + g] + ssum[40 + g] + ssum[56 + g];

  if (p.cluster_merge) {
    // ---- split merge inside the cluster: every CTA parks its unnormalised partial and softmax
    // statistics in its own shared memory, then merges one slice of the latent dims for all rows,
    // reading the peers' partials through distributed shared memory.  No global scratch. ----
    float* Osm = reinterpret_cast<float*>(smem_attn + S::kQBytes);          // [16][DL] over the dead KV tile
    float* Msm = ssum + 64;                                                  // [16] m, [16] l (after smax/ssum)
    __syncthreads();
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = g + half * 8;
      float* o = Osm + r * DL + warp * kDimsPerWarp + t4 * 2;
#pragma unroll
      for (int i = 0; i < kNT; ++i)
        *reinterpret_cast<float2*>(o + i * 8) = make_float2(o_acc[i][half * 2], o_acc[i][half * 2 + 1]);
      if (warp == 0 && t4 == 0) {
        Msm[r] = ok ? (half ? m_hi : m_lo) : -INFINITY;
        Msm[16 + r] = ok ? (half ? l_hi : l_lo) : 0.f;
      }
    }
    cluster_sync_all();
    if (tracing) p.trace[stamp++] = globaltimer_ns();                  // all splits parked their partials
    const int CS = static_cast<int>(cluster_nctarank());
    const int crank = static_cast<int>(cluster_ctarank());
    const int slice = DL / CS;                       // latent dims merged by this CTA
    const uint32_t osm_addr = smem_u32(Osm), msm_addr = smem_u32(Msm);
    float* wsm = smax;                               // [16][8] normalised split weights (CS <= 8)
    {
      // thread (r, c) fetches the statistics of split c for row r (one remote access each); the 8 lanes of a
      // row then combine them with shuffles, in split order
      const int r = tid >> 3, c = tid & 7;
      const int h = hblock * Hb + r % Hb;
      float mv = -INFINITY, lv = 0.f;
      if (c < CS) {
        const uint32_t ra = mapa_shared(msm_addr, c);
        // both loads in flight together (the compiler may not reorder the volatile form)
        asm("ld.shared::cluster.f32 %0, [%2];\n\tld.shared::cluster.f32 %1, [%3];"
            : "=f"(mv), "=f"(lv) : "r"(ra + r * 4), "r"(ra + (16 + r) * 4));
      }
      float M = mv;
#pragma unroll
      for (int o = 1; o < 8; o <<= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
      float sink_l = 0.f;
      if (p.sink && h < p.heads) {
        const float sk = p.sink[h] * 1.4426950408889634f;
        M = fmaxf(M, sk);
        sink_l = exp2f(sk - M);
      }
      const float w = (mv == -INFINITY || lv == 0.f) ? 0.f : exp2f(mv - M);
      // fixed-order sum over the splits (lane c holds term c)
      float L = sink_l;
      const int lane_base = lane & ~7;
#pragma unroll
      for (int cc = 0; cc < 8; ++cc) L += __shfl_sync(0xffffffffu, lv * w, lane_base + cc);
      const float inv = L > 0.f ? 1.f / L : 0.f;
      wsm[r * 8 + c] = w * inv;
    }
    __syncthreads();
    if (tracing) p.trace[stamp++] = globaltimer_ns();                  // split weights ready
    const int vec_per_row = slice / 4;
    for (int item = tid; item < 16 * vec_per_row; item += kAttnThreads) {
      const int r = item / vec_per_row, d = crank * slice + (item - r * vec_per_row) * 4;
      const int qr = qrow0 + r / Hb, h = hblock * Hb + r % Hb;
      if (r / Hb >= G || qr >= p.rows || h >= p.heads) continue;
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      // the partials of all splits are requested together (one round trip through distributed shared memory
      // instead of one per split), then added in split order
      float4 v[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        v[c] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < CS) {
          const uint32_t a = mapa_shared(osm_addr, c) + (r * DL + d) * 4;
          asm("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
              : "=f"(v[c].x), "=f"(v[c].y), "=f"(v[c].z), "=f"(v[c].w) : "r"(a));
        }
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        if (c < CS) {
          const float w = wsm[r * 8 + c];
          acc[0] += v[c].x * w; acc[1] += v[c].y * w; acc[2] += v[c].z * w; acc[3] += v[c].w * w;
        }
      }
      __nv_bfloat16* o = p.out + qr * p.ldo + static_cast<long long>(h) * DL + d;
      *reinterpret_cast<uint32_t*>(o) = pack_bf16(acc[0], acc[1]);
      *reinterpret_cast<uint32_t*>(o + 2) = pack_bf16(acc[2], acc[3]);
    }
    if (tracing) p.trace[stamp++] = globaltimer_ns();                  // merged slice written
    cluster_sync_all();   // peers may still be reading this CTA's shared memory
    if (tracing) p.trace[stamp++] = globaltimer_ns();
    return;
  }

  // ---- write ----
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = g + half * 8;
    const int qr = qrow0 + r / Hb, h = hblock * Hb + r % Hb;
    if (r / Hb >= G || qr >= p.rows || h >= p.heads) continue;
    float m = half ? m_hi : m_lo, l = half ? l_hi : l_lo;
    if (!ok) { m = -INFINITY; l = 0.f; }
    if (p.splits == 1) {
      if (p.sink) {
        const float sk = p.sink[h] * 1.4426950408889634f;
        const float mn = fmaxf(m, sk);
        const float a = m == -INFINITY ? 0.f : exp2f(m - mn);
        l = l * a + exp2f(sk - mn);
#pragma unroll
        for (int i = 0; i < kNT; ++i) { o_acc[i][half * 2] *= a; o_acc[i][half * 2 + 1] *= a; }
      }
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* o = p.out + qr * p.ldo + static_cast<long long>(h) * DL + warp * kDimsPerWarp + t4 * 2;
#pragma unroll
      for (int i = 0; i < kNT; ++i)
        *reinterpret_cast<uint32_t*>(o + i * 8) = pack_bf16(o_acc[i][half * 2] * inv, o_acc[i][half * 2 + 1] * inv);
    } else {
      const size_t idx = (static_cast<size_t>(qr) * p.splits + split) * p.heads + h;
      float* o = p.part_o + idx * DL + warp * kDimsPerWarp + t4 * 2;
#pragma unroll
      for (int i = 0; i < kNT; ++i)
        *reinterpret_cast<float2*>(o + i * 8) = make_float2(o_acc[i][half * 2], o_acc[i][half * 2 + 1]);
      if (warp == 0 && t4 == 0) {
        p.part_ml[idx * 2] = m;
        p.part_ml[idx * 2 + 1] = l;
      }
    }
  }
  if (p.splits == 1 || p.merge_ctr == nullptr) return;

  // ---- in-kernel merge: the CTA that finishes last for this (query group, head block) combines
  // the split partials, so no second launch is needed ----
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    unsigned int* c = p.merge_ctr + static_cast<size_t>(qgroup) * gridDim.z + hblock;
    const unsigned int done = atomicAdd(c, 1u);
    is_last = done == static_cast<unsigned int>(p.splits - 1);
    if (is_last) *c = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // per-row softmax statistics of all splits -> shared memory (weights w_s = 2^(m_s - M) / L)
  float* wts = reinterpret_cast<float*>(smem_attn);        // [16][splits], the tiles are dead by now
  for (int i = tid; i < 16 * p.splits; i += kAttnThreads) wts[i] = 0.f;
  __syncthreads();
  if (tid < 16) {
    const int r = tid;
    const int qr = qrow0 + r / Hb, h = hblock * Hb + r % Hb;
    if (r / Hb < G && qr < p.rows && h < p.heads) {
      float M = -INFINITY;
      for (int s2 = 0; s2 < p.splits; ++s2)
        M = fmaxf(M, p.part_ml[((static_cast<size_t>(qr) * p.splits + s2) * p.heads + h) * 2]);
      float L = 0.f;
      if (p.sink) {
        const float sk = p.sink[h] * 1.4426950408889634f;
        M = fmaxf(M, sk);
        L = exp2f(sk - M);
      }
      for (int s2 = 0; s2 < p.splits; ++s2) {
        const size_t idx = (static_cast<size_t>(qr) * p.splits + s2) * p.heads + h;
        const float m = p.part_ml[idx * 2], l = p.part_ml[idx * 2 + 1];
        const float w = (m == -INFINITY || l == 0.f) ? 0.f : exp2f(m - M);
        wts[r * p.splits + s2] = w;
        L += l * w;
      }
      const float inv = L > 0.f ? 1.f / L : 0.f;
      for (int s2 = 0; s2 < p.splits; ++s2) wts[r * p.splits + s2] *= inv;
    }
  }
  __syncthreads();
  // every thread combines independent (row, 4-dim) items; the split loads are independent
  constexpr int kVecPerRow = DL / 4;
  for (int item = tid; item < 16 * kVecPerRow; item += kAttnThreads) {
    const int r = item / kVecPerRow, d = (item - r * kVecPerRow) * 4;
    const int qr = qrow0 + r / Hb, h = hblock * Hb + r % Hb;
    if (r / Hb >= G || qr >= p.rows || h >= p.heads) continue;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int s2 = 0; s2 < p.splits; ++s2) {
      const float w = wts[r * p.splits + s2];
      const float4 v = *reinterpret_cast<const float4*>(
          p.part_o + ((static_cast<size_t>(qr) * p.splits + s2) * p.heads + h) * DL + d);
      acc[0] += v.x * w; acc[1] += v.y * w; acc[2] += v.z * w; acc[3] += v.w * w;
    }
    __nv_bfloat16* o = p.out + qr * p.ldo + static_cast<long long>(h) * DL + d;
    *reinterpret_cast<uint32_t*>(o) = pack_bf16(acc[0], acc[1]);
    *reinterpret_cast<uint32_t*>(o + 2) = pack_bf16(acc[2], acc[3]);
  }
}

// merge split partials: grid (rows, heads), DL/4 threads each handling 4 dims
template <int DL>
__global__ void mla_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                 const float* __restrict__ sink, __nv_bfloat16* __restrict__ out,
                                 long long ldo, int rows, int heads, int splits) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, h = blockIdx.y;
  if (r >= rows || h >= heads) return;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, part_ml[((static_cast<size_t>(r) * splits + s) * heads + h) * 2]);
  float sk = 0.f;
  if (sink) {
    sk = sink[h] * 1.4426950408889634f;
    M = fmaxf(M, sk);
  }
  const int d = threadIdx.x * 4;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float L = sink ? exp2f(sk - M) : 0.f;
  for (int s = 0; s < splits; ++s) {
    const size_t idx = (static_cast<size_t>(r) * splits + s) * heads + h;
    const float m = part_ml[idx * 2], l = part_ml[idx * 2 + 1];
    if (m == -INFINITY || l == 0.f) continue;
    const float w = exp2f(m - M);
    L += l * w;
    if (d < DL) {
      const float4 v = *reinterpret_cast<const float4*>(part_o + idx * DL + d);
      acc[0] += v.x * w; acc[1] += v.y * w; acc[2] += v.z * w; acc[3] += v.w * w;
    }
  }
  if (d < DL) {
    const float inv = L > 0.f ? 1.f / L : 0.f;
    __nv_bfloat16* o = out + r * ldo + static_cast<long long>(h) * DL + d;
    *reinterpret_cast<uint32_t*>(o) = pack_bf16(acc[0] * inv, acc[1] * inv);
    *reinterpret_cast<uint32_t*>(o + 2) = pack_bf16(acc[2] * inv, acc[3] * inv);
  }
}

template <int DL, int DR>
static int launch_attn(const AttnParams& p, cudaStream_t stream) {
  using S = AttnSmem<DL, DR>;
  auto kern = mla_attention_kernel<DL, DR>;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal) != cudaSuccess)
      return FB_ERR_LAUNCH;
    attr = true;
  }
  const int Hb = 16 / p.group_rows;
  dim3 grid((p.rows + p.group_rows - 1) / p.group_rows, p.splits, (p.heads + Hb - 1) / Hb);
  if (p.cluster_merge) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kAttnThreads);
    cfg.dynamicSmemBytes = S::kTotal;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = p.splits;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    if (cudaLaunchKernelEx(&cfg, kern, p) != cudaSuccess) return FB_ERR_LAUNCH;
    return cudaGetLastError() == cudaSuccess ? FB_OK : FB_ERR_LAUNCH;
  }
  launch_pdl(kern, dim3(grid), dim3(kAttnThreads), S::kTotal, stream, p);
  if (cudaGetLastError() != cudaSuccess) return FB_ERR_LAUNCH;
  if (p.splits > 1 && p.merge_ctr == nullptr) {
    dim3 mg(p.rows, p.heads);
    launch_pdl(mla_merge_kernel<DL>, dim3(mg), dim3(DL / 4), 0, stream, p.part_o, p.part_ml, p.sink, p.out, p.ldo, p.rows,
                                                   p.heads, p.splits);
    if (cudaGetLastError() != cudaSuccess) return FB_ERR_LAUNCH;
  }
  return FB_OK;
}

}  // namespace fb

using namespace fb;

extern "C" int fb_mla_attention(const FbAttnArgs* a, void* stream_) {
  if (!a || !a->q || !a->kv || !a->out) return FB_ERR_SHAPE;
  if (a->selection) {
    if (a->sel_width <= 0 || a->group_rows != 1) return FB_ERR_SHAPE;
  } else {
    if (!a->block_table || !a->row_seq || !a->row_pos) return FB_ERR_SHAPE;
    if (a->page_size <= 0 || a->max_blocks <= 0) return FB_ERR_SHAPE;
  }
  if (a->rows <= 0 || a->heads <= 0) return FB_ERR_SHAPE;
  if (a->group_rows != 1 && a->group_rows != 2 && a->group_rows != 4 && a->group_rows != 8 &&
      a->group_rows != 16)
    return FB_ERR_SHAPE;
  if (a->splits < 1 || a->split_tokens <= 0 || a->split_tokens % kKvTile != 0) return FB_ERR_SHAPE;
  // splits > 1 without scratch: the splits of a query tile form one cluster and merge on chip
  const bool cluster_merge = a->splits > 1 && !a->part_o;
  if (cluster_merge && a->splits != 2 && a->splits != 4 && a->splits != 8) return FB_ERR_SHAPE;
  if (a->splits > 1 && !cluster_merge && !a->part_ml) return FB_ERR_SHAPE;
  if ((a->ldq % 8) != 0 || (a->ldo % 2) != 0) return FB_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(a->kv) & 15) || (reinterpret_cast<uintptr_t>(a->q) & 15)) return FB_ERR_ALIGN;
  AttnParams p{};
  p.q = static_cast<const __nv_bfloat16*>(a->q);
  p.ldq = a->ldq;
  p.kv = static_cast<const __nv_bfloat16*>(a->kv);
  p.pool_rows = a->pool_rows;
  p.block_table = a->block_table;
  p.max_blocks = a->max_blocks;
  p.page_size = a->page_size;
  p.num_seqs = a->num_seqs;
  p.row_seq = a->row_seq;
  p.row_pos = a->row_pos;
  p.rows = a->rows;
  p.heads = a->heads;
  p.group_rows = a->group_rows;
  p.splits = a->splits;
  p.split_tokens = a->split_tokens;
  p.scale_log2 = a->softmax_scale * 1.4426950408889634f;
  p.sink = a->sink;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.ldo = a->ldo;
  p.part_o = a->part_o;
  p.part_ml = a->part_ml;
  p.merge_ctr = static_cast<unsigned int*>(a->merge_ctr);
  p.cluster_merge = cluster_merge ? 1 : 0;
  p.selection = a->selection;
  p.sel_width = a->sel_width;
  p.status = static_cast<DeviceStatus*>(a->status);
  p.trace = static_cast<unsigned long long*>(a->trace);
  p.prefetch_old = (a->decode_only && a->group_rows == 1 && a->selection == nullptr) ? 1 : 0;
  {
    static const bool enabled = [] {
      const char* e = getenv("FERRULE_W_EVICT_FIRST");
      return !(e && e[0] == '0');
    }();
    p.kv_stream = enabled && a->rows <= 128 && a->selection == nullptr;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a->kv_lora == 512 && a->rope_dim == 64) return launch_attn<512, 64>(p, stream);
  if (a->kv_lora == 64 && a->rope_dim == 16) return launch_attn<64, 16>(p, stream);
  if (a->kv_lora == 128 && a->rope_dim == 32) return launch_attn<128, 32>(p, stream);
  // single shared K = V head (DeepSeek-V4): scores and values both span the whole row
  if (a->kv_lora == 512 && a->rope_dim == 0) return launch_attn<512, 0>(p, stream);
  if (a->kv_lora == 64 && a->rope_dim == 0) return launch_attn<64, 0>(p, stream);
  return FB_ERR_SHAPE;
}
