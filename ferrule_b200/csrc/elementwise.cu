// Bandwidth-bound small operators of the decode / prefill step, each fused as far as
// its neighbours allow (sm_100a):
//
//   fb_embedding        token ids -> bf16 rows
//   fb_add_rmsnorm      (residual add) + RMSNorm, bf16 in/out, fp32 math
//   fb_mla_prep         per token: RMSNorm(latent kv) + RoPE(k_rope) -> paged KV append,
//                       RoPE(q_rope) per head -> query buffer
//   fb_router_topk      softmax / sigmoid(+bias, group-limited) / sqrt-softplus(+bias) / hash
//                       scoring + stable top-k + weight normalisation, one warp per token
//   fb_moe_plan         count -> scan -> scatter of routes into expert-major order plus the
//                       row-tile table the grouped GEMM walks (device side, no host sync)
//   fb_gather_rows      expert-major activation gather
//   fb_moe_reduce       fixed-order sum of a token's route rows (+ shared expert, + residual)
//   fb_argmax           greedy token (ties -> lower id) over fp32 logits
//   fb_topk_logits      top-k (k <= 64) logits + ids, sorted logit-desc / id-asc
//   fb_copy_pages       copy-on-write page copy for the paged KV pool
//
// Counterparts in the reference: portable/entrypoints.cu embedding_kernel :631-649,
// norm_kernel :651-712, rope_kernel :714-768, router_kernel :793-884,
// expert_group_route_plan_kernel :1382-1513, moe_kernel :1515-1612, data_kernel :478-629
// (crates/ferrule-backend/native/cuda/implementations/portable/entrypoints.cu).
#include "codec.cuh"
#include "common.cuh"
#include "ferrule_b200.h"
#include "launch.cuh"

namespace fb {

// ---------------------------------------------------------------------------------
// embedding
// ---------------------------------------------------------------------------------
__global__ void embedding_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                 __nv_bfloat16* __restrict__ out, int rows, int dim, int vocab,
                                 DeviceStatus* st) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  if (r >= rows) return;
  int id = ids[r];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) report_status(st, kStatusBadIndex, 0x10, r, id);
    id = 0;
  }
  const uint4* src = reinterpret_cast<const uint4*>(table + static_cast<size_t>(id) * dim);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * dim);
  for (int i = threadIdx.x; i < dim / 8; i += blockDim.x) dst[i] = src[i];
}

// ---------------------------------------------------------------------------------
// (add +) RMSNorm.  One CTA per row, 256 threads, 8 bf16 per thread per step.
// ---------------------------------------------------------------------------------
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < (blockDim.x >> 5)) ? red[l] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

__global__ void __launch_bounds__(256)
add_rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                   const __nv_bfloat16* __restrict__ delta, long long ldd,
                   const __nv_bfloat16* __restrict__ weight, __nv_bfloat16* __restrict__ res_out,
                   long long ldr, __nv_bfloat16* __restrict__ norm_out, long long ldn, int rows,
                   int dim, float eps, uint8_t* __restrict__ q_out, long long ldq,
                   uint8_t* __restrict__ q_scale, long long lds, int q_block) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[8];
  extern __shared__ float row[];  // dim floats
  const int r = blockIdx.x;
  if (r >= rows) return;
  const __nv_bfloat16* xr = x + r * ldx;
  const __nv_bfloat16* dr = delta ? delta + r * ldd : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < dim; i += blockDim.x * 8) {
    uint4 a = *reinterpret_cast<const uint4*>(xr + i);
    const __nv_bfloat16* ap = reinterpret_cast<const __nv_bfloat16*>(&a);
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __bfloat162float(ap[j]);
    if (dr) {
      uint4 d = *reinterpret_cast<const uint4*>(dr + i);
      const __nv_bfloat16* dp = reinterpret_cast<const __nv_bfloat16*>(&d);
      // the residual stream is kept in bf16: round the sum before it is normalised
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = bf16_round(v[j] + __bfloat162float(dp[j]));
      if (res_out) {
        __nv_bfloat16 o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16_rn(v[j]);
        *reinterpret_cast<uint4*>(res_out + r * ldr + i) = *reinterpret_cast<uint4*>(o);
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      row[i + j] = v[j];
      ss += v[j] * v[j];
    }
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / dim + eps);
  if (norm_out == nullptr) return;
  for (int i = threadIdx.x * 8; i < dim; i += blockDim.x * 8) {
    uint4 wv = *reinterpret_cast<const uint4*>(weight + i);
    const __nv_bfloat16* wp = reinterpret_cast<const __nv_bfloat16*>(&wv);
    __nv_bfloat16 o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16_rn(row[i + j] * inv * __bfloat162float(wp[j]));
    *reinterpret_cast<uint4*>(norm_out + r * ldn + i) = *reinterpret_cast<uint4*>(o);
    if (q_out != nullptr) {
      // the consumer is a block-scaled GEMM: the codes and scales of the normalised row, exactly what the row
      // quantiser would make of norm_out.  A scale block is 128 elements (16 lanes x 8) or 32 (4 lanes x 8);
      // dim % 128 == 0, so the lanes of a block always run the same iterations.
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(__bfloat162float(o[j])));
      const int glanes = q_block / 8;
      const uint32_t grp = (glanes == 16 ? 0xffffu : 0xfu) << (threadIdx.x & 31 & ~(glanes - 1));
      for (int d = glanes / 2; d >= 1; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(grp, amax, d));
      const uint8_t sb = fp8_block_scale(amax);
      const float sinv = 1.f / e8m0_to_float(sb);
      uint8_t c[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) c[j] = to_e4m3(__bfloat162float(o[j]) * sinv);
      *reinterpret_cast<uint2*>(q_out + r * ldq + i) = *reinterpret_cast<uint2*>(c);
      if ((threadIdx.x & (glanes - 1)) == 0) q_scale[r * lds + i / q_block] = sb;
    }
  }
}

// ---------------------------------------------------------------------------------
// MLA prep: latent-KV norm + RoPE + paged append, and query RoPE.
//   q row   : heads x [ nope (q_head_dim - rope_dim) | rope (rope_dim) ]
//   ckv row : [ c_kv (kv_lora) | k_rope (rope_dim) ]
//   q_out row     : per head [ latent slot (kv_lora, filled later by the absorb GEMM) | rope ]
// cos/sin tables are [max_pos, rope_dim/2] fp32 (any frequency scaling baked in).
// Rotation acts on interleaved pairs (x[2i], x[2i+1]).
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
mla_prep_kernel(const __nv_bfloat16* q, long long ldq, int q_head_dim,   // q may alias q_out (rotation in place)
                const __nv_bfloat16* __restrict__ ckv_in, long long ldckv, int heads, int kv_lora,
                int rope_dim,
                const __nv_bfloat16* __restrict__ kv_norm_w, float eps,
                const float* __restrict__ cos_t, const float* __restrict__ sin_t, int max_pos,
                const int* __restrict__ positions, const long long* __restrict__ write_slot,
                __nv_bfloat16* __restrict__ kv_pool, long long pool_rows,
                __nv_bfloat16* q_out, long long ldq_out, int rows, DeviceStatus* st) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[8];
  const int r = blockIdx.x;
  if (r >= rows) return;
  int pos = positions[r];
  if (pos < 0 || pos >= max_pos) {
    if (threadIdx.x == 0) report_status(st, kStatusBadIndex, 0x20, r, pos);
    pos = 0;
  }
  const int half = rope_dim / 2;
  const float* cr = cos_t + static_cast<size_t>(pos) * half;
  const float* sr = sin_t + static_cast<size_t>(pos) * half;

  // query rope
  const int nope = q_head_dim - rope_dim;
  for (int i = threadIdx.x; i < heads * half; i += blockDim.x) {
    const int h = i / half, p = i - h * half;
    const __nv_bfloat16* qh = q + r * ldq + h * q_head_dim + nope;
    const float a = __bfloat162float(qh[2 * p]), b = __bfloat162float(qh[2 * p + 1]);
    const float c = cr[p], s = sr[p];
    __nv_bfloat16* o = q_out + r * ldq_out + static_cast<long long>(h) * (kv_lora + rope_dim) + kv_lora;
    o[2 * p] = __float2bfloat16_rn(a * c - b * s);
    o[2 * p + 1] = __float2bfloat16_rn(a * s + b * c);
  }

  // latent kv: RMSNorm then append; k_rope: rotate then append
  const long long slot = write_slot[r];
  const bool slot_ok = slot >= 0 && slot < pool_rows;
  if (!slot_ok && slot != -1 && threadIdx.x == 0)
    report_status(st, kStatusBadIndex, 0x21, r, static_cast<uint32_t>(slot));
  const __nv_bfloat16* ckv = ckv_in + r * ldckv;
  float ss = 0.f;
  for (int i = threadIdx.x; i < kv_lora; i += blockDim.x) {
    const float v = __bfloat162float(ckv[i]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / kv_lora + eps);
  if (!slot_ok) return;
  __nv_bfloat16* dst = kv_pool + slot * (kv_lora + rope_dim);
  for (int i = threadIdx.x; i < kv_lora; i += blockDim.x)
    dst[i] = __float2bfloat16_rn(__bfloat162float(ckv[i]) * inv * __bfloat162float(kv_norm_w[i]));
  for (int p = threadIdx.x; p < half; p += blockDim.x) {
    const float a = __bfloat162float(ckv[kv_lora + 2 * p]), b = __bfloat162float(ckv[kv_lora + 2 * p + 1]);
    const float c = cr[p], s = sr[p];
    dst[kv_lora + 2 * p] = __float2bfloat16_rn(a * c - b * s);
    dst[kv_lora + 2 * p + 1] = __float2bfloat16_rn(a * s + b * c);
  }
}

// ---------------------------------------------------------------------------------
// router: one warp per token, experts <= 256 (8 per lane)
// ---------------------------------------------------------------------------------
enum { kScoreSoftmax = 0, kScoreSigmoid = 1, kScoreSqrtSoftplus = 2 };

// One warp routes one token.  `lr` points at the token's `experts` logits (global or shared).
__device__ __forceinline__ void route_one_token(const float* lr, int warp, int lane,
                                                const float* __restrict__ bias,
                                                const long long* __restrict__ hash_table,
                                                const int* __restrict__ token_ids, int experts, int topk,
                                                int score_fn, int n_groups, int topk_groups, int normalize,
                                                float route_scale, int* __restrict__ out_idx,
                                                float* __restrict__ out_w) {
  constexpr int kPer = 8;
  float score[kPer];   // the value weights are taken from
  float select[kPer];  // the value top-k is taken on (score + bias)
  // scores
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < kPer; ++j) {
    const int e = lane + 32 * j;
    score[j] = e < experts ? lr[e] : -INFINITY;
    mx = fmaxf(mx, score[j]);
  }
  if (score_fn == kScoreSoftmax) {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int e = lane + 32 * j;
      score[j] = e < experts ? __expf(score[j] - mx) : 0.f;
      sum += score[j];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int j = 0; j < kPer; ++j) score[j] /= sum;
  } else if (score_fn == kScoreSigmoid) {
#pragma unroll
    for (int j = 0; j < kPer; ++j) score[j] = 1.f / (1.f + __expf(-score[j]));
  } else {
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const float x = score[j];
      const float sp = x > 20.f ? x : log1pf(__expf(x));
      score[j] = sqrtf(sp);
    }
  }
#pragma unroll
  for (int j = 0; j < kPer; ++j) {
    const int e = lane + 32 * j;
    select[j] = e < experts ? score[j] + (bias ? bias[e] : 0.f) : -INFINITY;
  }

  int* oi = out_idx + static_cast<size_t>(warp) * topk;
  float* ow = out_w + static_cast<size_t>(warp) * topk;

  if (hash_table != nullptr) {
    // hash routing: experts come from the table row of the token id; weights from the scores
    const long long* hr = hash_table + static_cast<size_t>(token_ids[warp]) * topk;
    float wsum = 0.f;
    float mine = 0.f;
    for (int k = 0; k < topk; ++k) {
      int e = static_cast<int>(hr[k]);
      if (e < 0 || e >= experts) e = 0;
      float val = 0.f;
#pragma unroll
      for (int j = 0; j < kPer; ++j)
        if (j == (e >> 5)) val = __shfl_sync(0xffffffffu, score[j], e & 31);
      wsum += val;
      if (lane == k) { mine = val; oi[k] = e; }
    }
    if (lane < topk) ow[lane] = (normalize ? mine / wsum : mine) * route_scale;
    return;
  }

  // group-limited selection (sigmoid family): keep the topk_groups groups with the largest
  // sum of their two best selection values, mask the rest.
  if (n_groups > 1 && topk_groups < n_groups) {
    const int per_group = experts / n_groups;
    float gscore_mine = -INFINITY;  // lane g holds group g's score
    for (int g = 0; g < n_groups; ++g) {
      float b1 = -INFINITY, b2 = -INFINITY;
#pragma unroll
      for (int j = 0; j < kPer; ++j) {
        const int e = lane + 32 * j;
        if (e < experts && e / per_group == g) {
          const float v = select[j];
          if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) { b2 = v; }
        }
      }
      // merge (b1, b2) across lanes
      for (int o = 16; o > 0; o >>= 1) {
        const float o1 = __shfl_xor_sync(0xffffffffu, b1, o), o2 = __shfl_xor_sync(0xffffffffu, b2, o);
        const float n1 = fmaxf(b1, o1);
        const float n2 = fmaxf(fminf(b1, o1), fmaxf(b2, o2));
        b1 = n1; b2 = n2;
      }
      if (lane == g) gscore_mine = b1 + b2;
    }
    // pick topk_groups groups (ties -> lower group id)
    uint32_t keep = 0;
    for (int it = 0; it < topk_groups; ++it) {
      float v = (lane < n_groups && !((keep >> lane) & 1u)) ? gscore_mine : -INFINITY;
      int idx = lane;
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oidx = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oidx < idx)) { v = ov; idx = oidx; }
      }
      keep |= 1u << idx;
    }
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int e = lane + 32 * j;
      if (e < experts && !((keep >> (e / per_group)) & 1u)) select[j] = -INFINITY;
    }
  }

  // stable top-k: largest selection value, ties -> lower expert id
  float wsum = 0.f;
  float mine = 0.f;
  for (int k = 0; k < topk; ++k) {
    float v = -INFINITY;
    int idx = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int e = lane + 32 * j;
      if (e < experts && (select[j] > v || (select[j] == v && e < idx))) { v = select[j]; idx = e; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oidx = __shfl_xor_sync(0xffffffffu, idx, o);
      if (ov > v || (ov == v && oidx < idx)) { v = ov; idx = oidx; }
    }
    if (idx == 0x7fffffff) idx = 0;
    float val = 0.f;
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const float cand = __shfl_sync(0xffffffffu, score[j], idx & 31);
      if (j == (idx >> 5)) val = cand;
      if (j == (idx >> 5) && lane == (idx & 31)) select[j] = -INFINITY;
    }
    wsum += val;
    if (lane == k) { mine = val; oi[k] = idx; }
  }
  if (lane < topk) ow[lane] = (normalize ? mine / (wsum + 1e-20f) : mine) * route_scale;
}

__global__ void __launch_bounds__(128)
router_topk_kernel(const float* __restrict__ logits, long long ldl, const float* __restrict__ bias,
                   const long long* __restrict__ hash_table, const int* __restrict__ token_ids,
                   int rows, int experts, int topk, int score_fn, int n_groups, int topk_groups,
                   int normalize, float route_scale, int* __restrict__ out_idx,
                   float* __restrict__ out_w) {
  pdl_launch_dependents();
  pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= rows) return;
  route_one_token(logits + warp * ldl, warp, lane, bias, hash_table, token_ids, experts, topk, score_fn,
                  n_groups, topk_groups, normalize, route_scale, out_idx, out_w);
}

// ---------------------------------------------------------------------------------
// MoE plan: single CTA (routes are at most tokens * topk; the kernel is latency-bound)
//   topk_idx[route] in [0, experts) ; local experts are [e_lo, e_hi)
//   outputs (expert-major position p):
//     src_token[p], dst_row[p] = token * dst_slots + slot (route id when dst_slots == topk),
//     row_scale[p] = weight
//     tile table for row tiles of `ntok` rows: tile_group (local expert id), row0, rows
//     counts[local experts], meta = {num_tiles, num_rows}
// ---------------------------------------------------------------------------------
struct PlanOut {
  int* src_token;
  int* dst_row;
  float* row_scale;
  int* tile_group;
  int* tile_row0;
  int* tile_rows;
  int max_tiles;
  int* counts;
  int* meta;
};

// Executed by one whole CTA (any block size that is a multiple of 32).
__device__ __forceinline__ void moe_plan_body(const int* topk_idx, const float* topk_w, int routes,
                                              int topk, int e_lo, int e_hi, int ntok, int dst_slots,
                                              const PlanOut& o, DeviceStatus* st) {
  int* const src_token = o.src_token;
  int* const dst_row = o.dst_row;
  float* const row_scale = o.row_scale;
  int* const tile_group = o.tile_group;
  int* const tile_row0 = o.tile_row0;
  int* const tile_rows = o.tile_rows;
  const int max_tiles = o.max_tiles;
  int* const counts = o.counts;
  int* const meta = o.meta;
  __shared__ int cnt[256];
  __shared__ int off[257];
  __shared__ int s_idx[2048];   // decode-sized route lists are walked from shared memory
  __shared__ float s_w[2048];
  const bool staged = routes <= 2048;
  const int local = e_hi - e_lo;
  for (int i = threadIdx.x; i < 256; i += blockDim.x) cnt[i] = 0;
  __syncthreads();
  for (int r = threadIdx.x; r < routes; r += blockDim.x) {
    const int e = topk_idx[r];
    if (staged) {
      s_idx[r] = e;
      s_w[r] = topk_w ? topk_w[r] : 1.f;
    }
    if (e >= e_lo && e < e_hi) atomicAdd(&cnt[e - e_lo], 1);
  }
  __syncthreads();
  // Exclusive scans over experts (row offsets and tile offsets) by one warp: lane l owns experts
  // 8l .. 8l+7, so a serial walk over all experts (slow on one thread) is avoided.
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int c[8], rows_sum = 0, tiles_sum = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = lane * 8 + j;
      c[j] = e < local ? cnt[e] : 0;
      rows_sum += c[j];
      tiles_sum += (c[j] + ntok - 1) / ntok;
    }
    int row_off = rows_sum, tile_off = tiles_sum;       // inclusive warp scans
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int r = __shfl_up_sync(0xffffffffu, row_off, o);
      const int t = __shfl_up_sync(0xffffffffu, tile_off, o);
      if (lane >= o) { row_off += r; tile_off += t; }
    }
    const int total_rows = __shfl_sync(0xffffffffu, row_off, 31);
    int total_tiles = __shfl_sync(0xffffffffu, tile_off, 31);
    row_off -= rows_sum;
    tile_off -= tiles_sum;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = lane * 8 + j;
      if (e < local) {
        off[e] = row_off;
        counts[e] = c[j];
        for (int r0 = 0; r0 < c[j]; r0 += ntok) {
          if (tile_off < max_tiles) {
            tile_group[tile_off] = e;
            tile_row0[tile_off] = row_off + r0;
            tile_rows[tile_off] = min(ntok, c[j] - r0);
          }
          ++tile_off;
        }
        row_off += c[j];
      }
    }
    if (lane == 0) {
      off[local] = total_rows;
      if (total_tiles > max_tiles) {
        report_status(st, kStatusBadShape, 0x30, total_tiles, max_tiles);
        total_tiles = max_tiles;
      }
      meta[0] = total_tiles;
      meta[1] = total_rows;
    }
  }
  __syncthreads();
  // Placement keeps the routes of one expert in ascending route order (bit-stable buffers
  // from run to run): each warp walks all routes for its experts and ranks hits by ballot.
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int e = warp; e < local; e += nwarps) {
    int base = off[e];
    for (int r0 = 0; r0 < routes; r0 += 32) {
      const int r = r0 + lane;
      const bool hit = r < routes && (staged ? s_idx[r] : topk_idx[r]) == e + e_lo;
      const uint32_t mask = __ballot_sync(0xffffffffu, hit);
      if (hit) {
        const int p = base + __popc(mask & ((1u << lane) - 1u));
        src_token[p] = r / topk;
        dst_row[p] = (r / topk) * dst_slots + (r - (r / topk) * topk);
        row_scale[p] = staged ? s_w[r] : (topk_w ? topk_w[r] : 1.f);
      }
      base += __popc(mask);
    }
  }
}

__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ topk_idx, const float* __restrict__ topk_w, int routes,
                int topk, int e_lo, int e_hi, int ntok, int dst_slots, PlanOut o, DeviceStatus* st) {
  pdl_launch_dependents();
  pdl_wait();
  moe_plan_body(topk_idx, topk_w, routes, topk, e_lo, e_hi, ntok, dst_slots, o, st);
}

// Prefill-sized route lists: one CTA per local expert.  Every CTA counts all experts (cheap, coalesced),
// derives the row / tile offsets with the same warp scan as above, CTA 0 writes the tile table, and CTA e
// places expert e's routes in ascending route order with a block-wide ordered scan (1024 routes per step).
__global__ void __launch_bounds__(1024)
moe_plan_wide_kernel(const int* __restrict__ topk_idx, const float* __restrict__ topk_w, int routes, int topk,
                     int e_lo, int e_hi, int ntok, int dst_slots, PlanOut o, DeviceStatus* st) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int cnt[256];
  __shared__ int off[257];
  __shared__ int warp_tot[32];
  __shared__ int s_base;
  const int local = e_hi - e_lo;
  const int me = blockIdx.x;
  for (int i = threadIdx.x; i < 256; i += blockDim.x) cnt[i] = 0;
  __syncthreads();
  for (int r = threadIdx.x; r < routes; r += blockDim.x) {
    const int e = topk_idx[r];
    if (e >= e_lo && e < e_hi) atomicAdd(&cnt[e - e_lo], 1);
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int c[8], rows_sum = 0, tiles_sum = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = lane * 8 + j;
      c[j] = e < local ? cnt[e] : 0;
      rows_sum += c[j];
      tiles_sum += (c[j] + ntok - 1) / ntok;
    }
    int row_off = rows_sum, tile_off = tiles_sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int r = __shfl_up_sync(0xffffffffu, row_off, d);
      const int t = __shfl_up_sync(0xffffffffu, tile_off, d);
      if (lane >= d) { row_off += r; tile_off += t; }
    }
    const int total_rows = __shfl_sync(0xffffffffu, row_off, 31);
    int total_tiles = __shfl_sync(0xffffffffu, tile_off, 31);
    row_off -= rows_sum;
    tile_off -= tiles_sum;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = lane * 8 + j;
      if (e < local) {
        off[e] = row_off;
        if (me == 0) {
          o.counts[e] = c[j];
          for (int r0 = 0; r0 < c[j]; r0 += ntok) {
            if (tile_off < o.max_tiles) {
              o.tile_group[tile_off] = e;
              o.tile_row0[tile_off] = row_off + r0;
              o.tile_rows[tile_off] = min(ntok, c[j] - r0);
            }
            ++tile_off;
          }
        }
        row_off += c[j];
      }
    }
    if (lane == 0 && me == 0) {
      if (total_tiles > o.max_tiles) {
        report_status(st, kStatusBadShape, 0x30, total_tiles, o.max_tiles);
        total_tiles = o.max_tiles;
      }
      o.meta[0] = total_tiles;
      o.meta[1] = total_rows;
    }
  }
  if (threadIdx.x == 0) s_base = 0;
  __syncthreads();
  if (me >= local) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int first = off[me];
  for (int r0 = 0; r0 < routes; r0 += blockDim.x) {
    const int r = r0 + threadIdx.x;
    const bool hit = r < routes && topk_idx[r] == me + e_lo;
    const uint32_t mask = __ballot_sync(0xffffffffu, hit);
    if (lane == 0) warp_tot[warp] = __popc(mask);
    __syncthreads();
    if (hit) {
      int before = s_base;
      for (int w = 0; w < warp; ++w) before += warp_tot[w];
      const int pidx = first + before + __popc(mask & ((1u << lane) - 1u));
      o.src_token[pidx] = r / topk;
      o.dst_row[pidx] = (r / topk) * dst_slots + (r - (r / topk) * topk);
      o.row_scale[pidx] = topk_w ? topk_w[r] : 1.f;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int tot = 0;
      for (int w = 0; w < 32; ++w) tot += warp_tot[w];
      s_base += tot;
    }
    __syncthreads();
  }
}

// A second row-tile table over an existing plan's expert-major rows with another tile height: the two grouped
// GEMMs of a layer need not share one (the plain store / scatter GEMM takes 256-row tiles, the SwiGLU GEMM keeps
// two accumulators and stops at 128).  One warp; expert counts come from the plan.
__global__ void __launch_bounds__(32)
moe_retile_kernel(const int* __restrict__ counts, int local, int ntok, int* __restrict__ tile_group,
                  int* __restrict__ tile_row0, int* __restrict__ tile_rows, int max_tiles, int* __restrict__ meta,
                  DeviceStatus* st) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x;
  int c[8], rows_sum = 0, tiles_sum = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int e = lane * 8 + j;
    c[j] = e < local ? counts[e] : 0;
    rows_sum += c[j];
    tiles_sum += (c[j] + ntok - 1) / ntok;
  }
  int row_off = rows_sum, tile_off = tiles_sum;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int r = __shfl_up_sync(0xffffffffu, row_off, d);
    const int t = __shfl_up_sync(0xffffffffu, tile_off, d);
    if (lane >= d) { row_off += r; tile_off += t; }
  }
  const int total_rows = __shfl_sync(0xffffffffu, row_off, 31);
  int total_tiles = __shfl_sync(0xffffffffu, tile_off, 31);
  row_off -= rows_sum;
  tile_off -= tiles_sum;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int e = lane * 8 + j;
    if (e < local) {
      for (int r0 = 0; r0 < c[j]; r0 += ntok) {
        if (tile_off < max_tiles) {
          tile_group[tile_off] = e;
          tile_row0[tile_off] = row_off + r0;
          tile_rows[tile_off] = min(ntok, c[j] - r0);
        }
        ++tile_off;
      }
      row_off += c[j];
    }
  }
  if (lane == 0) {
    if (total_tiles > max_tiles) {
      report_status(st, kStatusBadShape, 0x31, total_tiles, max_tiles);
      total_tiles = max_tiles;
    }
    meta[0] = total_tiles;
    meta[1] = total_rows;
  }
}

// ---------------------------------------------------------------------------------
// Fused router for decode-sized batches: router logits (x . W_e, fp32 accumulate) + scoring +
// top-k per token (one CTA per token), then the CTA that finishes last builds the MoE plan.
// One launch instead of three (logit GEMM, top-k, plan).
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
router_plan_fused_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                         const __nv_bfloat16* __restrict__ w, int hidden,
                         const float* __restrict__ bias, const long long* __restrict__ hash_table,
                         const int* __restrict__ token_ids, int rows, int experts, int topk, int score_fn,
                         int n_groups, int topk_groups, int normalize, float route_scale,
                         int* __restrict__ out_idx, float* __restrict__ out_w, int e_lo, int e_hi, int ntok,
                         int dst_slots, PlanOut o, unsigned int* done_ctr, DeviceStatus* st) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float xs[];            // hidden floats, then `experts` logits
  float* logits = xs + hidden;
  __shared__ int is_last;
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(x + t * ldx + i);
    const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
    for (int j = 0; j < 8; ++j) xs[i + j] = __bfloat162float(vp[j]);
  }
  __syncthreads();
  // two experts per warp pass and four 16-byte loads per expert in flight: the weight rows come from L2 and
  // a serial chain of dependent-looking loads is what this phase would otherwise wait on
  for (int e = warp; e < experts; e += 2 * nwarps) {
    const int e2 = e + nwarps;
    const bool two = e2 < experts;
    const __nv_bfloat16* wr = w + static_cast<size_t>(e) * hidden;
    const __nv_bfloat16* wr2 = w + static_cast<size_t>(two ? e2 : e) * hidden;
    float acc = 0.f, acc2 = 0.f;
#pragma unroll 4
    for (int i = lane * 8; i < hidden; i += 256) {
      const uint4 v = *reinterpret_cast<const uint4*>(wr + i);
      const uint4 v2 = *reinterpret_cast<const uint4*>(wr2 + i);
      const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(&v);
      const __nv_bfloat16* vp2 = reinterpret_cast<const __nv_bfloat16*>(&v2);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        acc = fmaf(__bfloat162float(vp[j]), xs[i + j], acc);
        acc2 = fmaf(__bfloat162float(vp2[j]), xs[i + j], acc2);
      }
    }
    acc = warp_sum(acc);
    acc2 = warp_sum(acc2);
    if (lane == 0) {
      logits[e] = acc;
      if (two) logits[e2] = acc2;
    }
  }
  __syncthreads();
  if (warp == 0)
    route_one_token(logits, t, lane, bias, hash_table, token_ids, experts, topk, score_fn, n_groups,
                    topk_groups, normalize, route_scale, out_idx, out_w);
  // last CTA to finish plans for everyone
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(done_ctr, 1u);
    is_last = done == gridDim.x - 1;
    if (is_last) *done_ctr = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  moe_plan_body(out_idx, out_w, rows * topk, topk, e_lo, e_hi, ntok, dst_slots, o, st);
}

// ---------------------------------------------------------------------------------
// Router for decode-sized batches with a static plan: every local expert owns `slot_rows` consecutive rows of the
// expert-major buffers (slot_rows >= number of tokens, so no expert can overflow) and one GEMM row tile.  One CTA
// per token: router logits, scoring, top-k, then each route of the token reserves the next free row of its expert
// (atomicAdd on the expert's counter, zeroed once per step for all layers), records (source token, destination
// row, weight) there and copies the activation row into the gather buffer.  No plan kernel, no gather kernel and
// no inter-CTA dependency: the GEMMs take the counters as their per-tile row counts.  The order of an expert's
// rows depends on the atomics; every row is computed independently, so the outputs do not.
// ---------------------------------------------------------------------------------
// Optional prologue of router_append_kernel: residual add + RMSNorm of the token's row (see the kernel).
struct NormPrologue {
  const __nv_bfloat16* delta;     // sublayer output added to the residual row (may be null)
  long long ldd;
  const __nv_bfloat16* norm_w;    // null: no prologue, `x` already holds the normalised rows
  __nv_bfloat16* res_out;         // bf16(x + delta), the new residual stream (may be null)
  long long ldr;
  __nv_bfloat16* norm_out;        // normalised rows for other consumers (shared experts); may be null
  long long ldn;
  float eps;
};

// Optional: the rows gathered for the experts are quantised rows (codes + scale bytes) instead of bf16 rows.
struct QuantRows {
  const uint8_t* q_src;     // [rows, hidden] codes of the (already quantised) normalised rows; null: copy bf16 rows
  long long ldq;
  const uint8_t* s_src;     // [rows, s_cols] scale bytes
  long long lds;
  uint8_t* xg_q;            // expert-major destination of the codes
  long long ldxgq;
  uint8_t* xg_s;            // expert-major destination of the scales
  long long ldxgs;
  int s_cols;
};

__global__ void __launch_bounds__(1024)
router_append_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ w,
                     int hidden, const float* __restrict__ bias, const long long* __restrict__ hash_table,
                     const int* __restrict__ token_ids, int rows, int experts, int topk, int score_fn, int n_groups,
                     int topk_groups, int normalize, float route_scale, int* __restrict__ out_idx,
                     float* __restrict__ out_w, int e_lo, int e_hi, int slot_rows, int dst_slots,
                     int* __restrict__ cnt, int* __restrict__ src_token, int* __restrict__ dst_row,
                     float* __restrict__ row_scale, __nv_bfloat16* __restrict__ xg, long long ldxg, DeviceStatus* st,
                     NormPrologue np, QuantRows qr) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float xs[];            // hidden floats, then `experts` logits, then (norm prologue) hidden bf16
  float* logits = xs + hidden;
  __shared__ int rlist[32];
  __shared__ float red[8];
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  // rows copied into the expert-major buffer come from here: the input row, or the prologue's normalised row
  const __nv_bfloat16* xrow = x + t * ldx;
  if (np.norm_w != nullptr) {
    // ---- residual add + RMSNorm of this token's row, with the element -> thread mapping, the rounding points and
    // the reduction order of add_rmsnorm_kernel (256 threads x 8 elements, 8 warp sums combined by one warp), so
    // the result is bit-equal to running that kernel first.  x = residual stream, np.delta = the sublayer output. ----
    __nv_bfloat16* xb = reinterpret_cast<__nv_bfloat16*>(logits + experts);
    const __nv_bfloat16* dr = np.delta ? np.delta + t * np.ldd : nullptr;
    float ss = 0.f;
    if (threadIdx.x < 256) {
      for (int i = threadIdx.x * 8; i < hidden; i += 256 * 8) {
        uint4 a = *reinterpret_cast<const uint4*>(xrow + i);
        const __nv_bfloat16* ap = reinterpret_cast<const __nv_bfloat16*>(&a);
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __bfloat162float(ap[j]);
        if (dr) {
          uint4 d = *reinterpret_cast<const uint4*>(dr + i);
          const __nv_bfloat16* dp = reinterpret_cast<const __nv_bfloat16*>(&d);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = bf16_round(v[j] + __bfloat162float(dp[j]));
          if (np.res_out) {
            __nv_bfloat16 o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16_rn(v[j]);
            *reinterpret_cast<uint4*>(np.res_out + t * np.ldr + i) = *reinterpret_cast<uint4*>(o);
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xs[i + j] = v[j];
          ss += v[j] * v[j];
        }
      }
      ss = warp_sum(ss);
      if (lane == 0) red[warp] = ss;
    }
    __syncthreads();
    float tot = lane < 8 ? red[lane] : 0.f;
    tot = warp_sum(tot);
    const float inv = rsqrtf(tot / hidden + np.eps);
    if (threadIdx.x < 256) {
      for (int i = threadIdx.x * 8; i < hidden; i += 256 * 8) {
        uint4 wv = *reinterpret_cast<const uint4*>(np.norm_w + i);
        const __nv_bfloat16* wp = reinterpret_cast<const __nv_bfloat16*>(&wv);
        __nv_bfloat16 o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          o[j] = __float2bfloat16_rn(xs[i + j] * inv * __bfloat162float(wp[j]));
          xs[i + j] = __bfloat162float(o[j]);
        }
        *reinterpret_cast<uint4*>(xb + i) = *reinterpret_cast<uint4*>(o);
        if (np.norm_out) *reinterpret_cast<uint4*>(np.norm_out + t * np.ldn + i) = *reinterpret_cast<uint4*>(o);
      }
    }
    xrow = xb;
  } else {
    for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
      const uint4 v = *reinterpret_cast<const uint4*>(xrow + i);
      const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
      for (int j = 0; j < 8; ++j) xs[i + j] = __bfloat162float(vp[j]);
    }
  }
  __syncthreads();
  for (int e = warp; e < experts; e += 2 * nwarps) {
    const int e2 = e + nwarps;
    const bool two = e2 < experts;
    const __nv_bfloat16* wr = w + static_cast<size_t>(e) * hidden;
    const __nv_bfloat16* wr2 = w + static_cast<size_t>(two ? e2 : e) * hidden;
    float acc = 0.f, acc2 = 0.f;
#pragma unroll 4
    for (int i = lane * 8; i < hidden; i += 256) {
      const uint4 v = *reinterpret_cast<const uint4*>(wr + i);
      const uint4 v2 = *reinterpret_cast<const uint4*>(wr2 + i);
      const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(&v);
      const __nv_bfloat16* vp2 = reinterpret_cast<const __nv_bfloat16*>(&v2);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        acc = fmaf(__bfloat162float(vp[j]), xs[i + j], acc);
        acc2 = fmaf(__bfloat162float(vp2[j]), xs[i + j], acc2);
      }
    }
    acc = warp_sum(acc);
    acc2 = warp_sum(acc2);
    if (lane == 0) {
      logits[e] = acc;
      if (two) logits[e2] = acc2;
    }
  }
  __syncthreads();
  if (warp == 0) {
    route_one_token(logits, t, lane, bias, hash_table, token_ids, experts, topk, score_fn, n_groups,
                    topk_groups, normalize, route_scale, out_idx, out_w);
    __syncwarp();
    if (lane < topk) {
      const int e = out_idx[t * topk + lane];
      int r = -1;
      if (e >= e_lo && e < e_hi) {
        const int pos = atomicAdd(&cnt[e - e_lo], 1);
        if (pos < slot_rows) {
          r = (e - e_lo) * slot_rows + pos;
          src_token[r] = t;
          dst_row[r] = t * dst_slots + lane;
          row_scale[r] = out_w[t * topk + lane];
        } else {
          report_status(st, kStatusBadShape, 0x50, e, pos);
        }
      }
      rlist[lane] = r;
    }
  }
  __syncthreads();
  if (qr.q_src != nullptr) {
    // quantised activations: copy the token's codes (16 bytes per thread) and scale bytes into every reserved row
    const int vq = hidden / 16;
    for (int i = threadIdx.x; i < topk * vq; i += blockDim.x) {
      const int s = i / vq, c = i - s * vq;
      const int r = rlist[s];
      if (r >= 0)
        *reinterpret_cast<uint4*>(qr.xg_q + r * qr.ldxgq + c * 16) =
            *reinterpret_cast<const uint4*>(qr.q_src + t * qr.ldq + c * 16);
    }
    for (int i = threadIdx.x; i < topk * qr.s_cols; i += blockDim.x) {
      const int s = i / qr.s_cols, c = i - s * qr.s_cols;
      const int r = rlist[s];
      if (r >= 0) qr.xg_s[r * qr.ldxgs + c] = qr.s_src[t * qr.lds + c];
    }
    return;
  }
  // copy the token's activation row into every reserved row (16 bytes per thread)
  const int vec = hidden / 8;
  for (int i = threadIdx.x; i < topk * vec; i += blockDim.x) {
    const int s = i / vec, c = i - s * vec;
    const int r = rlist[s];
    if (r >= 0)
      *reinterpret_cast<uint4*>(xg + r * ldxg + c * 8) = *reinterpret_cast<const uint4*>(xrow + c * 8);
  }
}

// Asynchronous L2 prefetch of a byte range (weights that a later kernel will stream): every thread issues
// bulk prefetch requests of 8 KB; nothing is written and nothing waits.
__global__ void __launch_bounds__(128)
l2_prefetch_kernel(const uint8_t* __restrict__ base, long long bytes) {
  constexpr long long kChunk = 8192;
  const long long n = (bytes + kChunk - 1) / kChunk;
  for (long long c = blockIdx.x * blockDim.x + threadIdx.x; c < n; c += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long off = c * kChunk;
    const unsigned int sz = static_cast<unsigned int>(min(kChunk, bytes - off) & ~15ll);
    if (sz) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base + off), "r"(sz) : "memory");
  }
}

__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                   const int* __restrict__ src_token, const int* __restrict__ meta,
                                   __nv_bfloat16* __restrict__ out, long long ldo, int cap_rows,
                                   int dim, int src_rows, DeviceStatus* st) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int valid = min(meta[1], cap_rows);
  if (r >= valid) return;
  int t = src_token[r];
  if (t < 0 || t >= src_rows) {
    if (threadIdx.x == 0) report_status(st, kStatusBadIndex, 0x40, r, t);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(x + t * ldx);
  uint4* dst = reinterpret_cast<uint4*>(out + r * ldo);
  for (int i = threadIdx.x; i < dim / 8; i += blockDim.x) dst[i] = src[i];
}

// out[t] = residual[t] + sum_{slot} route_out[t*slots + slot] (only slots whose expert is local,
// or every slot >= topk, which carry dense contributions such as the shared expert)
__global__ void __launch_bounds__(256)
moe_reduce_kernel(const __nv_bfloat16* __restrict__ route_out, int slots, int topk,
                  const int* __restrict__ topk_idx, int e_lo, int e_hi,
                  const __nv_bfloat16* __restrict__ extra, long long lde,
                  const __nv_bfloat16* __restrict__ residual, long long ldr, void* __restrict__ out,
                  long long ldo, int out_fp32, int rows, int dim,
                  const __nv_bfloat16* __restrict__ norm_w, __nv_bfloat16* __restrict__ norm_out, long long ldn,
                  float eps) {
  pdl_launch_dependents();
  pdl_wait();
  // optional RMSNorm of the result (the next layer's input norm), with the element -> thread mapping, the bf16
  // rounding of the normalised value and the reduction order of add_rmsnorm_kernel: bit-equal to running it after
  __shared__ float red[8];
  extern __shared__ float nrow[];  // dim floats when norm_out is set
  const int t = blockIdx.x;
  if (t >= rows) return;
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < dim; i += blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int s = 0; s < slots; ++s) {
      if (s < topk) {
        const int e = topk_idx[t * topk + s];
        if (e < e_lo || e >= e_hi) continue;
      }
      const uint4 v = *reinterpret_cast<const uint4*>(route_out + (static_cast<size_t>(t) * slots + s) * dim + i);
      const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(vp[j]);
    }
    if (extra) {
      const uint4 v = *reinterpret_cast<const uint4*>(extra + t * lde + i);
      const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(vp[j]);
    }
    if (residual) {
      const uint4 v = *reinterpret_cast<const uint4*>(residual + t * ldr + i);
      const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(vp[j]);
    }
    if (out_fp32) {
      float* o = reinterpret_cast<float*>(out) + t * ldo + i;
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = acc[j];
    } else {
      __nv_bfloat16 o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16_rn(acc[j]);
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(out) + t * ldo + i) =
          *reinterpret_cast<uint4*>(o);
      if (norm_out) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float v = __bfloat162float(o[j]);
          nrow[i + j] = v;
          ss += v * v;
        }
      }
    }
  }
  if (norm_out == nullptr) return;
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / dim + eps);
  for (int i = threadIdx.x * 8; i < dim; i += blockDim.x * 8) {
    uint4 wv = *reinterpret_cast<const uint4*>(norm_w + i);
    const __nv_bfloat16* wp = reinterpret_cast<const __nv_bfloat16*>(&wv);
    __nv_bfloat16 o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16_rn(nrow[i + j] * inv * __bfloat162float(wp[j]));
    *reinterpret_cast<uint4*>(norm_out + t * ldn + i) = *reinterpret_cast<uint4*>(o);
  }
}

// ---------------------------------------------------------------------------------
// greedy argmax / top-k over the vocabulary.  One CTA per row.
// ---------------------------------------------------------------------------------
__device__ __forceinline__ bool better(float v, int i, float ov, int oi) {
  return v > ov || (v == ov && i < oi);
}

__global__ void __launch_bounds__(1024)
argmax_kernel(const float* __restrict__ logits, long long ldl, int rows, int vocab,
              int* __restrict__ out_id, float* __restrict__ out_val) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sv[32];
  __shared__ int si[32];
  const int r = blockIdx.x;
  if (r >= rows) return;
  const float* lr = logits + r * ldl;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = lr[i];
    if (v == v && better(v, i, best, bi)) { best = v; bi = i; }  // NaN never wins
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { sv[w] = best; si[w] = bi; }
  __syncthreads();
  if (w == 0) {
    best = l < (blockDim.x >> 5) ? sv[l] : -INFINITY;
    bi = l < (blockDim.x >> 5) ? si[l] : 0x7fffffff;
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
    }
    if (l == 0) {
      out_id[r] = bi == 0x7fffffff ? -1 : bi;  // -1: no finite candidate
      if (out_val) out_val[r] = best;
    }
  }
}

// Two-level argmax: grid (chunks, rows).  Every CTA scans one slice of the vocabulary and writes
// its (value, id) candidate; the CTA that finishes last for a row reduces the candidates.
__global__ void __launch_bounds__(256)
argmax_chunked_kernel(const float* __restrict__ logits, long long ldl, int rows, int vocab, int chunk,
                      float* __restrict__ part_val, int* __restrict__ part_id,
                      unsigned int* __restrict__ row_ctr, int* __restrict__ out_id,
                      float* __restrict__ out_val) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sv[8];
  __shared__ int si[8];
  __shared__ int is_last;
  const int c = blockIdx.x, r = blockIdx.y, chunks = gridDim.x;
  const float* lr = logits + r * ldl;
  const int lo = c * chunk, hi = min(vocab, lo + chunk);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = lo + threadIdx.x * 4; i < hi; i += blockDim.x * 4) {
    if (i + 3 < hi) {
      const float4 v = *reinterpret_cast<const float4*>(lr + i);
      const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (vv[j] == vv[j] && better(vv[j], i + j, best, bi)) { best = vv[j]; bi = i + j; }
    } else {
      for (int j = i; j < hi; ++j) {
        const float v = lr[j];
        if (v == v && better(v, j, best, bi)) { best = v; bi = j; }
      }
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { sv[w] = best; si[w] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int k = 1; k < (blockDim.x >> 5); ++k)
      if (better(sv[k], si[k], best, bi)) { best = sv[k]; bi = si[k]; }
    part_val[r * chunks + c] = best;
    part_id[r * chunks + c] = bi;
    __threadfence();
    const unsigned int done = atomicAdd(row_ctr + r, 1u);
    is_last = done == static_cast<unsigned int>(chunks - 1);
    if (is_last) row_ctr[r] = 0;
  }
  __syncthreads();
  if (!is_last || w != 0) return;
  __threadfence();
  best = -INFINITY;
  bi = 0x7fffffff;
  for (int k = l; k < chunks; k += 32) {
    const float v = part_val[r * chunks + k];
    const int id = part_id[r * chunks + k];
    if (better(v, id, best, bi)) { best = v; bi = id; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
  }
  if (l == 0) {
    out_id[r] = bi == 0x7fffffff ? -1 : bi;
    if (out_val) out_val[r] = best;
  }
}

// top-k by k rounds of block argmax with a "already taken" threshold (k small, rows few)
__global__ void __launch_bounds__(1024)
topk_logits_kernel(const float* __restrict__ logits, long long ldl, int rows, int vocab, int k,
                   int* __restrict__ out_id, float* __restrict__ out_val) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float last_v;
  __shared__ int last_i;
  const int r = blockIdx.x;
  if (r >= rows) return;
  const float* lr = logits + r * ldl;
  if (threadIdx.x == 0) { last_v = INFINITY; last_i = -1; }
  __syncthreads();
  for (int it = 0; it < k; ++it) {
    const float lv = last_v;
    const int li = last_i;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float v = lr[i];
      // candidates strictly after (lv, li) in (logit desc, id asc) order
      const bool after = v < lv || (v == lv && i > li);
      if (v == v && after && better(v, i, best, bi)) { best = v; bi = i; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
    }
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) { sv[w] = best; si[w] = bi; }
    __syncthreads();
    if (w == 0) {
      best = l < (blockDim.x >> 5) ? sv[l] : -INFINITY;
      bi = l < (blockDim.x >> 5) ? si[l] : 0x7fffffff;
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
      }
      if (l == 0) {
        out_id[r * k + it] = bi == 0x7fffffff ? -1 : bi;
        out_val[r * k + it] = best;
        last_v = best;
        last_i = bi;
      }
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------
// Greedy-token feedback for back-to-back decode steps.  The token a step produced becomes the next step's
// input without a trip through the host (ids < 0, "no finite candidate", are fed back as token 0: the host
// ends such a sequence when it reads the result).  With `advance` the whole input row moves one position on:
// position and visible length + 1, and the KV write slot is looked up in the sequence's page list (-1 when
// the list has no page for the position: the row then writes nothing).
// ---------------------------------------------------------------------------------
__global__ void decode_advance_kernel(const int* __restrict__ next_id, int* __restrict__ token_ids,
                                      int* __restrict__ positions, int* __restrict__ row_pos,
                                      long long* __restrict__ write_slot, const int* __restrict__ row_seq,
                                      const int* __restrict__ block_table, int max_blocks, int page_size,
                                      int num_seqs, int rows, int vocab, int advance) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  int id = next_id[r];
  if (id < 0 || id >= vocab) id = 0;
  token_ids[r] = id;
  if (!advance) return;
  if (row_pos[r] < 0) return;                     // padding row of a graph bucket
  const int pos = positions[r] + 1;
  positions[r] = pos;
  row_pos[r] = pos;
  const int seq = row_seq[r];
  long long slot = -1;
  const int blk = pos / page_size;
  if (seq >= 0 && seq < num_seqs && blk < max_blocks) {
    const int page = block_table[static_cast<long long>(seq) * max_blocks + blk];
    if (page >= 0) slot = static_cast<long long>(page) * page_size + pos % page_size;
  }
  write_slot[r] = slot;
}

// ---------------------------------------------------------------------------------
// paged pool: copy whole pages (all layers) for copy-on-write.  pool is
// [layers, pages, page_elems]; pairs = (src_page, dst_page).
// ---------------------------------------------------------------------------------
__global__ void copy_pages_kernel(__nv_bfloat16* pool, long long layer_stride, long long page_elems,
                                  const int* __restrict__ pairs, int n_pairs, int n_pages, int layers,
                                  DeviceStatus* st) {
  pdl_launch_dependents();
  pdl_wait();
  const int pair = blockIdx.x, layer = blockIdx.y;
  if (pair >= n_pairs || layer >= layers) return;
  const int src = pairs[2 * pair], dst = pairs[2 * pair + 1];
  if (src < 0 || src >= n_pages || dst < 0 || dst >= n_pages) {
    if (threadIdx.x == 0) report_status(st, kStatusBadIndex, 0x50, src, dst);
    return;
  }
  const uint4* s = reinterpret_cast<const uint4*>(pool + layer * layer_stride + src * page_elems);
  uint4* d = reinterpret_cast<uint4*>(pool + layer * layer_stride + dst * page_elems);
  for (long long i = threadIdx.x; i < page_elems / 8; i += blockDim.x) d[i] = s[i];
}

}  // namespace fb

using namespace fb;

#define FB_CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? FB_OK : FB_ERR_LAUNCH)

extern "C" int fb_status_bytes(void) { return static_cast<int>(sizeof(DeviceStatus)); }

extern "C" int fb_embedding(const int* ids, const void* table, void* out, int rows, int dim,
                            int vocab, void* status, void* stream) {
  if (rows <= 0 || dim % 8 != 0) return FB_ERR_SHAPE;
  launch_pdl(embedding_kernel, dim3(rows), dim3(128), 0, static_cast<cudaStream_t>(stream), 
      ids, static_cast<const __nv_bfloat16*>(table), static_cast<__nv_bfloat16*>(out), rows, dim,
      vocab, static_cast<DeviceStatus*>(status));
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_add_rmsnorm(const void* x, long long ldx, const void* delta, long long ldd,
                              const void* weight, void* res_out, long long ldr, void* norm_out,
                              long long ldn, int rows, int dim, float eps, void* stream) {
  return fb_add_rmsnorm_q(x, ldx, delta, ldd, weight, res_out, ldr, norm_out, ldn, rows, dim, eps, nullptr, 0, nullptr, 0,
                          128, stream);
}

extern "C" int fb_add_rmsnorm_q(const void* x, long long ldx, const void* delta, long long ldd,
                                const void* weight, void* res_out, long long ldr, void* norm_out,
                                long long ldn, int rows, int dim, float eps, void* q_out, long long ldq,
                                void* q_scale, long long lds, int q_block, void* stream) {
  if (rows <= 0 || dim % 8 != 0 || dim > 16384) return FB_ERR_SHAPE;
  if ((ldx | ldd | ldr | ldn) % 8 != 0) return FB_ERR_ALIGN;
  if (q_out != nullptr && (!q_scale || !norm_out || dim % 128 != 0 || ldq % 8 != 0 || (q_block != 128 && q_block != 32) ||
                           (reinterpret_cast<uintptr_t>(q_out) & 7)))
    return FB_ERR_SHAPE;
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(add_rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536);
    attr = true;
  }
  launch_pdl(add_rmsnorm_kernel, dim3(rows), dim3(256), dim * sizeof(float), static_cast<cudaStream_t>(stream), 
      static_cast<const __nv_bfloat16*>(x), ldx, static_cast<const __nv_bfloat16*>(delta), ldd,
      static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(res_out), ldr,
      static_cast<__nv_bfloat16*>(norm_out), ldn, rows, dim, eps, static_cast<uint8_t*>(q_out), ldq,
      static_cast<uint8_t*>(q_scale), lds, q_block);
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_mla_prep(const void* q, long long ldq, int q_head_dim, const void* ckv,
                           long long ldckv, int heads, int kv_lora, int rope_dim,
                           const void* kv_norm_w, float eps,
                           const float* cos_t, const float* sin_t, int max_pos,
                           const int* positions, const long long* write_slot, void* kv_pool,
                           long long pool_rows, void* q_out, long long ldq_out, int rows,
                           void* status, void* stream) {
  if (rows <= 0 || rope_dim % 2 != 0 || heads <= 0) return FB_ERR_SHAPE;
  launch_pdl(mla_prep_kernel, dim3(rows), dim3(256), 0, static_cast<cudaStream_t>(stream), 
      static_cast<const __nv_bfloat16*>(q), ldq, q_head_dim,
      static_cast<const __nv_bfloat16*>(ckv), ldckv, heads, kv_lora, rope_dim, static_cast<const __nv_bfloat16*>(kv_norm_w), eps, cos_t, sin_t, max_pos, positions,
      write_slot, static_cast<__nv_bfloat16*>(kv_pool), pool_rows,
      static_cast<__nv_bfloat16*>(q_out), ldq_out, rows, static_cast<DeviceStatus*>(status));
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_router_topk(const float* logits, long long ldl, const float* bias,
                              const long long* hash_table, const int* token_ids, int rows,
                              int experts, int topk, int score_fn, int n_groups, int topk_groups,
                              int normalize, float route_scale, int* out_idx, float* out_w,
                              void* stream) {
  if (rows <= 0 || experts <= 0 || experts > 256 || topk <= 0 || topk > 32 || topk > experts)
    return FB_ERR_SHAPE;
  if (n_groups > 32 || (n_groups > 1 && experts % n_groups != 0)) return FB_ERR_SHAPE;
  const int blocks = (rows + 3) / 4;
  launch_pdl(router_topk_kernel, dim3(blocks), dim3(128), 0, static_cast<cudaStream_t>(stream), 
      logits, ldl, bias, hash_table, token_ids, rows, experts, topk, score_fn, n_groups,
      topk_groups, normalize, route_scale, out_idx, out_w);
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_moe_plan(const int* topk_idx, const float* topk_w, int routes, int topk, int e_lo,
                           int e_hi, int ntok, int dst_slots, int* src_token, int* dst_row, float* row_scale,
                           int* tile_group, int* tile_row0, int* tile_rows, int max_tiles,
                           int* counts, int* meta, void* status, void* stream) {
  if (routes <= 0 || topk <= 0 || e_hi <= e_lo || e_hi - e_lo > 256 || ntok <= 0) return FB_ERR_SHAPE;
  PlanOut o{src_token, dst_row, row_scale, tile_group, tile_row0, tile_rows, max_tiles, counts, meta};
  if (routes > 2048)
    launch_pdl(moe_plan_wide_kernel, dim3(e_hi - e_lo), dim3(1024), 0, static_cast<cudaStream_t>(stream),
        topk_idx, topk_w, routes, topk, e_lo, e_hi, ntok, dst_slots < topk ? topk : dst_slots, o,
        static_cast<DeviceStatus*>(status));
  else
    launch_pdl(moe_plan_kernel, dim3(1), dim3(1024), 0, static_cast<cudaStream_t>(stream),
        topk_idx, topk_w, routes, topk, e_lo, e_hi, ntok, dst_slots < topk ? topk : dst_slots, o,
        static_cast<DeviceStatus*>(status));
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_moe_retile(const int* counts, int local_experts, int ntok, int* tile_group, int* tile_row0,
                             int* tile_rows, int max_tiles, int* meta, void* status, void* stream) {
  if (!counts || !tile_group || !tile_row0 || !tile_rows || !meta) return FB_ERR_SHAPE;
  if (local_experts <= 0 || local_experts > 256 || ntok <= 0 || max_tiles <= 0) return FB_ERR_SHAPE;
  launch_pdl(moe_retile_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), counts, local_experts, ntok,
             tile_group, tile_row0, tile_rows, max_tiles, meta, static_cast<DeviceStatus*>(status));
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_router_plan_fused(const void* x, long long ldx, const void* w, int hidden,
                                    const float* bias, const long long* hash_table,
                                    const int* token_ids, int rows, int experts, int topk, int score_fn,
                                    int n_groups, int topk_groups, int normalize, float route_scale,
                                    int* out_idx, float* out_w, int e_lo, int e_hi, int ntok, int dst_slots,
                                    int* src_token, int* dst_row, float* row_scale, int* tile_group,
                                    int* tile_row0, int* tile_rows, int max_tiles, int* counts, int* meta,
                                    void* done_ctr, void* status, void* stream) {
  if (rows <= 0 || experts <= 0 || experts > 256 || topk <= 0 || topk > 32 || topk > experts)
    return FB_ERR_SHAPE;
  if (hidden % 256 != 0 || hidden > 8192 || (ldx % 8) != 0) return FB_ERR_SHAPE;
  if (n_groups > 32 || (n_groups > 1 && experts % n_groups != 0)) return FB_ERR_SHAPE;
  if (e_hi <= e_lo || e_hi - e_lo > 256 || ntok <= 0 || !done_ctr) return FB_ERR_SHAPE;
  PlanOut o{src_token, dst_row, row_scale, tile_group, tile_row0, tile_rows, max_tiles, counts, meta};
  const size_t smem = static_cast<size_t>(hidden + experts) * sizeof(float);
  launch_pdl(router_plan_fused_kernel, dim3(rows), dim3(1024), smem, static_cast<cudaStream_t>(stream), 
      static_cast<const __nv_bfloat16*>(x), ldx, static_cast<const __nv_bfloat16*>(w), hidden, bias,
      hash_table, token_ids, rows, experts, topk, score_fn, n_groups, topk_groups, normalize, route_scale,
      out_idx, out_w, e_lo, e_hi, ntok, dst_slots < topk ? topk : dst_slots, o,
      static_cast<unsigned int*>(done_ctr), static_cast<DeviceStatus*>(status));
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_router_append(const void* x, long long ldx, const void* w, int hidden, const float* bias,
                                const long long* hash_table, const int* token_ids, int rows, int experts, int topk,
                                int score_fn, int n_groups, int topk_groups, int normalize, float route_scale,
                                int* out_idx, float* out_w, int e_lo, int e_hi, int slot_rows, int dst_slots, int* cnt,
                                int* src_token, int* dst_row, float* row_scale, void* xg, long long ldxg,
                                void* status, void* stream) {
  return fb_norm_router_append(x, ldx, nullptr, 0, nullptr, nullptr, 0, nullptr, 0, 0.f, w, hidden, bias, hash_table,
                               token_ids, rows, experts, topk, score_fn, n_groups, topk_groups, normalize, route_scale,
                               out_idx, out_w, e_lo, e_hi, slot_rows, dst_slots, cnt, src_token, dst_row, row_scale,
                               xg, ldxg, status, stream);
}

extern "C" int fb_norm_router_append(const void* x, long long ldx, const void* delta, long long ldd,
                                     const void* norm_w, void* res_out, long long ldr, void* norm_out, long long ldn,
                                     float eps, const void* w, int hidden, const float* bias,
                                     const long long* hash_table, const int* token_ids, int rows, int experts,
                                     int topk, int score_fn, int n_groups, int topk_groups, int normalize,
                                     float route_scale, int* out_idx, float* out_w, int e_lo, int e_hi,
                                     int slot_rows, int dst_slots, int* cnt, int* src_token, int* dst_row,
                                     float* row_scale, void* xg, long long ldxg, void* status, void* stream) {
  return fb_router_append_q(x, ldx, delta, ldd, norm_w, res_out, ldr, norm_out, ldn, eps, w, hidden, bias, hash_table,
                            token_ids, rows, experts, topk, score_fn, n_groups, topk_groups, normalize, route_scale,
                            out_idx, out_w, e_lo, e_hi, slot_rows, dst_slots, cnt, src_token, dst_row, row_scale, xg, ldxg,
                            nullptr, 0, nullptr, 0, nullptr, 0, nullptr, 0, 0, status, stream);
}

extern "C" int fb_router_append_q(const void* x, long long ldx, const void* delta, long long ldd,
                                  const void* norm_w, void* res_out, long long ldr, void* norm_out, long long ldn,
                                  float eps, const void* w, int hidden, const float* bias,
                                  const long long* hash_table, const int* token_ids, int rows, int experts,
                                  int topk, int score_fn, int n_groups, int topk_groups, int normalize,
                                  float route_scale, int* out_idx, float* out_w, int e_lo, int e_hi,
                                  int slot_rows, int dst_slots, int* cnt, int* src_token, int* dst_row,
                                  float* row_scale, void* xg, long long ldxg, const void* q_src, long long ldq,
                                  const void* s_src, long long lds, void* xg_q, long long ldxgq, void* xg_s,
                                  long long ldxgs, int s_cols, void* status, void* stream) {
  if (rows <= 0 || experts <= 0 || experts > 256 || topk <= 0 || topk > 32 || topk > experts) return FB_ERR_SHAPE;
  if (hidden % 256 != 0 || hidden > 8192 || (ldx % 8) != 0 || (ldxg % 8) != 0) return FB_ERR_SHAPE;
  if (slot_rows < rows || e_hi <= e_lo || !cnt || !src_token || !dst_row || !row_scale) return FB_ERR_SHAPE;
  if (q_src == nullptr && !xg) return FB_ERR_SHAPE;
  if (q_src != nullptr && (!s_src || !xg_q || !xg_s || s_cols <= 0 || (ldq % 16) != 0 || (ldxgq % 16) != 0 ||
                           (reinterpret_cast<uintptr_t>(q_src) & 15) || (reinterpret_cast<uintptr_t>(xg_q) & 15)))
    return FB_ERR_SHAPE;
  const QuantRows qr{static_cast<const uint8_t*>(q_src), ldq, static_cast<const uint8_t*>(s_src), lds,
                     static_cast<uint8_t*>(xg_q), ldxgq, static_cast<uint8_t*>(xg_s), ldxgs, s_cols};
  if (norm_w != nullptr && ((ldd % 8) != 0 || (ldr % 8) != 0 || (ldn % 8) != 0 || (experts % 4) != 0))
    return FB_ERR_SHAPE;
  const NormPrologue np{static_cast<const __nv_bfloat16*>(delta), ldd, static_cast<const __nv_bfloat16*>(norm_w),
                        static_cast<__nv_bfloat16*>(res_out), ldr, static_cast<__nv_bfloat16*>(norm_out), ldn, eps};
  const size_t smem = (static_cast<size_t>(hidden) + experts) * sizeof(float) +
                      (norm_w ? static_cast<size_t>(hidden) * 2 : 0);
  static bool attr_done = false;
  if (!attr_done) {
    cudaFuncSetAttribute(router_append_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    attr_done = true;
  }
  launch_pdl(router_append_kernel, dim3(rows), dim3(1024), smem, static_cast<cudaStream_t>(stream),
             static_cast<const __nv_bfloat16*>(x), ldx, static_cast<const __nv_bfloat16*>(w), hidden, bias, hash_table,
             token_ids, rows, experts, topk, score_fn, n_groups, topk_groups, normalize, route_scale, out_idx, out_w,
             e_lo, e_hi, slot_rows, dst_slots, cnt, src_token, dst_row, row_scale, static_cast<__nv_bfloat16*>(xg), ldxg,
             static_cast<DeviceStatus*>(status), np, qr);
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_l2_prefetch(const void* ptr, long long bytes, void* stream) {
  if (!ptr || bytes <= 0 || (reinterpret_cast<uintptr_t>(ptr) & 15)) return FB_ERR_SHAPE;
  l2_prefetch_kernel<<<8, 128, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint8_t*>(ptr), bytes);
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_gather_rows(const void* x, long long ldx, const int* src_token, const int* meta,
                              void* out, long long ldo, int cap_rows, int dim, int src_rows,
                              void* status, void* stream) {
  if (cap_rows <= 0 || dim % 8 != 0) return FB_ERR_SHAPE;
  launch_pdl(gather_rows_kernel, dim3(cap_rows), dim3(128), 0, static_cast<cudaStream_t>(stream), 
      static_cast<const __nv_bfloat16*>(x), ldx, src_token, meta, static_cast<__nv_bfloat16*>(out),
      ldo, cap_rows, dim, src_rows, static_cast<DeviceStatus*>(status));
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_moe_reduce(const void* route_out, int slots, int topk, const int* topk_idx,
                             int e_lo, int e_hi, const void* extra, long long lde,
                             const void* residual, long long ldr, void* out, long long ldo,
                             int out_fp32, int rows, int dim, void* stream) {
  if (rows <= 0 || dim % 8 != 0 || slots < topk) return FB_ERR_SHAPE;
  launch_pdl(moe_reduce_kernel, dim3(rows), dim3(256), 0, static_cast<cudaStream_t>(stream), 
      static_cast<const __nv_bfloat16*>(route_out), slots, topk, topk_idx, e_lo, e_hi,
      static_cast<const __nv_bfloat16*>(extra), lde, static_cast<const __nv_bfloat16*>(residual),
      ldr, out, ldo, out_fp32, rows, dim, static_cast<const __nv_bfloat16*>(nullptr),
      static_cast<__nv_bfloat16*>(nullptr), 0LL, 0.f);
  return FB_CHECK_LAUNCH();
}

// fb_moe_reduce with the RMSNorm of the (bf16) result written to norm_out as well
extern "C" int fb_moe_reduce_norm(const void* route_out, int slots, int topk, const int* topk_idx,
                                  int e_lo, int e_hi, const void* residual, long long ldr, void* out, long long ldo,
                                  int rows, int dim, const void* norm_w, void* norm_out, long long ldn, float eps,
                                  void* stream) {
  if (rows <= 0 || dim % 8 != 0 || slots < topk || !norm_w || !norm_out || dim > 16384) return FB_ERR_SHAPE;
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(moe_reduce_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536);
    attr = true;
  }
  launch_pdl(moe_reduce_kernel, dim3(rows), dim3(256), dim * sizeof(float), static_cast<cudaStream_t>(stream),
      static_cast<const __nv_bfloat16*>(route_out), slots, topk, topk_idx, e_lo, e_hi,
      static_cast<const __nv_bfloat16*>(nullptr), 0LL, static_cast<const __nv_bfloat16*>(residual),
      ldr, out, ldo, 0, rows, dim, static_cast<const __nv_bfloat16*>(norm_w),
      static_cast<__nv_bfloat16*>(norm_out), ldn, eps);
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_argmax(const float* logits, long long ldl, int rows, int vocab, int* out_id,
                         float* out_val, void* stream) {
  if (rows <= 0 || vocab <= 0) return FB_ERR_SHAPE;
  launch_pdl(argmax_kernel, dim3(rows), dim3(1024), 0, static_cast<cudaStream_t>(stream), logits, ldl, rows, vocab,
                                                                      out_id, out_val);
  return FB_CHECK_LAUNCH();
}

// scratch: part_val [rows * chunks] floats, part_id [rows * chunks] ints, row_ctr [rows] zeroed once
extern "C" int fb_argmax_chunked(const float* logits, long long ldl, int rows, int vocab, int chunks,
                                 float* part_val, int* part_id, void* row_ctr, int* out_id,
                                 float* out_val, void* stream) {
  if (rows <= 0 || vocab <= 0 || chunks <= 0 || chunks > 1024 || !part_val || !part_id || !row_ctr)
    return FB_ERR_SHAPE;
  if ((ldl % 4) != 0 || (reinterpret_cast<uintptr_t>(logits) & 15)) return FB_ERR_ALIGN;
  const int chunk = ((vocab + chunks - 1) / chunks + 3) / 4 * 4;
  dim3 grid(chunks, rows);
  launch_pdl(argmax_chunked_kernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream), 
      logits, ldl, rows, vocab, chunk, part_val, part_id, static_cast<unsigned int*>(row_ctr), out_id,
      out_val);
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_topk_logits(const float* logits, long long ldl, int rows, int vocab, int k,
                              int* out_id, float* out_val, void* stream) {
  if (rows <= 0 || vocab <= 0 || k <= 0 || k > 64) return FB_ERR_SHAPE;
  launch_pdl(topk_logits_kernel, dim3(rows), dim3(1024), 0, static_cast<cudaStream_t>(stream), logits, ldl, rows, vocab,
                                                                           k, out_id, out_val);
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_copy_pages(void* pool, long long layer_stride, long long page_elems,
                             const int* pairs, int n_pairs, int n_pages, int layers, void* status,
                             void* stream) {
  if (n_pairs <= 0) return FB_OK;
  if (page_elems % 8 != 0 || layers <= 0) return FB_ERR_SHAPE;
  dim3 grid(n_pairs, layers);
  launch_pdl(copy_pages_kernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream), 
      static_cast<__nv_bfloat16*>(pool), layer_stride, page_elems, pairs, n_pairs, n_pages, layers,
      static_cast<DeviceStatus*>(status));
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_decode_advance(const int* next_id, int* token_ids, int* positions, int* row_pos,
                                 long long* write_slot, const int* row_seq, const int* block_table,
                                 int max_blocks, int page_size, int num_seqs, int rows, int vocab, int advance,
                                 void* stream) {
  if (!next_id || !token_ids || rows <= 0 || vocab <= 0) return FB_ERR_SHAPE;
  if (advance && (!positions || !row_pos || !write_slot || !row_seq || !block_table || max_blocks <= 0 ||
                  page_size <= 0 || num_seqs <= 0))
    return FB_ERR_SHAPE;
  launch_pdl(decode_advance_kernel, dim3((rows + 127) / 128), dim3(128), 0, static_cast<cudaStream_t>(stream),
             next_id, token_ids, positions, row_pos, write_slot, row_seq, block_table, max_blocks, page_size,
             num_seqs, rows, vocab, advance);
  return cudaGetLastError() == cudaSuccess ? FB_OK : FB_ERR_LAUNCH;
}
