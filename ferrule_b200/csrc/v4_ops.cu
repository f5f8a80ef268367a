// DeepSeek-V4-only operators (sm_100a), all bandwidth- or latency-bound SIMT kernels:
//
//   fb_hc_pre            hyper-connection reduction: mixes = (W_fn . state) * rms(state), split into
//                        pre / post / comb (comb Sinkhorn-normalised), hidden = sum_j pre_j * state_j
//   fb_hc_post           out_j = post_j * hidden + sum_i comb[i][j] * residual_i
//   fb_compressor_pool   per-dimension softmax pooling of `ratio` (or 2 * ratio, overlapping) rows
//   fb_indexer_scores    per compressed row: bf16(sum_h bf16(relu(bf16(q_h . row)) * w_h))
//   fb_indexer_topk      stable top-k (k <= 512) of a score row: two-level radix select on the
//                        16-bit orderable key + bitonic sort of the winners; unused slots = -1
//   fb_rope_rows         forward / inverse interleaved RoPE on a slice of each row
//
// Counterparts in the reference: hc_kernel, compressor_kernel, indexer_kernel and rope_kernel of
// crates/ferrule-backend/native/cuda/implementations/portable/entrypoints.cu (:912-1266, :1614-1840,
// :714-768) and the host oracle crates/ferrule-model/src/hyper_connection.rs:175-420.
#include "common.cuh"
#include "ferrule_b200.h"
#include "launch.cuh"

namespace fb {

constexpr int kHcMaxMix = 24;   // 2 * hc + hc * hc for hc = 4

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// One CTA per token.  state bf16 [T, hc, hidden]; fn fp32 [nmix, hc * hidden]; scale fp32 [3]; base fp32 [nmix].
// nmix = 2 hc + hc^2 (full) or hc (head reduction: only `pre`).  coeff out fp32 [T, nmix].
template <int HC>
__global__ void __launch_bounds__(256)
hc_pre_kernel(const __nv_bfloat16* __restrict__ state, const float* __restrict__ fn,
              const float* __restrict__ scale, const float* __restrict__ base, void* __restrict__ hidden_out,
              int out_fp32, float* __restrict__ coeff, int tokens, int hidden, int nmix, float eps,
              float norm_eps, int sinkhorn_iters) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[8][kHcMaxMix + 1];
  __shared__ float mix[kHcMaxMix + 1];
  __shared__ float pre_s[HC];
  const int t = blockIdx.x;
  if (t >= tokens) return;
  const int n = HC * hidden;
  const __nv_bfloat16* x = state + static_cast<size_t>(t) * n;
  float acc[kHcMaxMix + 1];
#pragma unroll
  for (int m = 0; m <= kHcMaxMix; ++m) acc[m] = 0.f;
  for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) {
    const uint2 raw = *reinterpret_cast<const uint2*>(x + i);
    const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(&raw);
    float f[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) f[j] = __bfloat162float(v[j]);
    acc[kHcMaxMix] += f[0] * f[0] + f[1] * f[1] + f[2] * f[2] + f[3] * f[3];
#pragma unroll
    for (int m = 0; m < kHcMaxMix; ++m) {
      if (m < nmix) {
        const float4 w = *reinterpret_cast<const float4*>(fn + static_cast<size_t>(m) * n + i);
        acc[m] += f[0] * w.x + f[1] * w.y + f[2] * w.z + f[3] * w.w;
      }
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int m = 0; m <= kHcMaxMix; ++m) {
    const float s = warp_sum(acc[m]);
    if (lane == 0) red[warp][m] = s;
  }
  __syncthreads();
  if (threadIdx.x <= kHcMaxMix) {
    float s = 0.f;
    for (int w = 0; w < 8; ++w) s += red[w][threadIdx.x];
    mix[threadIdx.x] = s;
  }
  __syncthreads();
  if (warp == 0) {
    const float rms = rsqrtf(mix[kHcMaxMix] / static_cast<float>(n) + norm_eps);
    float* out = coeff + static_cast<size_t>(t) * nmix;
    if (lane < HC) {
      const float p = sigmoidf_(mix[lane] * rms * scale[0] + base[lane]) + eps;
      pre_s[lane] = p;
      out[lane] = p;
      if (nmix > HC) out[HC + lane] = 2.f * sigmoidf_(mix[HC + lane] * rms * scale[1] + base[HC + lane]);
    }
    if (nmix > HC) {
      // lane = i * HC + j holds comb[i][j]; rows reduce over xor masks < HC, columns over masks >= HC
      const bool on = lane < HC * HC;
      float c = on ? mix[2 * HC + lane] * rms * scale[2] + base[2 * HC + lane] : -INFINITY;
      float mx = c;
#pragma unroll
      for (int o = 1; o < HC; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      float e = on ? __expf(c - mx) : 0.f, s = e;
#pragma unroll
      for (int o = 1; o < HC; o <<= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      c = on ? e / s + eps : 0.f;
      auto col_norm = [&]() {
        float cs = c;
#pragma unroll
        for (int o = HC; o < HC * HC; o <<= 1) cs += __shfl_xor_sync(0xffffffffu, cs, o);
        c = c / (cs + eps);
      };
      auto row_norm = [&]() {
        float rs = c;
#pragma unroll
        for (int o = 1; o < HC; o <<= 1) rs += __shfl_xor_sync(0xffffffffu, rs, o);
        c = c / (rs + eps);
      };
      col_norm();
      for (int it = 1; it < sinkhorn_iters; ++it) {
        row_norm();
        col_norm();
      }
      if (on) out[2 * HC + lane] = c;
    }
  }
  __syncthreads();
  float p[HC];
#pragma unroll
  for (int j = 0; j < HC; ++j) p[j] = pre_s[j];
  for (int d = threadIdx.x * 4; d < hidden; d += blockDim.x * 4) {
    float h[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < HC; ++j) {
      const uint2 raw = *reinterpret_cast<const uint2*>(x + static_cast<size_t>(j) * hidden + d);
      const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
      for (int q = 0; q < 4; ++q) h[q] += p[j] * __bfloat162float(v[q]);
    }
    if (out_fp32) {
      *reinterpret_cast<float4*>(static_cast<float*>(hidden_out) + static_cast<size_t>(t) * hidden + d) =
          make_float4(h[0], h[1], h[2], h[3]);
    } else {
      __nv_bfloat16 o[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) o[q] = __float2bfloat16(h[q]);
      *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(hidden_out) + static_cast<size_t>(t) * hidden + d) =
          *reinterpret_cast<const uint2*>(o);
    }
  }
}

// Split variant for large hc * hidden: grid (tokens, chunks).  Every CTA reduces one chunk of the hc * hidden
// axis (partial dot products with the mixing rows + partial sum of squares) into scratch; the CTA that
// finishes last for a token adds the partials in chunk order, runs the split / Sinkhorn step and forms the
// weighted sum.  scratch: part [tokens][chunks][32] floats, ctr [tokens] zeroed once.
template <int HC>
__global__ void __launch_bounds__(256)
hc_pre_split_kernel(const __nv_bfloat16* __restrict__ state, const float* __restrict__ fn,
                    const float* __restrict__ scale, const float* __restrict__ base, void* __restrict__ hidden_out,
                    int out_fp32, float* __restrict__ coeff, int tokens, int hidden, int nmix, float eps,
                    float norm_eps, int sinkhorn_iters, float* __restrict__ part, unsigned int* __restrict__ ctr) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[8][kHcMaxMix + 1];
  __shared__ float mix[kHcMaxMix + 1];
  __shared__ float pre_s[HC];
  __shared__ int is_last;
  const int t = blockIdx.x, c = blockIdx.y, chunks = gridDim.y;
  const int n = HC * hidden;
  const int per = ((n + chunks - 1) / chunks + 3) / 4 * 4;
  const int lo = c * per, hi = min(n, lo + per);
  const __nv_bfloat16* x = state + static_cast<size_t>(t) * n;
  float acc[kHcMaxMix + 1];
#pragma unroll
  for (int m = 0; m <= kHcMaxMix; ++m) acc[m] = 0.f;
  for (int i = lo + threadIdx.x * 4; i < hi; i += blockDim.x * 4) {
    const uint2 raw = *reinterpret_cast<const uint2*>(x + i);
    const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(&raw);
    float f[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) f[j] = __bfloat162float(v[j]);
    acc[kHcMaxMix] += f[0] * f[0] + f[1] * f[1] + f[2] * f[2] + f[3] * f[3];
#pragma unroll
    for (int m = 0; m < kHcMaxMix; ++m) {
      if (m < nmix) {
        const float4 w = *reinterpret_cast<const float4*>(fn + static_cast<size_t>(m) * n + i);
        acc[m] += f[0] * w.x + f[1] * w.y + f[2] * w.z + f[3] * w.w;
      }
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int m = 0; m <= kHcMaxMix; ++m) {
    const float s = warp_sum(acc[m]);
    if (lane == 0) red[warp][m] = s;
  }
  __syncthreads();
  float* mine = part + (static_cast<size_t>(t) * chunks + c) * 32;
  if (threadIdx.x <= kHcMaxMix) {
    float s = 0.f;
    for (int w = 0; w < 8; ++w) s += red[w][threadIdx.x];
    mine[threadIdx.x] = s;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(ctr + t, 1u);
    is_last = done == static_cast<unsigned int>(chunks - 1);
    if (is_last) ctr[t] = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  if (threadIdx.x <= kHcMaxMix) {
    float s = 0.f;
    for (int k = 0; k < chunks; ++k) s += part[(static_cast<size_t>(t) * chunks + k) * 32 + threadIdx.x];
    mix[threadIdx.x] = s;
  }
  __syncthreads();
  if (warp == 0) {
    const float rms = rsqrtf(mix[kHcMaxMix] / static_cast<float>(n) + norm_eps);
    float* out = coeff + static_cast<size_t>(t) * nmix;
    if (lane < HC) {
      const float p = sigmoidf_(mix[lane] * rms * scale[0] + base[lane]) + eps;
      pre_s[lane] = p;
      out[lane] = p;
      if (nmix > HC) out[HC + lane] = 2.f * sigmoidf_(mix[HC + lane] * rms * scale[1] + base[HC + lane]);
    }
    if (nmix > HC) {
      const bool on = lane < HC * HC;
      float cv = on ? mix[2 * HC + lane] * rms * scale[2] + base[2 * HC + lane] : -INFINITY;
      float mx = cv;
#pragma unroll
      for (int o = 1; o < HC; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      float e = on ? __expf(cv - mx) : 0.f, s = e;
#pragma unroll
      for (int o = 1; o < HC; o <<= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      cv = on ? e / s + eps : 0.f;
      for (int it = 0; it < sinkhorn_iters; ++it) {
        if (it > 0) {
          float rs = cv;
#pragma unroll
          for (int o = 1; o < HC; o <<= 1) rs += __shfl_xor_sync(0xffffffffu, rs, o);
          cv = cv / (rs + eps);
        }
        float cs = cv;
#pragma unroll
        for (int o = HC; o < HC * HC; o <<= 1) cs += __shfl_xor_sync(0xffffffffu, cs, o);
        cv = cv / (cs + eps);
      }
      if (on) out[2 * HC + lane] = cv;
    }
  }
  __syncthreads();
  float p[HC];
#pragma unroll
  for (int j = 0; j < HC; ++j) p[j] = pre_s[j];
  for (int d = threadIdx.x * 4; d < hidden; d += blockDim.x * 4) {
    float h[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < HC; ++j) {
      const uint2 raw = *reinterpret_cast<const uint2*>(x + static_cast<size_t>(j) * hidden + d);
      const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
      for (int q = 0; q < 4; ++q) h[q] += p[j] * __bfloat162float(v[q]);
    }
    if (out_fp32) {
      *reinterpret_cast<float4*>(static_cast<float*>(hidden_out) + static_cast<size_t>(t) * hidden + d) =
          make_float4(h[0], h[1], h[2], h[3]);
    } else {
      __nv_bfloat16 o[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) o[q] = __float2bfloat16(h[q]);
      *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(hidden_out) + static_cast<size_t>(t) * hidden + d) =
          *reinterpret_cast<const uint2*>(o);
    }
  }
}

// out[t][j][d] = post[j] * hidden[t][d] + sum_i comb[i][j] * residual[t][i][d]; coeff = [pre | post | comb] per token
template <int HC>
__global__ void __launch_bounds__(256)
hc_post_kernel(const __nv_bfloat16* __restrict__ hidden_in, const __nv_bfloat16* __restrict__ residual,
               const float* __restrict__ coeff, __nv_bfloat16* __restrict__ out, int tokens, int hidden) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= tokens) return;
  const float* c = coeff + static_cast<size_t>(t) * (2 * HC + HC * HC);
  float post[HC], comb[HC][HC];
#pragma unroll
  for (int j = 0; j < HC; ++j) post[j] = c[HC + j];
#pragma unroll
  for (int i = 0; i < HC; ++i)
#pragma unroll
    for (int j = 0; j < HC; ++j) comb[i][j] = c[2 * HC + i * HC + j];
  const __nv_bfloat16* res = residual + static_cast<size_t>(t) * HC * hidden;
  __nv_bfloat16* o = out + static_cast<size_t>(t) * HC * hidden;
  for (int d = threadIdx.x * 4; d < hidden; d += blockDim.x * 4) {
    const uint2 hraw = *reinterpret_cast<const uint2*>(hidden_in + static_cast<size_t>(t) * hidden + d);
    const __nv_bfloat16* hv = reinterpret_cast<const __nv_bfloat16*>(&hraw);
    float r[HC][4];
#pragma unroll
    for (int i = 0; i < HC; ++i) {
      const uint2 raw = *reinterpret_cast<const uint2*>(res + static_cast<size_t>(i) * hidden + d);
      const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
      for (int q = 0; q < 4; ++q) r[i][q] = __bfloat162float(v[q]);
    }
#pragma unroll
    for (int j = 0; j < HC; ++j) {
      __nv_bfloat16 w[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float a = post[j] * __bfloat162float(hv[q]);
#pragma unroll
        for (int i = 0; i < HC; ++i) a += comb[i][j] * r[i][q];
        w[q] = __float2bfloat16(a);
      }
      *reinterpret_cast<uint2*>(o + static_cast<size_t>(j) * hidden + d) = *reinterpret_cast<const uint2*>(w);
    }
  }
}

// ---------------------------------------------------------------------------------
// Compressor pooling.  Group g pools window rows r = row0 + g * ratio + w (w < window); rows outside
// [0, n_rows) count as score -inf / value 0.  kv, gate fp32 [n_rows, ld] projected rows; ape fp32
// [ratio, cur_col + dim] contiguous; out bf16 [groups, dim].  With an overlapping window (window = 2 * ratio) the rows of the
// previous group are read from columns [0, dim) and the rows of the current group from columns
// [cur_col, cur_col + dim) of the projection (cur_col = dim), each with the position embedding of
// its position inside its group.  One thread per (group, dim); online softmax over the window.
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
compressor_pool_kernel(const float* __restrict__ kv, const float* __restrict__ gate, long long ld,
                       const float* __restrict__ ape, __nv_bfloat16* __restrict__ out, long long ldo,
                       int groups, int dim, int ratio, int window, int row0, int n_rows, int cur_col) {
  pdl_launch_dependents();
  pdl_wait();
  const int g = blockIdx.y;
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= groups || d >= dim) return;
  const int first = row0 + g * ratio;
  const int prev_rows = window - ratio;
  float m = -INFINITY, den = 0.f, num = 0.f;
  for (int w = 0; w < window; ++w) {
    const int r = first + w;
    if (r < 0 || r >= n_rows) continue;
    const int col = (w < prev_rows ? 0 : cur_col) + d;
    const int in_group = w < prev_rows ? w : w - prev_rows;
    const float s = gate[r * ld + col] + ape[static_cast<size_t>(in_group) * (cur_col + dim) + col];
    const float v = kv[r * ld + col];
    if (s > m) {
      const float c = __expf(m - s);   // exp(-inf) = 0 on the first valid row
      den *= c;
      num *= c;
      m = s;
    }
    const float e = __expf(s - m);
    den += e;
    num += e * v;
  }
  out[g * ldo + d] = __float2bfloat16(den > 0.f ? num / den : 0.f);
}

// Interleaved-pair RoPE on x[row][head][off : off + rdim], forward or inverse, in place (bf16).
__global__ void __launch_bounds__(256)
rope_rows_kernel(__nv_bfloat16* __restrict__ x, long long ld_row, long long ld_head, int rows, int heads,
                 int off, int rdim, const int* __restrict__ positions, const float* __restrict__ cos_t,
                 const float* __restrict__ sin_t, int max_pos, int inverse, DeviceStatus* st) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  if (r >= rows) return;
  int pos = positions[r];
  if (pos < 0 || pos >= max_pos) {
    if (threadIdx.x == 0) report_status(st, kStatusBadIndex, 0x70, r, pos);
    return;
  }
  const int half = rdim / 2;
  for (int i = threadIdx.x; i < heads * half; i += blockDim.x) {
    const int h = i / half, p = i - h * half;
    __nv_bfloat162* ptr = reinterpret_cast<__nv_bfloat162*>(x + r * ld_row + h * ld_head + off) + p;
    const float2 v = __bfloat1622float2(*ptr);
    const float c = cos_t[static_cast<size_t>(pos) * half + p];
    const float s = inverse ? -sin_t[static_cast<size_t>(pos) * half + p] : sin_t[static_cast<size_t>(pos) * half + p];
    *ptr = __floats2bfloat162_rn(v.x * c - v.y * s, v.x * s + v.y * c);
  }
}

// ---------------------------------------------------------------------------------
// Indexer scores.  q bf16 [queries, heads, d]; plane bf16 [n, d]; head_w fp32 [queries, heads];
// scores fp32 [queries, ld_s] (values are bf16-representable).  Grid (row chunks, queries); the
// query's heads sit in shared memory (rows padded by one word against bank conflicts); one warp
// per compressed row, each lane owning heads lane, lane + 32, ...
// ---------------------------------------------------------------------------------
__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16(v)); }

__global__ void __launch_bounds__(256)
indexer_scores_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ plane, long long ldp,
                      const float* __restrict__ head_w, float* __restrict__ scores, long long ld_s,
                      int heads, int d, int n, int rows_per_cta) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ uint32_t sm_idx[];
  const int words = d / 2, pitch = words + 1;
  uint32_t* qs = sm_idx;                                   // [heads][pitch]
  uint32_t* rowbuf = qs + heads * pitch;                   // [8 warps][words]
  const int qi = blockIdx.y;
  const uint32_t* qg = reinterpret_cast<const uint32_t*>(q + static_cast<size_t>(qi) * heads * d);
  for (int i = threadIdx.x; i < heads * words; i += blockDim.x) qs[(i / words) * pitch + (i % words)] = qg[i];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t* mine = rowbuf + warp * words;
  const int r_lo = blockIdx.x * rows_per_cta, r_hi = min(n, r_lo + rows_per_cta);
  for (int r = r_lo + warp; r < r_hi; r += 8) {
    const uint32_t* pg = reinterpret_cast<const uint32_t*>(plane + r * ldp);
    for (int i = lane; i < words; i += 32) mine[i] = pg[i];
    __syncwarp();
    float total = 0.f;
    for (int h = lane; h < heads; h += 32) {
      float dot = 0.f;
      const uint32_t* qh = qs + h * pitch;
      for (int i = 0; i < words; ++i) {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qh[i]));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&mine[i]));
        dot = fmaf(a.x, b.x, dot);
        dot = fmaf(a.y, b.y, dot);
      }
      const float w = bf16r(head_w[static_cast<size_t>(qi) * heads + h]);
      total += bf16r(fmaxf(bf16r(dot), 0.f) * w);
    }
    // fixed-order reduction: butterfly sums are order-stable for a given lane count
    total = warp_sum(total);
    if (lane == 0) scores[qi * ld_s + r] = bf16r(total);
    __syncwarp();
  }
}

// Head reduction of the indexer when the per-head dots come from the tensor-core GEMM
// (dots bf16 [queries * heads, n] = q . plane^T, already rounded to bf16 by the GEMM epilogue):
// score[q][n] = bf16(sum_h bf16(relu(dots[q*heads + h][n]) * bf16(w[q][h]))), heads summed in index order.
__global__ void __launch_bounds__(256)
indexer_reduce_kernel(const __nv_bfloat16* __restrict__ dots, long long ld, const float* __restrict__ head_w,
                      float* __restrict__ scores, long long ld_s, int heads, int n) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float w_s[];           // [heads] bf16-rounded weights of this query
  const int qi = blockIdx.y;
  for (int h = threadIdx.x; h < heads; h += blockDim.x) w_s[h] = bf16r(head_w[static_cast<size_t>(qi) * heads + h]);
  __syncthreads();
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (c >= n) return;
  const __nv_bfloat16* col = dots + static_cast<size_t>(qi) * heads * ld + c;
  float s0 = 0.f, s1 = 0.f;
  if (c + 1 < n) {
#pragma unroll 8
    for (int h = 0; h < heads; ++h) {
      const float2 d = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(col + h * ld));
      s0 += bf16r(fmaxf(d.x, 0.f) * w_s[h]);
      s1 += bf16r(fmaxf(d.y, 0.f) * w_s[h]);
    }
    scores[qi * ld_s + c] = bf16r(s0);
    scores[qi * ld_s + c + 1] = bf16r(s1);
  } else {
    for (int h = 0; h < heads; ++h) s0 += bf16r(fmaxf(__bfloat162float(col[h * ld]), 0.f) * w_s[h]);
    scores[qi * ld_s + c] = bf16r(s0);
  }
}

// ---------------------------------------------------------------------------------
// Stable top-k of one score row per CTA (1024 threads).  Scores hold bf16 values, so the 16-bit
// orderable key decides; ties go to the lower row id.  Non-finite scores never win.
//   pass 1: histogram of the key's high byte   -> byte b1 where the running count (from the top) reaches k
//   pass 2: histogram of the low byte inside b1 -> threshold key T and how many rows with key == T to take
//   pass 3: collect key > T (any order) and the first `need` rows with key == T (ordered scan)
//   pass 4: bitonic sort of (key desc, id asc) and write; the rest of the k slots = -1
// ---------------------------------------------------------------------------------
constexpr int kTopkMax = 512;

__device__ __forceinline__ uint32_t score_key(float s) {
  // bf16 bits -> ascending unsigned order; +1 keeps 0 free to mean "not a candidate"
  if (!isfinite(s)) return 0u;
  const uint32_t b = __float_as_uint(s) >> 16;
  const uint32_t k = (b & 0x8000u) ? (~b & 0xffffu) : (b | 0x8000u);
  return k + 1u;      // 1 .. 65536
}

__global__ void __launch_bounds__(1024)
indexer_topk_kernel(const float* __restrict__ scores, long long ld_s, const int* __restrict__ n_visible, int n_fixed,
                    int k, int* __restrict__ out_idx, long long ldo) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int hist[257];
  __shared__ unsigned long long win[kTopkMax];
  __shared__ int s_b1, s_above1, s_thr, s_need, s_count, s_eq_base;
  __shared__ int warp_tot[32];
  const int qi = blockIdx.x, tid = threadIdx.x;
  const int n = n_visible ? n_visible[qi] : n_fixed;
  const float* s = scores + qi * ld_s;
  int* out = out_idx + qi * ldo;
  for (int i = tid; i < k; i += blockDim.x) out[i] = -1;
  if (n <= 0) return;
  for (int i = tid; i < 257; i += blockDim.x) hist[i] = 0;
  for (int i = tid; i < kTopkMax; i += blockDim.x) win[i] = 0ull;
  if (tid == 0) { s_count = 0; s_eq_base = 0; }
  __syncthreads();
  for (int i = tid; i < n; i += blockDim.x) {
    const uint32_t key = score_key(s[i]);
    if (key) atomicAdd(&hist[(key - 1u) >> 8], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int run = 0, b = 255;
    for (; b >= 0; --b) {
      if (run + hist[b] >= k) break;
      run += hist[b];
    }
    s_b1 = b;          // -1: fewer than k candidates in total -> take them all
    s_above1 = run;
  }
  __syncthreads();
  const int b1 = s_b1;
  int thr_key = 0, need = 0;          // take key > thr_key, plus `need` rows with key == thr_key
  if (b1 >= 0) {
    __syncthreads();
    for (int i = tid; i < 257; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (int i = tid; i < n; i += blockDim.x) {
      const uint32_t key = score_key(s[i]);
      if (key && static_cast<int>((key - 1u) >> 8) == b1) atomicAdd(&hist[(key - 1u) & 255u], 1);
    }
    __syncthreads();
    if (tid == 0) {
      int run = s_above1, b = 255;
      for (; b >= 0; --b) {
        if (run + hist[b] >= k) break;
        run += hist[b];
      }
      s_thr = (b1 << 8) + b + 1;
      s_need = k - run;
    }
    __syncthreads();
    thr_key = s_thr;
    need = s_need;
  }
  // pass 3 (ordered over chunks of blockDim.x rows so that equal keys are taken lowest id first)
  const int warp = tid >> 5, lane = tid & 31;
  for (int base = 0; base < n; base += blockDim.x) {
    const int i = base + tid;
    const uint32_t key = i < n ? score_key(s[i]) : 0u;
    const bool above = key > static_cast<uint32_t>(thr_key);
    const bool equal = need > 0 && key != 0u && key == static_cast<uint32_t>(thr_key);
    const unsigned eq_mask = __ballot_sync(0xffffffffu, equal);
    if (lane == 0) warp_tot[warp] = __popc(eq_mask);
    __syncthreads();
    int before = s_eq_base;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    before += __popc(eq_mask & ((1u << lane) - 1u));
    const bool take = above || (equal && before < need);
    if (take) {
      const int slot = atomicAdd(&s_count, 1);
      if (slot < kTopkMax)
        win[slot] = (static_cast<unsigned long long>(key) << 32) | (0xffffffffu - static_cast<uint32_t>(i));
    }
    __syncthreads();
    if (tid == 0) {
      int tot = 0;
      for (int w = 0; w < 32; ++w) tot += warp_tot[w];
      s_eq_base += tot;
    }
    __syncthreads();
  }
  // pass 4: descending bitonic sort of 512 composite keys (zeros sink to the end)
  for (int size = 2; size <= kTopkMax; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      if (tid < kTopkMax / 2) {
        const int lo = (tid / stride) * stride * 2 + (tid % stride), hi = lo + stride;
        const bool desc = ((lo & size) == 0);
        const unsigned long long a = win[lo], b = win[hi];
        if ((a < b) == desc) { win[lo] = b; win[hi] = a; }
      }
      __syncthreads();
    }
  }
  const int got = min(s_count, k);
  for (int i = tid; i < got; i += blockDim.x)
    out[i] = static_cast<int>(0xffffffffu - static_cast<uint32_t>(win[i] & 0xffffffffull));
}

// ---------------------------------------------------------------------------------
// Markov proposal head, one draft step: id = argmax_t (logits[t] + W2[t] . W1[prev]) with ties to the
// lower id; prev is read from device memory (the anchor or the previous step's draft), so a block of
// draft steps needs no host round trip.  Grid = vocabulary chunks; the CTA that finishes last reduces
// the chunk candidates and writes (id, biased logit).
// ---------------------------------------------------------------------------------
__device__ __forceinline__ bool better_cand(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

__global__ void __launch_bounds__(256)
markov_step_kernel(const float* __restrict__ logits, const __nv_bfloat16* __restrict__ w1,
                   const __nv_bfloat16* __restrict__ w2, int vocab, int rank, int chunk,
                   const int* __restrict__ prev_token, float* __restrict__ part_val, int* __restrict__ part_id,
                   unsigned int* __restrict__ ctr, int* __restrict__ out_id, float* __restrict__ out_val,
                   DeviceStatus* st) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float w1_prev[];       // [rank]
  __shared__ float sv[8];
  __shared__ int si[8];
  __shared__ int is_last;
  int prev = *prev_token;
  if (prev < 0 || prev >= vocab) {
    if (threadIdx.x == 0 && blockIdx.x == 0) report_status(st, kStatusBadIndex, 0xB00, prev, vocab);
    prev = 0;
  }
  for (int i = threadIdx.x; i < rank; i += blockDim.x) w1_prev[i] = __bfloat162float(w1[static_cast<size_t>(prev) * rank + i]);
  __syncthreads();
  const int c = blockIdx.x, chunks = gridDim.x;
  const int lo = c * chunk, hi = min(vocab, lo + chunk);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int t = lo + threadIdx.x; t < hi; t += blockDim.x) {
    const uint4* row = reinterpret_cast<const uint4*>(w2 + static_cast<size_t>(t) * rank);
    float bias = 0.f;
    for (int i = 0; i < rank / 8; ++i) {
      const uint4 v = row[i];
      const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
      for (int j = 0; j < 8; ++j) bias = fmaf(__bfloat162float(b[j]), w1_prev[i * 8 + j], bias);
    }
    const float v = logits[t] + bias;
    if (v == v && better_cand(v, t, best, bi)) { best = v; bi = t; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better_cand(ov, oi, best, bi)) { best = ov; bi = oi; }
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { sv[w] = best; si[w] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int k = 1; k < 8; ++k)
      if (better_cand(sv[k], si[k], best, bi)) { best = sv[k]; bi = si[k]; }
    part_val[c] = best;
    part_id[c] = bi;
    __threadfence();
    const unsigned int done = atomicAdd(ctr, 1u);
    is_last = done == static_cast<unsigned int>(chunks - 1);
    if (is_last) *ctr = 0;
  }
  __syncthreads();
  if (!is_last || w != 0) return;
  __threadfence();
  best = -INFINITY;
  bi = 0x7fffffff;
  for (int k = l; k < chunks; k += 32) {
    const float v = part_val[k];
    const int id = part_id[k];
    if (better_cand(v, id, best, bi)) { best = v; bi = id; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better_cand(ov, oi, best, bi)) { best = ov; bi = oi; }
  }
  if (l == 0) {
    *out_id = bi == 0x7fffffff ? -1 : bi;
    *out_val = best;
  }
}

// Mean over the hc copies of the residual stream, scattered into a proposal tap:
// taps[t][tap_off : tap_off + hidden] = bf16(sum_j state[t][j][:] / hc)
__global__ void __launch_bounds__(256)
hc_mean_scatter_kernel(const __nv_bfloat16* __restrict__ state, __nv_bfloat16* __restrict__ taps, long long ld_taps,
                       int tap_off, int tokens, int hc, int hidden) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= tokens) return;
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
    float s = 0.f;
    for (int j = 0; j < hc; ++j) s += __bfloat162float(state[(static_cast<size_t>(t) * hc + j) * hidden + d]);
    taps[t * ld_taps + tap_off + d] = __float2bfloat16(s / static_cast<float>(hc));
  }
}

}  // namespace fb

using namespace fb;

#define FB_CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? FB_OK : FB_ERR_LAUNCH)

extern "C" int fb_hc_pre(const void* state, const float* fn, const float* scale, const float* base, void* hidden_out,
                         int out_fp32, float* coeff, int tokens, int hc, int hidden, int nmix, float eps,
                         float norm_eps, int sinkhorn_iters, void* stream) {
  if (tokens <= 0 || hidden % 4 != 0 || (hc != 2 && hc != 4)) return FB_ERR_SHAPE;
  if (nmix != hc && nmix != 2 * hc + hc * hc) return FB_ERR_SHAPE;
  auto st = static_cast<cudaStream_t>(stream);
  auto s = static_cast<const __nv_bfloat16*>(state);
  if (hc == 4)
    launch_pdl(hc_pre_kernel<4>, dim3(tokens), dim3(256), 0, st, s, fn, scale, base, hidden_out, out_fp32, coeff,
               tokens, hidden, nmix, eps, norm_eps, sinkhorn_iters);
  else
    launch_pdl(hc_pre_kernel<2>, dim3(tokens), dim3(256), 0, st, s, fn, scale, base, hidden_out, out_fp32, coeff,
               tokens, hidden, nmix, eps, norm_eps, sinkhorn_iters);
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_hc_post(const void* hidden_in, const void* residual, const float* coeff, void* out, int tokens,
                          int hc, int hidden, void* stream) {
  if (tokens <= 0 || hidden % 4 != 0 || (hc != 2 && hc != 4)) return FB_ERR_SHAPE;
  auto st = static_cast<cudaStream_t>(stream);
  auto h = static_cast<const __nv_bfloat16*>(hidden_in);
  auto r = static_cast<const __nv_bfloat16*>(residual);
  auto o = static_cast<__nv_bfloat16*>(out);
  if (hc == 4) launch_pdl(hc_post_kernel<4>, dim3(tokens), dim3(256), 0, st, h, r, coeff, o, tokens, hidden);
  else launch_pdl(hc_post_kernel<2>, dim3(tokens), dim3(256), 0, st, h, r, coeff, o, tokens, hidden);
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_compressor_pool(const float* kv, const float* gate, long long ld, const float* ape, void* out,
                                  long long ldo, int groups, int dim, int ratio, int window, int row0, int n_rows,
                                  int cur_col, void* stream) {
  if (groups <= 0 || dim <= 0 || ratio <= 0 || window < ratio || window > 2 * ratio || groups > 65535 ||
      cur_col < 0 || cur_col + dim > ld)
    return FB_ERR_SHAPE;
  launch_pdl(compressor_pool_kernel, dim3((dim + 255) / 256, groups), dim3(256), 0, static_cast<cudaStream_t>(stream),
             kv, gate, ld, ape, static_cast<__nv_bfloat16*>(out), ldo, groups, dim, ratio, window, row0, n_rows, cur_col);
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_rope_rows(void* x, long long ld_row, long long ld_head, int rows, int heads, int off, int rdim,
                            const int* positions, const float* cos_t, const float* sin_t, int max_pos, int inverse,
                            void* status, void* stream) {
  if (rows <= 0 || heads <= 0 || rdim <= 0 || rdim % 2 != 0 || off % 2 != 0 || ld_row % 2 != 0 || ld_head % 2 != 0)
    return FB_ERR_SHAPE;
  launch_pdl(rope_rows_kernel, dim3(rows), dim3(256), 0, static_cast<cudaStream_t>(stream),
             static_cast<__nv_bfloat16*>(x), ld_row, ld_head, rows, heads, off, rdim, positions, cos_t, sin_t, max_pos,
             inverse, static_cast<DeviceStatus*>(status));
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_indexer_scores(const void* q, const void* plane, long long ldp, const float* head_w, float* scores,
                                 long long ld_s, int queries, int heads, int d, int n, void* stream) {
  if (queries <= 0 || heads <= 0 || d <= 0 || d % 2 != 0 || n <= 0 || ldp % 2 != 0 || queries > 65535)
    return FB_ERR_SHAPE;
  const size_t smem = (static_cast<size_t>(heads) * (d / 2 + 1) + 8 * (d / 2)) * sizeof(uint32_t);
  if (smem > 200 * 1024) return FB_ERR_SHAPE;
  static bool attr_done = false;
  if (!attr_done) {
    cudaFuncSetAttribute(indexer_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    attr_done = true;
  }
  // enough CTAs to fill the GPU, at least 64 rows each so the query staging amortises
  int rows_per_cta = (n + 147) / 148;
  if (rows_per_cta < 64) rows_per_cta = 64;
  const int chunks = (n + rows_per_cta - 1) / rows_per_cta;
  launch_pdl(indexer_scores_kernel, dim3(chunks, queries), dim3(256), smem, static_cast<cudaStream_t>(stream),
             static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(plane), ldp, head_w, scores, ld_s,
             heads, d, n, rows_per_cta);
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_indexer_topk(const float* scores, long long ld_s, const int* n_visible, int n_fixed, int k,
                               int* out_idx, long long ldo, int queries, void* stream) {
  if (queries <= 0 || k <= 0 || k > kTopkMax) return FB_ERR_SHAPE;
  launch_pdl(indexer_topk_kernel, dim3(queries), dim3(1024), 0, static_cast<cudaStream_t>(stream), scores, ld_s,
             n_visible, n_fixed, k, out_idx, ldo);
  return FB_CHECK_LAUNCH();
}

// scratch: part_val [chunks] floats, part_id [chunks] ints, ctr one zeroed uint32; chunks <= 1024
extern "C" int fb_markov_step(const float* logits, const void* w1, const void* w2, int vocab, int rank, int chunks,
                              const int* prev_token, float* part_val, int* part_id, void* ctr, int* out_id,
                              float* out_val, void* status, void* stream) {
  if (vocab <= 0 || rank <= 0 || rank % 8 != 0 || rank > 4096 || chunks <= 0 || chunks > 1024 || !prev_token || !ctr)
    return FB_ERR_SHAPE;
  const int chunk = (vocab + chunks - 1) / chunks;
  launch_pdl(markov_step_kernel, dim3(chunks), dim3(256), rank * sizeof(float), static_cast<cudaStream_t>(stream),
             logits, static_cast<const __nv_bfloat16*>(w1), static_cast<const __nv_bfloat16*>(w2), vocab, rank, chunk,
             prev_token, part_val, part_id, static_cast<unsigned int*>(ctr), out_id, out_val,
             static_cast<DeviceStatus*>(status));
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_hc_mean_scatter(const void* state, void* taps, long long ld_taps, int tap_off, int tokens, int hc,
                                  int hidden, void* stream) {
  if (tokens <= 0 || hc <= 0 || hidden <= 0 || tap_off < 0) return FB_ERR_SHAPE;
  launch_pdl(hc_mean_scatter_kernel, dim3(tokens), dim3(256), 0, static_cast<cudaStream_t>(stream),
             static_cast<const __nv_bfloat16*>(state), static_cast<__nv_bfloat16*>(taps), ld_taps, tap_off, tokens, hc,
             hidden);
  return FB_CHECK_LAUNCH();
}

extern "C" int fb_indexer_reduce(const void* dots, long long ld, const float* head_w, float* scores, long long ld_s,
                                 int queries, int heads, int n, void* stream) {
  if (queries <= 0 || heads <= 0 || heads > 4096 || n <= 0 || ld % 2 != 0 || queries > 65535) return FB_ERR_SHAPE;
  launch_pdl(indexer_reduce_kernel, dim3((n + 511) / 512, queries), dim3(256), heads * sizeof(float),
             static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(dots), ld, head_w, scores, ld_s, heads, n);
  return FB_CHECK_LAUNCH();
}

// scratch (optional): part = floats [tokens * chunks * 32], ctr = zeroed uint32 [tokens]; with both given and
// chunks > 1 the reduction over hc * hidden is split over `chunks` CTAs per token
extern "C" int fb_hc_pre_split(const void* state, const float* fn, const float* scale, const float* base,
                               void* hidden_out, int out_fp32, float* coeff, int tokens, int hc, int hidden, int nmix,
                               float eps, float norm_eps, int sinkhorn_iters, int chunks, float* part, void* ctr,
                               void* stream) {
  if (tokens <= 0 || hidden % 4 != 0 || (hc != 2 && hc != 4) || chunks < 1 || chunks > 64 || !part || !ctr ||
      tokens > 65535)
    return FB_ERR_SHAPE;
  if (nmix != hc && nmix != 2 * hc + hc * hc) return FB_ERR_SHAPE;
  auto st = static_cast<cudaStream_t>(stream);
  auto s = static_cast<const __nv_bfloat16*>(state);
  auto c = static_cast<unsigned int*>(ctr);
  if (hc == 4)
    launch_pdl(hc_pre_split_kernel<4>, dim3(tokens, chunks), dim3(256), 0, st, s, fn, scale, base, hidden_out, out_fp32,
               coeff, tokens, hidden, nmix, eps, norm_eps, sinkhorn_iters, part, c);
  else
    launch_pdl(hc_pre_split_kernel<2>, dim3(tokens, chunks), dim3(256), 0, st, s, fn, scale, base, hidden_out, out_fp32,
               coeff, tokens, hidden, nmix, eps, norm_eps, sinkhorn_iters, part, c);
  return FB_CHECK_LAUNCH();
}
