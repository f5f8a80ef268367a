// Data movers (sm_100a): the small index / copy kernels between the compute kernels of a step, so that a
// step contains no library launch.  One kernel per kind, grid-stride over elements, 16-byte vectors where
// rows are moved.  Every index that addresses memory is range-checked: an out-of-range row is skipped and
// recorded in the status word.
//
//   fill / iota            dst[i] = value | start + i * step                                   (int32)
//   pack_pairs             out[2i] = id[i], out[2i+1] = bits(val[i])  -> one device->host copy of (id, value)
//   window_index_fill      sel[r, col0 + j] = position[r] - (window - 1 - j) >= 0 ? base[r] + that : -1
//   offset_index_fill      sel[r, col0 + j] = idx[r, j] >= 0 ? base[r] + idx[r, j] : -1        (top-k lists)
//   count_index_fill       sel[r, col0 + j] = j < count[r] ? base[r] + j : -1                  (all visible rows)
//   copy_rows              dst[dst_row0 + r] = src[r]                                          (copy into slot)
//   gather_rows            out[r] = src[idx[r]]
//   scatter_add_rows       dst[idx[r]] += src[r]                                               (fp32 atomics)
//   saxpy                  y += a * x                                                          (fp32)
//   ring_to_logical        combined-ring slot -> (logical position | compressed index, plane selector)
//   paged_row_scatter      pool[block_table[seq[r], pos[r] / page] * page + pos[r] % page] = src[r]
//
// Counterpart of the reference's data_kernel family
// (crates/ferrule-backend/native/cuda/implementations/portable/entrypoints.cu:478-629, paged addressing :450-476).
#include "common.cuh"
#include "ferrule_b200.h"
#include "launch.cuh"

namespace fb {
namespace mv {

constexpr int kThreads = 256;

__device__ __forceinline__ long long gtid() { return static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; }
__device__ __forceinline__ long long gstride() { return static_cast<long long>(gridDim.x) * blockDim.x; }

__global__ void fill_kernel(int* __restrict__ dst, long long n, int start, int step) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = gtid(); i < n; i += gstride()) dst[i] = start + static_cast<int>(i) * step;
}

__global__ void pack_pairs_kernel(const int* __restrict__ ids, const float* __restrict__ vals, int* __restrict__ out,
                                  int n) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = gtid(); i < n; i += gstride()) {
    out[2 * i] = ids[i];
    out[2 * i + 1] = __float_as_int(vals[i]);
  }
}

// mode 0: window (idx unused), 1: offset list idx [rows, width], 2: counts (idx [rows])
__global__ void index_fill_kernel(int* __restrict__ sel, long long lds, int col0, int rows, int width, int mode,
                                  const int* __restrict__ positions, const long long* __restrict__ base,
                                  const int* __restrict__ idx, long long ldi) {
  pdl_launch_dependents();
  pdl_wait();
  const long long n = static_cast<long long>(rows) * width;
  for (long long i = gtid(); i < n; i += gstride()) {
    const int r = static_cast<int>(i / width), j = static_cast<int>(i - static_cast<long long>(r) * width);
    long long v = -1;
    if (mode == 0) {
      const int p = positions[r] - (width - 1 - j);
      if (p >= 0) v = base[r] + p;
    } else if (mode == 1) {
      const int k = idx[r * ldi + j];
      if (k >= 0) v = base[r] + k;
    } else {
      if (j < idx[r]) v = base[r] + j;
    }
    sel[r * lds + col0 + j] = v > 0x7fffffffll ? -1 : static_cast<int>(v);
  }
}

// rows of `bytes` bytes (multiple of 16); idx == nullptr: dst row = dst_row0 + r (copy into slot); gather: src row =
// idx[r]; out-of-range source rows are skipped
__global__ void move_rows_kernel(uint8_t* __restrict__ dst, long long ldd, long long dst_row0,
                                 const uint8_t* __restrict__ src, long long lds, const int* __restrict__ idx,
                                 int rows, int src_rows, int bytes, DeviceStatus* st) {
  pdl_launch_dependents();
  pdl_wait();
  const int vec = bytes / 16;
  const long long n = static_cast<long long>(rows) * vec;
  for (long long i = gtid(); i < n; i += gstride()) {
    const int r = static_cast<int>(i / vec), c = static_cast<int>(i - static_cast<long long>(r) * vec);
    long long sr = r;
    if (idx != nullptr) {
      sr = idx[r];
      if (sr < 0 || sr >= src_rows) {
        if (c == 0) report_status(st, kStatusBadIndex, 0xa0, r, static_cast<uint32_t>(sr));
        continue;
      }
    }
    *reinterpret_cast<uint4*>(dst + (dst_row0 + r) * ldd + c * 16) =
        *reinterpret_cast<const uint4*>(src + sr * lds + c * 16);
  }
}

__global__ void scatter_add_kernel(float* __restrict__ dst, long long ldd, int dst_rows, const float* __restrict__ src,
                                   long long lds, const int* __restrict__ idx, int rows, int dim, DeviceStatus* st) {
  pdl_launch_dependents();
  pdl_wait();
  const long long n = static_cast<long long>(rows) * dim;
  for (long long i = gtid(); i < n; i += gstride()) {
    const int r = static_cast<int>(i / dim), c = static_cast<int>(i - static_cast<long long>(r) * dim);
    const int d = idx[r];
    if (d < 0 || d >= dst_rows) {
      if (c == 0) report_status(st, kStatusBadIndex, 0xa1, r, static_cast<uint32_t>(d));
      continue;
    }
    atomicAdd(dst + d * ldd + c, src[r * lds + c]);
  }
}

__global__ void saxpy_kernel(float* __restrict__ y, const float* __restrict__ x, float a, long long n) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = gtid(); i < n; i += gstride()) y[i] = fmaf(a, x[i], y[i]);
}

// Combined ring of the decode path: slots [0, window) hold the last `window` positions (slot = position % window),
// slots >= window name compressed rows.  out_index = the logical position (or the compressed row index), out_plane
// = 0 window / 1 compressed, -1 / -1 for an invalid or never-written slot.
__global__ void ring_to_logical_kernel(const int* __restrict__ slots, long long lds, int rows, int width, int window,
                                       const int* __restrict__ last_position, const int* __restrict__ n_compressed,
                                       int* __restrict__ out_index, int* __restrict__ out_plane, long long ldo) {
  pdl_launch_dependents();
  pdl_wait();
  const long long n = static_cast<long long>(rows) * width;
  for (long long i = gtid(); i < n; i += gstride()) {
    const int r = static_cast<int>(i / width), j = static_cast<int>(i - static_cast<long long>(r) * width);
    const int s = slots[r * lds + j];
    int index = -1, plane = -1;
    if (s >= 0 && s < window) {
      const int last = last_position[r];
      // the newest position p <= last with p % window == s
      const int p = last - ((last - s) % window + window) % window;
      if (p >= 0 && p > last - window) { index = p; plane = 0; }
    } else if (s >= window) {
      const int c = s - window;
      if (c < n_compressed[r]) { index = c; plane = 1; }
    }
    out_index[r * ldo + j] = index;
    out_plane[r * ldo + j] = plane;
  }
}

__global__ void paged_row_scatter_kernel(uint8_t* __restrict__ pool, long long pool_rows, int row_bytes,
                                         const int* __restrict__ block_table, int max_blocks, int num_seqs,
                                         int page_size, const int* __restrict__ row_seq,
                                         const int* __restrict__ positions, const uint8_t* __restrict__ src,
                                         long long lds, int rows, DeviceStatus* st) {
  pdl_launch_dependents();
  pdl_wait();
  const int vec = row_bytes / 16;
  const long long n = static_cast<long long>(rows) * vec;
  for (long long i = gtid(); i < n; i += gstride()) {
    const int r = static_cast<int>(i / vec), c = static_cast<int>(i - static_cast<long long>(r) * vec);
    const int seq = row_seq[r], pos = positions[r];
    if (pos < 0) continue;                                   // padding row
    const int blk = pos / page_size;
    long long slot = -1;
    if (seq >= 0 && seq < num_seqs && blk < max_blocks) {
      const int page = block_table[static_cast<long long>(seq) * max_blocks + blk];
      if (page >= 0) slot = static_cast<long long>(page) * page_size + pos % page_size;
    }
    if (slot < 0 || slot >= pool_rows) {
      if (c == 0) report_status(st, kStatusBadIndex, 0xa2, r, static_cast<uint32_t>(pos));
      continue;
    }
    *reinterpret_cast<uint4*>(pool + slot * row_bytes + c * 16) = *reinterpret_cast<const uint4*>(src + r * lds + c * 16);
  }
}

static inline dim3 grid_for(long long n) {
  long long b = (n + kThreads - 1) / kThreads;
  if (b < 1) b = 1;
  if (b > 1184) b = 1184;                                    // 8 CTAs per SM, grid-stride beyond
  return dim3(static_cast<unsigned>(b));
}

}  // namespace mv
}  // namespace fb

using namespace fb;
using namespace fb::mv;

#define MV_DONE() (cudaGetLastError() == cudaSuccess ? FB_OK : FB_ERR_LAUNCH)

extern "C" int fb_mv_fill(int* dst, long long n, int start, int step, void* stream) {
  if (!dst || n <= 0) return FB_ERR_SHAPE;
  launch_pdl(fill_kernel, grid_for(n), dim3(kThreads), 0, static_cast<cudaStream_t>(stream), dst, n, start, step);
  return MV_DONE();
}

extern "C" int fb_mv_pack_pairs(const int* ids, const float* vals, int* out, int n, void* stream) {
  if (!ids || !vals || !out || n <= 0) return FB_ERR_SHAPE;
  launch_pdl(pack_pairs_kernel, grid_for(n), dim3(kThreads), 0, static_cast<cudaStream_t>(stream), ids, vals, out, n);
  return MV_DONE();
}

extern "C" int fb_mv_index_fill(int* sel, long long lds, int col0, int rows, int width, int mode, const int* positions,
                                const long long* base, const int* idx, long long ldi, void* stream) {
  if (!sel || !base || rows <= 0 || width <= 0 || mode < 0 || mode > 2 || col0 < 0) return FB_ERR_SHAPE;
  if ((mode == 0 && !positions) || (mode != 0 && !idx)) return FB_ERR_SHAPE;
  launch_pdl(index_fill_kernel, grid_for(static_cast<long long>(rows) * width), dim3(kThreads), 0,
             static_cast<cudaStream_t>(stream), sel, lds, col0, rows, width, mode, positions, base, idx, ldi);
  return MV_DONE();
}

extern "C" int fb_mv_move_rows(void* dst, long long ldd_bytes, long long dst_row0, const void* src, long long lds_bytes,
                               const int* idx, int rows, int src_rows, int row_bytes, void* status, void* stream) {
  if (!dst || !src || rows <= 0 || row_bytes <= 0 || row_bytes % 16 != 0) return FB_ERR_SHAPE;
  if ((ldd_bytes % 16) || (lds_bytes % 16) || (reinterpret_cast<uintptr_t>(dst) & 15) ||
      (reinterpret_cast<uintptr_t>(src) & 15))
    return FB_ERR_ALIGN;
  launch_pdl(move_rows_kernel, grid_for(static_cast<long long>(rows) * (row_bytes / 16)), dim3(kThreads), 0,
             static_cast<cudaStream_t>(stream), static_cast<uint8_t*>(dst), ldd_bytes, dst_row0,
             static_cast<const uint8_t*>(src), lds_bytes, idx, rows, src_rows, row_bytes, static_cast<DeviceStatus*>(status));
  return MV_DONE();
}

extern "C" int fb_mv_scatter_add(float* dst, long long ldd, int dst_rows, const float* src, long long lds,
                                 const int* idx, int rows, int dim, void* status, void* stream) {
  if (!dst || !src || !idx || rows <= 0 || dim <= 0 || dst_rows <= 0) return FB_ERR_SHAPE;
  launch_pdl(scatter_add_kernel, grid_for(static_cast<long long>(rows) * dim), dim3(kThreads), 0,
             static_cast<cudaStream_t>(stream), dst, ldd, dst_rows, src, lds, idx, rows, dim,
             static_cast<DeviceStatus*>(status));
  return MV_DONE();
}

extern "C" int fb_mv_saxpy(float* y, const float* x, float a, long long n, void* stream) {
  if (!y || !x || n <= 0) return FB_ERR_SHAPE;
  launch_pdl(saxpy_kernel, grid_for(n), dim3(kThreads), 0, static_cast<cudaStream_t>(stream), y, x, a, n);
  return MV_DONE();
}

extern "C" int fb_mv_ring_to_logical(const int* slots, long long lds, int rows, int width, int window,
                                     const int* last_position, const int* n_compressed, int* out_index,
                                     int* out_plane, long long ldo, void* stream) {
  if (!slots || !last_position || !n_compressed || !out_index || !out_plane || rows <= 0 || width <= 0 || window <= 0)
    return FB_ERR_SHAPE;
  launch_pdl(ring_to_logical_kernel, grid_for(static_cast<long long>(rows) * width), dim3(kThreads), 0,
             static_cast<cudaStream_t>(stream), slots, lds, rows, width, window, last_position, n_compressed, out_index,
             out_plane, ldo);
  return MV_DONE();
}

extern "C" int fb_mv_paged_row_scatter(void* pool, long long pool_rows, int row_bytes, const int* block_table,
                                       int max_blocks, int num_seqs, int page_size, const int* row_seq,
                                       const int* positions, const void* src, long long lds_bytes, int rows,
                                       void* status, void* stream) {
  if (!pool || !block_table || !row_seq || !positions || !src || rows <= 0 || row_bytes <= 0 || row_bytes % 16 != 0 ||
      page_size <= 0 || max_blocks <= 0 || num_seqs <= 0)
    return FB_ERR_SHAPE;
  if ((lds_bytes % 16) || (reinterpret_cast<uintptr_t>(pool) & 15) || (reinterpret_cast<uintptr_t>(src) & 15))
    return FB_ERR_ALIGN;
  launch_pdl(paged_row_scatter_kernel, grid_for(static_cast<long long>(rows) * (row_bytes / 16)), dim3(kThreads), 0,
             static_cast<cudaStream_t>(stream), static_cast<uint8_t*>(pool), pool_rows, row_bytes, block_table,
             max_blocks, num_seqs, page_size, row_seq, positions, static_cast<const uint8_t*>(src), lds_bytes, rows,
             static_cast<DeviceStatus*>(status));
  return MV_DONE();
}
