"""Launchers of the data-mover kernels (csrc/data_movers.cu): the index fills and row copies between the
compute kernels of a step, so that a step launches no library kernel.

Role of the reference's twelve `data_kernel` kinds
(crates/ferrule-backend/native/cuda/implementations/portable/entrypoints.cu:478-629).
"""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import check, get_lib, status_tensor, stream_ptr


def fill_(t: torch.Tensor, value: int = 0) -> torch.Tensor:
    """int32 tensor (contiguous) <- value."""
    assert t.dtype == torch.int32 and t.is_contiguous()
    check(get_lib(True).fb_mv_fill(t.data_ptr(), t.numel(), value, 0, stream_ptr()), "fb_mv_fill")
    return t


def iota_(t: torch.Tensor, start: int = 0, step: int = 1) -> torch.Tensor:
    assert t.dtype == torch.int32 and t.is_contiguous()
    check(get_lib(True).fb_mv_fill(t.data_ptr(), t.numel(), start, step, stream_ptr()), "fb_mv_fill")
    return t


def pack_pairs(ids: torch.Tensor, vals: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """(int32 ids, fp32 values) -> interleaved int32 [n, 2] (value bits in the second word)."""
    n = ids.numel()
    if out is None:
        out = torch.empty(n, 2, dtype=torch.int32, device=ids.device)
    check(get_lib(True).fb_mv_pack_pairs(ids.data_ptr(), vals.data_ptr(), out.data_ptr(), n, stream_ptr()),
          "fb_mv_pack_pairs")
    return out


def window_index_fill(sel: torch.Tensor, col0: int, window: int, positions: torch.Tensor, base: torch.Tensor) -> None:
    """sel[r, col0 + j] = base[r] + p if p = positions[r] - (window - 1 - j) >= 0 else -1."""
    assert sel.dtype == torch.int32 and base.dtype == torch.int64 and positions.dtype == torch.int32
    check(get_lib(True).fb_mv_index_fill(sel.data_ptr(), sel.stride(0), col0, sel.shape[0], window, 0,
                                         positions.data_ptr(), base.data_ptr(), None, 0, stream_ptr()),
          "fb_mv_index_fill")


def offset_index_fill(sel: torch.Tensor, col0: int, idx: torch.Tensor, base: torch.Tensor) -> None:
    """sel[r, col0 + j] = base[r] + idx[r, j] where idx >= 0 else -1 (top-k lists)."""
    assert sel.dtype == torch.int32 and idx.dtype == torch.int32 and base.dtype == torch.int64
    check(get_lib(True).fb_mv_index_fill(sel.data_ptr(), sel.stride(0), col0, sel.shape[0], idx.shape[1], 1, None,
                                         base.data_ptr(), idx.data_ptr(), idx.stride(0), stream_ptr()),
          "fb_mv_index_fill")


def count_index_fill(sel: torch.Tensor, col0: int, width: int, counts: torch.Tensor, base: torch.Tensor) -> None:
    """sel[r, col0 + j] = base[r] + j for j < counts[r] else -1 (every visible row)."""
    assert sel.dtype == torch.int32 and counts.dtype == torch.int32 and base.dtype == torch.int64
    check(get_lib(True).fb_mv_index_fill(sel.data_ptr(), sel.stride(0), col0, sel.shape[0], width, 2, None,
                                         base.data_ptr(), counts.data_ptr(), 0, stream_ptr()), "fb_mv_index_fill")


def _row_bytes(t: torch.Tensor) -> int:
    assert t.dim() == 2 and t.stride(1) == 1
    return t.shape[1] * t.element_size()


def copy_rows(dst: torch.Tensor, dst_row0: int, src: torch.Tensor) -> None:
    """dst[dst_row0 : dst_row0 + rows] = src (rows of the same width, multiple of 16 bytes)."""
    rb = _row_bytes(src)
    assert _row_bytes(dst) == rb and dst_row0 + src.shape[0] <= dst.shape[0]
    es = src.element_size()
    check(get_lib(True).fb_mv_move_rows(dst.data_ptr(), dst.stride(0) * es, dst_row0, src.data_ptr(), src.stride(0) * es,
                                        None, src.shape[0], src.shape[0], rb, status_tensor(src.device).data_ptr(),
                                        stream_ptr()), "fb_mv_move_rows")


def gather_rows(src: torch.Tensor, idx: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r] = src[idx[r]] (idx int32)."""
    rb = _row_bytes(src)
    assert _row_bytes(out) == rb and idx.dtype == torch.int32 and out.shape[0] >= idx.shape[0]
    es = src.element_size()
    check(get_lib(True).fb_mv_move_rows(out.data_ptr(), out.stride(0) * es, 0, src.data_ptr(), src.stride(0) * es,
                                        idx.data_ptr(), idx.shape[0], src.shape[0], rb,
                                        status_tensor(src.device).data_ptr(), stream_ptr()), "fb_mv_move_rows")
    return out


def scatter_add_rows(dst: torch.Tensor, idx: torch.Tensor, src: torch.Tensor) -> None:
    """dst[idx[r]] += src[r] (fp32, atomic)."""
    assert dst.dtype == torch.float32 and src.dtype == torch.float32 and idx.dtype == torch.int32
    check(get_lib(True).fb_mv_scatter_add(dst.data_ptr(), dst.stride(0), dst.shape[0], src.data_ptr(), src.stride(0),
                                          idx.data_ptr(), src.shape[0], src.shape[1],
                                          status_tensor(src.device).data_ptr(), stream_ptr()), "fb_mv_scatter_add")


def saxpy_(y: torch.Tensor, x: torch.Tensor, a: float) -> torch.Tensor:
    assert y.dtype == torch.float32 and x.dtype == torch.float32 and y.is_contiguous() and x.is_contiguous()
    check(get_lib(True).fb_mv_saxpy(y.data_ptr(), x.data_ptr(), a, y.numel(), stream_ptr()), "fb_mv_saxpy")
    return y


def ring_to_logical(slots: torch.Tensor, window: int, last_position: torch.Tensor, n_compressed: torch.Tensor):
    """Combined-ring slots [rows, w] -> (logical index, plane selector), -1 / -1 where invalid."""
    idx = torch.empty_like(slots)
    plane = torch.empty_like(slots)
    check(get_lib(True).fb_mv_ring_to_logical(slots.data_ptr(), slots.stride(0), slots.shape[0], slots.shape[1], window,
                                              last_position.data_ptr(), n_compressed.data_ptr(), idx.data_ptr(),
                                              plane.data_ptr(), idx.stride(0), stream_ptr()), "fb_mv_ring_to_logical")
    return idx, plane


def paged_row_scatter(pool_rows: torch.Tensor, block_table: torch.Tensor, row_seq: torch.Tensor,
                      positions: torch.Tensor, src: torch.Tensor, page_size: int) -> None:
    """pool_rows [n_pool_rows, width]: row r of `src` goes to the pool row of (row_seq[r], positions[r]) according
    to the page lists in `block_table` (positions < 0 are padding rows)."""
    rb = _row_bytes(src)
    assert _row_bytes(pool_rows) == rb and pool_rows.is_contiguous()
    es = src.element_size()
    check(get_lib(True).fb_mv_paged_row_scatter(pool_rows.data_ptr(), pool_rows.shape[0], rb, block_table.data_ptr(),
                                                block_table.shape[1], block_table.shape[0], page_size,
                                                row_seq.data_ptr(), positions.data_ptr(), src.data_ptr(),
                                                src.stride(0) * es, src.shape[0], status_tensor(src.device).data_ptr(),
                                                stream_ptr()), "fb_mv_paged_row_scatter")
