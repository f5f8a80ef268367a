"""Launchers for the quantisation / packing kernels (csrc/quant.cu)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

import ctypes as C

from ._lib import check, get_lib, status_tensor, stream_ptr


def quant_fp8_rows(x: torch.Tensor, writeback: bool = False,
                   out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 [rows, n] -> (uint8 e4m3 codes, uint8 UE8M0 scales [rows, n/128]); writeback=True also
    overwrites x with the dequantised values (QAT).  `out` = preallocated (codes, scales) views."""
    lib = get_lib(True)
    rows, n = x.shape
    assert n % 128 == 0 and x.stride(1) == 1
    if out is None:
        q = torch.empty(rows, n, dtype=torch.uint8, device=x.device)
        s = torch.empty(rows, n // 128, dtype=torch.uint8, device=x.device)
    else:
        q, s = out
        assert q.shape == (rows, n) and s.shape == (rows, n // 128) and q.stride(1) == 1 and s.stride(1) == 1
    check(lib.fb_quant_fp8_rows(x.data_ptr(), x.stride(0), q.data_ptr(), q.stride(0), s.data_ptr(), s.stride(0), rows, n,
                                1 if writeback else 0, stream_ptr()), "fb_quant_fp8_rows")
    return q, s


def fp8_qat_(x: torch.Tensor) -> torch.Tensor:
    lib = get_lib(True)
    rows, n = x.shape
    check(lib.fb_quant_fp8_rows(x.data_ptr(), x.stride(0), None, 4, None, 0, rows, n, 1, stream_ptr()), "fb_quant_fp8_rows")
    return x


def dequant_fp8_block(q: torch.Tensor, scale: torch.Tensor, block: int = 128) -> torch.Tensor:
    lib = get_lib(True)
    rows, cols = q.shape
    out = torch.empty(rows, cols, dtype=torch.bfloat16, device=q.device)
    check(lib.fb_dequant_fp8_block(q.data_ptr(), scale.data_ptr(), out.data_ptr(), rows, cols, block, stream_ptr()),
          "fb_dequant_fp8_block")
    return out


def quant_mxfp4_rows(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    lib = get_lib(True)
    rows, n = x.shape
    p = torch.empty(rows, n // 2, dtype=torch.uint8, device=x.device)
    s = torch.empty(rows, n // 32, dtype=torch.uint8, device=x.device)
    check(lib.fb_quant_mxfp4_rows(x.data_ptr(), x.stride(0), p.data_ptr(), s.data_ptr(), rows, n, stream_ptr()),
          "fb_quant_mxfp4_rows")
    return p, s


def dequant_mxfp4(packed: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    lib = get_lib(True)
    rows, half = packed.shape
    out = torch.empty(rows, half * 2, dtype=torch.bfloat16, device=packed.device)
    check(lib.fb_dequant_mxfp4(packed.data_ptr(), scale.data_ptr(), out.data_ptr(), rows, half * 2, stream_ptr()),
          "fb_dequant_mxfp4")
    return out


def hadamard_(x: torch.Tensor) -> torch.Tensor:
    lib = get_lib(True)
    rows, n = x.shape
    check(lib.fb_hadamard_rows(x.data_ptr(), x.stride(0), rows, n, stream_ptr()), "fb_hadamard_rows")
    return x


class GemmFp8Args(C.Structure):
    _fields_ = [
        ("w", C.c_void_p), ("x", C.c_void_p), ("w_scale", C.c_void_p), ("x_scale", C.c_void_p), ("out", C.c_void_p),
        ("ldw", C.c_longlong), ("w_group_stride", C.c_longlong), ("ldx", C.c_longlong), ("ldxs", C.c_longlong),
        ("ldo", C.c_longlong),
        ("n_out", C.c_int), ("k", C.c_int), ("groups", C.c_int), ("w_rows_per_group", C.c_int), ("x_rows", C.c_int),
        ("ntok", C.c_int), ("epilogue", C.c_int), ("dual_offset", C.c_int), ("out_fp32", C.c_int),
        ("max_tok_tiles", C.c_int),
        ("tile_group", C.c_void_p), ("tile_row0", C.c_void_p), ("tile_rows", C.c_void_p), ("num_tok_tiles", C.c_void_p),
        ("dst_row", C.c_void_p), ("row_scale", C.c_void_p), ("act_limit", C.c_float), ("scale_group32", C.c_int),
        ("status", C.c_void_p),
        ("slot_cnt", C.c_void_p), ("slot_rows", C.c_int), ("out_scale", C.c_void_p), ("ldos", C.c_longlong),
    ]


def gemm_fp8(xq: torch.Tensor, xs: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor, out: Optional[torch.Tensor] = None,
             *, out_dtype=torch.bfloat16, epilogue: int = 0, plan=None, scatter_rows: Optional[int] = None,
             act_limit: float = 0.0, ntok: Optional[int] = None, group32: bool = False,
             slots=None, out_q=None) -> torch.Tensor:
    """Block-scaled FP8 GEMM on the tcgen05 path.

    xq uint8 e4m3 [rows, K] + xs UE8M0 [rows, K/128]; wq uint8 e4m3 [N, K] or [groups, N, K] + ws UE8M0
    [(groups,) ceil(N/128), ceil(K/128)].  epilogue 0 store, 1 SwiGLU (rows = [gate | up]), 2 scatter (plan).
    slots = (counts int32 [groups], slot_rows): static row slots instead of the plan's tile table - group g owns
    rows [g * slot_rows, (g + 1) * slot_rows), counts[g] of them are filled, groups without rows are skipped (the
    plan still supplies the scatter tables).  out_q = (codes u8 [rows, n_out], scales u8 [rows, n_out / 128]): the
    result leaves as 1 x 128 FP8 (what `quant_fp8_rows` makes of the bf16 result) instead of bf16.
    """
    lib = get_lib(True)
    if not hasattr(lib.fb_gemm_fp8, "_declared"):
        lib.fb_gemm_fp8.argtypes = [C.POINTER(GemmFp8Args), C.c_void_p]
        lib.fb_gemm_fp8.restype = C.c_int
        lib.fb_gemm_fp8._declared = True
    if wq.dim() == 2:
        wq, ws = wq.unsqueeze(0), ws.unsqueeze(0)
    groups, w_rows, K = wq.shape
    rows = xq.shape[0]
    dual = epilogue == 1
    n_out = w_rows // 2 if dual else w_rows
    if ntok is None:
        ntok = (plan.ntok if (plan is not None and slots is None)
                else (16 if (rows <= 16 or (slots is not None and slots[1] == 16))
                      else (32 if (rows <= 32 or dual or group32 or slots is not None) else 64)))
    out_s = None
    if out_q is not None:
        out, out_s = out_q
        assert out.dtype == torch.uint8 and out_s.dtype == torch.uint8 and out.shape[1] == n_out
    if out is None:
        orow = scatter_rows if (epilogue == 2 and scatter_rows) else rows
        out = torch.empty(orow, n_out, dtype=out_dtype, device=xq.device)
    a = GemmFp8Args()
    a.w, a.x, a.w_scale, a.x_scale, a.out = wq.data_ptr(), xq.data_ptr(), ws.data_ptr(), xs.data_ptr(), out.data_ptr()
    a.ldw, a.w_group_stride, a.ldx, a.ldxs, a.ldo = wq.stride(1), wq.stride(0), xq.stride(0), xs.stride(0), out.stride(0)
    a.n_out, a.k, a.groups, a.w_rows_per_group, a.x_rows = n_out, K, groups, w_rows, rows
    a.ntok, a.epilogue, a.dual_offset = ntok, epilogue, (w_rows // 2 if dual else 0)
    a.out_fp32 = 1 if out.dtype == torch.float32 else 0
    a.act_limit = act_limit
    a.scale_group32 = 1 if group32 else 0
    if plan is not None and slots is None:
        a.max_tok_tiles = plan.max_tiles
        a.tile_group, a.tile_row0, a.tile_rows = plan.tile_group.data_ptr(), plan.tile_row0.data_ptr(), plan.tile_rows.data_ptr()
        a.num_tok_tiles = plan.meta.data_ptr()
    if plan is not None and epilogue == 2:
        a.dst_row, a.row_scale = plan.dst_row.data_ptr(), plan.row_scale.data_ptr()
    if slots is not None:
        cnt, slot_rows = slots
        assert cnt.dtype == torch.int32 and cnt.numel() >= groups and slot_rows % ntok == 0
        a.slot_cnt, a.slot_rows = cnt.data_ptr(), slot_rows
    if out_s is not None:
        a.out_scale, a.ldos = out_s.data_ptr(), out_s.stride(0)
    a.status = status_tensor(xq.device).data_ptr()
    check(lib.fb_gemm_fp8(C.byref(a), stream_ptr()), "fb_gemm_fp8")
    return out


def mxfp4_to_e4m3_containers(packed: torch.Tensor) -> torch.Tensor:
    """Packed e2m1 [.., n/2] -> uint8 e4m3 codes [.., n] holding exactly the same values (load-time expansion
    for the group-scaled FP8 GEMM)."""
    from ..io import encoding as enc
    return enc.e4m3_encode(enc.fp4_unpack(packed))


# ---------------------------------------------------------------------------------------------------
# native MXFP4 x MXFP8 path (csrc/gemm_mxfp4.cu)
# ---------------------------------------------------------------------------------------------------
class GemmMxfp4Args(C.Structure):
    _fields_ = [
        ("w", C.c_void_p), ("x", C.c_void_p), ("w_sf", C.c_void_p), ("x_scale", C.c_void_p), ("out", C.c_void_p),
        ("out_scale", C.c_void_p),
        ("ldw_bytes", C.c_longlong), ("w_group_stride_bytes", C.c_longlong), ("ldx", C.c_longlong),
        ("ldxs", C.c_longlong), ("ldo", C.c_longlong), ("ldos", C.c_longlong),
        ("n_out", C.c_int), ("k", C.c_int), ("groups", C.c_int), ("w_rows_per_group", C.c_int), ("x_rows", C.c_int),
        ("ntok", C.c_int), ("epilogue", C.c_int), ("dual_offset", C.c_int), ("out_mode", C.c_int),
        ("max_tok_tiles", C.c_int),
        ("tile_group", C.c_void_p), ("tile_row0", C.c_void_p), ("tile_rows", C.c_void_p), ("num_tok_tiles", C.c_void_p),
        ("dst_row", C.c_void_p), ("row_scale", C.c_void_p), ("act_limit", C.c_float), ("status", C.c_void_p),
        ("w_tiled", C.c_int), ("w_fp8", C.c_int), ("slot_cnt", C.c_void_p), ("slot_rows", C.c_int),
    ]


def mxfp4_tile_major(packed: torch.Tensor) -> torch.Tensor:
    """Packed e2m1 weights [groups, rows, k/2] -> tile-major [groups, ceil(rows/128), k/128, 128, 64]: every
    (128 rows x 128 k) tile the GEMM loads is 8 KB of consecutive memory (rows padded with zeros)."""
    if packed.dim() == 2:
        packed = packed.unsqueeze(0)
    G, rows, half = packed.shape
    assert half % 64 == 0
    rt = (rows + 127) // 128
    if rt * 128 != rows:
        packed = torch.nn.functional.pad(packed, (0, 0, 0, rt * 128 - rows))
    return packed.view(G, rt, 128, half // 64, 64).permute(0, 1, 3, 2, 4).contiguous()


def _mx_lib():
    lib = get_lib(True)
    if not hasattr(lib.fb_gemm_mxfp4, "_declared"):
        vp, i, ll = C.c_void_p, C.c_int, C.c_longlong
        lib.fb_gemm_mxfp4.argtypes = [C.POINTER(GemmMxfp4Args), vp]
        lib.fb_gemm_mxfp4.restype = i
        lib.fb_mxfp4_prepare_sf.argtypes = [vp, vp, i, i, i, vp]
        lib.fb_mxfp4_prepare_sf.restype = i
        lib.fb_quant_mxfp8_rows.argtypes = [vp, ll, vp, ll, vp, ll, i, i, vp]
        lib.fb_quant_mxfp8_rows.restype = i
        lib.fb_gemm_mxfp4._declared = True
    return lib


def quant_mxfp8_rows(x: torch.Tensor, out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None
                     ) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 [rows, n] -> (uint8 e4m3 codes [rows, n], uint8 UE8M0 scales [rows, n/32]): MXFP8, 1 x 32 blocks."""
    lib = _mx_lib()
    rows, n = x.shape
    assert n % 128 == 0 and x.stride(1) == 1
    if out is None:
        q = torch.empty(rows, n, dtype=torch.uint8, device=x.device)
        s = torch.empty(rows, n // 32, dtype=torch.uint8, device=x.device)
    else:
        q, s = out
        assert q.shape == (rows, n) and s.shape == (rows, n // 32) and q.stride(1) == 1 and s.stride(1) == 1
    check(lib.fb_quant_mxfp8_rows(x.data_ptr(), x.stride(0), q.data_ptr(), q.stride(0), s.data_ptr(), s.stride(0),
                                  rows, n, stream_ptr()), "fb_quant_mxfp8_rows")
    return q, s


def mxfp4_prepare_sf(scale: torch.Tensor) -> torch.Tensor:
    """Weight scales UE8M0 [groups, rows, k/32] (or [rows, k/32]) -> the block layout the MXFP4 GEMM copies to
    TMEM: [groups, ceil(rows/128), k/128, 512] bytes."""
    lib = _mx_lib()
    if scale.dim() == 2:
        scale = scale.unsqueeze(0)
    scale = scale.contiguous()
    G, rows, kb32 = scale.shape
    k = kb32 * 32
    assert k % 128 == 0
    out = torch.empty(G, (rows + 127) // 128, k // 128, 512, dtype=torch.uint8, device=scale.device)
    check(lib.fb_mxfp4_prepare_sf(scale.data_ptr(), out.data_ptr(), G, rows, k, stream_ptr()), "fb_mxfp4_prepare_sf")
    return out


def gemm_mxfp4(xq: torch.Tensor, xs: torch.Tensor, w_packed: torch.Tensor, w_sf: torch.Tensor,
               out: Optional[torch.Tensor] = None, *, out_dtype=torch.bfloat16, epilogue: int = 0, plan=None,
               scatter_rows: Optional[int] = None, act_limit: float = 0.0, ntok: Optional[int] = None,
               out_mx: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, w_rows: Optional[int] = None,
               w_fp8: bool = False, slots=None) -> torch.Tensor:
    """MXFP4 (or, with `w_fp8`, e4m3) weights x MXFP8 activations on `tcgen05.mma kind::mxf8f6f4.block_scale`.

    w_fp8: `w_packed` holds e4m3 codes [groups, N, K], one byte per value, and `w_sf` their scales in the same
    per-32 layout (`fp8_block_sf` replicates a checkpoint's 128 x 128 block scales into it): the tensor core
    applies weight and activation scales itself, nothing is rescaled between k-blocks.
    slots = (counts int32 [groups], slot_rows): static row slots walked in `ntok`-row tiles instead of the plan's
    tile table (groups and sub-tiles without rows are skipped; the plan still supplies the scatter tables).

    xq uint8 e4m3 [rows, K] + xs UE8M0 [rows, K/32]; w_packed uint8 [groups, N, K/2] (two e2m1 per byte, low
    nibble first) + w_sf from `mxfp4_prepare_sf`.  epilogue 0 store, 1 SwiGLU (rows = [gate | up]), 2 scatter
    (plan).  `out_mx` = (codes [rows, n_out] uint8, scales [rows, n_out/32] uint8): the result is re-quantised
    to MXFP8 in the epilogue instead of being stored as bf16."""
    lib = _mx_lib()
    tiled = w_packed.dim() == 5            # from `mxfp4_tile_major`; `w_rows` = weight rows per group before padding
    if tiled:
        groups, rt, kb, _, _ = w_packed.shape
        K = kb * 128
        w_rows = rt * 128 if w_rows is None else w_rows
        half = K // 2
    else:
        if w_packed.dim() == 2:
            w_packed = w_packed.unsqueeze(0)
        groups, w_rows, half = w_packed.shape
        K = half if w_fp8 else half * 2
    rows = xq.shape[0]
    dual = epilogue == 1
    n_out = w_rows // 2 if dual else w_rows
    if ntok is None:
        ntok = plan.ntok if plan is not None else (16 if rows <= 16 else (32 if rows <= 32 else 64))
    a = GemmMxfp4Args()
    if out_mx is not None:
        oq, osc = out_mx
        assert oq.dtype == torch.uint8 and osc.dtype == torch.uint8 and oq.shape[1] == n_out
        a.out, a.out_scale, a.ldo, a.ldos, a.out_mode = oq.data_ptr(), osc.data_ptr(), oq.stride(0), osc.stride(0), 2
        out = oq
    else:
        if out is None:
            orow = scatter_rows if (epilogue == 2 and scatter_rows) else rows
            out = torch.empty(orow, n_out, dtype=out_dtype, device=xq.device)
        a.out, a.ldo = out.data_ptr(), out.stride(0)
        a.out_mode = 1 if out.dtype == torch.float32 else 0
    a.w, a.x, a.w_sf, a.x_scale = w_packed.data_ptr(), xq.data_ptr(), w_sf.data_ptr(), xs.data_ptr()
    if tiled:
        a.w_tiled, a.ldw_bytes, a.w_group_stride_bytes = 1, 64, w_packed.stride(0)
    else:
        a.ldw_bytes, a.w_group_stride_bytes = w_packed.stride(1), w_packed.stride(0)
    a.w_fp8 = 1 if w_fp8 else 0
    if slots is not None:
        cnt, slot_rows = slots
        assert cnt.dtype == torch.int32 and cnt.numel() >= groups and slot_rows % ntok == 0
        a.slot_cnt, a.slot_rows = cnt.data_ptr(), slot_rows
    a.ldx, a.ldxs = xq.stride(0), xs.stride(0)
    a.n_out, a.k, a.groups, a.w_rows_per_group, a.x_rows = n_out, K, groups, w_rows, rows
    a.ntok, a.epilogue, a.dual_offset = ntok, epilogue, (w_rows // 2 if dual else 0)
    a.act_limit = act_limit
    if plan is not None and slots is None:
        a.max_tok_tiles = plan.max_tiles
        a.tile_group, a.tile_row0, a.tile_rows = plan.tile_group.data_ptr(), plan.tile_row0.data_ptr(), plan.tile_rows.data_ptr()
        a.num_tok_tiles = plan.meta.data_ptr()
    if plan is not None and epilogue == 2:
        a.dst_row, a.row_scale = plan.dst_row.data_ptr(), plan.row_scale.data_ptr()
    a.status = status_tensor(xq.device).data_ptr()
    check(lib.fb_gemm_mxfp4(C.byref(a), stream_ptr()), "fb_gemm_mxfp4")
    return out


def fp8_block_sf(scale: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    """128 x 128 block scales UE8M0 [groups, ceil(rows/128), ceil(k/128)] (or 2-D) of e4m3 weights -> the per-32
    scale layout of the block-scaled GEMM: every block scale is repeated for its 128 rows and its four 32-column
    slices, so the products are exactly those of the 128 x 128 format (k % 128 == 0)."""
    assert k % 128 == 0
    if scale.dim() == 2:
        scale = scale.unsqueeze(0)
    G = scale.shape[0]
    out = None
    # group by group: the expanded [rows, k / 32] table of all groups at once can be large
    for g in range(G):
        per32 = scale[g].repeat_interleave(128, 0)[:rows].repeat_interleave(4, 1).contiguous()
        sf = mxfp4_prepare_sf(per32)
        if out is None:
            out = torch.empty((G,) + tuple(sf.shape[1:]), dtype=torch.uint8, device=scale.device)
        out[g] = sf[0]
    return out

