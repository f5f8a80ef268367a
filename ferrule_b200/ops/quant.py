"""Launchers for the quantisation / packing kernels (csrc/quant.cu)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ._lib import check, get_lib, ptr, stream_ptr


def quant_fp8_rows(x: torch.Tensor, writeback: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 [rows, n] -> (uint8 e4m3 codes, uint8 UE8M0 scales [rows, n/128]); writeback=True also
    overwrites x with the dequantised values (QAT)."""
    lib = get_lib(True)
    rows, n = x.shape
    q = torch.empty(rows, n, dtype=torch.uint8, device=x.device)
    s = torch.empty(rows, n // 128, dtype=torch.uint8, device=x.device)
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
