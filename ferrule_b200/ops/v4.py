"""ctypes wrappers of the DeepSeek-V4 operator kernels (`csrc/v4_ops.cu`) and of the attention
kernel's explicit-selection mode.  Shapes and math are those of `models/v4.py`, which holds the
PyTorch oracle each wrapper is tested against."""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from ._lib import AttnArgs, check, get_lib, ptr, status_tensor, stream_ptr


def hc_pre(state: torch.Tensor, fn: torch.Tensor, scale: torch.Tensor, base: torch.Tensor, cfg,
           out_fp32: bool = False, head_only: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """state bf16 [T, hc, hidden]; fn fp32 [nmix, hc*hidden] -> (hidden [T, hidden], coeff fp32 [T, nmix])."""
    lib = get_lib(True)
    T, hc, hidden = state.shape
    nmix = hc if head_only else 2 * hc + hc * hc
    assert state.dtype == torch.bfloat16 and state.is_contiguous()
    assert fn.dtype == torch.float32 and fn.shape == (nmix, hc * hidden) and fn.is_contiguous()
    out = torch.empty(T, hidden, dtype=torch.float32 if out_fp32 else torch.bfloat16, device=state.device)
    coeff = torch.empty(T, nmix, dtype=torch.float32, device=state.device)
    chunks = 16 if hc * hidden >= 8192 else 1
    if chunks > 1:
        part, ctr = _hc_scratch(state.device, T, chunks)
        check(lib.fb_hc_pre_split(state.data_ptr(), fn.data_ptr(), scale.data_ptr(), base.data_ptr(), out.data_ptr(),
                                  int(out_fp32), coeff.data_ptr(), T, hc, hidden, nmix, cfg.eps, cfg.norm_eps,
                                  cfg.sinkhorn_iters, chunks, part.data_ptr(), ctr.data_ptr(), stream_ptr()),
              "fb_hc_pre_split")
        return out, coeff
    check(lib.fb_hc_pre(state.data_ptr(), fn.data_ptr(), scale.data_ptr(), base.data_ptr(), out.data_ptr(),
                        int(out_fp32), coeff.data_ptr(), T, hc, hidden, nmix, cfg.eps, cfg.norm_eps,
                        cfg.sinkhorn_iters, stream_ptr()), "fb_hc_pre")
    return out, coeff


_HC_SCRATCH = {}


def _hc_scratch(device, tokens: int, chunks: int):
    """Partial-sum scratch + per-token arrival counters of the split hyper-connection reduction (grown on demand)."""
    key = torch.device(device)
    cur = _HC_SCRATCH.get(key)
    if cur is None or cur[0].numel() < tokens * chunks * 32 or cur[1].numel() < tokens:
        cap = max(tokens, 64)
        cur = (torch.empty(cap * chunks * 32, dtype=torch.float32, device=device),
               torch.zeros(cap, dtype=torch.int32, device=device))
        _HC_SCRATCH[key] = cur
    return cur


def hc_post(hidden: torch.Tensor, residual: torch.Tensor, coeff: torch.Tensor) -> torch.Tensor:
    """hidden bf16 [T, hidden]; residual bf16 [T, hc, hidden]; coeff fp32 [T, 2hc + hc^2] -> bf16 [T, hc, hidden]."""
    lib = get_lib(True)
    T, hc, dim = residual.shape
    assert hidden.dtype == residual.dtype == torch.bfloat16 and hidden.is_contiguous() and residual.is_contiguous()
    assert coeff.shape == (T, 2 * hc + hc * hc) and coeff.dtype == torch.float32
    out = torch.empty_like(residual)
    check(lib.fb_hc_post(hidden.data_ptr(), residual.data_ptr(), coeff.data_ptr(), out.data_ptr(), T, hc, dim,
                         stream_ptr()), "fb_hc_post")
    return out


def compressor_pool(kv: torch.Tensor, gate: torch.Tensor, ape: torch.Tensor, ratio: int, overlap: bool,
                    groups: Optional[int] = None, row0: Optional[int] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """kv, gate fp32 [n_rows, out_dim] projected rows; ape fp32 [ratio, out_dim] -> bf16 [groups, dim] with
    dim = out_dim (no overlap) or out_dim / 2.  `row0` is the row where group 0's window starts
    (default: ratio - window, i.e. the rows are a sequence from position 0)."""
    lib = get_lib(True)
    n_rows, out_dim = kv.shape
    dim = out_dim // 2 if overlap else out_dim
    W = ratio * (2 if overlap else 1)
    assert kv.dtype == gate.dtype == ape.dtype == torch.float32 and kv.stride() == gate.stride() and kv.stride(1) == 1
    assert ape.shape == (ratio, out_dim) and ape.is_contiguous()
    groups = n_rows // ratio if groups is None else groups
    row0 = ratio - W if row0 is None else row0
    if out is None:
        out = torch.empty(groups, dim, dtype=torch.bfloat16, device=kv.device)
    check(lib.fb_compressor_pool(kv.data_ptr(), gate.data_ptr(), kv.stride(0), ape.data_ptr(), out.data_ptr(),
                                 out.stride(0), groups, dim, ratio, W, row0, n_rows, dim if overlap else 0,
                                 stream_ptr()), "fb_compressor_pool")
    return out


def rope_rows(x: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, off: int, rdim: int,
              inverse: bool = False) -> torch.Tensor:
    """In place on x bf16 [rows, heads, head_dim]: rotate x[..., off:off+rdim] (interleaved pairs)."""
    lib = get_lib(True)
    rows, heads, hd = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(2) == 1 and positions.dtype == torch.int32
    assert cos.dtype == sin.dtype == torch.float32 and cos.shape[1] == rdim // 2 and cos.is_contiguous()
    check(lib.fb_rope_rows(x.data_ptr(), x.stride(0), x.stride(1), rows, heads, off, rdim, positions.data_ptr(),
                           cos.data_ptr(), sin.data_ptr(), cos.shape[0], int(inverse),
                           status_tensor(x.device).data_ptr(), stream_ptr()), "fb_rope_rows")
    return x


def indexer_scores(q: torch.Tensor, plane: torch.Tensor, head_w: torch.Tensor,
                   out: Optional[torch.Tensor] = None, use_gemm: Optional[bool] = None,
                   scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q bf16 [queries, heads, d]; plane bf16 [n, d]; head_w fp32 [queries, heads] -> fp32 [queries, n].

    Two paths with the same rounding chain: for a large plane the per-head dots are one tcgen05 GEMM
    ([queries * heads, d] x plane^T -> bf16) followed by the head-reduction kernel; small planes use the SIMT
    kernel that keeps the query heads in shared memory.  `scratch` (bf16 [queries * heads, >= n]) avoids the
    allocation of the GEMM path."""
    lib = get_lib(True)
    Q, H, d = q.shape
    n = plane.shape[0]
    assert q.dtype == plane.dtype == torch.bfloat16 and q.is_contiguous() and plane.stride(1) == 1
    assert head_w.dtype == torch.float32 and head_w.shape == (Q, H) and head_w.is_contiguous()
    if out is None:
        out = torch.empty(Q, n, dtype=torch.float32, device=q.device)
    if use_gemm is None:
        use_gemm = n >= 1024 and d % 8 == 0 and plane.stride(0) % 8 == 0
    if use_gemm:
        from . import kernels as K
        np2 = (n + 7) // 8 * 8
        dots = scratch[:Q * H, :np2] if scratch is not None else torch.empty(Q * H, np2, dtype=torch.bfloat16, device=q.device)
        K.gemm(q.view(Q * H, d), plane, out=dots, n_out=n)
        check(lib.fb_indexer_reduce(dots.data_ptr(), dots.stride(0), head_w.data_ptr(), out.data_ptr(), out.stride(0),
                                    Q, H, n, stream_ptr()), "fb_indexer_reduce")
        return out
    check(lib.fb_indexer_scores(q.data_ptr(), plane.data_ptr(), plane.stride(0), head_w.data_ptr(), out.data_ptr(),
                                out.stride(0), Q, H, d, n, stream_ptr()), "fb_indexer_scores")
    return out


def indexer_topk(scores: torch.Tensor, k: int, n_visible: Optional[torch.Tensor] = None) -> torch.Tensor:
    """scores fp32 [queries, n] holding bf16 values -> int32 [queries, k]; rows past n_visible[q] are not eligible."""
    lib = get_lib(True)
    Q, n = scores.shape
    assert scores.dtype == torch.float32 and scores.stride(1) == 1 and k <= 512
    if n_visible is not None:
        assert n_visible.dtype == torch.int32 and n_visible.numel() == Q
    out = torch.empty(Q, k, dtype=torch.int32, device=scores.device)
    check(lib.fb_indexer_topk(scores.data_ptr(), scores.stride(0), ptr(n_visible), n, k, out.data_ptr(), out.stride(0),
                              Q, stream_ptr()), "fb_indexer_topk")
    return out


def sparse_sink_attention(q: torch.Tensor, table: torch.Tensor, selection: torch.Tensor, kv_lora: int, rope_dim: int,
                          scale: float, sink: Optional[torch.Tensor] = None, splits: int = 1,
                          out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q bf16 [rows, heads, D]; table bf16 [n, D]; selection int32 [rows, W] (pool rows, -1 = masked).
    `splits` in (1, 2, 4, 8): the splits of one query merge on chip through a thread-block cluster."""
    lib = get_lib(True)
    rows, heads, D = q.shape
    W = selection.shape[1]
    assert D == kv_lora + rope_dim and q.stride(2) == 1 and q.stride(1) == D
    assert selection.dtype == torch.int32 and selection.is_contiguous() and table.is_contiguous()
    if out is None:
        out = torch.empty(rows, heads, kv_lora, dtype=torch.bfloat16, device=q.device)
    a = AttnArgs()
    a.q, a.kv, a.out = q.data_ptr(), table.data_ptr(), out.data_ptr()
    a.sink = ptr(sink)
    a.status = status_tensor(q.device).data_ptr()
    a.ldq, a.ldo = q.stride(0), out.stride(0)
    a.pool_rows = table.numel() // D
    a.rows, a.heads, a.kv_lora, a.rope_dim = rows, heads, kv_lora, rope_dim
    a.group_rows, a.splits = 1, splits
    a.split_tokens = ((W + splits - 1) // splits + 63) // 64 * 64
    a.softmax_scale = scale
    a.selection, a.sel_width = selection.data_ptr(), W
    check(lib.fb_mla_attention(C.byref(a), stream_ptr()), "fb_mla_attention(selection)")
    return out


class MarkovScratch:
    def __init__(self, device, chunks: int = 296):
        self.chunks = chunks
        self.part_val = torch.empty(chunks, dtype=torch.float32, device=device)
        self.part_id = torch.empty(chunks, dtype=torch.int32, device=device)
        self.ctr = torch.zeros(1, dtype=torch.int32, device=device)


def markov_head(logits: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, anchor: torch.Tensor,
                scratch: Optional[MarkovScratch] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """logits fp32 [gamma, vocab]; w1, w2 bf16 [vocab, rank]; anchor int32 [1] on the device.  One launch per
    draft step; each step reads the previous draft from device memory.  Returns (ids [gamma], values [gamma])."""
    lib = get_lib(True)
    gamma, vocab = logits.shape
    rank = w1.shape[1]
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and w1.dtype == w2.dtype == torch.bfloat16
    assert w1.is_contiguous() and w2.is_contiguous() and anchor.dtype == torch.int32
    scratch = scratch or MarkovScratch(logits.device)
    ids = torch.empty(gamma, dtype=torch.int32, device=logits.device)
    vals = torch.empty(gamma, dtype=torch.float32, device=logits.device)
    st = status_tensor(logits.device).data_ptr()
    for j in range(gamma):
        prev = anchor if j == 0 else ids[j - 1:j]
        check(lib.fb_markov_step(logits[j].data_ptr(), w1.data_ptr(), w2.data_ptr(), vocab, rank, scratch.chunks,
                                 prev.data_ptr(), scratch.part_val.data_ptr(), scratch.part_id.data_ptr(),
                                 scratch.ctr.data_ptr(), ids[j:j + 1].data_ptr(), vals[j:j + 1].data_ptr(), st,
                                 stream_ptr()), "fb_markov_step")
    return ids, vals


def hc_mean_scatter(state: torch.Tensor, taps: torch.Tensor, tap_index: int) -> torch.Tensor:
    """state bf16 [T, hc, hidden] -> taps[:, tap_index * hidden : +hidden] = bf16(mean over hc)."""
    lib = get_lib(True)
    T, hc, hidden = state.shape
    assert state.is_contiguous() and state.dtype == taps.dtype == torch.bfloat16 and taps.stride(1) == 1
    check(lib.fb_hc_mean_scatter(state.data_ptr(), taps.data_ptr(), taps.stride(0), tap_index * hidden, T, hc, hidden,
                                 stream_ptr()), "fb_hc_mean_scatter")
    return taps
