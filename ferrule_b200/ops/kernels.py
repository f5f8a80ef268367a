"""Python launchers for the sm_100a kernels.

Each function validates shapes on the host (the library's launchers validate again and
refuse instead of faulting), passes raw pointers through ctypes and launches on the
current torch CUDA stream.  Nothing here allocates unless the caller omitted an output
buffer, so every launcher is safe inside CUDA-graph capture when buffers are preallocated.

The typed-wrapper role matches the reference's operator context
(crates/ferrule-backend/src/cuda/context.rs:5706-6630 linear family, :8893-9955 MoE,
:10987-11630 attention).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from ._lib import AttnArgs, GemmArgs, check, get_lib, ptr, status_tensor, stream_ptr

EPI_STORE, EPI_SWIGLU, EPI_SCATTER, EPI_ALLREDUCE = 0, 1, 2, 3


def pick_ntok(rows: int, dual: bool = False) -> int:
    cap = 128 if dual else 256
    for n in (16, 32, 64, 128, 256):
        if rows <= n and n <= cap:
            return n
    return cap


@dataclass
class MoePlan:
    """Device-resident routing plan (expert-major order + row-tile table)."""
    ntok: int
    max_tiles: int
    cap_rows: int
    src_token: torch.Tensor
    dst_row: torch.Tensor
    row_scale: torch.Tensor
    tile_group: torch.Tensor
    tile_row0: torch.Tensor
    tile_rows: torch.Tensor
    counts: torch.Tensor
    meta: torch.Tensor       # [num_tiles, num_rows]

    @staticmethod
    def allocate(max_routes: int, local_experts: int, ntok: int, device) -> "MoePlan":
        max_tiles = (max_routes + ntok - 1) // ntok + local_experts
        i32 = dict(dtype=torch.int32, device=device)
        return MoePlan(ntok, max_tiles, max_routes,
                       torch.zeros(max_routes, **i32), torch.zeros(max_routes, **i32),
                       torch.zeros(max_routes, dtype=torch.float32, device=device),
                       torch.zeros(max_tiles, **i32), torch.zeros(max_tiles, **i32),
                       torch.zeros(max_tiles, **i32), torch.zeros(local_experts, **i32),
                       torch.zeros(2, **i32))


def _w3(w: torch.Tensor):
    """weights as [groups, rows, k] -> (groups, rows, k, ldw, group_stride)."""
    if w.dim() == 2:
        w = w.unsqueeze(0)
    assert w.dim() == 3 and w.dtype == torch.bfloat16 and w.stride(2) == 1
    return w, w.shape[0], w.shape[1], w.shape[2], w.stride(1), (w.stride(0) if w.shape[0] > 1 else w.shape[1] * w.stride(1))


def gemm(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, *,
         out_dtype=torch.bfloat16, epilogue: int = EPI_STORE, n_out: Optional[int] = None,
         dual_offset: int = 0, plan: Optional[MoePlan] = None, scatter_rows: Optional[int] = None,
         use_row_scale: bool = True, act_limit: float = 0.0, ntok: Optional[int] = None,
         x_group_koff: int = 0, out_group_coff: int = 0, k: Optional[int] = None,
         comm=None, residual: Optional[torch.Tensor] = None, split_k: int = 0,
         trace: Optional[torch.Tensor] = None, ep_combine=None) -> torch.Tensor:
    """out = x @ w^T on the tcgen05 path.

    x [rows, K] bf16 (row stride arbitrary multiple of 8), w [N, K] or [groups, N, K] bf16.
    plan        : grouped mode, x rows are in expert-major order.
    epilogue    : EPI_STORE | EPI_SWIGLU (w rows = [gate block | up block]) | EPI_SCATTER |
                  EPI_ALLREDUCE (comm = a parallel.symm.AllReduceChannel).
    x_group_koff: batched mode (groups > 1 without a plan): group g reads x[:, g*koff : g*koff+K]
                  and writes out[:, g*out_group_coff : +N].
    ep_combine  : EPI_SCATTER only, (rank, world, peer buffers, peer flags, ctr, remap_rank, remap_row, pitch):
                  output row r is stored as bf16 into rank remap_rank[r]'s buffer at row remap_row[r]
                  (expert-parallel combine over peer memory); `out` is then unused.
    """
    lib = get_lib(True)
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
    w, groups, w_rows, wk, ldw, gstride = _w3(w)
    K = wk if k is None else k
    rows = x.shape[0]
    dual = epilogue == EPI_SWIGLU
    if n_out is None:
        n_out = w_rows // 2 if dual else w_rows
    if dual and dual_offset == 0:
        dual_offset = w_rows // 2
    batched = plan is None and groups > 1
    if ntok is None:
        ntok = plan.ntok if plan is not None else pick_ntok(rows, dual)
    if out is None:
        cols = n_out * groups if batched else n_out
        orow = scatter_rows if (epilogue == EPI_SCATTER and scatter_rows) else rows
        out = torch.empty(orow, cols, dtype=out_dtype, device=x.device)
    assert out.stride(-1) == 1
    a = GemmArgs()
    a.w, a.x, a.out = w.data_ptr(), x.data_ptr(), out.data_ptr()
    a.ldw, a.w_group_stride, a.ldx, a.ldo = ldw, gstride, x.stride(0), out.stride(0)
    a.n_out, a.k, a.groups, a.w_rows_per_group = n_out, K, groups, w_rows
    a.x_rows, a.ntok, a.epilogue, a.dual_offset = rows, ntok, epilogue, dual_offset
    a.out_fp32 = 1 if out.dtype == torch.float32 else 0
    a.x_group_koff, a.out_group_coff = x_group_koff, out_group_coff
    a.act_limit = act_limit
    a.force_split = split_k
    a.trace = ptr(trace)
    if plan is not None:
        a.max_tok_tiles = plan.max_tiles
        a.tile_group, a.tile_row0, a.tile_rows = (plan.tile_group.data_ptr(), plan.tile_row0.data_ptr(),
                                                  plan.tile_rows.data_ptr())
        a.num_tok_tiles = plan.meta.data_ptr()
        if epilogue == EPI_SCATTER:
            a.dst_row = plan.dst_row.data_ptr()
            a.row_scale = plan.row_scale.data_ptr() if use_row_scale else None
    if epilogue == EPI_ALLREDUCE:
        comm.fill_gemm_args(a, rows, n_out, ntok)
        if residual is not None:
            a.residual, a.ldr = residual.data_ptr(), residual.stride(0)
    if ep_combine is not None:
        assert epilogue == EPI_SCATTER
        rank, world, bufs, flags, ctr, remap_rank, remap_row, pitch = ep_combine
        a.rank, a.world = rank, world
        for r in range(world):
            a.peer_recv[r], a.peer_flags[r] = bufs[r], flags[r]
        a.local_ctr = ctr.data_ptr()
        a.remap_rank, a.remap_row = remap_rank.data_ptr(), remap_row.data_ptr()
        a.ldo = pitch
    a.status = status_tensor(x.device).data_ptr()
    check(lib.fb_gemm_bf16(C.byref(a), stream_ptr()), "fb_gemm_bf16")
    return out


def embedding(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    lib = get_lib(True)
    rows, dim = ids.shape[0], table.shape[1]
    if out is None:
        out = torch.empty(rows, dim, dtype=torch.bfloat16, device=table.device)
    check(lib.fb_embedding(ids.data_ptr(), table.data_ptr(), out.data_ptr(), rows, dim, table.shape[0],
                           status_tensor(table.device).data_ptr(), stream_ptr()), "fb_embedding")
    return out


def add_rmsnorm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float,
                delta: Optional[torch.Tensor] = None, res_out: Optional[torch.Tensor] = None,
                norm_out: Optional[torch.Tensor] = None, want_norm: bool = True, quant_out=None,
                quant_block: int = 128):
    """(res_out, norm_out): res_out = bf16(x + delta) (if delta), norm_out = RMSNorm(res) * w.
    quant_out = (codes u8 [rows, dim], scales u8 [rows, dim / quant_block]): also the quantised form of norm_out,
    bit-equal to `quant_fp8_rows(norm_out)` (quant_block 128) or `quant_mxfp8_rows(norm_out)` (32): the consumer
    is a block-scaled GEMM and this saves the quantiser launch."""
    lib = get_lib(True)
    rows, dim = x.shape
    if delta is not None and res_out is None:
        res_out = torch.empty_like(x)
    if want_norm and norm_out is None:
        norm_out = torch.empty(rows, dim, dtype=torch.bfloat16, device=x.device)
    if quant_out is not None:
        q, sc = quant_out
        assert want_norm and q.shape[0] >= rows and q.shape[1] == dim and sc.shape[1] >= dim // quant_block
        lib.fb_add_rmsnorm_q.restype = C.c_int
        lib.fb_add_rmsnorm_q.argtypes = [C.c_void_p, C.c_longlong, C.c_void_p, C.c_longlong, C.c_void_p, C.c_void_p,
                                         C.c_longlong, C.c_void_p, C.c_longlong, C.c_int, C.c_int, C.c_float,
                                         C.c_void_p, C.c_longlong, C.c_void_p, C.c_longlong, C.c_int, C.c_void_p]
        check(lib.fb_add_rmsnorm_q(x.data_ptr(), x.stride(0), ptr(delta), delta.stride(0) if delta is not None else 0,
                                   ptr(weight), ptr(res_out), res_out.stride(0) if res_out is not None else 0,
                                   norm_out.data_ptr(), norm_out.stride(0), rows, dim, eps,
                                   q.data_ptr(), q.stride(0), sc.data_ptr(), sc.stride(0), quant_block, stream_ptr()),
              "fb_add_rmsnorm_q")
        return (res_out if delta is not None else x), norm_out
    check(lib.fb_add_rmsnorm(x.data_ptr(), x.stride(0), ptr(delta), delta.stride(0) if delta is not None else 0,
                             ptr(weight), ptr(res_out), res_out.stride(0) if res_out is not None else 0,
                             ptr(norm_out) if want_norm else None,
                             norm_out.stride(0) if (want_norm and norm_out is not None) else 0,
                             rows, dim, eps, stream_ptr()), "fb_add_rmsnorm")
    return (res_out if delta is not None else x), norm_out


def mla_prep(q: torch.Tensor, q_head_dim: int, ckv: torch.Tensor, heads: int, kv_lora: int,
             rope_dim: int, kv_norm_w: torch.Tensor, eps: float, cos: torch.Tensor, sin: torch.Tensor,
             positions: torch.Tensor, write_slot: torch.Tensor, kv_pool_layer: torch.Tensor,
             q_out: torch.Tensor) -> None:
    lib = get_lib(True)
    rows = q.shape[0]
    pool_rows = kv_pool_layer.numel() // (kv_lora + rope_dim)
    check(lib.fb_mla_prep(q.data_ptr(), q.stride(0), q_head_dim, ckv.data_ptr(), ckv.stride(0), heads,
                          kv_lora, rope_dim, kv_norm_w.data_ptr(), eps, cos.data_ptr(), sin.data_ptr(),
                          cos.shape[0], positions.data_ptr(), write_slot.data_ptr(),
                          kv_pool_layer.data_ptr(), pool_rows, q_out.data_ptr(), q_out.stride(0), rows,
                          status_tensor(q.device).data_ptr(), stream_ptr()), "fb_mla_prep")


def router_topk(logits: torch.Tensor, topk: int, score_fn: int, bias: Optional[torch.Tensor] = None,
                n_groups: int = 1, topk_groups: int = 1, normalize: bool = False,
                route_scale: float = 1.0, hash_table: Optional[torch.Tensor] = None,
                token_ids: Optional[torch.Tensor] = None, out_idx: Optional[torch.Tensor] = None,
                out_w: Optional[torch.Tensor] = None):
    lib = get_lib(True)
    rows, experts = logits.shape
    assert logits.dtype == torch.float32
    if out_idx is None:
        out_idx = torch.empty(rows, topk, dtype=torch.int32, device=logits.device)
    if out_w is None:
        out_w = torch.empty(rows, topk, dtype=torch.float32, device=logits.device)
    check(lib.fb_router_topk(logits.data_ptr(), logits.stride(0), ptr(bias), ptr(hash_table),
                             ptr(token_ids), rows, experts, topk, score_fn, n_groups, topk_groups,
                             1 if normalize else 0, route_scale, out_idx.data_ptr(), out_w.data_ptr(),
                             stream_ptr()), "fb_router_topk")
    return out_idx, out_w


def moe_plan(topk_idx: torch.Tensor, topk_w: Optional[torch.Tensor], plan: MoePlan, e_lo: int,
             e_hi: int, dst_slots: int = 0) -> MoePlan:
    lib = get_lib(True)
    rows, topk = topk_idx.shape
    assert rows * topk <= plan.cap_rows
    check(lib.fb_moe_plan(topk_idx.data_ptr(), ptr(topk_w), rows * topk, topk, e_lo, e_hi, plan.ntok, dst_slots,
                          plan.src_token.data_ptr(), plan.dst_row.data_ptr(), plan.row_scale.data_ptr(),
                          plan.tile_group.data_ptr(), plan.tile_row0.data_ptr(), plan.tile_rows.data_ptr(),
                          plan.max_tiles, plan.counts.data_ptr(), plan.meta.data_ptr(),
                          status_tensor(topk_idx.device).data_ptr(), stream_ptr()), "fb_moe_plan")
    return plan


def moe_retile(plan: MoePlan, ntok: int, tiles: Optional[MoePlan] = None) -> MoePlan:
    """A view of `plan` (same expert-major rows, scales and destinations) with row tiles of height `ntok`:
    fills and returns `tiles` (allocated on first use when None)."""
    lib = get_lib(True)
    local = plan.counts.shape[0]
    if tiles is None:
        max_tiles = (plan.cap_rows + ntok - 1) // ntok + local
        i32 = dict(dtype=torch.int32, device=plan.counts.device)
        tiles = MoePlan(ntok, max_tiles, plan.cap_rows, plan.src_token, plan.dst_row, plan.row_scale,
                        torch.zeros(max_tiles, **i32), torch.zeros(max_tiles, **i32), torch.zeros(max_tiles, **i32),
                        plan.counts, torch.zeros(2, **i32))
    lib.fb_moe_retile.restype = C.c_int
    lib.fb_moe_retile.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                  C.c_void_p, C.c_void_p, C.c_void_p]
    check(lib.fb_moe_retile(plan.counts.data_ptr(), local, ntok, tiles.tile_group.data_ptr(),
                            tiles.tile_row0.data_ptr(), tiles.tile_rows.data_ptr(), tiles.max_tiles,
                            tiles.meta.data_ptr(), status_tensor(plan.counts.device).data_ptr(), stream_ptr()),
          "fb_moe_retile")
    return tiles


def l2_prefetch(t: torch.Tensor, nbytes: int) -> None:
    """Ask the memory system to pull the first `nbytes` of `t` into L2 (asynchronous, on the current stream)."""
    lib = get_lib(True)
    nbytes = min(nbytes, t.numel() * t.element_size())
    check(lib.fb_l2_prefetch(t.data_ptr(), nbytes, stream_ptr()), "fb_l2_prefetch")


def gather_rows(x: torch.Tensor, plan: MoePlan, out: torch.Tensor, cap_rows: Optional[int] = None) -> torch.Tensor:
    lib = get_lib(True)
    cap = plan.cap_rows if cap_rows is None else cap_rows
    check(lib.fb_gather_rows(x.data_ptr(), x.stride(0), plan.src_token.data_ptr(), plan.meta.data_ptr(),
                             out.data_ptr(), out.stride(0), cap, x.shape[1], x.shape[0],
                             status_tensor(x.device).data_ptr(), stream_ptr()), "fb_gather_rows")
    return out


def moe_reduce(route_out: torch.Tensor, slots: int, topk: int, topk_idx: torch.Tensor, e_lo: int,
               e_hi: int, rows: int, dim: int, extra: Optional[torch.Tensor] = None,
               residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    lib = get_lib(True)
    if out is None:
        out = torch.empty(rows, dim, dtype=torch.bfloat16, device=route_out.device)
    check(lib.fb_moe_reduce(route_out.data_ptr(), slots, topk, topk_idx.data_ptr(), e_lo, e_hi,
                            ptr(extra), extra.stride(0) if extra is not None else 0, ptr(residual),
                            residual.stride(0) if residual is not None else 0, out.data_ptr(),
                            out.stride(0), 1 if out.dtype == torch.float32 else 0, rows, dim,
                            stream_ptr()), "fb_moe_reduce")
    return out


def moe_reduce_norm(route_out: torch.Tensor, slots: int, topk: int, topk_idx: torch.Tensor, e_lo: int, e_hi: int,
                    rows: int, dim: int, residual: torch.Tensor, out: torch.Tensor, norm_w: torch.Tensor,
                    norm_out: torch.Tensor, eps: float) -> torch.Tensor:
    """`moe_reduce` that also writes RMSNorm(out) * norm_w (bit-equal to `add_rmsnorm` run on `out` afterwards)."""
    lib = get_lib(True)
    check(lib.fb_moe_reduce_norm(route_out.data_ptr(), slots, topk, topk_idx.data_ptr(), e_lo, e_hi,
                                 residual.data_ptr(), residual.stride(0), out.data_ptr(), out.stride(0), rows, dim,
                                 norm_w.data_ptr(), norm_out.data_ptr(), norm_out.stride(0), eps, stream_ptr()),
          "fb_moe_reduce_norm")
    return out


def argmax(logits: torch.Tensor, out_id: Optional[torch.Tensor] = None,
           out_val: Optional[torch.Tensor] = None) -> torch.Tensor:
    lib = get_lib(True)
    rows, vocab = logits.shape
    if out_id is None:
        out_id = torch.empty(rows, dtype=torch.int32, device=logits.device)
    check(lib.fb_argmax(logits.data_ptr(), logits.stride(0), rows, vocab, out_id.data_ptr(), ptr(out_val),
                        stream_ptr()), "fb_argmax")
    return out_id


@dataclass
class ArgmaxScratch:
    chunks: int
    part_val: torch.Tensor
    part_id: torch.Tensor
    row_ctr: torch.Tensor

    @staticmethod
    def allocate(max_rows: int, device, chunks: int = 64) -> "ArgmaxScratch":
        return ArgmaxScratch(chunks, torch.zeros(max_rows * chunks, dtype=torch.float32, device=device),
                             torch.zeros(max_rows * chunks, dtype=torch.int32, device=device),
                             torch.zeros(max_rows, dtype=torch.int32, device=device))


def argmax_chunked(logits: torch.Tensor, scratch: ArgmaxScratch, out_id: torch.Tensor,
                   out_val: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Greedy token with the vocabulary scan spread over rows x chunks CTAs (one launch)."""
    lib = get_lib(True)
    rows, vocab = logits.shape
    assert rows * scratch.chunks <= scratch.part_val.numel()
    check(lib.fb_argmax_chunked(logits.data_ptr(), logits.stride(0), rows, vocab, scratch.chunks,
                                scratch.part_val.data_ptr(), scratch.part_id.data_ptr(),
                                scratch.row_ctr.data_ptr(), out_id.data_ptr(), ptr(out_val), stream_ptr()),
          "fb_argmax_chunked")
    return out_id


def router_plan_fused(x: torch.Tensor, w: torch.Tensor, topk: int, score_fn: int, plan: "MoePlan", e_lo: int,
                      e_hi: int, out_idx: torch.Tensor, out_w: torch.Tensor, done_ctr: torch.Tensor, *,
                      bias: Optional[torch.Tensor] = None, n_groups: int = 1, topk_groups: int = 1,
                      normalize: bool = False, route_scale: float = 1.0,
                      hash_table: Optional[torch.Tensor] = None, token_ids: Optional[torch.Tensor] = None,
                      dst_slots: int = 0) -> None:
    """Router logits + scoring + top-k + MoE plan in one launch (one CTA per token)."""
    lib = get_lib(True)
    rows, hidden = x.shape
    experts = w.shape[0]
    assert rows * topk <= plan.cap_rows and w.is_contiguous()
    check(lib.fb_router_plan_fused(x.data_ptr(), x.stride(0), w.data_ptr(), hidden, ptr(bias), ptr(hash_table),
                                   ptr(token_ids), rows, experts, topk, score_fn, n_groups, topk_groups,
                                   1 if normalize else 0, route_scale, out_idx.data_ptr(), out_w.data_ptr(),
                                   e_lo, e_hi, plan.ntok, dst_slots, plan.src_token.data_ptr(),
                                   plan.dst_row.data_ptr(), plan.row_scale.data_ptr(), plan.tile_group.data_ptr(),
                                   plan.tile_row0.data_ptr(), plan.tile_rows.data_ptr(), plan.max_tiles,
                                   plan.counts.data_ptr(), plan.meta.data_ptr(), done_ctr.data_ptr(),
                                   status_tensor(x.device).data_ptr(), stream_ptr()), "fb_router_plan_fused")


def static_plan(ntok: int, local_experts: int, counts: torch.Tensor, shared: Optional[MoePlan] = None) -> MoePlan:
    """Plan with one row tile per local expert at fixed rows [e * ntok, (e + 1) * ntok); `counts` (the per-expert
    row counters the router fills) doubles as the tile row counts.  `shared` lends its row tables (they are
    rewritten by every router launch, so the layers of a model can share them)."""
    dev = counts.device
    i32 = dict(dtype=torch.int32, device=dev)
    cap = local_experts * ntok
    if shared is None:
        ar = torch.arange(local_experts, **i32)
        return MoePlan(ntok, local_experts, cap, torch.zeros(cap, **i32), torch.zeros(cap, **i32),
                       torch.zeros(cap, dtype=torch.float32, device=dev), ar, ar * ntok, counts, counts,
                       torch.tensor([local_experts, cap], **i32))
    return MoePlan(ntok, local_experts, cap, shared.src_token, shared.dst_row, shared.row_scale, shared.tile_group,
                   shared.tile_row0, counts, counts, shared.meta)


def router_append(x: torch.Tensor, w: torch.Tensor, topk: int, score_fn: int, plan: MoePlan, e_lo: int, e_hi: int,
                  out_idx: torch.Tensor, out_w: torch.Tensor, xg: torch.Tensor, *,
                  bias: Optional[torch.Tensor] = None, n_groups: int = 1, topk_groups: int = 1,
                  normalize: bool = False, route_scale: float = 1.0, hash_table: Optional[torch.Tensor] = None,
                  token_ids: Optional[torch.Tensor] = None, dst_slots: int = 0,
                  norm_w: Optional[torch.Tensor] = None, eps: float = 0.0, delta: Optional[torch.Tensor] = None,
                  res_out: Optional[torch.Tensor] = None, norm_out: Optional[torch.Tensor] = None,
                  quant_rows=None) -> None:
    """Router + top-k + row reservation in a static plan + activation gather, one launch (one CTA per token).
    `plan.counts` must be zero on entry.  With `norm_w` the kernel first forms the row itself: `x` is then the
    residual stream, res_out = bf16(x + delta), norm_out = RMSNorm(res_out) * norm_w (bit-equal to `add_rmsnorm`),
    and the router reads that normalised row.  `quant_rows` = (codes [rows, hidden] u8, scales [rows, c] u8,
    xg codes, xg scales): the gathered rows are the token's quantised codes and scale bytes (`xg` is unused)."""
    lib = get_lib(True)
    rows, hidden = x.shape
    assert rows <= plan.ntok and w.is_contiguous()
    assert plan.max_tiles == e_hi - e_lo
    if quant_rows is not None:
        q, sc, xgq, xgs = quant_rows
        assert xgq.shape[0] >= plan.cap_rows and xgq.shape[1] == hidden and xgs.shape[1] == sc.shape[1]
        check(lib.fb_router_append_q(x.data_ptr(), x.stride(0), ptr(delta), delta.stride(0) if delta is not None else 0,
                                     ptr(norm_w), ptr(res_out), res_out.stride(0) if res_out is not None else 0,
                                     ptr(norm_out), norm_out.stride(0) if norm_out is not None else 0, eps,
                                     w.data_ptr(), hidden, ptr(bias), ptr(hash_table),
                                     ptr(token_ids), rows, w.shape[0], topk, score_fn, n_groups, topk_groups,
                                     1 if normalize else 0, route_scale, out_idx.data_ptr(), out_w.data_ptr(), e_lo,
                                     e_hi, plan.ntok, dst_slots, plan.counts.data_ptr(), plan.src_token.data_ptr(),
                                     plan.dst_row.data_ptr(), plan.row_scale.data_ptr(), None, 8,
                                     q.data_ptr(), q.stride(0), sc.data_ptr(), sc.stride(0), xgq.data_ptr(),
                                     xgq.stride(0), xgs.data_ptr(), xgs.stride(0), sc.shape[1],
                                     status_tensor(x.device).data_ptr(), stream_ptr()), "fb_router_append_q")
        return
    assert xg.shape[0] >= plan.cap_rows and xg.shape[1] == hidden
    check(lib.fb_norm_router_append(x.data_ptr(), x.stride(0), ptr(delta), delta.stride(0) if delta is not None else 0,
                                    ptr(norm_w), ptr(res_out), res_out.stride(0) if res_out is not None else 0,
                                    ptr(norm_out), norm_out.stride(0) if norm_out is not None else 0, eps,
                                    w.data_ptr(), hidden, ptr(bias), ptr(hash_table),
                                    ptr(token_ids), rows, w.shape[0], topk, score_fn, n_groups, topk_groups,
                                    1 if normalize else 0, route_scale, out_idx.data_ptr(), out_w.data_ptr(), e_lo, e_hi,
                                    plan.ntok, dst_slots, plan.counts.data_ptr(), plan.src_token.data_ptr(),
                                    plan.dst_row.data_ptr(), plan.row_scale.data_ptr(), xg.data_ptr(), xg.stride(0),
                                    status_tensor(x.device).data_ptr(), stream_ptr()), "fb_norm_router_append")


def decode_advance(next_id: torch.Tensor, batch, vocab: int, page_size: int, advance: bool) -> None:
    """Feed a decode step's greedy tokens back as the next step's input ids on the device (`batch`: the
    DeviceBatch of the step, one row per sequence).  `advance` also moves positions, visible lengths and KV
    write slots one token on, using the page lists already in `batch.block_table`."""
    lib = get_lib(True)
    rows = batch.token_ids.shape[0]
    check(lib.fb_decode_advance(next_id.data_ptr(), batch.token_ids.data_ptr(), batch.positions.data_ptr(),
                                batch.row_pos.data_ptr(), batch.write_slot.data_ptr(), batch.row_seq.data_ptr(),
                                batch.block_table.data_ptr(), batch.block_table.shape[1], page_size,
                                batch.block_table.shape[0], rows, vocab, 1 if advance else 0, stream_ptr()),
          "fb_decode_advance")


def topk_logits(logits: torch.Tensor, k: int):
    lib = get_lib(True)
    rows, vocab = logits.shape
    ids = torch.empty(rows, k, dtype=torch.int32, device=logits.device)
    vals = torch.empty(rows, k, dtype=torch.float32, device=logits.device)
    check(lib.fb_topk_logits(logits.data_ptr(), logits.stride(0), rows, vocab, k, ids.data_ptr(),
                             vals.data_ptr(), stream_ptr()), "fb_topk_logits")
    return ids, vals


def copy_pages(pool: torch.Tensor, pairs: torch.Tensor) -> None:
    """pool [layers, pages, page_size, D] bf16; pairs int32 [n, 2] = (src page, dst page)."""
    lib = get_lib(True)
    layers, pages = pool.shape[0], pool.shape[1]
    page_elems = pool.stride(1)
    check(lib.fb_copy_pages(pool.data_ptr(), pool.stride(0), page_elems, pairs.data_ptr(), pairs.shape[0],
                            pages, layers, status_tensor(pool.device).data_ptr(), stream_ptr()),
          "fb_copy_pages")


@dataclass
class AttnWorkspace:
    part_o: torch.Tensor
    part_ml: torch.Tensor
    max_rows: int
    splits: int
    merge_ctr: Optional[torch.Tensor] = None      # zeroed int32 [max_rows * head blocks]: in-kernel merge


def prefill_tiles(segments, heads: int, min_rows: int = 1):
    """Tile table of `mla_prefill_tc` and what is left for the row-tile kernel.

    segments: (sequence index, first query row, query rows, position of the first row) per sequence of the batch,
    in row order.  Sequences with at least `min_rows` rows are cut into tiles of 128 / heads consecutive
    positions; -> (tiles [n, 4] int32 numpy array sorted by KV length, longest first, and the list of
    (first row, end row) ranges of the other sequences, merged where adjacent)."""
    import numpy as np
    G = 128 // heads
    tiles, rest = [], []
    for seq, r0, n, p0 in segments:
        if n >= min_rows:
            for o in range(0, n, G):
                tiles.append((seq, r0 + o, min(G, n - o), p0 + o))
        elif rest and rest[-1][1] == r0:
            rest[-1] = (rest[-1][0], r0 + n)
        else:
            rest.append((r0, r0 + n))
    tiles.sort(key=lambda t: -(t[3] + t[2]))
    return np.asarray(tiles, dtype=np.int32).reshape(-1, 4), rest


def prefill_tc_supported(heads: int, kv_lora: int, rope_dim: int, page_size: int) -> bool:
    return (kv_lora == 512 and rope_dim == 64 and 0 < heads <= 128 and 128 % heads == 0
            and page_size >= 8 and page_size & (page_size - 1) == 0)


def mla_prefill_tc(q: torch.Tensor, kv_layer: torch.Tensor, block_table: torch.Tensor, tiles: torch.Tensor,
                   n_tiles: int, page_size: int, kv_lora: int, rope_dim: int, scale: float, out: torch.Tensor,
                   sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Prefill attention on tcgen05: q [rows, heads, 576] bf16 contiguous, tiles [>= n_tiles, 4] int32 on the
    device (see `prefill_tiles`); rows that no tile covers are left untouched in `out` [rows, heads, 512]."""
    lib = get_lib(True)
    rows, heads, D = q.shape
    assert D == kv_lora + rope_dim and q.is_contiguous() and tiles.dtype == torch.int32 and tiles.stride(-1) == 1
    a = _lib.PrefillAttnArgs()
    a.q, a.kv, a.out, a.tiles = q.data_ptr(), kv_layer.data_ptr(), out.data_ptr(), tiles.data_ptr()
    a.block_table, a.sink = block_table.data_ptr(), ptr(sink)
    a.status = status_tensor(q.device).data_ptr()
    a.ldq, a.ldo = q.stride(0), out.stride(0)
    a.pool_rows = kv_layer.numel() // D
    a.n_tiles, a.rows, a.heads, a.kv_lora, a.rope_dim = n_tiles, rows, heads, kv_lora, rope_dim
    a.num_seqs, a.max_blocks, a.page_size = block_table.shape[0], block_table.shape[1], page_size
    a.softmax_scale = scale
    check(lib.fb_mla_prefill_tc(C.byref(a), stream_ptr()), "fb_mla_prefill_tc")
    return out


def mla_attention(q: torch.Tensor, kv_layer: torch.Tensor, block_table: torch.Tensor,
                  row_seq: torch.Tensor, row_pos: torch.Tensor, page_size: int, kv_lora: int,
                  rope_dim: int, scale: float, out: torch.Tensor, *, splits: int = 1,
                  split_tokens: int = 1 << 20, ws: Optional[AttnWorkspace] = None,
                  sink: Optional[torch.Tensor] = None, group_rows: int = 1,
                  trace: Optional[torch.Tensor] = None, decode_only: bool = False) -> torch.Tensor:
    """q [rows, heads, D] bf16; kv_layer [..., D] bf16 (any leading shape, contiguous rows).
    decode_only: one query row per sequence, and every KV row below its position predates the running step
    (the kernel then requests its first KV tile before waiting for the preceding kernel)."""
    lib = get_lib(True)
    rows, heads, D = q.shape
    assert D == kv_lora + rope_dim and q.stride(2) == 1 and q.stride(1) == D
    a = AttnArgs()
    a.q, a.kv, a.out = q.data_ptr(), kv_layer.data_ptr(), out.data_ptr()
    a.block_table, a.row_seq, a.row_pos = block_table.data_ptr(), row_seq.data_ptr(), row_pos.data_ptr()
    a.sink = ptr(sink)
    if splits > 1 and ws is not None:      # ws=None: the splits merge on chip through a thread-block cluster
        assert ws.max_rows >= rows and ws.splits >= splits
        a.part_o, a.part_ml = ws.part_o.data_ptr(), ws.part_ml.data_ptr()
        a.merge_ctr = ptr(ws.merge_ctr)
    a.status = status_tensor(q.device).data_ptr()
    a.ldq, a.ldo = q.stride(0), out.stride(0)
    a.pool_rows = kv_layer.numel() // D
    a.rows, a.heads, a.kv_lora, a.rope_dim = rows, heads, kv_lora, rope_dim
    a.num_seqs, a.max_blocks, a.page_size = block_table.shape[0], block_table.shape[1], page_size
    a.group_rows, a.splits, a.split_tokens = group_rows, splits, split_tokens
    a.softmax_scale = scale
    a.trace = ptr(trace)
    a.decode_only = 1 if (decode_only and group_rows == 1) else 0
    check(lib.fb_mla_attention(C.byref(a), stream_ptr()), "fb_mla_attention")
    return out
