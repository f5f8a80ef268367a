"""Tensor / expert parallel execution of one model replica over the GPUs of a node.

Sharding: attention heads, dense/shared FFN inner dimension and the vocabulary are split
across ranks; routed experts are split by expert id while activations stay replicated
between the two collectives of a layer, so expert parallelism needs no token dispatch.
Each layer therefore has two reductions of a [rows, hidden] tensor:

  attention o_proj -> all-reduce (+ residual)   : fused into the tcgen05 GEMM epilogue
  MoE / FFN output -> all-reduce (+ residual)   : fused into the route-reduce kernel (MoE) or
                                                  the down-projection GEMM epilogue (dense)

Decode-sized batches use the fused one-shot kernels over NVLink peer stores; larger batches
(prefill) and `fused=False` use NCCL, which is also the baseline the fused path is measured
against.  The greedy token of a vocabulary-sharded LM head is resolved by a (logit, id)
all-gather between ranks.

The reference is single-GPU (crates/ferrule-model/src/support/policies.rs:56-77 keeps an inert
parallelism plan; docs/ROADMAP.md:34-41 lists distributed execution as future work).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import kernels as K
from ..ops._lib import check, get_lib, status_tensor, stream_ptr
from .symm import Channel


class TensorParallel:
    def __init__(self, rank: int, world: int, device, fused: bool = True, fused_max_rows: int = 64,
                 group=None, wait_ns: int = 3_000_000_000, payload: str = "fp32", collective: str = "ll",
                 multicast_push: bool = False):
        self.rank, self.world, self.device, self.group = rank, world, torch.device(device), group
        self.fused = fused and self.device.type == "cuda"
        self.fused_max_rows = fused_max_rows
        # what the fused all-reduces push over NVLink: fp32 partials (as exact as an fp32 all-reduce) or bf16
        # partials (half the bytes; each rank's partial is rounded to bf16 before the fixed-order sum)
        assert payload in ("fp32", "bf16")
        self.payload_bf16 = 1 if payload == "bf16" else 0
        self.wait_ns = wait_ns
        # "ll": tagged peer pushes, every rank sums in rank order (works on any peer-mapped memory);
        # "multimem": two-shot reduce + broadcast inside the NVLink switch (needs NVLS; rows up to mm_max_rows)
        assert collective in ("ll", "multimem")
        self.collective = collective
        self.mm = None
        self.mm_max_rows = 512
        # "ll" pushes through an NVLink multicast address when the node has NVLS: one store reaches every rank
        self.multicast_push = multicast_push
        self.gemm_ch: Optional[Channel] = None
        self.moe_ch: Optional[Channel] = None
        self.arg_ch: Optional[Channel] = None
        self.hidden = 0
        self.calls_fused = 0
        self.calls_nccl = 0

    # ------------------------------------------------------------------ setup
    def attach(self, fwd) -> None:
        """Allocate the channels for a CudaForward (hidden size and decode row capacity)."""
        H = fwd.cfg.hidden
        self.hidden = H
        rows = self.fused_max_rows
        self._tmp32 = torch.zeros(fwd.ws.max_rows, H, dtype=torch.float32, device=self.device)
        self._no_idx = torch.zeros(8, dtype=torch.int32, device=self.device)     # top-k table of a route-free reduce
        self._pairs = torch.zeros(self.world, fwd.ws.max_logit_rows, 2, dtype=torch.float32, device=self.device)
        if not self.fused:
            return
        if self.collective == "multimem":
            from .symm import McChannel
            self.mm = McChannel(self.rank, self.world, self.device, self.mm_max_rows, H, self.group, self.wait_ns)
            self._partial = torch.zeros(self.mm_max_rows, H, dtype=torch.bfloat16, device=self.device)
        n_tiles = (H + 127) // 128
        self.gemm_ch = Channel(self.rank, self.world, self.device, rows * H, n_tiles * ((rows + 15) // 16),
                               self.group, self.wait_ns, multicast=self.multicast_push)
        self.moe_ch = Channel(self.rank, self.world, self.device, rows * H, rows, self.group, self.wait_ns,
                              multicast=self.multicast_push)
        self.arg_ch = Channel(self.rank, self.world, self.device, max(fwd.ws.max_logit_rows, 1) * 2, 1, self.group,
                              self.wait_ns)

    def close(self) -> None:
        for ch in (self.gemm_ch, self.moe_ch, self.arg_ch, self.mm):
            if ch is not None:
                ch.close()

    def fill_gemm_args(self, a, rows: int, n_out: int, ntok: int) -> None:
        ch = self.gemm_ch
        a.rank, a.world, a.rows_cap, a.flag_capacity = self.rank, self.world, self.fused_max_rows, ch.n_flags
        for r in range(self.world):
            a.peer_recv[r] = ch.recv[r]
            a.peer_flags[r] = ch.flags[r]
        a.local_ctr = ch.ctr.data_ptr()
        a.peer_wait_ns = self.wait_ns
        a.ar_payload_bf16 = self.payload_bf16
        a.mc_recv = ch.mc_recv or None

    # ------------------------------------------------------------------ fused collectives
    def gemm_allreduce(self, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor, out: torch.Tensor,
                       T: int) -> torch.Tensor:
        """out = bf16(residual + sum over ranks of x @ w^T)."""
        if self.mm is not None and T <= self.mm_max_rows and w.shape[-2] == self.hidden:
            # the GEMM leaves this rank's partial in local memory, the switch reduces and broadcasts it
            K.gemm(x, w, out=self._partial[:T])
            self.mm.collective(3, out, T, src=self._partial[:T], residual=residual)
            self.calls_fused += 1
            return out
        if self.fused and T <= self.fused_max_rows and w.shape[-2] == self.hidden:
            K.gemm(x, w, out=out, epilogue=K.EPI_ALLREDUCE, comm=self, residual=residual, ntok=K.pick_ntok(T))
            self.calls_fused += 1
            return out
        tmp = self._tmp32[:T]
        K.gemm(x, w, out=tmp)
        dist.all_reduce(tmp, group=self.group)
        torch.add(tmp, residual, out=tmp)
        out.copy_(tmp)
        self.calls_nccl += 1
        return out

    def moe_reduce_allreduce(self, route_out: torch.Tensor, slots: int, topk: int, idx: torch.Tensor,
                             e_lo: int, e_hi: int, residual: torch.Tensor, out: torch.Tensor, T: int) -> torch.Tensor:
        H = self.hidden
        if self.mm is not None and T <= self.mm_max_rows:
            self.mm.collective(3, out, T, src=route_out, slots=slots, topk=topk, topk_idx=idx, e_lo=e_lo, e_hi=e_hi,
                               residual=residual)
            self.calls_fused += 1
            return out
        if self.fused and T <= self.fused_max_rows:
            ch = self.moe_ch
            lib = get_lib(True)
            check(lib.fb_moe_reduce_allreduce_mc(route_out.data_ptr(), slots, topk, idx.data_ptr(), e_lo, e_hi,
                                                 residual.data_ptr(), residual.stride(0), out.data_ptr(),
                                                 out.stride(0), T, H, self.rank, self.world, self.fused_max_rows,
                                                 ch.recv, ch.flags, ch.ctr.data_ptr(), self.payload_bf16,
                                                 self.wait_ns, ch.mc_recv or None,
                                                 status_tensor(self.device).data_ptr(), stream_ptr()),
                  "fb_moe_reduce_allreduce_mc")
            self.calls_fused += 1
            return out
        tmp = self._tmp32[:T]
        K.moe_reduce(route_out, slots, topk, idx, e_lo, e_hi, T, H, out=tmp)
        dist.all_reduce(tmp, group=self.group)
        torch.add(tmp, residual, out=tmp)
        out.copy_(tmp)
        self.calls_nccl += 1
        return out

    def reduce_scatter(self, partial: torch.Tensor, out_slice: torch.Tensor, T: int,
                       residual_slice: Optional[torch.Tensor] = None) -> torch.Tensor:
        """out_slice [ceil(T / world), hidden] = this rank's rows of the sum over ranks of `partial` [T, hidden]
        (+ residual_slice): rows are owned in contiguous slices.  In-switch reduction; NCCL otherwise."""
        per = (T + self.world - 1) // self.world
        if self.mm is not None and T <= self.mm_max_rows:
            self.mm.collective(1, out_slice, T, src=partial, residual=residual_slice)
            self.calls_fused += 1
            return out_slice
        pad = torch.zeros(per * self.world, partial.shape[1], dtype=torch.float32, device=partial.device)
        pad[:T] = partial.float()
        o = torch.empty(per, partial.shape[1], dtype=torch.float32, device=partial.device)
        dist.reduce_scatter_tensor(o, pad, group=self.group)
        if residual_slice is not None:
            o[:residual_slice.shape[0]] += residual_slice.float()
        out_slice.copy_(o[:out_slice.shape[0]])
        self.calls_nccl += 1
        return out_slice

    def all_gather(self, slice_rows: torch.Tensor, out: torch.Tensor, T: int) -> torch.Tensor:
        """out [T, hidden] = the ranks' row slices (ceil(T / world) rows each, the last ones possibly short)."""
        per = (T + self.world - 1) // self.world
        if self.mm is not None and T <= self.mm_max_rows:
            self.mm.collective(2, out, T, src=slice_rows)
            self.calls_fused += 1
            return out
        mine = torch.zeros(per, out.shape[1], dtype=out.dtype, device=out.device)
        mine[:slice_rows.shape[0]] = slice_rows
        full = torch.empty(per * self.world, out.shape[1], dtype=out.dtype, device=out.device)
        dist.all_gather_into_tensor(full, mine, group=self.group)
        out.copy_(full[:T])
        self.calls_nccl += 1
        return out

    def add_allreduce(self, delta: torch.Tensor, residual: torch.Tensor, out: torch.Tensor, T: int) -> torch.Tensor:
        """out = residual + sum over ranks of delta [T, hidden]: the partial result of a row-parallel linear
        whose GEMM has no collective epilogue (FP8 weights).  Runs the one-shot push all-reduce with a single
        dense slot per token."""
        return self.moe_reduce_allreduce(delta, 1, 0, self._no_idx, 0, 0, residual, out, T)

    def argmax_across_vocab(self, ids: torch.Tensor, vals: torch.Tensor, vocab_lo: int, L: int) -> None:
        """In place: local (id, logit) of a vocabulary shard -> global greedy token on every rank."""
        if self.fused and self.arg_ch is not None:
            ch = self.arg_ch
            lib = get_lib(True)
            check(lib.fb_argmax_allgather(ids.data_ptr(), vals.data_ptr(), vocab_lo, L, self.rank, self.world,
                                          ch.payload_floats // 2, ch.recv, ch.flags, ch.ctr.data_ptr(),
                                          self.wait_ns, status_tensor(self.device).data_ptr(), stream_ptr()),
                  "fb_argmax_allgather")
            return
        pairs = self._pairs[:, :L]
        mine = torch.stack([vals[:L], torch.where(ids[:L] < 0, -1.0, (ids[:L] + vocab_lo).float())], dim=-1)
        self._gather_pairs(pairs, mine)
        v, gid = pairs[..., 0], pairs[..., 1]
        v = torch.where(gid < 0, torch.full_like(v, float("-inf")), v)
        best = v.max(0).values
        cand = torch.where((v == best) & (gid >= 0), gid, torch.full_like(gid, 3.0e38))
        win = cand.min(0).values
        ids[:L] = torch.where(win > 1.0e38, torch.full_like(win, -1.0), win).to(torch.int32)
        vals[:L] = best

    def _gather_pairs(self, pairs: torch.Tensor, mine: torch.Tensor) -> None:
        bufs = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(bufs, mine.contiguous(), group=self.group)
        for r, b in enumerate(bufs):
            pairs[r].copy_(b)

    # ------------------------------------------------------------------ reference path (any backend)
    # ------------------------------------------------------------------ sequence parallelism
    def gemm_reduce_scatter(self, x: torch.Tensor, w: torch.Tensor, residual_rows: torch.Tensor, out_rows: torch.Tensor,
                            T: int) -> torch.Tensor:
        """out_rows = bf16(residual_rows + this rank's rows of the sum over ranks of x @ w^T): the GEMM leaves its
        fp32 partial in local memory, the reduce-scatter (in-switch when bound, NCCL otherwise) sums and cuts it."""
        tmp = self._tmp32[:T]
        K.gemm(x, w, out=tmp)
        return self.reduce_scatter(tmp, out_rows, T, residual_slice=residual_rows)

    def moe_reduce_scatter(self, route_out: torch.Tensor, slots: int, topk: int, idx: torch.Tensor, e_lo: int, e_hi: int,
                           residual_rows: torch.Tensor, out_rows: torch.Tensor, T: int) -> torch.Tensor:
        tmp = self._tmp32[:T]
        K.moe_reduce(route_out, slots, topk, idx, e_lo, e_hi, T, self.hidden, out=tmp)
        return self.reduce_scatter(tmp, out_rows, T, residual_slice=residual_rows)

    def row_range(self, T: int):
        """Rows of a T-row batch this rank owns between a reduce-scatter and the next all-gather (contiguous
        slices of ceil(T / world) rows; the last ranks' slices may be short or empty)."""
        per = (T + self.world - 1) // self.world
        lo = min(self.rank * per, T)
        return lo, min(lo + per, T)

    def reduce_scatter_reference(self, t: torch.Tensor) -> torch.Tensor:
        """Host path: this rank's rows of the sum over ranks of `t` [T, hidden]."""
        T = t.shape[0]
        per = (T + self.world - 1) // self.world
        pad = torch.zeros(per * self.world, t.shape[1], dtype=t.dtype, device=t.device)
        pad[:T] = t
        try:
            out = torch.empty(per, t.shape[1], dtype=t.dtype, device=t.device)
            dist.reduce_scatter_tensor(out, pad, group=self.group)
        except (RuntimeError, NotImplementedError):          # a backend without reduce-scatter (gloo on CPU)
            dist.all_reduce(pad, group=self.group)
            out = pad[self.rank * per:(self.rank + 1) * per]
        lo, hi = self.row_range(T)
        return out[:hi - lo].contiguous()

    def all_gather_reference(self, rows: torch.Tensor, T: int) -> torch.Tensor:
        """Host path: the ranks' row slices put back together -> [T, hidden]."""
        per = (T + self.world - 1) // self.world
        mine = torch.zeros(per, rows.shape[1], dtype=rows.dtype, device=rows.device)
        mine[:rows.shape[0]] = rows
        bufs = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(bufs, mine, group=self.group)
        return torch.cat(bufs, dim=0)[:T].contiguous()

    def allreduce_reference(self, t: torch.Tensor) -> torch.Tensor:
        t = t.contiguous()
        dist.all_reduce(t, group=self.group)
        return t

    def gather_vocab_reference(self, logits: torch.Tensor) -> torch.Tensor:
        bufs = [torch.empty_like(logits) for _ in range(self.world)]
        dist.all_gather(bufs, logits.contiguous(), group=self.group)
        return torch.cat(bufs, dim=-1)
