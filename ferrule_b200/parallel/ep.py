"""Expert parallelism with token dispatch: every rank holds a slice of the tokens and a slice of the
experts; routes travel to the rank that owns their expert and the weighted outputs travel back.

Fused path (default): the all-to-alls are plain peer stores issued from inside the kernels
(`csrc/ep_moe.cu` + the scatter epilogue of the grouped down-projection GEMM):

    dispatch (push rows + records into the owners' receive segments, signal)
      -> collect (wait for all sources, build the route list) -> route plan -> gather
      -> grouped gate|up GEMM + SwiGLU -> grouped down GEMM whose epilogue stores each weighted row
         into the token owner's combine buffer and signals
      -> combine-reduce (wait for all owners, fixed-order top-k sum + shared + residual
         [, all-gather push]).

Baseline path (`fused=False`): the same math with `torch.distributed.all_to_all_single` (NCCL) for
both exchanges; it is what the fused path is measured against.

The reference keeps all experts on one GPU and streams them from host memory instead
(crates/ferrule-model/src/moe/streaming.rs); its ParallelismPlan is inert
(crates/ferrule-model/src/support/policies.rs:56-77).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import kernels as K
from ..ops._lib import check, get_lib, ptr, status_tensor, stream_ptr
from .symm import SymmetricBuffer


class EpArgs(C.Structure):
    _fields_ = [("base", C.c_void_p * 8),
                ("off_recv_x", C.c_longlong), ("off_recv_meta", C.c_longlong), ("off_recv_cnt", C.c_longlong),
                ("off_comb", C.c_longlong), ("off_disp_flag", C.c_longlong), ("off_comb_flag", C.c_longlong),
                ("off_gath_flag", C.c_longlong), ("off_gath_out", C.c_longlong),
                ("rank", C.c_int), ("world", C.c_int), ("cap", C.c_int), ("hidden", C.c_int), ("topk", C.c_int),
                ("experts_local", C.c_int), ("tcap", C.c_int),
                ("wait_ns", C.c_ulonglong), ("status", C.c_void_p)]


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


class ExpertParallelMoE:
    """One MoE call site family (all layers of a model can share it: calls are strictly ordered)."""

    def __init__(self, rank: int, world: int, device, hidden: int, inter: int, topk: int, n_experts: int,
                 max_local_tokens: int, group=None, fused: bool = True, wait_ns: int = 3_000_000_000,
                 allgather: bool = False):
        assert n_experts % world == 0 and hidden % 8 == 0
        self.rank, self.world, self.device, self.group = rank, world, torch.device(device), group
        self.H, self.I, self.k, self.E = hidden, inter, topk, n_experts
        self.el = n_experts // world
        self.e_lo = rank * self.el
        self.tcap = max_local_tokens
        # worst case: every route of every local token goes to one rank
        self.cap = max_local_tokens * min(topk, self.el)
        self.fused = fused
        self.rows = world * self.cap
        dev = self.device
        i32 = dict(dtype=torch.int32, device=dev)
        self.ntok = 16 if self.rows // max(self.el, 1) <= 16 else 32
        self.plan = K.MoePlan.allocate(self.rows, self.el, self.ntok, dev)
        self.r_idx = torch.full((self.rows,), -1, **i32)
        self.r_w = torch.zeros(self.rows, dtype=torch.float32, device=dev)
        self.remap_rank = torch.zeros(self.rows, **i32)
        self.remap_row = torch.zeros(self.rows, **i32)
        self.xg = torch.zeros(self.rows, hidden, dtype=torch.bfloat16, device=dev)
        self.hmid = torch.zeros(self.rows, inter, dtype=torch.bfloat16, device=dev)
        self.calls = 0
        if not fused:
            return
        lib = get_lib(True)
        for name, args in (("fb_ep_dispatch", [C.POINTER(EpArgs), C.c_void_p, C.c_longlong, C.c_void_p, C.c_void_p,
                                               C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
                           ("fb_ep_collect", [C.POINTER(EpArgs), C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                              C.c_void_p, C.c_void_p]),
                           ("fb_ep_combine_reduce", [C.POINTER(EpArgs), C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p,
                                                     C.c_longlong, C.c_void_p, C.c_longlong, C.c_int, C.c_int,
                                                     C.c_int, C.c_void_p]),
                           ("fb_ep_gather_wait", [C.POINTER(EpArgs), C.c_void_p, C.c_void_p])):
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = args, C.c_int
        self.lib = lib
        a = EpArgs()
        off = 0
        a.off_disp_flag, off = off, off + 256
        a.off_comb_flag, off = off, off + 256
        a.off_gath_flag, off = off, off + 256
        a.off_recv_cnt, off = off, off + 256
        a.off_recv_meta, off = off, _align(off + self.rows * 16)
        a.off_recv_x, off = off, _align(off + self.rows * hidden * 2)
        a.off_comb, off = off, _align(off + self.tcap * topk * hidden * 2)
        a.off_gath_out = off
        if allgather:
            off = _align(off + world * self.tcap * hidden * 2)
        self.sym = SymmetricBuffer(off, rank, world, group)
        for r in range(world):
            a.base[r] = self.sym.ptrs[r]
        a.rank, a.world, a.cap, a.hidden, a.topk, a.experts_local, a.tcap = rank, world, self.cap, hidden, topk, self.el, self.tcap
        a.wait_ns = wait_ns
        a.status = status_tensor(dev).data_ptr()
        self.args = a
        self.has_gather = allgather
        self.comb_ptrs = self.sym.ptr_array(a.off_comb)
        self.comb_flags = self.sym.ptr_array(a.off_comb_flag)
        # private counters: dispatch [cnt_local(world) | ctr(2)], collect ctr, gemm ctr, reduce ctr, gather ctr
        self.ctr = torch.zeros(32, **i32)
        self.cnt_local = self.ctr[:8]
        self.ctr_disp, self.ctr_coll, self.ctr_gemm, self.ctr_red, self.ctr_gath = (self.ctr[8 + 2 * i:10 + 2 * i]
                                                                                      for i in range(5))
        # views of the local segment of the symmetric buffer (for the gather kernel and tests)
        self._recv_x_ptr = self.sym.local_ptr + a.off_recv_x
        self._gath_ptr = self.sym.local_ptr + a.off_gath_out

    # ------------------------------------------------------------------ fused
    def forward(self, x: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor, e_w13: torch.Tensor, e_w2: torch.Tensor,
                residual: Optional[torch.Tensor] = None, extra: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, act_limit: float = 0.0, allgather: bool = False,
                gather_row0: int = -1):
        """x bf16 [T, H] (this rank's tokens), idx int32 [T, k] global expert ids, wts fp32 [T, k].
        Returns out bf16 [T, H] = residual + extra + sum_k w * expert(x); with `allgather` also the
        [world, tcap, H] buffer holding every rank's rows (`gather_row0` >= 0: this rank's rows go to rows
        gather_row0 ... of the flat [world * tcap, H] buffer instead, so that slices of a batch line up)."""
        T = x.shape[0]
        assert T <= self.tcap and idx.shape == (T, self.k) and idx.dtype == torch.int32
        if out is None:
            out = torch.empty(T, self.H, dtype=torch.bfloat16, device=x.device)
        self.calls += 1
        if not self.fused:
            return self._forward_nccl(x, idx, wts, e_w13, e_w2, residual, extra, out, act_limit)
        lib, a, sp = self.lib, self.args, stream_ptr()
        check(lib.fb_ep_dispatch(C.byref(a), x.data_ptr(), x.stride(0), idx.data_ptr(), wts.data_ptr(), T,
                                 self.cnt_local.data_ptr(), self.ctr_disp.data_ptr(), sp), "fb_ep_dispatch")
        check(lib.fb_ep_collect(C.byref(a), self.ctr_coll.data_ptr(), self.e_lo, self.r_idx.data_ptr(),
                                self.r_w.data_ptr(), self.remap_rank.data_ptr(), self.remap_row.data_ptr(), sp),
              "fb_ep_collect")
        plan = self.plan
        K.moe_plan(self.r_idx.view(self.rows, 1), self.r_w.view(self.rows, 1), plan, self.e_lo, self.e_lo + self.el,
                   dst_slots=1)
        recv_x = _wrap_device_pointer(self._recv_x_ptr, (self.rows, self.H), torch.bfloat16, self.device)
        K.gather_rows(recv_x, plan, self.xg, cap_rows=self.rows)
        K.gemm(self.xg, e_w13, out=self.hmid, epilogue=K.EPI_SWIGLU, plan=plan, act_limit=act_limit)
        K.gemm(self.hmid, e_w2, out=out, epilogue=K.EPI_SCATTER, plan=plan, scatter_rows=self.rows,
               ep_combine=(self.rank, self.world, self.comb_ptrs, self.comb_flags, self.ctr_gemm,
                           self.remap_rank, self.remap_row, self.H))
        ag = 1 if (allgather and self.has_gather) else 0
        check(lib.fb_ep_combine_reduce(C.byref(a), self.ctr_red.data_ptr(), ptr(extra),
                                       extra.stride(0) if extra is not None else 0, ptr(residual),
                                       residual.stride(0) if residual is not None else 0, out.data_ptr(),
                                       out.stride(0), T, ag, gather_row0 if ag else -1, sp), "fb_ep_combine_reduce")
        if ag:
            check(lib.fb_ep_gather_wait(C.byref(a), self.ctr_gath.data_ptr(), sp), "fb_ep_gather_wait")
            return out, _wrap_device_pointer(self._gath_ptr, (self.world, self.tcap, self.H), torch.bfloat16,
                                             self.device)
        return out

    # ------------------------------------------------------------------ NCCL baseline
    def _forward_nccl(self, x, idx, wts, e_w13, e_w2, residual, extra, out, act_limit):
        T, k, H, W = x.shape[0], self.k, self.H, self.world
        flat_e = idx.reshape(-1).long()
        dest = flat_e // self.el
        order = torch.argsort(dest, stable=True)
        send_counts = torch.bincount(dest, minlength=W)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        tok = (order // k)
        send_x = x[tok].contiguous()
        send_e = (flat_e[order] % self.el).to(torch.int32).contiguous()
        n_recv = sum(rc)
        recv_x = torch.empty(n_recv, H, dtype=x.dtype, device=x.device)
        recv_e = torch.empty(n_recv, dtype=torch.int32, device=x.device)
        dist.all_to_all_single(recv_x, send_x, rc, sc, group=self.group)
        dist.all_to_all_single(recv_e, send_e, rc, sc, group=self.group)
        y = torch.zeros(n_recv, H, dtype=torch.bfloat16, device=x.device)
        if n_recv:
            plan = self.plan
            r_idx = torch.full((self.rows,), -1, dtype=torch.int32, device=x.device)
            r_idx[:n_recv] = recv_e + self.e_lo
            r_w = torch.ones(self.rows, dtype=torch.float32, device=x.device)
            K.moe_plan(r_idx.view(self.rows, 1), r_w.view(self.rows, 1), plan, self.e_lo, self.e_lo + self.el, dst_slots=1)
            xin = torch.zeros(self.rows, H, dtype=torch.bfloat16, device=x.device)
            xin[:n_recv] = recv_x
            K.gather_rows(xin, plan, self.xg, cap_rows=self.rows)
            K.gemm(self.xg, e_w13, out=self.hmid, epilogue=K.EPI_SWIGLU, plan=plan, act_limit=act_limit)
            yfull = torch.zeros(self.rows, H, dtype=torch.bfloat16, device=x.device)
            K.gemm(self.hmid, e_w2, out=yfull, epilogue=K.EPI_SCATTER, plan=plan, scatter_rows=self.rows)
            y = yfull[:n_recv].contiguous()
        back = torch.empty(T * k, H, dtype=torch.bfloat16, device=x.device)
        dist.all_to_all_single(back, y, sc, rc, group=self.group)
        routes = torch.empty(T * k, H, dtype=torch.float32, device=x.device)
        routes[order] = back.float() * wts.reshape(-1)[order].unsqueeze(-1)
        acc = routes.bfloat16().float().view(T, k, H).sum(1)
        if extra is not None:
            acc = acc + extra.float()
        if residual is not None:
            acc = acc + residual.float()
        out.copy_(acc.to(out.dtype))
        return out

    def close(self) -> None:
        if self.fused:
            self.sym.close()


def _wrap_device_pointer(p: int, shape, dtype, device) -> torch.Tensor:
    """Zero-copy tensor over device memory this process allocated outside the PyTorch allocator."""
    n = 1
    for s in shape:
        n *= s
    esize = torch.empty((), dtype=dtype).element_size()

    class _Holder:
        pass

    h = _Holder()
    typestr = {torch.bfloat16: "<i2", torch.float32: "<f4", torch.int32: "<i4", torch.uint8: "|u1"}[dtype]
    h.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (p, False), "version": 3}
    t = torch.as_tensor(h, device=device)
    if dtype == torch.bfloat16:
        t = t.view(torch.bfloat16)
    assert t.element_size() == esize
    return t.view(*shape)
