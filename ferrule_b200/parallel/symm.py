"""Symmetric peer memory: one device buffer per rank, mapped into every rank of the node.

Buffers come from `cudaMalloc` inside the native library (not from the PyTorch caching
allocator), their CUDA IPC handles are exchanged through the process group's store, and
every rank opens every peer's handle, which yields NVLink peer pointers usable from kernels
(plain loads/stores; no multicast objects are bound, so a rank that exits between steps
cannot fault its peers).

A `Channel` bundles what one fused collective call site needs: a double-buffered receive
area (one slot per source rank), arrival counters, and private call/consumed counters.

The reference has no counterpart (single GPU); this is the communication substrate the
tensor/expert-parallel paths stand on.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops._lib import check, get_lib


class SymmetricBuffer:
    def __init__(self, nbytes: int, rank: int, world: int, group=None):
        lib = get_lib(True)
        self.lib, self.rank, self.world, self.nbytes = lib, rank, world, nbytes
        hb = lib.fb_ipc_handle_bytes()
        handle = C.create_string_buffer(hb)
        local = C.c_void_p()
        check(lib.fb_ipc_alloc(C.byref(local), nbytes, handle), "fb_ipc_alloc")
        self.local_ptr = local.value
        handles: List[Optional[bytes]] = [None] * world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        self.ptrs: List[int] = []
        self._opened: List[int] = []
        for r in range(world):
            if r == rank:
                self.ptrs.append(self.local_ptr)
                continue
            p = C.c_void_p()
            buf = C.create_string_buffer(handles[r], hb)
            check(lib.fb_ipc_open(buf, C.byref(p)), f"fb_ipc_open(rank {r})")
            self.ptrs.append(p.value)
            self._opened.append(p.value)
        dist.barrier(group=group)

    def ptr_array(self, offset: int = 0):
        arr = (C.c_void_p * 8)()
        for r in range(self.world):
            arr[r] = self.ptrs[r] + offset
        return arr

    def close(self) -> None:
        for p in self._opened:
            self.lib.fb_ipc_close(C.c_void_p(p))
        self._opened = []
        if self.local_ptr:
            self.lib.fb_ipc_free(C.c_void_p(self.local_ptr))
            self.local_ptr = 0


class Channel:
    """Receive area + arrival flags for one call-site family.

    payload_floats: floats per source slot (rows_cap * width).  n_flags: arrival counters.
    """

    def __init__(self, rank: int, world: int, device, payload_floats: int, n_flags: int, group=None,
                 wait_ns: int = 3_000_000_000, multicast: bool = False):
        self.rank, self.world, self.wait_ns = rank, world, wait_ns
        self.payload_floats, self.n_flags = payload_floats, n_flags
        self.flag_bytes = ((n_flags * 4 + 255) // 256) * 256
        # every fp32 travels as an 8-byte (value, tag) pair; two parities; one slot per source rank
        recv_bytes = 2 * world * payload_floats * 8
        # `multicast`: the buffer is also bound to an NVLink multicast address (NVLS), so that a pusher reaches all
        # ranks' slots with one `multimem.st`; `mc_recv` stays 0 when the node offers none
        self.mc_recv = 0
        self.buf = None
        if multicast:
            try:
                self.buf = McSymmetricBuffer(self.flag_bytes + recv_bytes, rank, world, device, group)
                self.mc_recv = self.buf.mc_ptr + self.flag_bytes
            except Exception:  # noqa: BLE001 - no NVLS here: plain peer stores
                self.buf = None
        if self.buf is None:
            self.buf = SymmetricBuffer(self.flag_bytes + recv_bytes, rank, world, group)
        self.flags = self.buf.ptr_array(0)
        self.recv = self.buf.ptr_array(self.flag_bytes)
        # private: [calls, ctas_done, consumed[n_flags]]
        self.ctr = torch.zeros(2 + n_flags, dtype=torch.int32, device=device)

    def close(self) -> None:
        self.buf.close()


class McSymmetricBuffer:
    """Symmetric buffer with peer mappings and an NVLink multicast mapping (allocated and exchanged by
    `torch.distributed._symmetric_memory`); same interface as `SymmetricBuffer` plus `mc_ptr`."""

    def __init__(self, nbytes: int, rank: int, world: int, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.rank, self.world, self.nbytes = rank, world, nbytes
        self.t = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.t.zero_()
        torch.cuda.synchronize(device)
        grp = group if group is not None else dist.group.WORLD
        try:
            self.hdl = symm_mem.rendezvous(self.t, grp)
        except Exception:  # noqa: BLE001
            symm_mem.enable_symm_mem_for_group(grp.group_name)
            self.hdl = symm_mem.rendezvous(self.t, grp.group_name)
        self.mc_ptr = int(self.hdl.multicast_ptr or 0)
        if not self.mc_ptr:
            raise RuntimeError("this node offers no NVLink multicast (NVLS)")
        self.ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        self.local_ptr = self.ptrs[rank]
        dist.barrier(group=group)

    def ptr_array(self, offset: int = 0):
        arr = (C.c_void_p * 8)()
        for r in range(self.world):
            arr[r] = self.ptrs[r] + offset
        return arr

    def close(self) -> None:
        self.hdl = None
        self.t = None


class McChannel:
    """One symmetric buffer bound to an NVLink multicast object (NVLS), for the `multimem` collectives of
    `csrc/comm_mm.cu`: [flags 256 B | stage x 2 | result x 2], each area `rows_cap x dim` bf16.

    Allocation, handle exchange and the multicast binding are done by `torch.distributed._symmetric_memory`
    (plumbing); the kernels that reduce and broadcast through the switch are this library's own.  All call sites
    of a model share one channel: their calls are strictly ordered on every rank.  `available()` tells whether
    the node offers multicast at all (NVSwitch + driver support)."""

    def __init__(self, rank: int, world: int, device, rows_cap: int, dim: int, group=None,
                 wait_ns: int = 3_000_000_000):
        import torch.distributed._symmetric_memory as symm_mem
        self.rank, self.world, self.wait_ns = rank, world, wait_ns
        self.rows_cap, self.dim = rows_cap, dim
        self.buf_bytes = (rows_cap * dim * 2 + 255) // 256 * 256
        self.flag_bytes = 256
        total = self.flag_bytes + 4 * self.buf_bytes
        self.t = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self.t.zero_()
        torch.cuda.synchronize(device)
        grp = group if group is not None else dist.group.WORLD
        try:
            self.hdl = symm_mem.rendezvous(self.t, grp)
        except Exception:  # noqa: BLE001 - older call convention: the group has to be enabled by name first
            symm_mem.enable_symm_mem_for_group(grp.group_name)
            self.hdl = symm_mem.rendezvous(self.t, grp.group_name)
        self.mc_ptr = int(self.hdl.multicast_ptr or 0)
        if not self.mc_ptr:
            raise RuntimeError("this node offers no NVLink multicast (NVLS): multimem collectives are unavailable")
        self.local_ptr = self.t.data_ptr()
        self.stage_off = self.flag_bytes
        self.result_off = self.flag_bytes + 2 * self.buf_bytes
        self.priv = torch.zeros(4, dtype=torch.int32, device=device)
        dist.barrier(group=group)

    def collective(self, mode: int, out: torch.Tensor, rows: int, src: Optional[torch.Tensor] = None, slots: int = 1,
                   topk: int = 0, topk_idx: Optional[torch.Tensor] = None, e_lo: int = 0, e_hi: int = 0,
                   residual: Optional[torch.Tensor] = None, norm_w: Optional[torch.Tensor] = None,
                   norm_out: Optional[torch.Tensor] = None, eps: float = 0.0) -> torch.Tensor:
        """mode 1 reduce-scatter, 2 all-gather, 3 all-reduce (see `fb_mm_collective`)."""
        from ..ops._lib import ptr, status_tensor, stream_ptr
        lib = get_lib(True)
        # a rank whose row slice is empty (more ranks than rows) still takes part: it owns nothing and reads no
        # row of `src`, but the launcher wants a pointer
        src_ptr = ptr(src) if (src is None or src.numel()) else out.data_ptr()
        check(lib.fb_mm_collective(src_ptr, src.stride(0) if src is not None else 0, slots, topk, ptr(topk_idx), e_lo,
                                   e_hi, ptr(residual), residual.stride(0) if residual is not None else 0,
                                   out.data_ptr(), out.stride(0), rows, self.dim, mode, ptr(norm_w), ptr(norm_out),
                                   norm_out.stride(0) if norm_out is not None else 0, eps, self.local_ptr, self.mc_ptr,
                                   self.stage_off, self.result_off, self.buf_bytes, self.priv.data_ptr(), self.rank,
                                   self.world, self.wait_ns, status_tensor(out.device).data_ptr(), stream_ptr()),
              "fb_mm_collective")
        return out

    def close(self) -> None:
        self.hdl = None
        self.t = None

