"""Host-pinned expert streaming: checkpoint slices -> pinned slabs -> device slots.

Pieces:
  ExpertSourceCatalog   where each routed expert's tensors live in the checkpoint (file, offset,
                        length per tensor), its payload size and its exact MaterializationKey
  PinnedSlabPool        one registered pinned host buffer cut into aligned slabs, leased to reads
  HostStagedExpertCache LRU of expert payloads kept in host memory (pinned first, pageable second)
                        so a re-streamed expert does not touch storage again
  ExpertArena           fixed-frame device arena: `slots` frames of `frame_bytes` per layer
  ExpertMaterializationProvider
                        the MaterializationProvider the LoadRegistry drives: reserve (slot ticket +
                        slab) -> read (native direct reader or the staged cache) -> async upload on
                        a dedicated low-priority stream, completion gated by a CUDA event ->
                        install (activate + publish the slot, bump its generation)
On a CPU-only machine the same code runs with host "device" buffers and synchronous copies, which
is what the unit tests exercise.

Counterpart of crates/ferrule-model/src/moe/streaming.rs:278-520 (catalog), :696-1140 (planner),
:1423-2150 (reader), :2337-2800 (host staged cache); moe/cuda_materialization.rs:45-210, :385-700,
:2299-3180 (provider); crates/ferrule-backend/src/cuda/context.rs:561-940, :5049-5290 (arena, uploads).
"""
from __future__ import annotations

import os
import threading
from collections import deque
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass
from typing import Deque, Dict, List, Optional, Sequence, Tuple

import torch

from ..utils.failpoints import FAILPOINTS, FailpointTriggered
from ..utils.memory import MemoryPoolLimits, OwnerMemoryLru
from .expert_residency import ExpertResidencyController, InstallTicket, ResidencyError
from .io_protocol import (CompletionEvent, CompletionOutcome, FailureReason, LoadStage, MaterializationKey,
                          MaterializationResourcePlan, PinnedSlabLease, ResourceId, ResourceKind, SlabLeaseState)
from .provider import MaterializationProvider, ProviderError

ALIGN = 4096


@dataclass(frozen=True)
class TensorSlice:
    name: str
    file: str
    offset: int
    length: int
    payload_offset: int          # where the tensor sits inside the packed expert payload


@dataclass(frozen=True)
class ExpertSource:
    layer: int
    expert: int
    slices: Tuple[TensorSlice, ...]
    payload_bytes: int


class ExpertSourceCatalog:
    """Built once per prepared model generation from the checkpoint index."""

    def __init__(self, model: str, checkpoint, layers: Sequence[int], n_experts: int,
                 name_fn=None, device: int = 0, backend: str = "cuda-sm100a", payload_encoding: int = 1,
                 destination_generation: int = 0):
        self.model, self.ck, self.device, self.backend = model, checkpoint, device, backend
        self.payload_encoding, self.destination_generation = payload_encoding, destination_generation
        self.source_identity = checkpoint.source_identity()
        self.sources: Dict[Tuple[int, int], ExpertSource] = {}
        name_fn = name_fn or (lambda l, e: [f"model.layers.{l}.mlp.experts.{e}.{p}.{s}"
                                            for p in ("gate_proj", "up_proj", "down_proj")
                                            for s in ("weight", "scale", "weight_scale_inv")])
        for l in layers:
            for e in range(n_experts):
                off, sl = 0, []
                for n in name_fn(l, e):
                    if not checkpoint.has(n):
                        continue
                    i = checkpoint.info(n)
                    sl.append(TensorSlice(n, i.file, i.start, i.nbytes, off))
                    off += (i.nbytes + 255) // 256 * 256
                if sl:
                    self.sources[(l, e)] = ExpertSource(l, e, tuple(sl), off)

    def source(self, layer: int, expert: int) -> ExpertSource:
        return self.sources[(layer, expert)]

    def key(self, layer: int, expert: int) -> MaterializationKey:
        src = self.sources[(layer, expert)]
        content = self.ck.content_hash([s.name for s in src.slices])
        return MaterializationKey(self.model, self.source_identity, content,
                                  ResourceId(ResourceKind.ROUTED_EXPERT, layer, expert), self.payload_encoding,
                                  self.backend, self.device, 0, self.destination_generation)

    def max_payload_bytes(self) -> int:
        return max((s.payload_bytes for s in self.sources.values()), default=0)


class PinnedSlabPool:
    def __init__(self, slab_bytes: int, n_slabs: int, pin: bool = True):
        self.slab_bytes = (slab_bytes + ALIGN - 1) // ALIGN * ALIGN
        self.n_slabs = n_slabs
        # over-allocate so the first slab can start on a 4 KiB boundary (direct I/O needs it)
        self.buffer = torch.empty(self.slab_bytes * n_slabs + ALIGN, dtype=torch.uint8)
        self.pinned = False
        if pin and torch.cuda.is_available():
            self.buffer = self.buffer.pin_memory()
            self.pinned = True
        self.base = (-self.buffer.data_ptr()) % ALIGN
        self.leases = [PinnedSlabLease(i, self.base + i * self.slab_bytes, self.slab_bytes, ALIGN,
                                       base_address=self.buffer.data_ptr()) for i in range(n_slabs)]
        self._free: Deque[int] = deque(range(n_slabs))
        self.high_water = 0

    def acquire(self, op: int) -> Optional[PinnedSlabLease]:
        if not self._free:
            return None
        l = self.leases[self._free.popleft()]
        l.advance(SlabLeaseState.LEASED)
        l.operation = op
        l.validate()
        self.high_water = max(self.high_water, self.n_slabs - len(self._free))
        return l

    def release(self, lease: PinnedSlabLease) -> None:
        if lease.state != SlabLeaseState.RELEASED:
            lease.advance(SlabLeaseState.RELEASED)
        lease.advance(SlabLeaseState.FREE)
        lease.operation = None
        self._free.append(lease.slab)

    def view(self, lease: PinnedSlabLease, nbytes: Optional[int] = None) -> torch.Tensor:
        return self.buffer[lease.offset:lease.offset + (nbytes if nbytes is not None else lease.nbytes)]

    @property
    def in_use(self) -> int:
        return self.n_slabs - len(self._free)


class HostStagedExpertCache:
    """Two-level host LRU of packed expert payloads: pinned (fast to upload) then pageable."""

    def __init__(self, pinned_bytes: int, pageable_bytes: int):
        self.pageable: OwnerMemoryLru = OwnerMemoryLru(MemoryPoolLimits(pageable_bytes))
        self.pinned: OwnerMemoryLru = OwnerMemoryLru(MemoryPoolLimits(pinned_bytes), self._demote)
        self.hits_pinned = self.hits_pageable = self.misses = 0

    def _demote(self, key, value: torch.Tensor) -> None:
        self.pageable.put(key, value.clone() if value.is_pinned() else value, value.numel())

    def get(self, key) -> Optional[torch.Tensor]:
        v = self.pinned.get(key)
        if v is not None:
            self.hits_pinned += 1
            return v
        v = self.pageable.get(key)
        if v is not None:
            self.hits_pageable += 1
            return v
        self.misses += 1
        return None

    def put(self, key, payload: torch.Tensor) -> None:
        if self.pinned.put(key, payload, payload.numel()):
            self.pageable.pop(key)                  # an older demoted copy would only hold pageable bytes
        else:
            self.pageable.put(key, payload, payload.numel())


class ExpertArena:
    """Fixed-frame device arena: frame s of layer l holds whichever expert currently owns slot s."""

    def __init__(self, layers: Sequence[int], slots: Dict[int, int], frame_bytes: int, device):
        self.frame_bytes = (frame_bytes + 255) // 256 * 256
        self.device = torch.device(device)
        self.frames = {l: torch.zeros(slots[l], self.frame_bytes, dtype=torch.uint8, device=self.device) for l in layers}

    def frame(self, layer: int, slot: int) -> torch.Tensor:
        return self.frames[layer][slot]

    def nbytes(self) -> int:
        return sum(f.numel() for f in self.frames.values())


class PythonDirectReader:
    """Positioned reads on a small thread pool (fallback for the native O_DIRECT reader)."""

    def __init__(self, threads: int = 4):
        self.pool = ThreadPoolExecutor(max_workers=threads, thread_name_prefix="ferrule-read")
        self._fds: Dict[str, int] = {}
        self._lock = threading.Lock()

    def _fd(self, path: str) -> int:
        with self._lock:
            fd = self._fds.get(path)
            if fd is None:
                fd = self._fds[path] = os.open(path, os.O_RDONLY)
            return fd

    def submit(self, src: ExpertSource, dst: torch.Tensor, done) -> None:
        def work():
            try:
                n = 0
                mv = memoryview(dst.numpy())
                for s in src.slices:
                    got = os.preadv(self._fd(s.file), [mv[s.payload_offset:s.payload_offset + s.length]], s.offset)
                    if got != s.length:
                        return done(False, n + got)
                    n += got
                done(True, src.payload_bytes)
            except Exception:  # noqa: BLE001 - reported as a failed read
                done(False, 0)
        self.pool.submit(work)

    def close(self) -> None:
        self.pool.shutdown(wait=True)
        for fd in self._fds.values():
            os.close(fd)
        self._fds.clear()


@dataclass
class _OpState:
    op: int
    key: MaterializationKey
    source: ExpertSource
    ticket: InstallTicket
    slab: Optional[PinnedSlabLease] = None
    cached: Optional[torch.Tensor] = None
    event: Optional[object] = None
    generation: int = 0
    cancelled: bool = False


class ExpertMaterializationProvider(MaterializationProvider):
    def __init__(self, catalog: ExpertSourceCatalog, residency: ExpertResidencyController, arena: ExpertArena,
                 slabs: PinnedSlabPool, cache: Optional[HostStagedExpertCache] = None, reader=None,
                 on_install=None, hub=None, max_upload_inflight: int = 32):
        self.catalog, self.residency, self.arena, self.slabs = catalog, residency, arena, slabs
        self.cache, self.reader = cache, reader or PythonDirectReader()
        self.on_install = on_install        # callback(layer, expert, slot, generation, frame) after publish
        self.hub = hub
        self.max_upload_inflight = max_upload_inflight
        self.ops: Dict[int, _OpState] = {}
        self._done: Deque[CompletionEvent] = deque()
        self._lock = threading.Lock()
        self._uploads: List[_OpState] = []
        self._waiting_reads: Deque[int] = deque()
        self.cuda = arena.device.type == "cuda"
        self.upload_stream = torch.cuda.Stream(device=arena.device, priority=0) if self.cuda else None
        self.bytes_read = self.bytes_uploaded = self.cache_served = 0

    # ---- helpers ----
    def _push(self, ev: CompletionEvent) -> None:
        with self._lock:
            self._done.append(ev)
        if self.hub is not None:
            self.hub.notify()

    def _ev(self, st: _OpState, stage: LoadStage, ok: bool, nbytes: int, failure=None) -> CompletionEvent:
        outcome = CompletionOutcome.OK if ok else (CompletionOutcome.CANCELLED if st.cancelled else CompletionOutcome.FAILED)
        return CompletionEvent(st.op, st.key, stage, st.generation, outcome, nbytes if ok else 0,
                               None if ok else (FailureReason.CANCELLED if st.cancelled else failure))

    # ---- provider API ----
    def plan(self, key: MaterializationKey) -> MaterializationResourcePlan:
        src = self.catalog.source(key.resource.group, key.resource.item)
        p = MaterializationResourcePlan.for_payload(src.payload_bytes, ALIGN)
        return p

    def reserve(self, op: int, key: MaterializationKey) -> None:
        layer, expert = key.resource.group, key.resource.item
        src = self.catalog.source(layer, expert)
        if src.payload_bytes > self.arena.frame_bytes:
            raise ProviderError("expert payload larger than an arena frame")
        try:
            FAILPOINTS.check("arena_acquire")
            ticket = self.residency.layer(layer).prepare(expert)
        except (ResidencyError, FailpointTriggered) as exc:
            raise ProviderError(str(exc)) from exc
        self.ops[op] = _OpState(op, key, src, ticket)

    def submit_read(self, op: int, key: MaterializationKey, generation: int) -> None:
        st = self.ops[op]
        st.generation = generation
        cached = self.cache.get((key.resource.group, key.resource.item)) if self.cache else None
        if cached is not None:
            st.cached = cached
            self.cache_served += 1
            return self._push(self._ev(st, LoadStage.READ_SUBMITTED, True, st.source.payload_bytes))
        slab = self.slabs.acquire(op)
        if slab is None:
            # every slab is on loan: the read starts as soon as an upload gives one back
            self._waiting_reads.append(op)
            return
        self._start_read(st, slab)

    def _start_read(self, st: _OpState, slab: PinnedSlabLease) -> None:
        st.slab = slab
        dst = self.slabs.view(slab, st.source.payload_bytes)

        def done(ok: bool, n: int) -> None:
            if ok:
                slab.advance(SlabLeaseState.FILLED)
                self.bytes_read += n
            self._push(self._ev(st, LoadStage.READ_SUBMITTED, ok, n,
                                FailureReason.SHORT_READ if n else FailureReason.READ_ERROR))
        try:
            FAILPOINTS.check("checkpoint_read")
        except FailpointTriggered:
            return done(False, 0)
        self.reader.submit(st.source, dst, done)

    def submit_upload(self, op: int, key: MaterializationKey, generation: int) -> None:
        st = self.ops[op]
        st.generation = generation
        try:
            FAILPOINTS.check("expert_upload")
        except FailpointTriggered:
            return self._push(self._ev(st, LoadStage.UPLOAD_SUBMITTED, False, 0, FailureReason.UPLOAD_ERROR))
        n = st.source.payload_bytes
        host = st.cached[:n] if st.cached is not None else self.slabs.view(st.slab, n)
        frame = self.arena.frame(st.ticket.layer, st.ticket.slot)
        if st.slab is not None:
            st.slab.advance(SlabLeaseState.UPLOADING)
        if self.cuda:
            with torch.cuda.stream(self.upload_stream):
                frame[:n].copy_(host, non_blocking=True)
                st.event = torch.cuda.Event()
                st.event.record(self.upload_stream)
            self._uploads.append(st)
        else:
            frame[:n].copy_(host)
            self._finish_upload(st)

    def _finish_upload(self, st: _OpState) -> None:
        n = st.source.payload_bytes
        self.bytes_uploaded += n
        if st.slab is not None:
            if self.cache is not None:
                self.cache.put((st.key.resource.group, st.key.resource.item), self.slabs.view(st.slab, n).clone())
            self._release_slab(st)
        self._push(self._ev(st, LoadStage.UPLOAD_SUBMITTED, True, n))

    def _release_slab(self, st: _OpState) -> None:
        self.slabs.release(st.slab)
        st.slab = None
        while self._waiting_reads:
            nxt = self.ops.get(self._waiting_reads.popleft())
            if nxt is None or nxt.cancelled:
                if nxt is not None:
                    self._push(self._ev(nxt, LoadStage.READ_SUBMITTED, False, 0))
                continue
            slab = self.slabs.acquire(nxt.op)
            if slab is None:
                self._waiting_reads.appendleft(nxt.op)
            else:
                self._start_read(nxt, slab)
            break

    def poll_install(self, op: int, key: MaterializationKey, generation: int) -> None:
        st = self.ops[op]
        st.generation = generation
        try:
            FAILPOINTS.check("resource_install")
            coord = self.residency.layer(st.ticket.layer)
            coord.activate(st.ticket)
            coord.publish(st.ticket)
            if self.on_install is not None:
                self.on_install(st.ticket.layer, st.ticket.expert, st.ticket.slot, st.ticket.generation,
                                self.arena.frame(st.ticket.layer, st.ticket.slot))
        except (ResidencyError, FailpointTriggered):
            return self._push(self._ev(st, LoadStage.INSTALLING, False, 0, FailureReason.INSTALL_ERROR))
        self._push(self._ev(st, LoadStage.INSTALLING, True, st.source.payload_bytes))

    def cancel(self, op: int) -> None:
        st = self.ops.get(op)
        if st is not None:
            st.cancelled = True
            if op in self._waiting_reads:          # never started: answer the owed completion now
                self._waiting_reads.remove(op)
                self._push(self._ev(st, LoadStage.READ_SUBMITTED, False, 0))

    def retire(self, op: int, key: MaterializationKey) -> None:
        st = self.ops.pop(op, None)
        if st is None:
            return
        if op in self._waiting_reads:
            self._waiting_reads.remove(op)
        if st.slab is not None and st.slab.state in (SlabLeaseState.LEASED, SlabLeaseState.FILLED):
            self._release_slab(st)
        coord = self.residency.layer(st.ticket.layer)
        if coord.in_flight(st.ticket.expert):
            try:
                coord.cancel(st.ticket)
            except ResidencyError:
                pass
        else:
            coord.evict(st.ticket.expert)

    def next_completion(self) -> Optional[CompletionEvent]:
        if self._uploads:
            still = []
            for st in self._uploads:
                if st.event.query():
                    self._finish_upload(st)
                else:
                    still.append(st)
            self._uploads = still
        with self._lock:
            return self._done.popleft() if self._done else None

    def close(self) -> None:
        if hasattr(self.reader, "close"):
            self.reader.close()
