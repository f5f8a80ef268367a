"""Asynchronous routed-expert streaming for the real model: the forward stops at a MoE layer whose experts are
not resident, the engine parks the transaction (`Waiting`), the load registry drives this provider (pinned host
copy -> device frame -> slot-table install) and the transaction resumes at the layer it stopped at.

* `NeedExperts` - raised inside the forward, between routing and the expert GEMMs, when the batch routes to
  experts that are not in the arena.  Nothing of the layer has been committed at that point (the layer's input
  buffer is only overwritten by its last kernel), so the layer is simply run again on resume.
* `expert_key` - the `MaterializationKey` of (layer, expert); the destination generation counts how often the
  expert has been evicted, so a reload after an eviction is a new payload for the registry.
* `ArenaProvider` - `MaterializationProvider` over `ExpertArena`: `reserve` takes a frame (evicting the least
  recently used unleased expert and retiring its registry entry), `submit_read` completes at once (the source
  is pinned host memory), `submit_upload` starts the copy on the upload stream and completes when its event
  has fired, `poll_install` publishes the frame in the coordinator and the device table.

Counterpart of the CUDA materialization provider and the suspend / resume path of the reference
(crates/ferrule-model/src/moe/cuda_materialization.rs:27-900, crates/ferrule-model/src/runner.rs:221-236,
crates/ferrule-runtime/src/engine/driver.rs:3282-3444).
"""
from __future__ import annotations

from collections import deque
from typing import Deque, Dict, List, Optional, Tuple

import torch

from ..runtime.io_protocol import (CompletionEvent, CompletionOutcome, FailureReason, LoadStage, MaterializationKey,
                                   MaterializationResourcePlan, ResourceId, ResourceKind, content_hash)
from ..runtime.provider import MaterializationProvider, ProviderError
from .expert_arena import ExpertArena


class NeedExperts(Exception):
    """The batch routes to experts of `layer` that are not resident."""

    def __init__(self, layer: int, missing: List[int]):
        super().__init__(f"layer {layer}: experts {missing} are not resident")
        self.layer, self.missing = layer, list(missing)
        self.hidden: Optional[torch.Tensor] = None      # the layer's input rows (filled by the forward loop)


def expert_key(model: str, layer: int, expert: int, generation: int = 0, device: int = 0) -> MaterializationKey:
    ident = f"{model}/{layer}/{expert}".encode()
    return MaterializationKey(model, content_hash(b"pinned-host", ident), content_hash(ident),
                              ResourceId(ResourceKind.ROUTED_EXPERT, layer, expert), 0, "cuda-sm100a", device, 0,
                              generation)


class ArenaProvider(MaterializationProvider):
    def __init__(self, arena: ExpertArena, model: str = "model"):
        self.arena, self.model = arena, model
        self.registry = None                           # set by `attach`: evictions retire the victim's entry
        self._gen: Dict[Tuple[int, int], int] = {}     # (layer, expert) -> times evicted
        self._ops: Dict[int, dict] = {}
        self._ready: Deque[CompletionEvent] = deque()
        self._uploading: List[Tuple[int, MaterializationKey, int]] = []
        # uploads that found every frame of their layer leased: retried at every poll (a transaction that ends gives
        # its frames back); op -> [key, generation, polls without a frame]
        self._starved: Dict[int, list] = {}
        self._resident_op: Dict[Tuple[int, int], Tuple[int, MaterializationKey]] = {}
        self.clock_ns = 0

    def attach(self, registry) -> None:
        self.registry = registry

    def key(self, layer: int, expert: int) -> MaterializationKey:
        return expert_key(self.model, layer, expert, self._gen.get((layer, expert), 0))

    # ---- provider API --------------------------------------------------------------------
    def plan(self, key: MaterializationKey) -> MaterializationResourcePlan:
        la = self.arena.layers[key.resource.group]
        return MaterializationResourcePlan.for_payload(la.expert_bytes)

    def reserve(self, op: int, key: MaterializationKey) -> None:
        layer, expert = key.resource.group, key.resource.item
        if key.destination_generation != self._gen.get((layer, expert), 0):
            raise ProviderError(f"stale destination generation for layer {layer} expert {expert}")
        self._ops[op] = {"key": key, "ticket": None, "event": None}

    def _emit(self, op: int, key: MaterializationKey, stage: LoadStage, generation: int,
              outcome: CompletionOutcome = CompletionOutcome.OK, failure: Optional[FailureReason] = None) -> None:
        self.clock_ns += 1000
        la = self.arena.layers[key.resource.group]
        done = la.expert_bytes if outcome == CompletionOutcome.OK else 0
        self._ready.append(CompletionEvent(op, key, stage, generation, outcome, done, failure, self.clock_ns))

    def submit_read(self, op: int, key: MaterializationKey, generation: int) -> None:
        self._emit(op, key, LoadStage.READ_SUBMITTED, generation)      # the source already sits in pinned memory

    def submit_upload(self, op: int, key: MaterializationKey, generation: int) -> None:
        layer, expert = key.resource.group, key.resource.item
        if not self._start_upload(op, key, generation):
            self._starved[op] = [key, generation, 0]     # every frame is leased right now: try again at the next polls

    def _start_upload(self, op: int, key: MaterializationKey, generation: int) -> bool:
        layer, expert = key.resource.group, key.resource.item
        st = self._ops[op]
        if self.registry is not None:
            # payloads a parked transaction waits for stay put from their install until that transaction resumes
            # and leases them itself
            awaited = self.registry.awaited_ops()
            self.arena.layers[layer].coord.protected = {e for (l, e), (o, _) in self._resident_op.items()
                                                        if l == layer and o in awaited}
        try:
            ticket, event = self.arena.begin_upload(layer, expert)
        except Exception:  # noqa: BLE001 - no frame without a lease
            return False
        st["ticket"], st["event"] = ticket, event
        if ticket.evicted is not None:
            self._evicted(layer, ticket.evicted)
        self._uploading.append((op, key, generation))
        return True

    def starving(self, min_polls: int = 8) -> List[int]:
        """Operations that have found no free frame for at least `min_polls` polls: the transactions that lease the
        frames are parked themselves, nobody will give one up by itself."""
        return [op for op, (_, _, n) in self._starved.items() if n >= min_polls]

    def _evicted(self, layer: int, expert: int) -> None:
        self._gen[(layer, expert)] = self._gen.get((layer, expert), 0) + 1
        old = self._resident_op.pop((layer, expert), None)
        if old is not None and self.registry is not None:
            try:
                self.registry.cancel(old[0])            # resident and unleased: retires the entry
            except RuntimeError:
                pass                                    # a parked transaction still holds it; its resume re-checks

    def poll_install(self, op: int, key: MaterializationKey, generation: int) -> None:
        st = self._ops[op]
        self.arena.finish_install(key.resource.group, st["ticket"])
        self._resident_op[(key.resource.group, key.resource.item)] = (op, key)
        self._emit(op, key, LoadStage.INSTALLING, generation)

    def cancel(self, op: int) -> None:
        st = self._ops.get(op)
        if st is None:
            return
        starved = self._starved.pop(op, None)
        if starved is not None:                          # never got a frame: nothing to undo
            self._emit(op, starved[0], LoadStage.UPLOAD_SUBMITTED, starved[1], CompletionOutcome.CANCELLED,
                       FailureReason.CANCELLED)
            return
        for i, (o, key, gen) in enumerate(self._uploading):
            if o == op:
                del self._uploading[i]
                if st["event"] is not None:
                    st["event"].synchronize()
                self.arena.layers[key.resource.group].coord.cancel(st["ticket"])
                self._emit(op, key, LoadStage.UPLOAD_SUBMITTED, gen, CompletionOutcome.CANCELLED,
                           FailureReason.CANCELLED)
                return

    def retire(self, op: int, key: MaterializationKey) -> None:
        self._ops.pop(op, None)

    def next_completion(self) -> Optional[CompletionEvent]:
        for op in list(self._starved):
            key, gen, _ = self._starved[op]
            if self._start_upload(op, key, gen):
                del self._starved[op]
            else:
                self._starved[op][2] += 1
        still = []
        for op, key, gen in self._uploading:
            ev = self._ops[op]["event"]
            if ev is None or ev.query():
                self._emit(op, key, LoadStage.UPLOAD_SUBMITTED, gen)
            else:
                still.append((op, key, gen))
        self._uploading = still
        return self._ready.popleft() if self._ready else None
