"""Routed-expert arena: a fixed number of device frames per MoE layer, the full expert set in pinned host
memory, stable slots with generations and leases, event-gated uploads.

Per MoE layer:
  * host: every local expert's `[2I, H]` and `[H, I]` matrices in pinned memory (the streaming source);
  * device: `frames` slots of the same shapes (`e_w13` / `e_w2` of the layer's `LayerWeights` become the
    arena tensors, so the grouped GEMM indexes slots instead of experts);
  * `ExpertResidencyCoordinator` decides which slot an incoming expert takes (least recently used, never
    a leased one); the device table (expert -> slot) is updated by a kernel on the compute stream after
    it has waited for the upload event.

`ensure(layer, experts)` is called between routing and the expert GEMMs with the experts the batch
needs.  Resident ones are leased; missing ones are copied on the upload stream (which first waits for the
compute event recorded after the layer's previous GEMMs: no frame is overwritten while a kernel may still
read it), then the compute stream waits for the upload event.  `release(layer)` drops the leases and
records the consumer event.

Counterpart of the routed-expert arena and slot table of the reference's device runtime
(crates/ferrule-backend/src/cuda/context.rs:8044-8320, expert_table.rs:20-500) and of its CUDA
materialization provider (crates/ferrule-model/src/moe/cuda_materialization.rs:27-900).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..ops._lib import check, get_lib, status_tensor, stream_ptr
from ..runtime.expert_residency import ExpertResidencyCoordinator
from .weights import ModelWeights, QuantWeight


@dataclass
class ArenaStats:
    hits: int = 0
    misses: int = 0
    uploads: int = 0
    upload_bytes: int = 0
    evictions: int = 0
    ensure_calls: int = 0


_QW_PARTS = ("q", "scale", "packed", "sf")


def _parts(w) -> List[torch.Tensor]:
    """The per-expert tensors of an expert weight: the bf16 tensor itself, or the codes / scales / packed values /
    arranged scale factors of a quantised one (each indexed by expert in its first dimension)."""
    if isinstance(w, QuantWeight):
        return [getattr(w, n) for n in _QW_PARTS if getattr(w, n) is not None]
    return [w]


def _like(w, parts: List[torch.Tensor]):
    """`w` rebuilt over other tensors of the same kinds (frames instead of the full expert set)."""
    if not isinstance(w, QuantWeight):
        return parts[0]
    it = iter(parts)
    kw = {n: (next(it) if getattr(w, n) is not None else None) for n in _QW_PARTS}
    return QuantWeight(kw["q"], kw["scale"], w.group32, kw["packed"], kw["sf"])


class _LayerArena:
    def __init__(self, layer: int, w13, w2, frames: int, device):
        """w13 / w2: bf16 tensors [experts, ...] or `QuantWeight`s (FP8 blocks, MXFP4 containers or packed MXFP4):
        a frame holds one expert in the model's own form, so streamed experts cost their quantised bytes."""
        src = _parts(w13) + _parts(w2)
        self.n13 = len(_parts(w13))
        E = src[0].shape[0]
        self.layer, self.n_experts, self.frames = layer, E, frames
        self.host = [t.cpu().pin_memory() if device.type == "cuda" else t.cpu() for t in src]
        self.dev = [torch.zeros(frames, *t.shape[1:], dtype=t.dtype, device=device) for t in src]
        self.dev13, self.dev2 = _like(w13, self.dev[:self.n13]), _like(w2, self.dev[self.n13:])
        i32 = dict(dtype=torch.int32, device=device)
        self.expert_to_slot = torch.full((E,), -1, **i32)
        self.slot_expert = torch.full((frames,), -1, **i32)
        self.slot_gen = torch.zeros(frames, **i32)
        self.miss = torch.zeros(64, **i32)
        self.coord = ExpertResidencyCoordinator(layer, frames, E)
        self.leases: List[tuple] = []
        self.consumer_event: Optional[torch.cuda.Event] = None
        self.expert_bytes = sum(t[0].numel() * t.element_size() for t in self.host)

    def copy_in(self, slot: int, expert: int, non_blocking: bool = False) -> None:
        for d, h in zip(self.dev, self.host):
            d[slot].copy_(h[expert], non_blocking=non_blocking)


class ExpertArena:
    def __init__(self, weights: ModelWeights, resident_fraction: float = 0.5, min_frames: int = 0,
                 replace_weights: bool = True, mtp_resident: bool = True):
        """Moves the routed experts of every MoE layer of `weights` to pinned host memory and replaces the
        layer's expert tensors by arena frames (in place: `weights` is the streaming model afterwards).
        `replace_weights=False` keeps the model's tensors (the fp32 oracle reads them directly) and runs the
        residency protocol beside it.  `mtp_resident`: the proposal stages keep all their experts on the device
        (one stage is 1 / n_layers of the expert bytes): drafting runs between transactions, where nothing can
        park and wait for an upload, so with streamed proposal experts every draft would upload inline."""
        self.device = weights.embed.device
        self.cuda = self.device.type == "cuda"
        self.layers: Dict[int, _LayerArena] = {}
        self.stats = ArenaStats()
        self.upload_stream = torch.cuda.Stream(device=self.device) if self.cuda else None
        all_layers = list(weights.layers) + ([] if mtp_resident else [m.layer for m in weights.mtp])
        for i, lw in enumerate(all_layers):
            if not lw.is_moe or lw.e_w13 is None:
                continue
            E = lw.e_w13.shape[0]
            frames = max(min_frames, min(E, int(round(E * resident_fraction))), 1)
            la = _LayerArena(i, lw.e_w13, lw.e_w2, frames, self.device)
            if replace_weights:
                lw.e_w13, lw.e_w2 = la.dev13, la.dev2
            self.layers[i] = la

    def frames(self, layer: int) -> int:
        return self.layers[layer].frames

    def resident(self, layer: int) -> List[int]:
        return self.layers[layer].coord.resident()

    # ------------------------------------------------------------------ per-step protocol
    def ensure(self, layer: int, experts: Sequence[int]) -> int:
        """Make `experts` resident and leased; returns the number of uploads issued."""
        la = self.layers[layer]
        self.stats.ensure_calls += 1
        need = sorted(set(int(e) for e in experts))
        if len(need) > la.frames:
            raise RuntimeError(f"layer {layer}: the batch needs {len(need)} distinct experts but only {la.frames} frames exist")
        missing = []
        for e in need:
            if la.coord.resolve(e) is not None:
                la.leases.append(la.coord.lease(e))
                self.stats.hits += 1
            else:
                missing.append(e)
                self.stats.misses += 1
        if not missing:
            return 0
        tickets = [la.coord.prepare(e, required=True) for e in missing]
        n = len(tickets)
        updates = []
        if self.cuda:
            up = self.upload_stream
            if la.consumer_event is not None:
                up.wait_event(la.consumer_event)        # no frame is overwritten under a running kernel
            with torch.cuda.stream(up):
                for t in tickets:
                    la.copy_in(t.slot, t.expert, non_blocking=True)
                done = torch.cuda.Event()
                done.record(up)
            torch.cuda.current_stream().wait_event(done)
        else:
            for t in tickets:
                la.copy_in(t.slot, t.expert)
        for j, t in enumerate(tickets):
            la.coord.activate(t)
            la.coord.publish(t)
            la.leases.append(la.coord.lease(t.expert))
            updates.append([t.slot, t.expert, t.generation, -1 if t.evicted is None else t.evicted])
            self.stats.evictions += 0 if t.evicted is None else 1
        self.stats.uploads += n
        self.stats.upload_bytes += n * la.expert_bytes
        self._apply(la, updates)
        return n

    # ------------------------------------------------------------------ asynchronous protocol (one expert at a time)
    def missing(self, layer: int, experts: Sequence[int]) -> List[int]:
        la = self.layers[layer]
        return [int(e) for e in sorted(set(int(x) for x in experts)) if la.coord.resolve(int(e)) is None]

    def lease_resident(self, layer: int, experts: Sequence[int]) -> Dict[int, tuple]:
        """Lease every expert of `experts` that is resident -> {expert: lease}; the caller releases them with
        `release_leases`."""
        la = self.layers[layer]
        out = {}
        for e in sorted(set(int(x) for x in experts)):
            if la.coord.resolve(e) is not None:
                out[e] = la.coord.lease(e)
                self.stats.hits += 1
        return out

    def release_leases(self, layer: int, leases: Sequence[tuple]) -> None:
        la = self.layers[layer]
        for slot, gen in leases:
            la.coord.release(slot, gen)
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            la.consumer_event = ev

    def begin_upload(self, layer: int, expert: int):
        """Pick a frame for `expert` (evicting the least recently used unleased one) and start its copy on the
        upload stream -> (ticket, event or None).  Raises when every frame is leased."""
        la = self.layers[layer]
        t = la.coord.prepare(int(expert), required=True)
        self.stats.misses += 1
        ev = None
        if self.cuda:
            up = self.upload_stream
            if la.consumer_event is not None:
                up.wait_event(la.consumer_event)
            with torch.cuda.stream(up):
                la.copy_in(t.slot, t.expert, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(up)
        else:
            la.copy_in(t.slot, t.expert)
        return t, ev

    def finish_install(self, layer: int, ticket) -> None:
        """The copy has completed: publish the frame in the coordinator and in the device table."""
        la = self.layers[layer]
        la.coord.activate(ticket)
        la.coord.publish(ticket)
        self.stats.uploads += 1
        self.stats.upload_bytes += la.expert_bytes
        self.stats.evictions += 0 if ticket.evicted is None else 1
        self._apply(la, [[ticket.slot, ticket.expert, ticket.generation, -1 if ticket.evicted is None else ticket.evicted]])

    def _apply(self, la: _LayerArena, updates: List[List[int]]) -> None:
        n = len(updates)
        if self.cuda:
            # a pageable source makes this copy synchronous with the host, so the list can be reused at once
            upd = torch.tensor(updates, dtype=torch.int32).to(self.device)
            lib = get_lib(True)
            check(lib.fb_expert_table_apply(la.expert_to_slot.data_ptr(), la.slot_expert.data_ptr(), la.slot_gen.data_ptr(),
                                            upd.data_ptr(), n, la.n_experts, la.frames,
                                            status_tensor(self.device).data_ptr(), stream_ptr()), "fb_expert_table_apply")
        else:
            for slot, e, gen, ev in updates:
                if ev >= 0 and int(la.expert_to_slot[ev]) == slot:
                    la.expert_to_slot[ev] = -1
                prev = int(la.slot_expert[slot])
                if prev >= 0 and int(la.expert_to_slot[prev]) == slot:
                    la.expert_to_slot[prev] = -1
                la.slot_expert[slot], la.slot_gen[slot], la.expert_to_slot[e] = e, gen, slot

    def resolve_plan(self, layer: int, plan) -> None:
        """Rewrite the plan's per-tile expert ids into arena slots (device side)."""
        la = self.layers[layer]
        lib = get_lib(True)
        la.miss.zero_()
        check(lib.fb_expert_table_resolve(plan.tile_group.data_ptr(), plan.tile_rows.data_ptr(), plan.meta.data_ptr(),
                                          plan.max_tiles, la.expert_to_slot.data_ptr(), la.n_experts, la.miss.data_ptr(),
                                          stream_ptr()), "fb_expert_table_resolve")

    def release(self, layer: int) -> None:
        la = self.layers[layer]
        for slot, gen in la.leases:
            la.coord.release(slot, gen)
        la.leases = []
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            la.consumer_event = ev
