"""Expert residency: stable device slots, generations and leases for streamed routed experts.

A layer owns `capacity` stable slots.  Bringing an expert in is two-phase: `prepare(expert)`
picks a victim slot (least recently used among slots that are neither leased nor reserved),
reserves it and hands back a ticket; once the upload has landed `activate(ticket)` binds the
expert to the slot with a new generation, and `publish(ticket)` makes it resolvable; `cancel`
returns the slot.  `resolve` answers (slot, generation) for resident experts and records misses;
`lease` pins a resident expert for the duration of a dispatch, so eviction can never pull
weights from under a running kernel.  A prefetch-prepared install can be promoted to required.

Counterpart of crates/ferrule-common/src/expert_residency.rs:247-294 (control trait), :297-826
(coordinator) and crates/ferrule-runtime/src/expert_residency.rs:18-130 (per-layer controller).
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Dict, List, Optional, Tuple


class ResidencyError(RuntimeError):
    pass


class SlotState(Enum):
    EMPTY = "empty"
    PREPARING = "preparing"      # reserved for an install in flight
    ACTIVE = "active"            # bound, not yet visible
    READY = "ready"              # resolvable


@dataclass
class Slot:
    index: int
    expert: Optional[int] = None
    generation: int = 0
    state: SlotState = SlotState.EMPTY
    leases: int = 0
    last_use: int = 0
    incoming: Optional[int] = None
    required: bool = False


@dataclass(frozen=True)
class InstallTicket:
    layer: int
    slot: int
    expert: int
    generation: int
    evicted: Optional[int]


@dataclass
class ResidencyStats:
    hits: int = 0
    misses: int = 0
    installs: int = 0
    evictions: int = 0
    cancelled: int = 0
    promoted: int = 0
    stale_resolves: int = 0
    lease_high_water: int = 0


class ExpertResidencyCoordinator:
    def __init__(self, layer: int, capacity: int, n_experts: int):
        if capacity <= 0:
            raise ResidencyError("capacity must be positive")
        self.layer, self.capacity, self.n_experts = layer, capacity, n_experts
        self.slots = [Slot(i) for i in range(capacity)]
        self.where: Dict[int, int] = {}            # expert -> slot (READY only)
        self.incoming: Dict[int, int] = {}         # expert -> slot (PREPARING / ACTIVE)
        # resident experts that must not be evicted although nobody leases them yet: installed for a parked
        # transaction that has not been resumed (set by the provider before it asks for a slot)
        self.protected: set = set()
        self._clock = 0
        self._leases_out = 0
        self.stats = ResidencyStats()

    # ------------------------------------------------------------------ lookup
    def resolve(self, expert: int) -> Optional[Tuple[int, int]]:
        s = self.where.get(expert)
        if s is None:
            self.stats.misses += 1
            return None
        self._clock += 1
        self.slots[s].last_use = self._clock
        self.stats.hits += 1
        return s, self.slots[s].generation

    def is_current(self, slot: int, generation: int) -> bool:
        ok = 0 <= slot < self.capacity and self.slots[slot].generation == generation and \
            self.slots[slot].state == SlotState.READY
        if not ok:
            self.stats.stale_resolves += 1
        return ok

    def resident(self) -> List[int]:
        return sorted(self.where)

    def in_flight(self, expert: int) -> bool:
        return expert in self.incoming

    # ------------------------------------------------------------------ install
    def _victim(self) -> Optional[Slot]:
        cands = [s for s in self.slots if s.state in (SlotState.EMPTY, SlotState.READY) and s.leases == 0
                 and (s.expert is None or s.expert not in self.protected)]
        if not cands:
            return None
        empties = [s for s in cands if s.state == SlotState.EMPTY]
        return empties[0] if empties else min(cands, key=lambda s: s.last_use)

    def prepare(self, expert: int, required: bool = True) -> InstallTicket:
        if not 0 <= expert < self.n_experts:
            raise ResidencyError(f"expert {expert} out of range")
        if expert in self.where:
            raise ResidencyError(f"expert {expert} is already resident")
        if expert in self.incoming:
            raise ResidencyError(f"expert {expert} is already being installed")
        v = self._victim()
        if v is None:
            raise ResidencyError("every slot is leased or reserved")
        evicted = v.expert if v.state == SlotState.READY else None
        if evicted is not None:
            del self.where[evicted]
            self.stats.evictions += 1
        v.state, v.expert, v.incoming, v.required = SlotState.PREPARING, None, expert, required
        v.generation += 1
        self.incoming[expert] = v.index
        return InstallTicket(self.layer, v.index, expert, v.generation, evicted)

    def promote(self, expert: int) -> bool:
        """A prefetch install became required by an execution."""
        s = self.incoming.get(expert)
        if s is None or self.slots[s].required:
            return False
        self.slots[s].required = True
        self.stats.promoted += 1
        return True

    def _slot_of(self, t: InstallTicket) -> Slot:
        s = self.slots[t.slot]
        if s.generation != t.generation or s.incoming != t.expert:
            raise ResidencyError("ticket does not match the slot any more")
        return s

    def activate(self, t: InstallTicket) -> None:
        s = self._slot_of(t)
        if s.state != SlotState.PREPARING:
            raise ResidencyError(f"slot {t.slot} is {s.state.value}, cannot activate")
        s.state, s.expert = SlotState.ACTIVE, t.expert

    def publish(self, t: InstallTicket) -> None:
        s = self._slot_of(t)
        if s.state != SlotState.ACTIVE:
            raise ResidencyError(f"slot {t.slot} is {s.state.value}, cannot publish")
        s.state, s.incoming = SlotState.READY, None
        self._clock += 1
        s.last_use = self._clock
        del self.incoming[t.expert]
        self.where[t.expert] = s.index
        self.stats.installs += 1

    def cancel(self, t: InstallTicket) -> None:
        s = self._slot_of(t)
        if s.state not in (SlotState.PREPARING, SlotState.ACTIVE):
            raise ResidencyError("nothing to cancel")
        s.state, s.expert, s.incoming = SlotState.EMPTY, None, None
        s.generation += 1
        del self.incoming[t.expert]
        self.stats.cancelled += 1

    # ------------------------------------------------------------------ leases
    def lease(self, expert: int) -> Tuple[int, int]:
        s = self.where.get(expert)
        if s is None:
            raise ResidencyError(f"expert {expert} is not resident")
        self.slots[s].leases += 1
        self._leases_out += 1
        self.stats.lease_high_water = max(self.stats.lease_high_water, self._leases_out)
        return s, self.slots[s].generation

    def release(self, slot: int, generation: int) -> None:
        s = self.slots[slot]
        if s.generation != generation or s.leases <= 0:
            raise ResidencyError("lease does not match the slot")
        s.leases -= 1
        self._leases_out -= 1

    def evict(self, expert: int) -> bool:
        s = self.where.get(expert)
        if s is None or self.slots[s].leases:
            return False
        sl = self.slots[s]
        sl.state, sl.expert = SlotState.EMPTY, None
        sl.generation += 1
        del self.where[expert]
        self.stats.evictions += 1
        return True


class ExpertResidencyController:
    """One coordinator per MoE layer."""

    def __init__(self, layers: List[int], capacity_per_layer: Dict[int, int], n_experts: int):
        self.layers = {l: ExpertResidencyCoordinator(l, capacity_per_layer[l], n_experts) for l in layers}

    def layer(self, l: int) -> ExpertResidencyCoordinator:
        return self.layers[l]

    def stats(self) -> Dict[int, ResidencyStats]:
        return {l: c.stats for l, c in self.layers.items()}


def plan_residency(device_budget_bytes: int, expert_bytes: int, moe_layers: List[int], n_experts: int,
                   min_per_layer: int, max_fraction: float = 1.0) -> Dict[int, int]:
    """Device budget -> expert slots per layer (equal split, at least top-k + shared working set, at
    most `max_fraction` of the experts).  Counterpart of crates/ferrule-model/src/moe/residency.rs."""
    if not moe_layers:
        return {}
    per_layer = device_budget_bytes // max(len(moe_layers), 1) // max(expert_bytes, 1)
    cap = max(min_per_layer, min(per_layer, int(n_experts * max_fraction)))
    if cap * expert_bytes * len(moe_layers) > device_budget_bytes and cap > min_per_layer:
        cap = max(min_per_layer, per_layer)
    return {l: min(cap, n_experts) for l in moe_layers}
