"""Hard-resource broker: bounded credits for everything physical the runtime consumes.

A claim names amounts of several resource kinds and is granted atomically or not at all.
Each kind has a capacity and an *execution reserve*: background work (prefetch, warm-up) may
not dip into the reserve, required work may.  Once a grant is marked submitted (the physical
operation is in flight) it cannot be revoked; it is returned only by `complete`.

Counterpart of crates/ferrule-runtime/src/scheduling/resources.rs:28-62 (kinds), :100-215
(claims/grants), :285-288 (submitted irrevocable), :375-520 (broker).
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Dict, Optional


class ResourceKind(Enum):
    READ_SLOTS = "read_slots"
    PINNED_BYTES = "pinned_bytes"
    STORAGE_BYTES = "storage_bytes"
    UPLOAD_SLOTS = "upload_slots"
    UPLOAD_BYTES = "upload_bytes"
    INSTALL_SLOTS = "install_slots"
    INSTALL_BYTES = "install_bytes"
    RESIDENT_BYTES = "resident_bytes"
    RESIDENCY_LEASES = "residency_leases"
    ARENAS = "arenas"
    KV_PAGES = "kv_pages"
    CONTINUATIONS = "continuations"
    WAITERS = "waiters"
    LOAD_OPS = "load_ops"
    READY_COHORTS = "ready_cohorts"


class ResourceError(RuntimeError):
    pass


@dataclass
class ResourceLimit:
    capacity: int
    execution_reserve: int = 0


@dataclass
class Grant:
    grant_id: int
    amounts: Dict[ResourceKind, int]
    required: bool
    submitted: bool = False
    released: bool = False


@dataclass
class ResourceUsage:
    in_use: int = 0
    high_water: int = 0
    denied: int = 0


class PhysicalResourceBroker:
    def __init__(self, limits: Optional[Dict[ResourceKind, ResourceLimit]] = None):
        self.limits: Dict[ResourceKind, ResourceLimit] = {k: ResourceLimit(1 << 62) for k in ResourceKind}
        if limits:
            self.limits.update(limits)
        self.usage: Dict[ResourceKind, ResourceUsage] = {k: ResourceUsage() for k in ResourceKind}
        self._grants: Dict[int, Grant] = {}
        self._next = 0

    def set_limit(self, kind: ResourceKind, capacity: int, execution_reserve: int = 0) -> None:
        if execution_reserve > capacity:
            raise ResourceError("reserve larger than capacity")
        self.limits[kind] = ResourceLimit(capacity, execution_reserve)

    def available(self, kind: ResourceKind, required: bool = True) -> int:
        lim = self.limits[kind]
        cap = lim.capacity if required else lim.capacity - lim.execution_reserve
        return max(cap - self.usage[kind].in_use, 0)

    def try_claim(self, amounts: Dict[ResourceKind, int], required: bool = True) -> Optional[Grant]:
        """All-or-nothing multi-kind claim."""
        for kind, n in amounts.items():
            if n < 0:
                raise ResourceError("negative claim")
            if n > self.available(kind, required):
                self.usage[kind].denied += 1
                return None
        for kind, n in amounts.items():
            u = self.usage[kind]
            u.in_use += n
            u.high_water = max(u.high_water, u.in_use)
        g = Grant(self._next, dict(amounts), required)
        self._next += 1
        self._grants[g.grant_id] = g
        return g

    def mark_submitted(self, grant: Grant) -> None:
        if grant.released:
            raise ResourceError("grant already released")
        grant.submitted = True

    def revoke(self, grant: Grant) -> None:
        """Give back a grant whose operation was never started."""
        if grant.submitted:
            raise ResourceError("submitted grants cannot be revoked; wait for completion")
        self._release(grant)

    def complete(self, grant: Grant) -> None:
        """The physical operation finished (or was proven never to run)."""
        self._release(grant)

    def shrink(self, grant: Grant, kind: ResourceKind, amount: int) -> None:
        """Return part of a grant (e.g. speculative KV pages that were rejected)."""
        if grant.released:
            raise ResourceError("grant already released")
        have = grant.amounts.get(kind, 0)
        if amount < 0 or amount > have:
            raise ResourceError("shrinking below zero" if amount > have else "negative shrink")
        grant.amounts[kind] = have - amount
        self.usage[kind].in_use -= amount

    def _release(self, grant: Grant) -> None:
        if grant.released:
            raise ResourceError("grant released twice")
        for kind, n in grant.amounts.items():
            self.usage[kind].in_use -= n
            if self.usage[kind].in_use < 0:
                raise ResourceError(f"{kind.value} underflow")
        grant.released = True
        self._grants.pop(grant.grant_id, None)

    def outstanding(self) -> int:
        return len(self._grants)

    def snapshot(self) -> Dict[str, Dict[str, int]]:
        return {k.value: {"in_use": u.in_use, "high_water": u.high_water, "denied": u.denied,
                          "capacity": self.limits[k].capacity}
                for k, u in self.usage.items() if u.high_water or u.denied}
