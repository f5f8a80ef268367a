"""Memory policy types: topology, pools, limits, and an owner-thread LRU bounded by entries and bytes.

Counterpart of crates/ferrule-common/src/memory.rs:13-19 (topology), :45-83 (pools and limits),
:115-230 (OwnerMemoryLru).
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass
from enum import Enum
from typing import Callable, Dict, Generic, Hashable, List, Optional, TypeVar


class MemoryTopology(Enum):
    DISCRETE = "discrete"                   # separate host and device memory (B200 + x86 host)
    COHERENT_UNIFIED = "coherent_unified"   # one coherent pool (e.g. Grace-class systems)


class MemoryPoolKind(Enum):
    DEVICE_WEIGHTS = "device_weights"
    DEVICE_KV = "device_kv"
    DEVICE_ARENA = "device_arena"
    DEVICE_EXPERT_SLOTS = "device_expert_slots"
    HOST_PINNED = "host_pinned"
    HOST_PAGEABLE = "host_pageable"


@dataclass(frozen=True)
class MemoryPoolLimits:
    max_bytes: int
    max_entries: int = 1 << 30
    reserve_bytes: int = 0                  # kept free for execution

    def usable(self) -> int:
        return max(self.max_bytes - self.reserve_bytes, 0)


K = TypeVar("K", bound=Hashable)
V = TypeVar("V")


class OwnerMemoryLru(Generic[K, V]):
    """LRU limited by entry count and bytes; single owner thread, no locking.  Pinned keys are never
    evicted.  `on_evict(key, value)` runs for every entry pushed out."""

    def __init__(self, limits: MemoryPoolLimits, on_evict: Optional[Callable[[K, V], None]] = None):
        self.limits = limits
        self._d: "OrderedDict[K, Tuple[V, int]]" = OrderedDict()
        self._pinned: Dict[K, int] = {}
        self.bytes = 0
        self.hits = self.misses = self.evictions = 0
        self._on_evict = on_evict

    def __len__(self) -> int:
        return len(self._d)

    def __contains__(self, k: K) -> bool:
        return k in self._d

    def get(self, k: K) -> Optional[V]:
        e = self._d.get(k)
        if e is None:
            self.misses += 1
            return None
        self._d.move_to_end(k)
        self.hits += 1
        return e[0]

    def pin(self, k: K) -> None:
        self._pinned[k] = self._pinned.get(k, 0) + 1

    def unpin(self, k: K) -> None:
        n = self._pinned.get(k, 0) - 1
        if n <= 0:
            self._pinned.pop(k, None)
        else:
            self._pinned[k] = n

    def put(self, k: K, v: V, nbytes: int) -> bool:
        """Insert (replacing an older value); False if it cannot fit even after evicting everything
        that is not pinned."""
        if nbytes > self.limits.usable():
            return False
        old = self._d.pop(k, None)
        if old is not None:
            self.bytes -= old[1]
        while (self.bytes + nbytes > self.limits.usable() or len(self._d) + 1 > self.limits.max_entries):
            victim = next((key for key in self._d if key not in self._pinned), None)
            if victim is None:
                if old is not None:                 # the value that was there stays (it fitted before)
                    self._d[k] = old
                    self.bytes += old[1]
                return False
            val, nb = self._d.pop(victim)
            self.bytes -= nb
            self.evictions += 1
            if self._on_evict:
                self._on_evict(victim, val)
        self._d[k] = (v, nbytes)
        self.bytes += nbytes
        return True

    def pop(self, k: K) -> Optional[V]:
        e = self._d.pop(k, None)
        if e is None:
            return None
        self.bytes -= e[1]
        return e[0]

    def keys_lru_first(self) -> List[K]:
        return list(self._d)
