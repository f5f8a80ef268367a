"""Three-band deficit-round-robin queue for materialization work.

Bands, highest first: REQUIRED (a transaction is blocked on it), PREFETCH (declared ahead of
need), BACKGROUND (warm-up).  Each band earns `quantum[band]` credit per round and spends the
item's cost; a band whose head waited `aging_ticks` rounds is served regardless of credit, and no
band may run a debt larger than `debt_bound` times its quantum.  `starvation_ticks` reports how
long the oldest queued item of each band has waited.

Counterpart of crates/ferrule-runtime/src/io/fairness.rs:10-33 (bands/config), :35-90 (queue),
:144-180 (pop policy).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from enum import IntEnum
from typing import Deque, Dict, Generic, Optional, Tuple, TypeVar

T = TypeVar("T")


class Band(IntEnum):
    REQUIRED = 0
    PREFETCH = 1
    BACKGROUND = 2


@dataclass
class FairQueueConfig:
    quantum: Tuple[int, int, int] = (8, 3, 1)
    aging_ticks: int = 32
    debt_bound: int = 4


@dataclass
class _Entry(Generic[T]):
    item: T
    cost: int
    enqueued_tick: int


class FairQueue(Generic[T]):
    def __init__(self, cfg: Optional[FairQueueConfig] = None):
        if cfg is not None and (len(cfg.quantum) != len(Band) or min(cfg.quantum) <= 0 or cfg.aging_ticks <= 0
                                or cfg.debt_bound < 0):
            raise ValueError("fair queue: every band needs a positive quantum, aging_ticks > 0, debt_bound >= 0")
        self.cfg = cfg or FairQueueConfig()
        self._q: Dict[Band, Deque[_Entry[T]]] = {b: deque() for b in Band}
        self._credit: Dict[Band, int] = {b: 0 for b in Band}
        self._tick = 0
        self.served: Dict[Band, int] = {b: 0 for b in Band}
        self.aged: Dict[Band, int] = {b: 0 for b in Band}

    def push(self, band: Band, item: T, cost: int = 1) -> None:
        self._q[band].append(_Entry(item, max(cost, 1), self._tick))

    def promote(self, item: T, to: Band) -> bool:
        """Move an item to a more urgent band (a prefetch became required)."""
        for band in Band:
            if band <= to:
                continue
            for e in self._q[band]:
                if e.item == item:
                    self._q[band].remove(e)
                    self._q[to].append(_Entry(item, e.cost, e.enqueued_tick))
                    return True
        return False

    def remove(self, item: T) -> bool:
        for band in Band:
            for e in self._q[band]:
                if e.item == item:
                    self._q[band].remove(e)
                    return True
        return False

    def __len__(self) -> int:
        return sum(len(q) for q in self._q.values())

    def starvation_ticks(self) -> Dict[Band, int]:
        return {b: (self._tick - q[0].enqueued_tick if q else 0) for b, q in self._q.items()}

    def pop(self) -> Optional[Tuple[Band, T]]:
        if not len(self):
            return None
        self._tick += 1
        # 1. aging: the longest-waiting head beyond the limit goes first
        oldest: Optional[Band] = None
        for b in Band:
            q = self._q[b]
            if q and self._tick - q[0].enqueued_tick > self.cfg.aging_ticks:
                if oldest is None or q[0].enqueued_tick < self._q[oldest][0].enqueued_tick:
                    oldest = b
        if oldest is not None:
            self.aged[oldest] += 1
            return self._serve(oldest)
        # 2. deficit round robin in priority order
        for _ in range(2 * self.cfg.debt_bound + 2):
            for b in Band:
                q = self._q[b]
                if not q:
                    self._credit[b] = 0
                    continue
                floor = -self.cfg.debt_bound * self.cfg.quantum[b]
                if self._credit[b] >= q[0].cost or (self._credit[b] > 0 and self._credit[b] - q[0].cost >= floor):
                    return self._serve(b)
            for b in Band:
                if self._q[b]:
                    self._credit[b] += self.cfg.quantum[b]
        for b in Band:                      # costs larger than any reachable credit: serve by priority
            if self._q[b]:
                return self._serve(b)
        return None

    def _serve(self, b: Band) -> Tuple[Band, T]:
        e = self._q[b].popleft()
        # forced progress (aging, oversized costs) is served on credit the band does not have: the debt is capped,
        # so a band that was pushed ahead for a while does not pay for it forever
        self._credit[b] = max(self._credit[b] - e.cost, -self.cfg.debt_bound * self.cfg.quantum[b])
        self.served[b] += 1
        return b, e.item
