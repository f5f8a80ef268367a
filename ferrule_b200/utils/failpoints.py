"""Operation counters and one-shot failpoints.

Counters tally launches, allocations, synchronisations, uploads per operator family.  A failpoint
is armed by name for the next N hits; code that is about to do the named thing calls
`FAILPOINTS.check(name)`, which raises `FailpointTriggered` when armed.  Failures are injected on
the host, before a launch or copy is issued; nothing here makes a GPU fault.

Counterpart of crates/ferrule-backend/src/cuda/counters.rs:9-126 (failpoints), :128-163 (counters).
"""
from __future__ import annotations

import threading
from collections import Counter
from typing import Dict

FAILPOINT_NAMES = ("device_allocation", "arena_acquire", "kv_preserve_copy", "expert_upload",
                   "compressor_transition", "indexer_transition", "resource_install", "graph_capture",
                   "checkpoint_read")


class FailpointTriggered(RuntimeError):
    def __init__(self, name: str):
        super().__init__(f"failpoint '{name}' triggered")
        self.name = name
        self.retryable = False


class Failpoints:
    def __init__(self):
        self._armed: Dict[str, int] = {}
        self._lock = threading.Lock()
        self.triggered = Counter()

    def arm(self, name: str, times: int = 1) -> None:
        if name not in FAILPOINT_NAMES:
            raise KeyError(f"unknown failpoint {name}")
        with self._lock:
            self._armed[name] = self._armed.get(name, 0) + times

    def disarm_all(self) -> None:
        with self._lock:
            self._armed.clear()

    def check(self, name: str) -> None:
        with self._lock:
            n = self._armed.get(name, 0)
            if n <= 0:
                return
            if n == 1:
                del self._armed[name]
            else:
                self._armed[name] = n - 1
            self.triggered[name] += 1
        raise FailpointTriggered(name)


class OpCounters:
    def __init__(self):
        self._c = Counter()
        self._lock = threading.Lock()

    def add(self, name: str, n: int = 1) -> None:
        with self._lock:
            self._c[name] += n

    def snapshot(self) -> Dict[str, int]:
        with self._lock:
            return dict(self._c)

    def reset(self) -> None:
        with self._lock:
            self._c.clear()


FAILPOINTS = Failpoints()
COUNTERS = OpCounters()
