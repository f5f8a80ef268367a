"""Materialization providers: the physical side the LoadRegistry drives.

A provider owns storage reads, pinned staging, host->device uploads and slot installs.  The
registry calls `reserve` / `submit_read` / `submit_upload` / `poll_install` / `cancel`, and collects
`CompletionEvent`s from `next_completion`.  `FakeMaterializationProvider` is the scriptable
stand-in used to test every ordering, loss and failure on the CPU.

Counterpart of crates/ferrule-runtime/src/io/provider.rs:125-195 (trait), :197-330 (shared
provider), :504-760 (unavailable + fake provider with script_next / lose_next / reject_next /
fail_next_reserve / push_completion).
"""
from __future__ import annotations

from collections import deque
from dataclasses import replace
from typing import Deque, Dict, List, Optional

from .io_protocol import (CompletionEvent, CompletionOutcome, FailureReason, LoadStage, MaterializationKey,
                          MaterializationResourcePlan)


class ProviderError(RuntimeError):
    pass


class MaterializationProvider:
    def plan(self, key: MaterializationKey) -> MaterializationResourcePlan:
        raise NotImplementedError

    def reserve(self, op: int, key: MaterializationKey) -> None:
        """Claim a destination slot / staging for the operation; raise ProviderError if impossible."""
        raise NotImplementedError

    def submit_read(self, op: int, key: MaterializationKey, generation: int) -> None:
        raise NotImplementedError

    def submit_upload(self, op: int, key: MaterializationKey, generation: int) -> None:
        raise NotImplementedError

    def poll_install(self, op: int, key: MaterializationKey, generation: int) -> None:
        raise NotImplementedError

    def cancel(self, op: int) -> None:
        raise NotImplementedError

    def retire(self, op: int, key: MaterializationKey) -> None:
        """The registry dropped the operation: free its slot / staging."""

    def next_completion(self) -> Optional[CompletionEvent]:
        raise NotImplementedError


class UnavailableMaterializationProvider(MaterializationProvider):
    """Placeholder for builds without streaming: every request fails at reserve."""

    def plan(self, key):
        return MaterializationResourcePlan()

    def reserve(self, op, key):
        raise ProviderError("materialization is not available in this configuration")

    def next_completion(self):
        return None

    def cancel(self, op):
        pass


class FakeMaterializationProvider(MaterializationProvider):
    """auto=True completes every submitted stage on the next `next_completion`; auto=False keeps
    submissions in `pending` until the test calls `complete(op)`."""

    def __init__(self, auto: bool = True, payload_bytes: int = 4096):
        self.auto = auto
        self.payload_bytes = payload_bytes
        self.pending: Dict[int, CompletionEvent] = {}
        self._ready: Deque[CompletionEvent] = deque()
        self.calls: List[tuple] = []
        self.reserved: Dict[int, MaterializationKey] = {}
        self.cancelled: List[int] = []
        self.retired: List[int] = []
        self._script: Deque[str] = deque()          # outcomes for the next submissions
        self._fail_reserve = 0
        self.clock_ns = 0

    # ---- scripting ----
    def script_next(self, *outcomes: str) -> None:
        """'ok' | 'fail' | 'short' | 'lose' (never completes) | 'reject' (completion for a wrong key) |
        'dup' (completes twice) | 'stale' (old generation)."""
        self._script.extend(outcomes)

    def lose_next(self) -> None:
        self.script_next("lose")

    def reject_next(self) -> None:
        self.script_next("reject")

    def fail_next_reserve(self, n: int = 1) -> None:
        self._fail_reserve += n

    def push_completion(self, ev: CompletionEvent) -> None:
        self._ready.append(ev)

    def complete(self, op: int) -> None:
        self._ready.append(self.pending.pop(op))

    # ---- provider API ----
    def plan(self, key):
        return MaterializationResourcePlan.for_payload(self.payload_bytes)

    def reserve(self, op, key):
        self.calls.append(("reserve", op))
        if self._fail_reserve > 0:
            self._fail_reserve -= 1
            raise ProviderError("scripted reserve failure")
        self.reserved[op] = key

    def _submit(self, what: str, stage: LoadStage, op: int, key: MaterializationKey, generation: int) -> None:
        self.calls.append((what, op))
        self.clock_ns += 1000
        mode = self._script.popleft() if self._script else "ok"
        ev = CompletionEvent(op, key, stage, generation, CompletionOutcome.OK, self.payload_bytes, None, self.clock_ns)
        if mode == "lose":
            return
        if mode == "fail":
            ev = replace(ev, outcome=CompletionOutcome.FAILED, bytes_done=0, failure=FailureReason.READ_ERROR)
        elif mode == "short":
            ev = replace(ev, bytes_done=self.payload_bytes // 2)
        elif mode == "reject":
            ev = replace(ev, key=replace(key, destination_generation=key.destination_generation + 99))
        elif mode == "stale":
            ev = replace(ev, generation=generation - 1)
        if self.auto:
            self._ready.append(ev)
            if mode == "dup":
                self._ready.append(ev)
        else:
            self.pending[op] = ev

    def submit_read(self, op, key, generation):
        self._submit("read", LoadStage.READ_SUBMITTED, op, key, generation)

    def submit_upload(self, op, key, generation):
        self._submit("upload", LoadStage.UPLOAD_SUBMITTED, op, key, generation)

    def poll_install(self, op, key, generation):
        self._submit("install", LoadStage.INSTALLING, op, key, generation)

    def cancel(self, op):
        self.calls.append(("cancel", op))
        self.cancelled.append(op)
        ev = self.pending.pop(op, None)
        if ev is not None:
            self._ready.append(replace(ev, outcome=CompletionOutcome.CANCELLED, bytes_done=0,
                                       failure=FailureReason.CANCELLED))

    def retire(self, op, key):
        self.retired.append(op)
        self.reserved.pop(op, None)

    def next_completion(self):
        return self._ready.popleft() if self._ready else None
