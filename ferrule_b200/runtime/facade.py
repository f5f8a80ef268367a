"""Engine facade, owner-thread guard and the validated executor adapter.

* `InferenceEngine` - the surface a front end programs against: submit / cancel / step / has_work / stats.
  `runtime.engine.Engine` implements it.
* `NativeExecutor` - thin adapter over a `ModelRunner` that validates every batch against the runner's
  capabilities before it reaches the backend and every output against the batch after it comes back
  (strictly increasing rows, sorted finite candidates), so a misbehaving backend fails the transaction
  instead of corrupting scheduler state.
* `InferenceCompletionOwner` - runs an engine on the thread that constructed it and refuses calls from
  any other thread (device state, graphs and pinned staging are not thread-safe); its loop is the
  race-free `listen -> step -> wait` pattern over a `CompletionHub`: a notification that arrives between
  the step and the wait is not lost because the ticket was taken before the step.

Counterpart of crates/ferrule-runtime/src/engine/inference.rs:374-411 (trait), :19-215 (completion owner,
affinity guard) and crates/ferrule-runtime/src/engine/native_executor.rs:24-245.
"""
from __future__ import annotations

import threading
from typing import Callable, Dict, List, Optional, Sequence

from ..utils.async_wake import CompletionHub
from .execution import ExecutionBatch, ExecutionCapabilities, KvLayoutSchema
from .runner import Complete, EndIntent, EndStatus, ModelRunner, Proposal, Waiting


class InferenceEngine:
    """Interface of an inference engine (structural: `Engine` provides these methods)."""

    def submit(self, request) -> None:
        raise NotImplementedError

    def cancel_request(self, request_id: str) -> bool:
        raise NotImplementedError

    def step(self, emit: Callable) -> bool:
        raise NotImplementedError

    def has_work(self) -> bool:
        raise NotImplementedError

    def snapshot_stats(self) -> Dict[str, object]:
        raise NotImplementedError


class AffinityError(RuntimeError):
    pass


class NativeExecutor(ModelRunner):
    """Validating pass-through: everything else is delegated to the wrapped runner."""

    def __init__(self, inner: ModelRunner):
        self.inner = inner
        self._batches: Dict[int, ExecutionBatch] = {}
        self.validated_batches = 0
        self.validated_outputs = 0

    def __getattr__(self, name):          # vocab_size, eos_token_id, stats, ...
        return getattr(self.inner, name)

    def capabilities(self) -> ExecutionCapabilities:
        return self.inner.capabilities()

    def kv_schema(self) -> KvLayoutSchema:
        return self.inner.kv_schema()

    def prepare_batch(self, txn_id: int, batch: ExecutionBatch) -> None:
        batch.validate(self.inner.capabilities())
        self.validated_batches += 1
        self._batches[txn_id] = batch
        self.inner.prepare_batch(txn_id, batch)

    def _check(self, txn_id: int, progress):
        if isinstance(progress, Complete):
            progress.output.validate(self._batches[txn_id])
            self.validated_outputs += 1
        elif not isinstance(progress, Waiting):
            raise TypeError(f"runner returned {type(progress).__name__}, expected Complete or Waiting")
        return progress

    def execute(self, txn_id: int):
        return self._check(txn_id, self.inner.execute(txn_id))

    def resume(self, txn_id: int):
        return self._check(txn_id, self.inner.resume(txn_id))

    def end_transaction(self, txn_id: int, intent: EndIntent) -> EndStatus:
        st = self.inner.end_transaction(txn_id, intent)
        if st == EndStatus.COMPLETE:
            self._batches.pop(txn_id, None)
        return st

    def retain_provisional_prefixes(self, txn_id: int, rows_by_slot: Dict[int, int]) -> None:
        b = self._batches.get(txn_id)
        if b is not None:
            by_slot = {s.state_slot: s.query_len for s in b.sequences}
            for slot, rows in rows_by_slot.items():
                if slot not in by_slot or not 0 <= rows <= by_slot[slot]:
                    raise ValueError(f"retained prefix of slot {slot} is outside the verified rows")
        self.inner.retain_provisional_prefixes(txn_id, rows_by_slot)

    def release_pages(self, pages: Sequence[int]) -> None:
        self.inner.release_pages(pages)

    def snapshot_pages(self, pages: Sequence[int]):
        return self.inner.snapshot_pages(pages)

    def restore_pages(self, pages: Sequence[int], snapshot) -> None:
        self.inner.restore_pages(pages, snapshot)

    def release_slot(self, state_slot: int) -> None:
        self.inner.release_slot(state_slot)

    def proposals_enabled(self) -> bool:
        return self.inner.proposals_enabled()

    def propose(self, slots, anchors, positions, views, max_draft) -> List[Proposal]:
        out = self.inner.propose(slots, anchors, positions, views, max_draft)
        if len(out) != len(slots) or any(len(p.tokens) > max_draft or len(p.tokens) != len(p.confidence) for p in out):
            raise ValueError("runner returned malformed proposals")
        return out

    def observability(self) -> Dict[str, object]:
        d = dict(self.inner.observability())
        d["validated_batches"], d["validated_outputs"] = self.validated_batches, self.validated_outputs
        return d

    def shutdown(self) -> None:
        self.inner.shutdown()


class InferenceCompletionOwner:
    """Owns an engine on one thread; producers on other threads only touch `hub.notify()`."""

    def __init__(self, engine, hub: Optional[CompletionHub] = None):
        self.engine = engine
        self.hub = hub or CompletionHub()
        self._owner = threading.get_ident()
        self.steps = 0
        self.idle_waits = 0

    def _guard(self) -> None:
        if threading.get_ident() != self._owner:
            raise AffinityError("the engine may only be driven from the thread that owns it")

    def submit(self, request) -> None:
        self._guard()
        self.engine.submit(request)
        self.hub.notify()

    def cancel(self, request_id: str) -> bool:
        self._guard()
        return self.engine.cancel_request(request_id)

    def run_once(self, emit: Callable, idle_timeout: float = 0.05) -> bool:
        """listen -> step -> (if nothing progressed) wait.  Returns whether the engine made progress."""
        self._guard()
        ticket = self.hub.listen()
        progressed = self.engine.step(emit)
        self.steps += 1
        if not progressed and not self.engine.has_work():
            self.idle_waits += 1
            self.hub.wait(ticket, idle_timeout)
        return progressed

    def run_until_idle(self, emit: Callable, max_steps: int = 100000) -> int:
        self._guard()
        n = 0
        while self.engine.has_work() and n < max_steps:
            self.run_once(emit, idle_timeout=0.0)
            n += 1
        return n
