"""LoadRegistry: the single owner of every materialization in flight.

* exact-key single flight: a second request for the same `MaterializationKey` attaches to the
  operation already in flight (or is satisfied at once if it is resident);
* owners: executions (REQUIRED) and prefetch owners (model warm-up, a transaction's declared
  prefetch, external hints); an execution request promotes an active prefetch without a second
  transfer;
* a fair queue of next actions (reserve / submit read / submit upload / poll install), each gated
  by hard credits from the resource broker; submitted credits are held until the completion;
* every completion is validated against the recorded expectation; anything that does not match
  (wrong operation, key, stage, generation, byte count, duplicate) is rejected and kept as evidence;
* continuations (suspended transactions) wait on sets of keys and become ready when all are
  resident, or failed when one cannot be provided;
* custody: resident payloads stay leased while a stage / transaction / persistent owner holds them;
  only unleased ones may be retired; shutdown drains everything that was submitted.

Counterpart of crates/ferrule-runtime/src/io/registry.rs:489-526 (state), :918-1095 (requests and
owners), :1097-1445 (waiters), :1446-1730 (scheduling and completions), :1753-1990 (resume leases),
:2013-2100 (shutdown), :2560-2925 (apply/publish), waiters.rs:41-110, resolver.rs:32-140.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Deque, Dict, Iterable, List, Optional, Set, Tuple

from .fairness import Band, FairQueue, FairQueueConfig
from .io_protocol import (IoProtocolError, CompletionEvent, CompletionExpectation, CompletionOutcome, DependencySet, FailureReason,
                          LoadStage, MaterializationKey, Purpose, RetirementReason, RetirementToken,
                          validate_transition)
from .ledger import CriticalPathLedger, LedgerPhase
from .provider import MaterializationProvider, ProviderError
from .resources import Grant, PhysicalResourceBroker
from .resources import ResourceKind as RK


class OwnerKind(Enum):
    EXECUTION = "execution"
    MODEL_WARMUP = "model_warmup"
    TRANSACTION_PREFETCH = "transaction_prefetch"
    EXTERNAL = "external"


class Retention(Enum):
    STAGE = "stage"
    TRANSACTION = "transaction"
    PERSISTENT = "persistent"


@dataclass
class Operation:
    op_id: int
    key: MaterializationKey
    stage: LoadStage = LoadStage.RESERVED
    purpose: Purpose = Purpose.PREFETCH
    generation: int = 0
    owners: Set[Tuple[OwnerKind, int]] = field(default_factory=set)
    waiters: Set[int] = field(default_factory=set)            # continuation (transaction) ids
    expectation: Optional[CompletionExpectation] = None
    grants: List[Grant] = field(default_factory=list)
    resident_grant: Optional[Grant] = None
    leases: int = 0
    reserved_at_provider: bool = False
    failure: Optional[FailureReason] = None
    cancel_requested: bool = False
    t_stage_ns: int = 0
    last_use: int = 0


@dataclass
class Continuation:
    txn_id: int
    needs: Set[int]                       # op ids still outstanding
    all_ops: List[int]
    failed: bool = False
    failure: Optional[FailureReason] = None      # why the first of its payloads failed
    t_wait_start_ns: int = 0
    current: Set[int] = field(default_factory=set)      # operations named by the latest registration (this wait)
    resumed: bool = False                        # handed to the engine by pop_ready since that registration


@dataclass
class RegistryStats:
    requests: int = 0
    coalesced: int = 0
    satisfied_resident: int = 0
    promoted: int = 0
    submitted_reads: int = 0
    submitted_uploads: int = 0
    submitted_installs: int = 0
    published: int = 0
    failed: int = 0
    rejected_completions: int = 0
    credit_denials: int = 0
    retired: int = 0
    cancelled: int = 0
    continuations: int = 0
    resumed: int = 0


@dataclass
class Rejection:
    event: CompletionEvent
    reason: str


_NEXT_ACTION = {LoadStage.RESERVED: "read", LoadStage.HOST_READY: "upload", LoadStage.UPLOAD_SUBMITTED: None}


class LoadRegistry:
    def __init__(self, provider: MaterializationProvider, broker: Optional[PhysicalResourceBroker] = None,
                 fair: Optional[FairQueueConfig] = None, ledger: Optional[CriticalPathLedger] = None,
                 clock=time.perf_counter_ns):
        self.provider = provider
        self.broker = broker or PhysicalResourceBroker()
        self.queue: FairQueue[int] = FairQueue(fair)
        self.ledger = ledger or CriticalPathLedger()
        self.clock = clock
        self.ops: Dict[int, Operation] = {}
        self.by_key: Dict[MaterializationKey, int] = {}
        self.conts: Dict[int, Continuation] = {}
        self._ready: Deque[int] = deque()
        self._failed: Deque[int] = deque()
        self.rejections: List[Rejection] = []
        self.stats = RegistryStats()
        self._next_op = 0
        self._use = 0
        self._shutdown = False
        self._queued: Set[int] = set()

    # ------------------------------------------------------------------ requests
    def _band(self, op: Operation) -> Band:
        if op.purpose == Purpose.EXECUTION:
            return Band.REQUIRED
        if any(k == OwnerKind.MODEL_WARMUP for k, _ in op.owners):
            return Band.BACKGROUND
        return Band.PREFETCH

    def request(self, key: MaterializationKey, owner: Tuple[OwnerKind, int], purpose: Purpose = Purpose.PREFETCH) -> int:
        if self._shutdown:
            raise RuntimeError("registry is shut down")
        self.stats.requests += 1
        op_id = self.by_key.get(key)
        if op_id is not None:
            op = self.ops[op_id]
            if op.stage in (LoadStage.FAILED, LoadStage.STALE, LoadStage.DRAINING, LoadStage.RETIRED):
                op_id = None                 # dead operation: start a fresh one below
            else:
                op.owners.add(owner)
                if op.stage == LoadStage.RESIDENT:
                    self.stats.satisfied_resident += 1
                else:
                    self.stats.coalesced += 1
                if purpose == Purpose.EXECUTION and op.purpose != Purpose.EXECUTION:
                    op.purpose = Purpose.EXECUTION
                    self.stats.promoted += 1
                    self.queue.promote(op.op_id, Band.REQUIRED)
                self._touch(op)
                return op.op_id
        op = Operation(self._next_op, key, purpose=purpose, owners={owner}, t_stage_ns=self.clock())
        self._next_op += 1
        self.ops[op.op_id] = op
        self.by_key[key] = op.op_id
        self._enqueue(op)
        self._touch(op)
        return op.op_id

    def prefetch(self, keys: Iterable[MaterializationKey], owner: Tuple[OwnerKind, int]) -> List[int]:
        return [self.request(k, owner, Purpose.PREFETCH) for k in keys]

    def _touch(self, op: Operation) -> None:
        self._use += 1
        op.last_use = self._use

    def _enqueue(self, op: Operation) -> None:
        if op.op_id not in self._queued:
            self._queued.add(op.op_id)
            self.queue.push(self._band(op), op.op_id)

    # ------------------------------------------------------------------ continuations
    def register_continuation(self, txn_id: int, deps) -> None:
        keys = deps.keys if isinstance(deps, DependencySet) else list(deps)
        # checked before anything is touched: a rejected registration leaves no owner, lease or operation behind
        prev = self.conts.get(txn_id)
        if prev is not None and (prev.needs or prev.failed):
            raise IoProtocolError(f"continuation {txn_id} is already registered and unresolved")
        if len(set(keys)) != len(keys):
            raise IoProtocolError(f"continuation {txn_id} names a dependency twice")
        if self._shutdown:
            raise RuntimeError("registry is shut down")
        # a transaction that was resumed and has to wait again extends its continuation: it keeps the custody of
        # what it already holds and takes a lease on the new payloads only
        held = set(prev.all_ops) if prev is not None else set()
        needs, all_ops = set(), list(prev.all_ops) if prev is not None else []
        for k in keys:
            op_id = self.request(k, (OwnerKind.EXECUTION, txn_id), Purpose.EXECUTION)
            op = self.ops[op_id]
            if op_id not in held:
                all_ops.append(op_id)
                held.add(op_id)
                op.leases += 1                   # transaction custody from the start
            if op.stage != LoadStage.RESIDENT:
                needs.add(op_id)
                op.waiters.add(txn_id)
        c = Continuation(txn_id, needs, all_ops, t_wait_start_ns=self.clock(),
                         current={self.by_key[k] for k in keys if k in self.by_key})
        self.conts[txn_id] = c
        self.stats.continuations += 1
        if not needs:
            self._ready.append(txn_id)

    def cancel_continuation(self, txn_id: int) -> None:
        c = self.conts.pop(txn_id, None)
        if c is None:
            return
        for op_id in c.all_ops:
            op = self.ops.get(op_id)
            if op is None:
                continue
            op.waiters.discard(txn_id)
            op.leases = max(op.leases - 1, 0)
            op.owners.discard((OwnerKind.EXECUTION, txn_id))
        for q in (self._ready, self._failed):
            if txn_id in q:
                q.remove(txn_id)

    def pop_ready(self) -> List[int]:
        out = list(self._ready)
        self._ready.clear()
        now = self.clock()
        for t in out:
            c = self.conts.get(t)
            if c is not None:
                c.resumed = True
                self.ledger.record_wait(t, c.t_wait_start_ns, now)
        self.stats.resumed += len(out)
        return out

    def pop_failed(self) -> List[int]:
        out = list(self._failed)
        self._failed.clear()
        return out

    def awaited_ops(self) -> Set[int]:
        """Operations that a parked transaction named in its current wait and has not been resumed for yet.  Their
        payloads are about to be used: a provider must not evict them to make room for another load (between the
        install and the resume nobody holds a lease on them)."""
        out: Set[int] = set()
        for c in self.conts.values():
            if not c.resumed and not c.failed:
                out |= c.current
        return out

    def failure_of(self, txn_id: int) -> Optional[FailureReason]:
        """Why the continuation of `txn_id` failed (None: it did not, or it is gone already)."""
        c = self.conts.get(txn_id)
        return c.failure if c is not None else None

    def release_transaction(self, txn_id: int) -> None:
        """The transaction ended: drop its custody of every payload it used."""
        self.cancel_continuation(txn_id)

    # ------------------------------------------------------------------ owner loop
    def drive(self, max_actions: int = 64) -> int:
        n = self._collect_completions()
        n += self._schedule(max_actions)
        return n

    def _collect_completions(self) -> int:
        n = 0
        while True:
            ev = self.provider.next_completion()
            if ev is None:
                return n
            n += 1
            self._process_completion(ev)

    def _reject(self, ev: CompletionEvent, why: str) -> None:
        self.stats.rejected_completions += 1
        self.rejections.append(Rejection(ev, why))
        if len(self.rejections) > 1024:
            del self.rejections[:512]

    def _process_completion(self, ev: CompletionEvent) -> None:
        op = self.ops.get(ev.operation)
        if op is None:
            return self._reject(ev, "unknown operation")
        if op.expectation is None:
            return self._reject(ev, "no completion is owed (duplicate or unsolicited)")
        why = op.expectation.check(ev)
        if why is None:
            self._apply_completion(op, ev)
        elif why.startswith("byte count"):
            # a short transfer answers the right submission: it is a failure, not a stray event
            self._fail(op, FailureReason.SHORT_READ)
        else:
            self._reject(ev, why)

    def _release_grants(self, op: Operation) -> None:
        for g in op.grants:
            self.broker.complete(g)
        op.grants.clear()

    def _apply_completion(self, op: Operation, ev: CompletionEvent) -> None:
        now = self.clock()
        phase = {LoadStage.READ_SUBMITTED: LedgerPhase.READ, LoadStage.UPLOAD_SUBMITTED: LedgerPhase.UPLOAD,
                 LoadStage.INSTALLING: LedgerPhase.PUBLISH}[op.stage]
        self.ledger.record_operation(op.op_id, phase, op.t_stage_ns, now)
        op.expectation = None
        self._release_grants(op)
        if ev.outcome == CompletionOutcome.CANCELLED or op.cancel_requested:
            self._set_stage(op, LoadStage.DRAINING)
            self._retire(op, RetirementReason.CANCELLED)
            self.stats.cancelled += 1
            return
        if ev.outcome == CompletionOutcome.FAILED:
            self._fail(op, ev.failure or FailureReason.PROVIDER_LOST)
            return
        if op.stage == LoadStage.READ_SUBMITTED:
            self._set_stage(op, LoadStage.HOST_READY)
            self._enqueue(op)
        elif op.stage == LoadStage.UPLOAD_SUBMITTED:
            self._set_stage(op, LoadStage.INSTALLING)
            self._submit_install(op)
        elif op.stage == LoadStage.INSTALLING:
            self._set_stage(op, LoadStage.RESIDENT)
            self._publish(op)

    def _set_stage(self, op: Operation, nxt: LoadStage) -> None:
        validate_transition(op.stage, nxt)
        op.stage = nxt
        op.t_stage_ns = self.clock()

    def _fail(self, op: Operation, reason: FailureReason) -> None:
        self.stats.failed += 1
        op.failure = reason
        op.expectation = None
        self._release_grants(op)
        if op.stage != LoadStage.RESERVED:          # a reservation that never started goes straight to retired
            self._set_stage(op, LoadStage.FAILED)
        for txn in list(op.waiters):
            c = self.conts.get(txn)
            if c is not None and not c.failed:
                c.failed, c.failure = True, reason
                self._failed.append(txn)
        op.waiters.clear()
        self._retire(op, RetirementReason.FAILED)

    def _publish(self, op: Operation) -> None:
        self.stats.published += 1
        plan = self.provider.plan(op.key)
        op.resident_grant = self.broker.try_claim({RK.RESIDENT_BYTES: plan.resident_bytes}, required=True)
        for txn in list(op.waiters):
            c = self.conts.get(txn)
            if c is None:
                continue
            c.needs.discard(op.op_id)
            if not c.needs and not c.failed:
                self._ready.append(txn)
        op.waiters.clear()

    # ------------------------------------------------------------------ scheduling
    def _claim(self, op: Operation, amounts) -> Optional[Grant]:
        g = self.broker.try_claim(amounts, required=op.purpose == Purpose.EXECUTION)
        if g is None:
            self.stats.credit_denials += 1
        return g

    def _schedule(self, max_actions: int) -> int:
        n = 0
        deferred: List[int] = []
        while n < max_actions:
            item = self.queue.pop()
            if item is None:
                break
            _, op_id = item
            self._queued.discard(op_id)
            op = self.ops.get(op_id)
            if op is None or op.cancel_requested:
                continue
            plan = self.provider.plan(op.key)
            if op.stage == LoadStage.RESERVED:
                if not op.reserved_at_provider:
                    try:
                        self.provider.reserve(op.op_id, op.key)
                        op.reserved_at_provider = True
                    except ProviderError:
                        self._fail(op, FailureReason.RESOURCE_EXHAUSTED)
                        n += 1
                        continue
                g = self._claim(op, {RK.READ_SLOTS: plan.read_slots, RK.STORAGE_BYTES: plan.storage_bytes,
                                     RK.PINNED_BYTES: plan.pinned_bytes, RK.LOAD_OPS: 1})
                if g is None:
                    deferred.append(op_id)
                    continue
                op.grants.append(g)
                op.generation += 1
                op.expectation = CompletionExpectation(op.op_id, op.key, LoadStage.READ_SUBMITTED, op.generation,
                                                       self._payload_bytes(op))
                self._set_stage(op, LoadStage.READ_SUBMITTED)
                self.broker.mark_submitted(g)
                self.provider.submit_read(op.op_id, op.key, op.generation)
                self.stats.submitted_reads += 1
                n += 1
            elif op.stage == LoadStage.HOST_READY:
                g = self._claim(op, {RK.UPLOAD_SLOTS: plan.upload_slots, RK.UPLOAD_BYTES: plan.h2d_bytes,
                                     RK.PINNED_BYTES: plan.pinned_bytes})
                if g is None:
                    deferred.append(op_id)
                    continue
                op.grants.append(g)
                op.generation += 1
                op.expectation = CompletionExpectation(op.op_id, op.key, LoadStage.UPLOAD_SUBMITTED, op.generation,
                                                       self._payload_bytes(op))
                self._set_stage(op, LoadStage.UPLOAD_SUBMITTED)
                self.broker.mark_submitted(g)
                self.provider.submit_upload(op.op_id, op.key, op.generation)
                self.stats.submitted_uploads += 1
                n += 1
        for op_id in deferred:                      # out of credits: try again on a later drive
            self._enqueue(self.ops[op_id])
        return n

    def _payload_bytes(self, op: Operation) -> int:
        return self.provider.plan(op.key).h2d_bytes

    def _submit_install(self, op: Operation) -> None:
        plan = self.provider.plan(op.key)
        g = self._claim(op, {RK.INSTALL_SLOTS: plan.install_slots, RK.INSTALL_BYTES: plan.device_install_bytes})
        if g is not None:
            op.grants.append(g)
            self.broker.mark_submitted(g)
        op.generation += 1
        op.expectation = CompletionExpectation(op.op_id, op.key, LoadStage.INSTALLING, op.generation,
                                               self._payload_bytes(op))
        self.provider.poll_install(op.op_id, op.key, op.generation)
        self.stats.submitted_installs += 1

    # ------------------------------------------------------------------ cancel / retire / evict
    def detach(self, op_id: int, owner: Tuple[OwnerKind, int]) -> bool:
        """`owner` no longer wants the payload.  The operation goes on while anyone else owns it, waits for it or
        leases it; the last owner's detach cancels it (at once if nothing was submitted, after the completion of
        submitted work otherwise).  -> True when this detach cancelled the operation.  Detaching twice, or an owner
        that never attached, is a protocol error."""
        op = self.ops.get(op_id)
        if op is None:
            raise IoProtocolError(f"unknown operation {op_id}")
        if owner not in op.owners:
            raise IoProtocolError(f"operation {op_id}: {owner} is not an owner (duplicate detach?)")
        op.owners.discard(owner)
        if op.owners or op.waiters or op.leases or op.stage in (LoadStage.RESIDENT, LoadStage.RETIRED):
            return False
        self.cancel(op_id)
        return True

    def cancel(self, op_id: int) -> None:
        op = self.ops.get(op_id)
        if op is None or op.stage in (LoadStage.RETIRED,):
            return
        if op.waiters or op.leases:
            raise RuntimeError("operation still has waiters or leases")
        if op.stage == LoadStage.RESERVED:
            self.queue.remove(op_id)
            self._queued.discard(op_id)
            self._retire(op, RetirementReason.CANCELLED)
            self.stats.cancelled += 1
        elif op.expectation is not None:
            op.cancel_requested = True           # submitted work cannot be revoked: wait for its completion
            self.provider.cancel(op_id)
        elif op.stage == LoadStage.HOST_READY:
            self.queue.remove(op_id)
            self._queued.discard(op_id)
            self._set_stage(op, LoadStage.STALE)
            self._retire(op, RetirementReason.CANCELLED)
            self.stats.cancelled += 1
        elif op.stage == LoadStage.RESIDENT:
            self._retire(op, RetirementReason.EVICTED)

    def _retire(self, op: Operation, reason: RetirementReason) -> RetirementToken:
        if op.stage != LoadStage.RETIRED:
            if op.stage in (LoadStage.RESERVED, LoadStage.RESIDENT, LoadStage.FAILED, LoadStage.STALE,
                            LoadStage.DRAINING):
                self._set_stage(op, LoadStage.RETIRED)
        token = RetirementToken(op.op_id, reason)
        token.consume()
        self._release_grants(op)
        if op.resident_grant is not None:
            self.broker.complete(op.resident_grant)
            op.resident_grant = None
        if op.reserved_at_provider:
            self.provider.retire(op.op_id, op.key)
            op.reserved_at_provider = False
        if self.by_key.get(op.key) == op.op_id:
            del self.by_key[op.key]
        self.stats.retired += 1
        return token

    def evict_candidates(self) -> List[int]:
        """Resident operations nobody leases, least recently used first."""
        c = [o for o in self.ops.values() if o.stage == LoadStage.RESIDENT and o.leases == 0]
        return [o.op_id for o in sorted(c, key=lambda o: o.last_use)]

    def evict(self, n: int = 1) -> int:
        done = 0
        for op_id in self.evict_candidates()[:n]:
            self._retire(self.ops[op_id], RetirementReason.EVICTED)
            done += 1
        return done

    def is_resident(self, key: MaterializationKey) -> bool:
        op_id = self.by_key.get(key)
        return op_id is not None and self.ops[op_id].stage == LoadStage.RESIDENT

    # ------------------------------------------------------------------ shutdown
    def shutdown(self) -> bool:
        """Stop taking requests, cancel what was not submitted, keep collecting completions of what
        was.  Returns True when nothing is in flight and no credit is outstanding."""
        self._shutdown = True
        for op in list(self.ops.values()):
            if op.stage in (LoadStage.RESERVED, LoadStage.HOST_READY) and op.expectation is None:
                op.waiters.clear()
                op.leases = 0
                self.cancel(op.op_id)
            elif op.expectation is not None and not op.cancel_requested:
                op.waiters.clear()
                op.leases = 0
                op.cancel_requested = True
                self.provider.cancel(op.op_id)
        self._collect_completions()
        busy = any(op.expectation is not None for op in self.ops.values())
        if not busy:
            for op in list(self.ops.values()):
                if op.stage == LoadStage.RESIDENT:
                    op.leases = 0
                    self._retire(op, RetirementReason.SHUTDOWN)
        return not busy

    def residual(self) -> Dict[str, int]:
        """What is still held; all zeros after a clean shutdown."""
        return {"in_flight": sum(1 for o in self.ops.values() if o.expectation is not None),
                "resident": sum(1 for o in self.ops.values() if o.stage == LoadStage.RESIDENT),
                "grants": self.broker.outstanding(), "continuations": len(self.conts)}
