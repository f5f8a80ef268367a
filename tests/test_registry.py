"""LoadRegistry state machine against the scriptable fake provider (CPU)."""
import pytest

from ferrule_b200.runtime.fairness import Band, FairQueue, FairQueueConfig
from ferrule_b200.runtime.io_protocol import (CompletionEvent, CompletionOutcome, IoProtocolError, LoadStage,
                                              MaterializationKey, ResourceId, ResourceKind, RetirementReason,
                                              RetirementToken, can_transition, validate_transition)
from ferrule_b200.runtime.ledger import CriticalPathLedger, LedgerPhase, union_length
from ferrule_b200.runtime.provider import FakeMaterializationProvider
from ferrule_b200.runtime.registry import LoadRegistry, OwnerKind
from ferrule_b200.runtime.resources import PhysicalResourceBroker
from ferrule_b200.runtime.resources import ResourceKind as RK


def key(e, layer=1, gen=0):
    return MaterializationKey("m", b"src", bytes([e]), ResourceId(ResourceKind.ROUTED_EXPERT, layer, e), 1,
                              "cuda-sm100a", 0, 0, gen)


def drive_all(reg, n=20):
    for _ in range(n):
        reg.drive()


def test_load_stage_table():
    assert can_transition(LoadStage.RESERVED, LoadStage.READ_SUBMITTED)
    assert can_transition(LoadStage.INSTALLING, LoadStage.RESIDENT)
    assert not can_transition(LoadStage.RESIDENT, LoadStage.READ_SUBMITTED)
    assert not can_transition(LoadStage.RETIRED, LoadStage.RESERVED)
    with pytest.raises(IoProtocolError):
        validate_transition(LoadStage.HOST_READY, LoadStage.RESIDENT)
    t = RetirementToken(1, RetirementReason.EVICTED)
    t.consume()
    with pytest.raises(IoProtocolError):
        t.consume()


def test_single_flight_and_key_exactness():
    p = FakeMaterializationProvider()
    reg = LoadRegistry(p)
    a = reg.request(key(3), (OwnerKind.EXTERNAL, 0))
    b = reg.request(key(3), (OwnerKind.EXTERNAL, 1))
    c = reg.request(key(3, gen=1), (OwnerKind.EXTERNAL, 2))        # destination generation differs
    assert a == b and c != a and reg.stats.coalesced == 1
    drive_all(reg)
    assert reg.is_resident(key(3)) and reg.is_resident(key(3, gen=1))
    assert [x for x in p.calls if x[0] == "read"] == [("read", a), ("read", c)]
    d = reg.request(key(3), (OwnerKind.EXTERNAL, 3))
    assert d == a and reg.stats.satisfied_resident == 1


def test_continuation_ready_after_all_dependencies_and_promotion():
    p = FakeMaterializationProvider(auto=False)
    reg = LoadRegistry(p)
    pre = reg.request(key(1), (OwnerKind.TRANSACTION_PREFETCH, 7))
    reg.register_continuation(7, [key(1), key(2)])
    assert reg.stats.promoted == 1 and reg.pop_ready() == []
    for _ in range(8):
        reg.drive()
        for op in list(p.pending):
            p.complete(op)
    assert reg.pop_ready() == [7]
    assert reg.ops[pre].leases == 1
    reg.release_transaction(7)
    assert reg.ops[pre].leases == 0 and set(reg.evict_candidates()) == {0, 1}


def test_wrong_stale_duplicate_and_lost_completions_are_rejected_or_survived():
    p = FakeMaterializationProvider()
    reg = LoadRegistry(p)
    p.script_next("reject")                    # completion names a different key
    a = reg.request(key(1), (OwnerKind.EXTERNAL, 0))
    reg.drive(); reg.drive()
    assert reg.stats.rejected_completions == 1 and reg.ops[a].stage == LoadStage.READ_SUBMITTED
    assert "key" in reg.rejections[0].reason
    # the right completion arrives later: the operation carries on
    exp = reg.ops[a].expectation
    p.push_completion(CompletionEvent(a, key(1), exp.stage, exp.generation, CompletionOutcome.OK, exp.bytes_expected))
    drive_all(reg)
    assert reg.is_resident(key(1))
    # duplicate of an already consumed completion
    p.push_completion(CompletionEvent(a, key(1), LoadStage.INSTALLING, reg.ops[a].generation, CompletionOutcome.OK, 4096))
    reg.drive()
    assert reg.stats.rejected_completions == 2
    # stale generation
    p.script_next("stale")
    b = reg.request(key(2), (OwnerKind.EXTERNAL, 0))
    reg.drive(); reg.drive()
    assert reg.stats.rejected_completions == 3 and reg.ops[b].stage == LoadStage.READ_SUBMITTED
    # unknown operation
    p.push_completion(CompletionEvent(999, key(9), LoadStage.READ_SUBMITTED, 1, CompletionOutcome.OK, 4096))
    reg.drive()
    assert reg.stats.rejected_completions == 4


def test_failure_and_short_read_fail_the_waiters():
    p = FakeMaterializationProvider()
    reg = LoadRegistry(p)
    p.script_next("ok", "short")               # read ok, upload comes back short
    reg.register_continuation(1, [key(1)])
    drive_all(reg)
    assert reg.pop_failed() == [1] and reg.pop_ready() == []
    assert reg.stats.failed == 1 and reg.broker.outstanding() == 0
    # a new request for the same key starts a fresh operation
    reg.release_transaction(1)
    reg.register_continuation(2, [key(1)])
    drive_all(reg)
    assert reg.pop_ready() == [2]
    p.fail_next_reserve()
    reg.register_continuation(3, [key(5)])
    drive_all(reg)
    assert reg.pop_failed() == [3]


def test_cancellation_at_every_stage():
    p = FakeMaterializationProvider(auto=False)
    reg = LoadRegistry(p)
    a = reg.request(key(1), (OwnerKind.EXTERNAL, 0))
    reg.cancel(a)                               # still reserved: retire at once
    assert reg.ops[a].stage == LoadStage.RETIRED
    b = reg.request(key(2), (OwnerKind.EXTERNAL, 0))
    reg.drive()                                 # read submitted
    reg.cancel(b)                               # submitted work cannot be revoked
    assert reg.ops[b].stage == LoadStage.READ_SUBMITTED and reg.broker.outstanding() == 1
    reg.drive()                                 # provider answers CANCELLED
    assert reg.ops[b].stage == LoadStage.RETIRED and reg.broker.outstanding() == 0
    c = reg.request(key(3), (OwnerKind.EXTERNAL, 0))
    reg.drive(); p.complete(c); reg.drive()     # host ready (upload submitted by the same drive)
    assert reg.ops[c].stage == LoadStage.UPLOAD_SUBMITTED
    reg.cancel(c); reg.drive()
    assert reg.ops[c].stage == LoadStage.RETIRED
    assert reg.stats.cancelled == 3 and set(p.retired) >= {b, c}


def test_credit_exhaustion_defers_and_required_may_use_the_reserve():
    broker = PhysicalResourceBroker()
    broker.set_limit(RK.READ_SLOTS, 2, execution_reserve=1)
    p = FakeMaterializationProvider(auto=False)
    reg = LoadRegistry(p, broker)
    ops = [reg.request(key(i), (OwnerKind.EXTERNAL, 0)) for i in range(3)]
    reg.drive()
    assert reg.stats.submitted_reads == 1 and reg.stats.credit_denials >= 1      # prefetch may not touch the reserve
    reg.register_continuation(9, [key(7)])
    reg.drive()
    assert reg.stats.submitted_reads == 2                                        # required work may
    for _ in range(12):
        for op in list(p.pending):
            p.complete(op)
        reg.drive()
    assert all(reg.ops[o].stage == LoadStage.RESIDENT for o in ops) and reg.pop_ready() == [9]
    assert broker.usage[RK.READ_SLOTS].high_water == 2


def test_shutdown_drains_submitted_work():
    p = FakeMaterializationProvider(auto=False)
    reg = LoadRegistry(p)
    reg.request(key(1), (OwnerKind.EXTERNAL, 0))
    reg.request(key(2), (OwnerKind.EXTERNAL, 0))
    reg.drive()
    assert not reg.shutdown() or reg.residual()["in_flight"] == 0
    for _ in range(5):
        if reg.shutdown():
            break
    assert reg.residual() == {"in_flight": 0, "resident": 0, "grants": 0, "continuations": 0}
    with pytest.raises(RuntimeError):
        reg.request(key(3), (OwnerKind.EXTERNAL, 0))


def test_fair_queue_bands_aging_and_promotion():
    q = FairQueue(FairQueueConfig(quantum=(4, 2, 1), aging_ticks=10, debt_bound=2))
    for i in range(20):
        q.push(Band.REQUIRED, ("r", i))
        q.push(Band.PREFETCH, ("p", i))
    q.push(Band.BACKGROUND, ("b", 0))
    order = [q.pop() for _ in range(41)]
    first12 = [b for b, _ in order[:14]]
    assert first12.count(Band.REQUIRED) > first12.count(Band.PREFETCH) > 0
    pos_bg = [i for i, (b, _) in enumerate(order) if b == Band.BACKGROUND][0]
    assert pos_bg <= 14 and q.aged[Band.BACKGROUND] + q.served[Band.BACKGROUND] >= 1     # never starved
    assert q.pop() is None
    q.push(Band.BACKGROUND, "x")
    assert q.promote("x", Band.REQUIRED) and q.pop() == (Band.REQUIRED, "x")


def test_ledger_union_and_cover():
    assert union_length([(0, 10), (5, 20), (30, 40)]) == 30
    led = CriticalPathLedger()
    led.record_operation(1, LedgerPhase.READ, 0, 100)
    led.record_operation(2, LedgerPhase.READ, 50, 150)
    assert led.shared_wait([1, 2]) == 150
    led.record_wait(7, 0, 150)
    led.record_runnable_work(20, 60)
    led.record_runnable_work(100, 400)
    s = led.snapshot_for_token(7, 0)
    assert (s.wait_ns, s.covered_ns, s.uncovered_ns) == (150, 90, 60)
    assert abs(led.summary()["covered_fraction"] - 0.6) < 1e-9
