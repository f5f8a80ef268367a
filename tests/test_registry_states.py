"""LoadRegistry: one test per named state-machine case (success path, single flight, ownership, cancellation at
every stage, failures, stale / wrong / duplicate / lost / out-of-order completions, credits, fairness, targeted
wake-ups, shutdown, retry).  Everything runs against the scriptable fake provider on the CPU.

The case list follows the reference's registry suite (crates/ferrule-runtime/src/io/tests.rs:310-2366)."""
import random

import pytest

from ferrule_b200.runtime.fairness import Band, FairQueue, FairQueueConfig
from ferrule_b200.runtime.io_protocol import (CompletionEvent, CompletionOutcome, FailureReason, IoProtocolError, LoadStage,
                                              MaterializationKey, Purpose, ResourceId, ResourceKind, can_transition,
                                              validate_transition)
from ferrule_b200.runtime.provider import FakeMaterializationProvider
from ferrule_b200.runtime.registry import LoadRegistry, OwnerKind
from ferrule_b200.runtime.resources import PhysicalResourceBroker
from ferrule_b200.runtime.resources import ResourceKind as RK


def key(e, layer=1, gen=0, src=b"src", kind=ResourceKind.ROUTED_EXPERT):
    return MaterializationKey("m", src, bytes([e]), ResourceId(kind, layer, e), 1, "cuda-sm100a", 0, 0, gen)


EXT = (OwnerKind.EXTERNAL, 0)


def manual():
    p = FakeMaterializationProvider(auto=False)
    return p, LoadRegistry(p)


def to_stage(p, reg, op, stage):
    """Drive a manual registry until `op` sits in `stage` (READ_SUBMITTED, UPLOAD_SUBMITTED or INSTALLING)."""
    order = [LoadStage.READ_SUBMITTED, LoadStage.UPLOAD_SUBMITTED, LoadStage.INSTALLING]
    for _ in range(order.index(stage) + 1):
        reg.drive()
        if reg.ops[op].stage == stage:
            return
        p.complete(op)
    reg.drive()
    assert reg.ops[op].stage == stage, reg.ops[op].stage


def finish(p, reg, n=12):
    for _ in range(n):
        for op in list(p.pending):
            p.complete(op)
        reg.drive()


# ------------------------------------------------------------------------------------------ success path
def test_initial_stage_is_reserved_without_claims_or_provider_reservation():
    p, reg = manual()
    a = reg.request(key(1), EXT)
    op = reg.ops[a]
    assert op.stage == LoadStage.RESERVED and op.expectation is None and not op.grants
    assert reg.broker.outstanding() == 0 and p.calls == [] and not op.reserved_at_provider


def test_every_stage_is_reached_once_and_in_order():
    p, reg = manual()
    a = reg.request(key(1), EXT)
    seen = [reg.ops[a].stage]
    for _ in range(8):
        reg.drive()
        if reg.ops[a].stage != seen[-1]:
            seen.append(reg.ops[a].stage)
        if a in p.pending:
            p.complete(a)
    # HOST_READY is left by the same drive that reaches it (the upload is submitted at once)
    assert seen == [LoadStage.RESERVED, LoadStage.READ_SUBMITTED, LoadStage.UPLOAD_SUBMITTED, LoadStage.INSTALLING,
                    LoadStage.RESIDENT]
    assert [c[0] for c in p.calls] == ["reserve", "read", "upload", "install"]
    assert reg.stats.published == 1 and reg.broker.outstanding() == 1          # the residency credit


def test_read_completion_reaches_host_ready_before_the_upload_is_scheduled():
    p, reg = manual()
    a = reg.request(key(1), EXT)
    reg.drive()
    p.complete(a)
    reg._collect_completions()
    assert reg.ops[a].stage == LoadStage.HOST_READY and reg.ops[a].expectation is None and not reg.ops[a].grants


def test_upload_completion_reaches_installing_with_a_new_generation():
    p, reg = manual()
    a = reg.request(key(1), EXT)
    to_stage(p, reg, a, LoadStage.UPLOAD_SUBMITTED)
    g_up = reg.ops[a].generation
    p.complete(a)
    reg.drive()
    assert reg.ops[a].stage == LoadStage.INSTALLING and reg.ops[a].generation == g_up + 1
    assert reg.ops[a].expectation.stage == LoadStage.INSTALLING


def test_published_binding_carries_the_exact_destination_generation():
    p = FakeMaterializationProvider()
    reg = LoadRegistry(p)
    a = reg.request(key(1, gen=4), EXT)
    for _ in range(6):
        reg.drive()
    assert reg.is_resident(key(1, gen=4)) and not reg.is_resident(key(1, gen=3)) and not reg.is_resident(key(1, gen=5))
    assert reg.ops[a].key.destination_generation == 4


def test_successful_operation_retires_exactly_once_and_keeps_its_key():
    p = FakeMaterializationProvider()
    reg = LoadRegistry(p)
    a = reg.request(key(1), EXT)
    for _ in range(6):
        reg.drive()
    assert reg.evict() == 1 and reg.ops[a].stage == LoadStage.RETIRED and p.retired == [a]
    assert reg.evict() == 0 and reg.stats.retired == 1 and p.retired == [a]
    assert reg.ops[a].key == key(1) and not reg.is_resident(key(1))           # the id still names its key
    assert reg.broker.outstanding() == 0


# ------------------------------------------------------------------------------------------ single flight
def test_n_waiters_issue_one_physical_read():
    p, reg = manual()
    for t in range(5):
        reg.register_continuation(t, [key(1)])
    finish(p, reg)
    assert sum(1 for c in p.calls if c[0] == "read") == 1 and sorted(reg.pop_ready()) == [0, 1, 2, 3, 4]
    assert reg.ops[0].leases == 5


def test_resource_kinds_never_join_across_kinds():
    p = FakeMaterializationProvider()
    reg = LoadRegistry(p)
    ids = {reg.request(key(1, kind=k), EXT) for k in ResourceKind}
    assert len(ids) == len(list(ResourceKind)) and reg.stats.coalesced == 0


def test_different_source_generation_never_joins():
    p, reg = manual()
    a = reg.request(key(1, src=b"v1"), EXT)
    b = reg.request(key(1, src=b"v2"), EXT)
    assert a != b and reg.stats.coalesced == 0


def test_duplicate_dependency_and_duplicate_waiter_are_rejected_before_side_effects():
    p, reg = manual()
    with pytest.raises(IoProtocolError):
        reg.register_continuation(1, [key(1), key(2), key(1)])
    assert not reg.ops and not reg.conts and reg.stats.requests == 0
    reg.register_continuation(1, [key(1)])
    with pytest.raises(IoProtocolError):
        reg.register_continuation(1, [key(2)])
    assert len(reg.ops) == 1 and reg.ops[0].leases == 1


# ------------------------------------------------------------------------------------------ ownership
def test_prefetch_owns_an_operation_without_execution_state():
    p, reg = manual()
    a = reg.request(key(1), (OwnerKind.TRANSACTION_PREFETCH, 3))
    op = reg.ops[a]
    assert op.purpose == Purpose.PREFETCH and not op.waiters and op.leases == 0 and not reg.conts


def test_execution_joins_an_active_prefetch_without_second_io():
    p, reg = manual()
    a = reg.request(key(1), (OwnerKind.TRANSACTION_PREFETCH, 3))
    reg.drive()
    reg.register_continuation(3, [key(1)])
    assert reg.stats.promoted == 1 and reg.ops[a].purpose == Purpose.EXECUTION
    finish(p, reg)
    assert sum(1 for c in p.calls if c[0] == "read") == 1 and reg.pop_ready() == [3]


def test_cancelling_the_prefetch_owner_does_not_cancel_the_joined_execution():
    p, reg = manual()
    a = reg.request(key(1), (OwnerKind.TRANSACTION_PREFETCH, 3))
    reg.drive()
    reg.register_continuation(8, [key(1)])
    assert reg.detach(a, (OwnerKind.TRANSACTION_PREFETCH, 3)) is False
    finish(p, reg)
    assert reg.pop_ready() == [8] and p.cancelled == []


def test_cancelling_one_of_several_prefetch_owners_keeps_the_operation():
    p, reg = manual()
    a = reg.request(key(1), (OwnerKind.TRANSACTION_PREFETCH, 1))
    assert reg.request(key(1), (OwnerKind.TRANSACTION_PREFETCH, 2)) == a
    assert reg.detach(a, (OwnerKind.TRANSACTION_PREFETCH, 1)) is False and reg.ops[a].stage == LoadStage.RESERVED
    assert reg.detach(a, (OwnerKind.TRANSACTION_PREFETCH, 2)) is True and reg.ops[a].stage == LoadStage.RETIRED


def test_duplicate_detach_is_detected():
    p, reg = manual()
    a = reg.request(key(1), (OwnerKind.TRANSACTION_PREFETCH, 1))
    reg.request(key(1), (OwnerKind.TRANSACTION_PREFETCH, 2))
    reg.detach(a, (OwnerKind.TRANSACTION_PREFETCH, 1))
    with pytest.raises(IoProtocolError):
        reg.detach(a, (OwnerKind.TRANSACTION_PREFETCH, 1))
    with pytest.raises(IoProtocolError):
        reg.detach(a, (OwnerKind.EXTERNAL, 9))
    with pytest.raises(IoProtocolError):
        reg.detach(77, (OwnerKind.EXTERNAL, 9))


def test_prefetch_of_a_resident_payload_creates_no_operation_and_takes_no_credit():
    p = FakeMaterializationProvider()
    reg = LoadRegistry(p)
    a = reg.request(key(1), EXT)
    for _ in range(6):
        reg.drive()
    n_ops, credit, calls = len(reg.ops), reg.broker.outstanding(), len(p.calls)
    assert reg.prefetch([key(1)], (OwnerKind.TRANSACTION_PREFETCH, 5)) == [a]
    assert (len(reg.ops), reg.broker.outstanding(), len(p.calls)) == (n_ops, credit, calls)
    assert reg.stats.satisfied_resident == 1


def test_cancelling_one_shared_waiter_keeps_the_demand_load():
    p, reg = manual()
    reg.register_continuation(1, [key(1)])
    reg.register_continuation(2, [key(1)])
    reg.drive()
    reg.cancel_continuation(1)
    assert reg.ops[0].waiters == {2} and reg.ops[0].leases == 1 and p.cancelled == []
    finish(p, reg)
    assert reg.pop_ready() == [2]


# ------------------------------------------------------------------------------------------ cancellation
def test_cancelling_the_last_reserved_owner_retires_immediately():
    p, reg = manual()
    a = reg.request(key(1), EXT)
    assert reg.detach(a, EXT) is True
    assert reg.ops[a].stage == LoadStage.RETIRED and p.calls == [] and reg.broker.outstanding() == 0


@pytest.mark.parametrize("stage", [LoadStage.READ_SUBMITTED, LoadStage.UPLOAD_SUBMITTED, LoadStage.INSTALLING])
def test_cancelling_submitted_work_waits_for_its_completion(stage):
    p, reg = manual()
    a = reg.request(key(1), EXT)
    to_stage(p, reg, a, stage)
    held = reg.broker.outstanding()
    reg.cancel(a)
    assert reg.ops[a].stage == stage and reg.broker.outstanding() == held      # nothing is revoked under the hardware
    assert p.cancelled == [a]
    reg.drive()                                                               # CANCELLED completion arrives
    assert reg.ops[a].stage == LoadStage.RETIRED and reg.broker.outstanding() == 0 and p.retired == [a]


def test_success_that_beats_the_cancel_still_ends_in_cleanup():
    """The read had completed before the last owner cancelled: the operation is at HOST_READY with nothing in
    flight, so the cancel retires it through STALE without another completion."""
    p, reg = manual()
    a = reg.request(key(1), EXT)
    reg.drive()
    p.complete(a)
    reg._collect_completions()
    assert reg.ops[a].stage == LoadStage.HOST_READY
    reg.cancel(a)
    assert reg.ops[a].stage == LoadStage.RETIRED and reg.broker.outstanding() == 0
    reg.drive()
    assert sum(1 for c in p.calls if c[0] == "upload") == 0


def test_demand_load_is_not_cancellable_while_a_waiter_remains():
    p, reg = manual()
    reg.register_continuation(1, [key(1)])
    with pytest.raises(RuntimeError):
        reg.cancel(0)
    assert reg.ops[0].stage == LoadStage.RESERVED


def test_all_shared_waiters_cancelled_requests_one_physical_cancel():
    p, reg = manual()
    for t in (1, 2, 3):
        reg.register_continuation(t, [key(1)])
    reg.drive()
    for t in (1, 2, 3):
        reg.cancel_continuation(t)
    reg.cancel(0)
    assert p.cancelled == [0]
    reg.drive()
    assert reg.ops[0].stage == LoadStage.RETIRED


def test_cancelling_an_unsubmitted_load_releases_its_place_for_the_next_one():
    broker = PhysicalResourceBroker()
    broker.set_limit(RK.READ_SLOTS, 1)
    p = FakeMaterializationProvider(auto=False)
    reg = LoadRegistry(p, broker)
    a = reg.request(key(1), EXT)
    b = reg.request(key(2), EXT)
    reg.drive()
    assert reg.ops[a].stage == LoadStage.READ_SUBMITTED and reg.ops[b].stage == LoadStage.RESERVED
    reg.cancel(b)
    c = reg.request(key(3), EXT)
    p.complete(a)
    reg.drive()
    assert reg.ops[c].stage == LoadStage.READ_SUBMITTED


# ------------------------------------------------------------------------------------------ failures
@pytest.mark.parametrize("script,reads,uploads,installs", [(("fail",), 1, 0, 0), (("ok", "fail"), 1, 1, 0),
                                                            (("ok", "ok", "fail"), 1, 1, 1)])
def test_failure_at_any_stage_fails_the_waiter_and_retires(script, reads, uploads, installs):
    p = FakeMaterializationProvider()
    reg = LoadRegistry(p)
    p.script_next(*script)
    reg.register_continuation(1, [key(1)])
    for _ in range(8):
        reg.drive()
    assert reg.pop_failed() == [1] and reg.pop_ready() == []
    assert (reg.stats.submitted_reads, reg.stats.submitted_uploads, reg.stats.submitted_installs) == (reads, uploads, installs)
    assert reg.ops[0].stage == LoadStage.RETIRED and reg.ops[0].failure == FailureReason.READ_ERROR
    assert reg.broker.outstanding() == 0 and p.retired == [0] and not reg.is_resident(key(1))


def test_failure_is_targeted_and_an_unrelated_load_goes_on():
    p = FakeMaterializationProvider()
    reg = LoadRegistry(p)
    p.script_next("fail")
    reg.register_continuation(1, [key(1)])
    reg.register_continuation(2, [key(2)])
    for _ in range(8):
        reg.drive()
    assert reg.pop_failed() == [1] and reg.pop_ready() == [2]


def test_reserve_failure_rolls_back_every_claim():
    p = FakeMaterializationProvider()
    reg = LoadRegistry(p)
    p.fail_next_reserve()
    reg.register_continuation(1, [key(1)])
    reg.drive()
    assert reg.pop_failed() == [1] and reg.broker.outstanding() == 0 and reg.ops[0].stage == LoadStage.RETIRED
    assert reg.ops[0].failure == FailureReason.RESOURCE_EXHAUSTED and p.reserved == {}


def test_retry_after_failure_gets_a_new_identity_and_old_completions_cannot_touch_it():
    p = FakeMaterializationProvider(auto=False)
    reg = LoadRegistry(p)
    a = reg.request(key(1), EXT)
    reg.drive()
    old = p.pending[a]
    p.pending[a] = CompletionEvent(a, old.key, old.stage, old.generation, CompletionOutcome.FAILED, 0,
                                   FailureReason.READ_ERROR, old.timestamp_ns)
    p.complete(a)
    reg.drive()
    assert reg.ops[a].stage == LoadStage.RETIRED
    b = reg.request(key(1), EXT)
    assert b != a
    reg.drive()
    p.push_completion(old)                                 # the first attempt's success shows up late
    reg._collect_completions()
    assert reg.stats.rejected_completions == 1 and reg.ops[b].stage == LoadStage.READ_SUBMITTED
    finish(p, reg)
    assert reg.is_resident(key(1))


# ------------------------------------------------------------------------------------------ bad completions
@pytest.mark.parametrize("stage", [LoadStage.READ_SUBMITTED, LoadStage.UPLOAD_SUBMITTED, LoadStage.INSTALLING])
def test_stale_completion_never_publishes(stage):
    p, reg = manual()
    a = reg.request(key(1), EXT)
    to_stage(p, reg, a, stage)
    ev = p.pending.pop(a)
    p.push_completion(CompletionEvent(a, ev.key, ev.stage, ev.generation - 1, ev.outcome, ev.bytes_done, None, ev.timestamp_ns))
    reg.drive()
    assert reg.ops[a].stage == stage and reg.stats.rejected_completions == 1 and not reg.is_resident(key(1))
    assert "generation" in reg.rejections[-1].reason


def test_wrong_operation_wrong_key_and_wrong_stage_completions_fail_closed():
    p, reg = manual()
    a = reg.request(key(1), EXT)
    b = reg.request(key(2), EXT)
    reg.drive()
    ea, eb = p.pending[a], p.pending[b]
    p.push_completion(CompletionEvent(a, eb.key, ea.stage, ea.generation, CompletionOutcome.OK, ea.bytes_done))     # key
    p.push_completion(CompletionEvent(a, ea.key, LoadStage.INSTALLING, ea.generation, CompletionOutcome.OK, ea.bytes_done))
    p.push_completion(CompletionEvent(55, ea.key, ea.stage, ea.generation, CompletionOutcome.OK, ea.bytes_done))    # op
    reg._collect_completions()
    assert reg.stats.rejected_completions == 3
    assert reg.ops[a].stage == LoadStage.READ_SUBMITTED and reg.ops[b].stage == LoadStage.READ_SUBMITTED
    assert [r.reason for r in reg.rejections][2] == "unknown operation"


def test_short_success_is_a_failure_not_a_stray_event():
    p = FakeMaterializationProvider()
    reg = LoadRegistry(p)
    p.script_next("short")
    reg.register_continuation(1, [key(1)])
    for _ in range(4):
        reg.drive()
    assert reg.pop_failed() == [1] and reg.ops[0].failure == FailureReason.SHORT_READ
    assert reg.stats.rejected_completions == 0


def test_duplicate_completion_is_diagnosed_without_a_second_release():
    p = FakeMaterializationProvider()
    reg = LoadRegistry(p)
    p.script_next("dup")
    a = reg.request(key(1), EXT)
    for _ in range(6):
        reg.drive()
    assert reg.is_resident(key(1)) and reg.stats.rejected_completions == 1
    assert reg.broker.outstanding() == 1 and reg.stats.submitted_uploads == 1      # one upload, one residency credit


def test_out_of_order_completion_does_not_advance_the_owner():
    p, reg = manual()
    a = reg.request(key(1), EXT)
    reg.drive()
    ev = p.pending[a]
    p.push_completion(CompletionEvent(a, ev.key, LoadStage.UPLOAD_SUBMITTED, ev.generation + 1, CompletionOutcome.OK,
                                      ev.bytes_done))
    reg._collect_completions()
    assert reg.ops[a].stage == LoadStage.READ_SUBMITTED and reg.stats.rejected_completions == 1
    finish(p, reg)
    assert reg.is_resident(key(1))


def test_lost_completion_keeps_its_credit_and_never_publishes():
    p = FakeMaterializationProvider()
    reg = LoadRegistry(p)
    p.lose_next()
    a = reg.request(key(1), EXT)
    for _ in range(10):
        reg.drive()
    assert reg.ops[a].stage == LoadStage.READ_SUBMITTED and reg.broker.outstanding() == 1
    assert not reg.is_resident(key(1)) and reg.stats.published == 0


def test_completion_queue_rejects_the_bad_event_and_applies_the_good_one_behind_it():
    p, reg = manual()
    a = reg.request(key(1), EXT)
    reg.drive()
    ev = p.pending.pop(a)
    p.push_completion(CompletionEvent(a, ev.key, ev.stage, ev.generation + 7, ev.outcome, ev.bytes_done))
    p.push_completion(ev)
    reg._collect_completions()
    assert reg.stats.rejected_completions == 1 and reg.ops[a].stage == LoadStage.HOST_READY


def test_every_illegal_stage_transition_is_rejected():
    legal = 0
    for a in LoadStage:
        for b in LoadStage:
            if can_transition(a, b):
                legal += 1
                validate_transition(a, b)
            else:
                with pytest.raises(IoProtocolError):
                    validate_transition(a, b)
    assert 0 < legal < len(list(LoadStage)) ** 2 // 2
    assert not any(can_transition(LoadStage.RETIRED, b) for b in LoadStage)
    assert not can_transition(LoadStage.RESERVED, LoadStage.RESIDENT) and not can_transition(LoadStage.FAILED, LoadStage.RESIDENT)


# ------------------------------------------------------------------------------------------ credits
def test_upload_backpressure_lets_reads_go_on_up_to_the_pinned_capacity():
    broker = PhysicalResourceBroker()
    broker.set_limit(RK.UPLOAD_SLOTS, 1)
    p = FakeMaterializationProvider(auto=False, payload_bytes=4096)
    broker.set_limit(RK.PINNED_BYTES, 3 * FakeMaterializationProvider().plan(key(0)).pinned_bytes)
    reg = LoadRegistry(p, broker)
    ops = [reg.request(key(i), EXT) for i in range(4)]
    reg.drive()
    reading = [o for o in ops if reg.ops[o].stage == LoadStage.READ_SUBMITTED]
    assert len(reading) == 3 and reg.stats.credit_denials >= 1                   # the fourth waits for pinned bytes
    for o in reading:
        p.complete(o)
    reg.drive()
    stages = [reg.ops[o].stage for o in ops]
    assert stages.count(LoadStage.UPLOAD_SUBMITTED) == 1                         # one upload slot
    assert broker.usage[RK.UPLOAD_SLOTS].high_water == 1
    finish(p, reg, 30)
    assert all(reg.ops[o].stage == LoadStage.RESIDENT for o in ops)


def test_install_slots_bound_concurrent_installs():
    broker = PhysicalResourceBroker()
    broker.set_limit(RK.INSTALL_SLOTS, 1)
    p = FakeMaterializationProvider(auto=False)
    reg = LoadRegistry(p, broker)
    ops = [reg.request(key(i), EXT) for i in range(3)]
    finish(p, reg, 30)
    assert all(reg.ops[o].stage == LoadStage.RESIDENT for o in ops)
    assert broker.usage[RK.INSTALL_SLOTS].high_water <= 1


def test_operation_larger_than_a_physical_limit_never_starves_the_queue_behind_it():
    broker = PhysicalResourceBroker()
    broker.set_limit(RK.STORAGE_BYTES, 1024)                 # smaller than one payload
    p = FakeMaterializationProvider(auto=False, payload_bytes=4096)
    reg = LoadRegistry(p, broker)
    a = reg.request(key(1), EXT)
    for _ in range(5):
        reg.drive()
    assert reg.ops[a].stage == LoadStage.RESERVED and reg.stats.credit_denials >= 5 and reg.broker.outstanding() == 0


def test_multi_claim_admission_is_atomic():
    broker = PhysicalResourceBroker()
    broker.set_limit(RK.READ_SLOTS, 4)
    broker.set_limit(RK.PINNED_BYTES, 100)
    assert broker.try_claim({RK.READ_SLOTS: 1, RK.PINNED_BYTES: 200}) is None
    assert broker.outstanding() == 0 and broker.usage[RK.READ_SLOTS].in_use == 0
    g = broker.try_claim({RK.READ_SLOTS: 1, RK.PINNED_BYTES: 60})
    assert g is not None and broker.try_claim({RK.READ_SLOTS: 1, RK.PINNED_BYTES: 60}) is None
    assert broker.usage[RK.READ_SLOTS].in_use == 1
    broker.complete(g)
    assert broker.outstanding() == 0


def test_submitted_grant_cannot_be_revoked_and_completes_once():
    broker = PhysicalResourceBroker()
    broker.set_limit(RK.READ_SLOTS, 1)
    g = broker.try_claim({RK.READ_SLOTS: 1})
    broker.mark_submitted(g)
    with pytest.raises(Exception):
        broker.revoke(g)
    broker.complete(g)
    with pytest.raises(Exception):
        broker.complete(g)
    assert broker.outstanding() == 0


def test_prefetch_cannot_use_the_execution_reserve_but_required_work_can():
    broker = PhysicalResourceBroker()
    broker.set_limit(RK.LOAD_OPS, 2, execution_reserve=1)
    assert broker.try_claim({RK.LOAD_OPS: 1}, required=False) is not None
    assert broker.try_claim({RK.LOAD_OPS: 1}, required=False) is None
    assert broker.try_claim({RK.LOAD_OPS: 1}, required=True) is not None
    assert broker.try_claim({RK.LOAD_OPS: 1}, required=True) is None


# ------------------------------------------------------------------------------------------ fairness
def test_required_work_runs_first_without_freezing_background_warmup():
    p, reg = manual()
    warm = [reg.request(key(i), (OwnerKind.MODEL_WARMUP, 0)) for i in range(30)]
    reg.register_continuation(1, [key(100 + i) for i in range(6)])
    reg.drive(max_actions=8)
    started = [o for o, op in reg.ops.items() if op.stage == LoadStage.READ_SUBMITTED]
    req = [o for o in started if reg.ops[o].purpose == Purpose.EXECUTION]
    assert len(req) >= 5 and len(started) == 8
    for _ in range(40):
        reg.drive(max_actions=8)
        for o in list(p.pending):
            p.complete(o)
    assert all(reg.ops[o].stage == LoadStage.RESIDENT for o in warm)


def test_fair_queue_serves_ten_thousand_entries_in_order_within_a_band():
    q = FairQueue(FairQueueConfig())
    for i in range(10_000):
        q.push(Band.PREFETCH, i)
    out = [q.pop()[1] for _ in range(10_000)]
    assert out == list(range(10_000)) and q.pop() is None


def test_fair_queue_drops_removed_entries_lazily():
    q = FairQueue(FairQueueConfig())
    for i in range(10):
        q.push(Band.REQUIRED, i)
    for i in range(0, 10, 2):
        q.remove(i)
    assert [q.pop()[1] for _ in range(5)] == [1, 3, 5, 7, 9] and q.pop() is None


def test_aged_prefetch_makes_progress_under_required_pressure_and_debt_stays_bounded():
    cfg = FairQueueConfig(quantum=(8, 1, 1), aging_ticks=4, debt_bound=2)
    q = FairQueue(cfg)
    q.push(Band.PREFETCH, ("p", 0))
    served = []
    for i in range(40):                       # required work keeps arriving: every head is younger than the prefetch
        q.push(Band.REQUIRED, ("r", 2 * i))
        q.push(Band.REQUIRED, ("r", 2 * i + 1))
        served.append(q.pop()[0])
    assert Band.PREFETCH in served[:12] and q.aged[Band.PREFETCH] == 1 and q.served[Band.PREFETCH] == 1
    assert all(c >= -cfg.debt_bound * cfg.quantum[b] for b, c in q._credit.items())


def test_fair_queue_rejects_zero_quantum():
    with pytest.raises(Exception):
        FairQueue(FairQueueConfig(quantum=(0, 1, 1)))


def test_fairness_never_bypasses_feasibility():
    """The head of the required band cannot be admitted (no credit); prefetch work behind it that fits does run,
    and the blocked head keeps its place."""
    broker = PhysicalResourceBroker()
    broker.set_limit(RK.READ_SLOTS, 1)
    p = FakeMaterializationProvider(auto=False)
    reg = LoadRegistry(p, broker)
    a = reg.request(key(1), EXT)
    reg.drive()
    reg.register_continuation(5, [key(2)])                   # needs a read slot: none left
    reg.drive()
    assert reg.ops[1].stage == LoadStage.RESERVED and reg.stats.credit_denials >= 1
    p.complete(a)
    reg.drive()
    assert reg.ops[1].stage == LoadStage.READ_SUBMITTED


# ------------------------------------------------------------------------------------------ waiters
def test_continuation_needs_all_its_dependencies():
    p, reg = manual()
    reg.register_continuation(1, [key(1), key(2), key(3)])
    reg.drive()
    for o in (0, 1):
        to_done = [o]
        while reg.ops[o].stage != LoadStage.RESIDENT:
            if o in p.pending:
                p.complete(o)
            reg.drive()
    assert reg.pop_ready() == [] and reg.conts[1].needs == {2}
    finish(p, reg)
    assert reg.pop_ready() == [1]


def test_targeted_ready_does_not_wake_an_unrelated_continuation():
    p, reg = manual()
    reg.register_continuation(1, [key(1)])
    reg.register_continuation(2, [key(2)])
    reg.drive()
    while reg.ops[1].stage != LoadStage.RESIDENT:           # complete only the second one's payload
        if 1 in p.pending:
            p.complete(1)
        reg.drive()
    assert reg.pop_ready() == [2] and reg.conts[1].needs == {0}


def test_reverse_completion_order_wakes_in_completion_order():
    p, reg = manual()
    for t in range(4):
        reg.register_continuation(t, [key(t)])
    reg.drive()
    woke = []
    for o in (3, 2, 1, 0):
        while reg.ops[o].stage != LoadStage.RESIDENT:
            if o in p.pending:
                p.complete(o)
            reg.drive()
        woke += reg.pop_ready()
    assert woke == [3, 2, 1, 0]


def test_waiter_index_is_kept_in_both_directions():
    p, reg = manual()
    reg.register_continuation(1, [key(1), key(2)])
    reg.register_continuation(2, [key(2)])
    assert reg.ops[0].waiters == {1} and reg.ops[1].waiters == {1, 2}
    assert reg.conts[1].needs == {0, 1} and reg.conts[2].needs == {1}
    reg.cancel_continuation(1)
    assert reg.ops[0].waiters == set() and reg.ops[1].waiters == {2} and 1 not in reg.conts


def test_resident_attach_is_ready_at_once_without_a_second_read():
    p = FakeMaterializationProvider()
    reg = LoadRegistry(p)
    reg.request(key(1), EXT)
    for _ in range(6):
        reg.drive()
    reads = reg.stats.submitted_reads
    reg.register_continuation(4, [key(1)])
    assert reg.pop_ready() == [4] and reg.stats.submitted_reads == reads and reg.ops[0].leases == 1


def test_residency_lease_is_held_from_registration_until_release():
    p = FakeMaterializationProvider()
    reg = LoadRegistry(p)
    reg.register_continuation(4, [key(1)])
    for _ in range(6):
        reg.drive()
    assert reg.pop_ready() == [4] and reg.ops[0].leases == 1 and reg.evict_candidates() == [] and reg.evict() == 0
    reg.release_transaction(4)
    assert reg.ops[0].leases == 0 and reg.evict_candidates() == [0]


def test_shared_wait_is_counted_once_not_per_waiter():
    t = [0]
    p = FakeMaterializationProvider(auto=False)
    reg = LoadRegistry(p, clock=lambda: t[0])
    for w in (1, 2, 3):
        reg.register_continuation(w, [key(1)])
    reg.drive()
    for _ in range(3):
        t[0] += 100
        if 0 in p.pending:
            p.complete(0)
        reg.drive()
    assert sorted(reg.pop_ready()) == [1, 2, 3]
    assert reg.ledger.shared_wait([0]) <= 300


# ------------------------------------------------------------------------------------------ shutdown
def test_shutdown_drains_mixed_queued_and_submitted_work_without_a_grant_leak():
    broker = PhysicalResourceBroker()
    broker.set_limit(RK.READ_SLOTS, 2)
    p = FakeMaterializationProvider(auto=False)
    reg = LoadRegistry(p, broker)
    for i in range(5):
        reg.request(key(i), EXT)
    reg.drive()
    assert sum(1 for o in reg.ops.values() if o.stage == LoadStage.READ_SUBMITTED) == 2
    for _ in range(4):
        if reg.shutdown():
            break
    assert reg.residual() == {"in_flight": 0, "resident": 0, "grants": 0, "continuations": 0}
    assert all(o.stage == LoadStage.RETIRED for o in reg.ops.values())


def test_shutdown_releases_residency_and_continuation_custody():
    p = FakeMaterializationProvider()
    reg = LoadRegistry(p)
    reg.register_continuation(1, [key(1), key(2)])
    for _ in range(6):
        reg.drive()
    assert reg.pop_ready() == [1] and reg.broker.outstanding() == 2
    reg.release_transaction(1)
    while not reg.shutdown():
        pass
    assert reg.residual() == {"in_flight": 0, "resident": 0, "grants": 0, "continuations": 0}


def test_shutdown_with_a_lost_completion_is_explicit_and_can_be_retried():
    p = FakeMaterializationProvider()
    reg = LoadRegistry(p)
    p.lose_next()
    a = reg.request(key(1), EXT)
    reg.drive()
    assert reg.shutdown() is False and reg.shutdown() is False        # the owed completion never came
    assert reg.residual()["in_flight"] == 1 and reg.residual()["grants"] == 1
    exp = reg.ops[a].expectation
    p.push_completion(CompletionEvent(a, key(1), exp.stage, exp.generation, CompletionOutcome.CANCELLED, 0,
                                      FailureReason.CANCELLED))
    assert reg.shutdown() is True and reg.residual()["grants"] == 0


def test_new_requests_and_continuations_are_refused_once_shutdown_began():
    p, reg = manual()
    reg.shutdown()
    with pytest.raises(RuntimeError):
        reg.request(key(1), EXT)
    with pytest.raises(RuntimeError):
        reg.register_continuation(1, [key(1)])
    assert not reg.ops and not reg.conts


def test_resumed_transaction_that_waits_again_extends_its_continuation():
    """A transaction resumed after its first wait may need more payloads: the second registration keeps the
    custody (one lease per payload, never two) and waits for the new ones only; registering again while the
    first wait is unresolved stays an error."""
    p, reg = manual()
    reg.register_continuation(1, [key(1)])
    with pytest.raises(IoProtocolError):
        reg.register_continuation(1, [key(2)])
    finish(p, reg)
    assert reg.pop_ready() == [1]
    reg.register_continuation(1, [key(1), key(2)])
    assert reg.ops[0].leases == 1 and reg.ops[1].leases == 1 and reg.conts[1].needs == {1}
    finish(p, reg)
    assert reg.pop_ready() == [1] and sorted(reg.conts[1].all_ops) == [0, 1]
    reg.release_transaction(1)
    assert reg.ops[0].leases == 0 and reg.ops[1].leases == 0 and sorted(reg.evict_candidates()) == [0, 1]


# ---------------------------------------------------------------------------------------------- randomised soak
def _soak(seed):
    rnd = random.Random(seed)
    p = FakeMaterializationProvider(auto=False)
    reg = LoadRegistry(p)
    txns = {}          # txn -> state: "waiting" | "ready"
    next_txn = 0
    prefetch_owned = {}   # (op, owner)
    for step in range(600):
        a = rnd.random()
        if a < 0.20:
            t = next_txn
            next_txn += 1
            ks = [key(e, gen=0) for e in rnd.sample(range(12), rnd.randrange(1, 4))]
            reg.register_continuation(t, ks)
            txns[t] = "waiting"
        elif a < 0.30:
            o = (OwnerKind.TRANSACTION_PREFETCH, rnd.randrange(1000, 1010))
            op = reg.request(key(rnd.randrange(12)), o)
            prefetch_owned.setdefault(op, set()).add(o)
        elif a < 0.36 and prefetch_owned:
            op = rnd.choice(sorted(prefetch_owned))
            o = prefetch_owned[op].pop()
            if not prefetch_owned[op]:
                del prefetch_owned[op]
            x = reg.ops.get(op)
            if x is not None and o in x.owners:
                reg.detach(op, o)
        elif a < 0.60 and p.pending:
            op = rnd.choice(sorted(p.pending))
            p.complete(op)
        elif a < 0.66:
            p.script_next(rnd.choice(["fail", "short", "lose", "reject", "dup", "stale", "ok", "ok"]))
        elif a < 0.74 and txns:
            t = rnd.choice(sorted(txns))
            reg.release_transaction(t)
            del txns[t]
        elif a < 0.78:
            # a ready transaction waits again (extension)
            ready = [t for t, s in txns.items() if s == "ready"]
            if ready:
                t = rnd.choice(ready)
                ks = [key(e, gen=0) for e in rnd.sample(range(12), rnd.randrange(1, 3))]
                try:
                    reg.register_continuation(t, ks)
                    txns[t] = "waiting"
                except IoProtocolError:
                    pass
        reg.drive()
        for t in reg.pop_ready():
            if t in txns:
                txns[t] = "ready"
        for t in reg.pop_failed():
            if t in txns:
                reg.release_transaction(t)
                del txns[t]
        # invariants
        for op in reg.ops.values():
            assert op.leases >= 0
            if op.stage == LoadStage.RETIRED:
                assert not op.waiters and op.leases == 0, (seed, step, op)
        for t, c in reg.conts.items():
            for o in c.needs:
                assert t in reg.ops[o].waiters or reg.ops[o].stage in (LoadStage.FAILED, LoadStage.RETIRED), (seed, step, t, o, reg.ops[o].stage)
    # wind down: release all, complete everything
    for t in list(txns):
        reg.release_transaction(t)
    for op, owners in list(prefetch_owned.items()):
        for o in owners:
            x = reg.ops.get(op)
            if x is not None and o in x.owners:
                reg.detach(op, o)
    for _ in range(50):
        for op in list(p.pending):
            p.complete(op)
        reg.drive()
    res = reg.residual()
    assert res.get("continuations", 0) == 0, res
    assert all(op.leases == 0 and not op.waiters for op in reg.ops.values()), [(o.op_id, o.stage, o.leases, o.waiters) for o in reg.ops.values() if o.leases or o.waiters]
    return res



@pytest.mark.parametrize("seed", range(8))
def test_registry_soak(seed):
    """Random interleavings of continuations (one to three payloads, re-waits that extend them), prefetch owners
    that attach and detach, completions in any order, scripted failures, short reads, lost, rejected, duplicate
    and stale completions, and transactions that end at any time: no lease or waiter survives a retired operation,
    every outstanding dependency has its waiter registered, and after the wind-down nothing holds anything."""
    _soak(seed)


def test_broker_accounting_survives_random_claims_shrinks_and_releases():
    """in_use equals the sum of live grants after every operation; a released grant refuses every further use; a
    shrink can neither go negative nor grow the grant."""
    import random
    from ferrule_b200.runtime.resources import PhysicalResourceBroker, ResourceError, ResourceKind, ResourceLimit
    for seed in range(60):
        r = random.Random(seed)
        ks = r.sample(list(ResourceKind), 3)
        lim = {k: ResourceLimit(cap, r.randint(0, cap)) for k in ks for cap in [r.randint(1, 40)]}
        b = PhysicalResourceBroker(lim)
        live = []
        for _ in range(200):
            op = r.random()
            if op < 0.45:
                req = r.random() < 0.6
                am = {k: r.randint(0, 12) for k in r.sample(ks, r.randint(1, 3))}
                fits = all(n <= max(lim[k].capacity - (0 if req else lim[k].execution_reserve) - b.usage[k].in_use, 0)
                           for k, n in am.items())
                g = b.try_claim(am, req)
                assert (g is not None) == fits
                if g:
                    live.append(g)
            elif op < 0.6 and live:
                b.mark_submitted(r.choice(live))
            elif op < 0.8 and live:
                g = live.pop(r.randrange(len(live)))
                if g.submitted:
                    with pytest.raises(ResourceError):
                        b.revoke(g)
                    b.complete(g)
                else:
                    (b.revoke if r.random() < 0.5 else b.complete)(g)
                for again in (lambda: b.complete(g), lambda: b.shrink(g, ks[0], 0), lambda: b.mark_submitted(g)):
                    with pytest.raises(ResourceError):
                        again()
            elif live:
                g = r.choice(live)
                k = r.choice(list(g.amounts))
                n = r.randint(-1, g.amounts[k] + 1)
                if 0 <= n <= g.amounts[k]:
                    b.shrink(g, k, n)
                else:
                    with pytest.raises(ResourceError):
                        b.shrink(g, k, n)
            for k in ks:
                assert b.usage[k].in_use == sum(g.amounts.get(k, 0) for g in live)
                assert 0 <= b.usage[k].in_use <= lim[k].capacity
            assert b.outstanding() == len(live)


def test_ledger_interval_math_matches_a_bitmap():
    import random
    from ferrule_b200.runtime.ledger import intersect, union_length
    r = random.Random(0)

    def ticks(spans):
        return {t for s, e in spans for t in range(s, e)}
    for _ in range(300):
        a = [(s, s + r.randint(-3, 40)) for s in (r.randint(0, 200) for _ in range(r.randint(0, 8)))]
        b = [(s, s + r.randint(-3, 40)) for s in (r.randint(0, 200) for _ in range(r.randint(0, 8)))]
        assert union_length(a) == len(ticks(a))
        assert union_length(intersect(a, b)) == len(ticks(a) & ticks(b))
