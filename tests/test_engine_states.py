"""Engine owner loop: transactions that overlap (a waiting one, endings that stay pending) and finish out of
order, speculation under page exhaustion, custody after every kind of ending.  Mock runner, CPU.

Cases follow the reference's driver suite (crates/ferrule-runtime/src/engine/driver.rs:5686-10737: waiting cohorts,
pending endings, reverse completion order, zero-accept cycles, exhaustion)."""

from ferrule_b200.runtime.engine import Engine, EngineConfig, FinishEvent, TokenEvent
from ferrule_b200.runtime.io_protocol import MaterializationKey, ResourceId, ResourceKind
from ferrule_b200.runtime.provider import FakeMaterializationProvider
from ferrule_b200.runtime.registry import LoadRegistry
from ferrule_b200.runtime.runner import MockRunner
from ferrule_b200.runtime.scheduler import SchedulerConfig
from ferrule_b200.runtime.session import FinishReason, GenerateRequest


def key(e):
    return MaterializationKey("m", b"s", bytes([e]), ResourceId(ResourceKind.ROUTED_EXPERT, 1, e), 1, "cuda", 0, 0, 0)


def engine(runner, registry=None, pages=64, **kw):
    sched = SchedulerConfig(max_active_sequences=8, max_decode_batch=kw.pop("max_decode", 8), max_batch_tokens=64,
                            prefill_chunk_size=16, ctx_size=256, mixed_batches=kw.pop("mixed", True))
    return Engine(runner, EngineConfig(scheduler=sched, kv_pages=pages, page_size=16, **kw), registry=registry)


def expected(r, prompt, n):
    out, tok, pos = [], prompt[-1], len(prompt) - 1
    for _ in range(n):
        tok = r.next_token_fn(tok, pos)
        pos += 1
        out.append(tok)
    return out


def toks(ev, rid):
    return [e.token for e in ev if isinstance(e, TokenEvent) and e.request_id == rid]


def clean(eng):
    eng.kv.check_invariants()
    st = eng.kv.stats()
    assert st.used_pages == 0 and st.open_reservations == 0 and st.quarantined_pages == 0
    assert eng.broker.outstanding() == 0


def test_a_waiting_transaction_does_not_hold_up_the_others_and_resumes_last():
    """Transaction 0 waits for a payload that arrives late; the request submitted after it runs to completion
    meanwhile (its transactions start and end while 0 is parked); 0 then resumes with its reservation intact."""
    r = MockRunner()
    prov = FakeMaterializationProvider(auto=False)
    eng = engine(r, LoadRegistry(prov))
    r.wait_next = [[key(1)]]
    eng.submit(GenerateRequest("late", [5, 6, 7], max_new_tokens=3))
    ev = []
    eng.step(ev.append)                                   # transaction 0 parks
    assert eng.stats.waits == 1 and 0 in eng._waiting
    eng.submit(GenerateRequest("fast", [9, 8], max_new_tokens=4))
    for _ in range(40):
        eng.step(ev.append)
    assert toks(ev, "fast") == expected(r, [9, 8], 4) and toks(ev, "late") == []
    assert any(isinstance(e, FinishEvent) and e.request_id == "fast" for e in ev)
    assert 0 in eng._waiting and eng.kv.stats().open_reservations == 1     # the parked batch keeps its pages
    for op in list(prov.pending):                          # the payload arrives
        prov.complete(op)
    for _ in range(60):
        for op in list(prov.pending):
            prov.complete(op)
        eng.step(ev.append)
    assert toks(ev, "late") == expected(r, [5, 6, 7], 3) and eng.stats.resumes == 1
    ends = [c for c in r.calls if c[0].startswith("end_")]
    assert ends[-1][1] != 0 or ends.index(("end_publish", 0)) > 0          # 0 did not end first
    assert [c[1] for c in ends].index(0) > 0
    clean(eng)


def test_endings_that_stay_pending_complete_out_of_order_without_mixing_custody():
    """Transaction 0's ending stays PENDING for many polls (the backend is still draining it) while later
    transactions of other sequences start, end and publish; nothing of 0 is visible until its own ending
    completes, and every page finds its way back."""
    r = MockRunner()
    eng = engine(r, max_decode=1, mixed=False)
    eng.submit(GenerateRequest("a", [1, 2, 3], max_new_tokens=2))
    ev = []
    r._pending_left[0] = 6                                 # only the first transaction drains slowly
    eng.step(ev.append)                                    # prefill of a executes; its ending is pending
    assert len(eng._ending) == 1 and eng.kv.sequence(0).committed_tokens == 0
    eng.submit(GenerateRequest("b", [7, 7], max_new_tokens=2))
    for _ in range(4):
        eng.step(ev.append)
    assert eng.kv.sequence(0).committed_tokens == 0 and toks(ev, "a") == []        # still invisible
    assert len(toks(ev, "b")) >= 1                                                 # b published meanwhile
    ev += _drain(eng)
    assert toks(ev, "a") == expected(r, [1, 2, 3], 2) and toks(ev, "b") == expected(r, [7, 7], 2)
    order = [c[1] for c in r.calls if c[0] == "end_publish"]
    first_done = {t: i for i, t in reversed(list(enumerate(order)))}
    last_seen = {t: i for i, t in enumerate(order)}
    assert last_seen[0] > first_done[1]                    # 0 completed after a later transaction did
    clean(eng)


def _drain(eng):
    ev = []
    eng.run_until_idle(ev.append, max_steps=10000)
    return ev


def test_execute_failure_of_one_transaction_leaves_a_parked_one_untouched():
    r = MockRunner()
    prov = FakeMaterializationProvider(auto=False)
    eng = engine(r, LoadRegistry(prov))
    r.wait_next = [[key(4)]]
    eng.submit(GenerateRequest("parked", [3, 4, 5], max_new_tokens=2))
    ev = []
    eng.step(ev.append)
    r.fail_next_execute = 1
    eng.submit(GenerateRequest("boom", [6, 6], max_new_tokens=2))
    for _ in range(10):
        eng.step(ev.append)
    fin = [e for e in ev if isinstance(e, FinishEvent)]
    assert [f.request_id for f in fin] == ["boom"] and fin[0].reason == FinishReason.ERROR
    assert 0 in eng._waiting and eng.kv.stats().open_reservations == 1
    for _ in range(40):
        for op in list(prov.pending):
            prov.complete(op)
        eng.step(ev.append)
    assert toks(ev, "parked") == expected(r, [3, 4, 5], 2)
    clean(eng)


def test_cancelling_a_parked_request_releases_its_reservation_and_its_continuation():
    r = MockRunner()
    prov = FakeMaterializationProvider(auto=False)
    reg = LoadRegistry(prov)
    eng = engine(r, reg)
    r.wait_next = [[key(2)]]
    eng.submit(GenerateRequest("gone", [3, 4, 5], max_new_tokens=2))
    ev = []
    eng.step(ev.append)
    assert reg.conts and eng.kv.stats().open_reservations == 1
    eng.cancel_request("gone")
    for _ in range(20):
        for op in list(prov.pending):
            prov.complete(op)
        eng.step(ev.append)
    fin = [e for e in ev if isinstance(e, FinishEvent)]
    assert [f.reason for f in fin] == [FinishReason.CANCELLED] and toks(ev, "gone") == []
    assert not reg.conts and not eng._waiting
    clean(eng)


def test_zero_accept_speculation_under_page_exhaustion_stays_exact_and_leaks_nothing():
    """Every draft is wrong and the pool is so small that verification batches (anchor + drafts per sequence)
    often cannot reserve their pages: cycles fall back to plain decoding or stall, the streams stay those of greedy
    decoding, rejected suffix pages and unused copies all return."""
    def always_wrong(slot, j, nxt):
        return (nxt + 1) % 1000
    prompts = {f"r{i}": [(i * 31 + j) % 997 + 1 for j in range(14 + i)] for i in range(4)}
    want = {}
    base_r = MockRunner()
    base = engine(base_r, pages=64)
    for rid, p in prompts.items():
        base.submit(GenerateRequest(rid, p, max_new_tokens=24))
    eb = _drain(base)
    r = MockRunner(draft_len=3, draft_accuracy=always_wrong)
    eng = engine(r, pages=10, speculative=True, max_draft=3)          # 4 sequences x (38 tokens -> 3 pages) need 12
    for rid, p in prompts.items():
        eng.submit(GenerateRequest(rid, p, max_new_tokens=24))
    ev = _drain(eng)
    for rid in prompts:
        assert toks(ev, rid) == toks(eb, rid) and len(toks(ev, rid)) == 24, rid
    m = eng.spec.metrics
    assert m.cycles > 0 and m.accepted == 0 and m.drafted > 0 and m.accepted_prefix_hist.get(0, 0) == m.cycles_with_drafts \
        if hasattr(m, "cycles_with_drafts") else m.accepted == 0
    assert eng.stats.kv_stalls > 0, "the pool was meant to be too small"
    clean(eng)


def test_speculation_with_auto_preempt_under_exhaustion_completes_every_request():
    def half_right(slot, j, nxt):
        return nxt if (slot + j) % 2 else (nxt + 5) % 1000
    prompts = {f"r{i}": [(i * 13 + j) % 997 + 1 for j in range(20)] for i in range(4)}
    base = engine(MockRunner(), pages=64)
    for rid, p in prompts.items():
        base.submit(GenerateRequest(rid, p, max_new_tokens=30))
    eb = _drain(base)
    eng = engine(MockRunner(draft_len=2, draft_accuracy=half_right), pages=9, speculative=True, max_draft=2,
                 auto_preempt=True)
    for rid, p in prompts.items():
        eng.submit(GenerateRequest(rid, p, max_new_tokens=30))
    ev = []
    for _ in range(20000):
        if not eng.has_work() and not eng.scheduler.suspended:
            break
        eng.step(ev.append)
        eng.maybe_restore_suspended()
    for rid in prompts:
        assert toks(ev, rid) == toks(eb, rid), rid
    assert eng.stats.auto_preemptions > 0 and eng.kv.stats().preemptions == eng.stats.auto_preemptions
    clean(eng)


def test_finish_while_another_sequence_of_the_same_batch_continues():
    """Sequences of one decode cohort finish at different steps (length budgets 1..5): each leaves the cohort at
    its own step, its pages retire while the cohort goes on, and the later ones are unaffected."""
    r = MockRunner()
    eng = engine(r)
    for i in range(5):
        eng.submit(GenerateRequest(f"r{i}", [10 + i, 20 + i], max_new_tokens=i + 1))
    ev = _drain(eng)
    for i in range(5):
        assert toks(ev, f"r{i}") == expected(r, [10 + i, 20 + i], i + 1)
    fins = [e.request_id for e in ev if isinstance(e, FinishEvent)]
    assert fins == [f"r{i}" for i in range(5)]
    clean(eng)


def test_shutdown_with_a_parked_transaction_and_a_pending_ending_returns_all_custody():
    r = MockRunner()
    prov = FakeMaterializationProvider(auto=False)
    reg = LoadRegistry(prov)
    eng = engine(r, reg)
    r.wait_next = [[key(1)]]
    eng.submit(GenerateRequest("parked", [3, 4, 5], max_new_tokens=2))
    eng.step(lambda e: None)
    r._pending_left[1] = 3
    eng.submit(GenerateRequest("ending", [6, 7], max_new_tokens=2))
    eng.step(lambda e: None)
    for _ in range(200):
        for op in list(prov.pending):
            prov.complete(op)
        if eng.shutdown():
            break
    else:
        raise AssertionError("shutdown did not drain")
    clean(eng)
    while not reg.shutdown():
        for op in list(prov.pending):
            prov.complete(op)
    assert reg.residual() == {"in_flight": 0, "resident": 0, "grants": 0, "continuations": 0}


def test_page_deadlock_without_preemption_ends_the_youngest_request_with_an_error():
    """Every running sequence needs a page, none is free and nothing will return one: without `auto_preempt` the
    engine ends the youngest stalled request (error) instead of spinning; the others then finish normally."""
    r = MockRunner()
    eng = engine(r, pages=4)
    for i in range(3):
        eng.submit(GenerateRequest(f"r{i}", [(7 * i + j) % 990 + 1 for j in range(14)], max_new_tokens=30))
    ev = _drain(eng)
    fins = {e.request_id: e.reason for e in ev if isinstance(e, FinishEvent)}
    assert len(fins) == 3 and eng.stats.page_deadlocks >= 1
    errs = [k for k, v in fins.items() if v == FinishReason.ERROR]
    assert errs and "r0" not in errs, "the oldest request is the last to be given up"
    for rid, reason in fins.items():
        if reason != FinishReason.ERROR:
            assert toks(ev, rid) == expected(r, [(7 * int(rid[1]) + j) % 990 + 1 for j in range(14)], 30)
    clean(eng)


def test_restore_waits_for_headroom_instead_of_bouncing():
    """A swapped-out sequence returns only when its pages plus one page per running sequence are free."""
    r = MockRunner()
    eng = engine(r, pages=6, auto_preempt=True)
    for i in range(3):
        eng.submit(GenerateRequest(f"r{i}", [(5 * i + j) % 990 + 1 for j in range(15)], max_new_tokens=20))
    ev = _drain(eng)                                        # the owner loop itself brings them back
    assert all(len(toks(ev, f"r{i}")) == 20 for i in range(3))
    assert 1 <= eng.stats.auto_preemptions <= 4, "a handful of swaps, not one per step"
    clean(eng)
