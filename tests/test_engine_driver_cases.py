"""Named owner-loop cases (CPU, deterministic mock runner): request edges, policy isolation inside one batch,
event delivery, capability checks, failure write-back, exact forks, session continuation, cancellation reports."""
import pytest

from ferrule_b200.runtime.engine import Engine, EngineConfig, FinishEvent, TokenEvent
from ferrule_b200.runtime.execution import Intent, LogitsKind
from ferrule_b200.runtime.runner import MockRunner
from ferrule_b200.runtime.scheduler import SchedulerConfig
from ferrule_b200.runtime.session import FinishReason, GenerateRequest


def make(runner=None, **kw):
    sched = SchedulerConfig(max_active_sequences=kw.pop("max_active", 8), max_decode_batch=kw.pop("max_decode", 8),
                            max_batch_tokens=kw.pop("max_batch_tokens", 64),
                            prefill_chunk_size=kw.pop("chunk", 16), mixed_batches=kw.pop("mixed", True),
                            ctx_size=kw.pop("ctx", 256))
    cfg = EngineConfig(scheduler=sched, kv_pages=kw.pop("pages", 64), page_size=kw.pop("page", 16), **kw)
    r = runner or MockRunner(page_size=cfg.page_size)
    return Engine(r, cfg), r


def run(engine):
    events = []
    engine.run_until_idle(events.append, max_steps=10000)
    return events


def toks(events, rid):
    return [e.token for e in events if isinstance(e, TokenEvent) and e.request_id == rid]


def fin(events, rid):
    return [e for e in events if isinstance(e, FinishEvent) and e.request_id == rid][0]


def expected(r, prompt, n):
    out, tok, pos = [], prompt[-1], len(prompt) - 1
    for _ in range(n):
        tok = r.next_token_fn(tok, pos)
        pos += 1
        out.append(tok)
    return out


class Recording(MockRunner):
    """Keeps every executed batch."""

    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self.batches = []

    def execute(self, txn_id):
        self.batches.append(self.txns[txn_id])
        return super().execute(txn_id)


def test_max_new_zero_finishes_after_prefill():
    eng, r = make(Recording())
    eng.submit(GenerateRequest("z", list(range(1, 21)), max_new_tokens=0))
    ev = run(eng)
    assert toks(ev, "z") == [] and fin(ev, "z").reason == FinishReason.MAX_TOKENS and fin(ev, "z").generated_tokens == 0
    assert sum(b.rows for b in r.batches) == 20, "the prompt was prefilled, nothing was decoded"
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0


def test_final_decode_skips_the_logits_nobody_reads():
    eng, r = make(Recording(skip_unread_logits=True))
    prompt = list(range(3, 12))
    eng.submit(GenerateRequest("a", prompt, max_new_tokens=4))
    eng.submit(GenerateRequest("b", prompt[:5], max_new_tokens=7))
    ev = run(eng)
    assert toks(ev, "a") == expected(r, prompt, 4) and toks(ev, "b") == expected(r, prompt[:5], 7)
    # every generated token is committed through the model; the last one of a request asks for no logits
    last_a = next(b for b in r.batches if toks(ev, "a")[-1] in b.token_ids and len(b.sequences) <= 2 and b.rows <= 2)
    row = last_a.token_ids.index(toks(ev, "a")[-1])
    assert last_a.logits[row].kind == LogitsKind.NONE
    other = [i for i in range(last_a.rows) if i != row]
    assert all(last_a.logits[i].kind != LogitsKind.NONE for i in other), "the other request of the batch keeps its logits"
    none_rows = sum(1 for b in r.batches for i in range(b.rows)
                    if b.logits[i].kind == LogitsKind.NONE and any(s.phase.name == "DECODE" and s.query_start == i for s in b.sequences))
    assert none_rows == 2, "one unread row per request"
    # a runner that replays a captured step keeps the uniform request
    eng2, r2 = make(Recording())
    eng2.submit(GenerateRequest("a", prompt, max_new_tokens=4))
    run(eng2)
    assert all(b.logits[s.query_start].kind != LogitsKind.NONE for b in r2.batches for s in b.sequences
               if s.phase.name == "DECODE")


def test_mixed_requests_isolate_ignore_eos_policy():
    r = MockRunner(eos=7, next_token_fn=lambda t, p: 7 if p >= 6 else 20 + p)
    eng, _ = make(r)
    eng.submit(GenerateRequest("stop", [1, 2, 3, 4], max_new_tokens=8))
    eng.submit(GenerateRequest("go", [1, 2, 3, 4], max_new_tokens=8, ignore_eos=True))
    ev = run(eng)
    assert fin(ev, "stop").reason == FinishReason.EOS and 7 not in toks(ev, "stop") and len(toks(ev, "stop")) == 3
    assert fin(ev, "go").reason == FinishReason.MAX_TOKENS and toks(ev, "go").count(7) == 5
    assert eng.kv.stats().used_pages == 0


def test_callback_failure_retains_the_committed_event_and_does_not_poison_the_engine():
    eng, r = make()
    prompt = [5, 6, 7, 8]
    eng.submit(GenerateRequest("a", prompt, max_new_tokens=5))
    seen, fail = [], {"left": 1}

    def emit(e):
        if isinstance(e, TokenEvent) and e.index == 2 and fail["left"]:
            fail["left"] -= 1
            raise ConnectionError("consumer went away for a moment")
        seen.append(e)

    with pytest.raises(ConnectionError):
        eng.run_until_idle(emit, max_steps=1000)
    # the committed token is still in the outbox: the next steps deliver it, in order, exactly once
    eng.run_until_idle(emit, max_steps=1000)
    assert toks(seen, "a") == expected(r, prompt, 5)
    assert [e.index for e in seen if isinstance(e, TokenEvent)] == [0, 1, 2, 3, 4]
    assert fin(seen, "a").reason == FinishReason.MAX_TOKENS
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0


def test_requests_beyond_the_runner_capabilities_are_refused_before_any_work_is_consumed():
    class Small(MockRunner):
        def capabilities(self):
            from dataclasses import replace
            return replace(super().capabilities(), max_batch_rows=8)
    with pytest.raises(ValueError):
        make(Small(), chunk=16)              # a prefill chunk of 16 rows can never fit an 8-row runner
    eng, r = make(Small(), chunk=8, max_batch_tokens=8, max_decode=8)
    eng.submit(GenerateRequest("a", list(range(1, 20)), max_new_tokens=3))
    ev = run(eng)
    assert toks(ev, "a") == expected(r, list(range(1, 20)), 3)


def test_failed_batch_writes_back_every_sequence_and_the_engine_carries_on():
    eng, r = make()
    for rid in ("a", "b", "c"):
        eng.submit(GenerateRequest(rid, [ord(rid), 2, 3, 4, 5], max_new_tokens=4))
    ev = []
    eng.step(ev.append)                      # one mixed batch prefills all three
    r.fail_next_execute = 1
    while eng.has_work():
        eng.step(ev.append)
    reasons = {rid: fin(ev, rid).reason for rid in ("a", "b", "c")}
    assert set(reasons.values()) == {FinishReason.ERROR}, "every sequence of the failed batch ends with an error"
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0 and eng.stats.aborted_transactions >= 1
    eng.submit(GenerateRequest("d", [9, 9, 9], max_new_tokens=2))
    ev2 = run(eng)
    assert toks(ev2, "d") == expected(r, [9, 9, 9], 2)


def test_lowering_failure_fails_the_dequeued_sequence_only():
    eng, r = make()
    eng.submit(GenerateRequest("bad", [1, 2, 3], max_new_tokens=2))
    eng.submit(GenerateRequest("ok", [4, 5, 6], max_new_tokens=2))
    orig = eng._lower
    state = {"n": 0}

    def lower(txn):
        state["n"] += 1
        if state["n"] == 1:
            raise RuntimeError("cannot lower this batch")
        return orig(txn)

    eng._lower = lower
    ev = run(eng)
    done = {e.request_id: e.reason for e in ev if isinstance(e, FinishEvent)}
    assert FinishReason.ERROR in done.values()
    eng._lower = orig
    eng.submit(GenerateRequest("after", [7, 8], max_new_tokens=2))
    ev2 = run(eng)
    assert toks(ev2, "after") == expected(r, [7, 8], 2)
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0


def test_retained_session_continues_across_turns_and_can_reset():
    eng, r = make(Recording())
    eng.submit(GenerateRequest("t1", [1, 2, 3, 4, 5], max_new_tokens=3, session_id="s", retain_session=True))
    ev = run(eng)
    first = toks(ev, "t1")
    used = eng.kv.stats().used_pages
    assert used > 0, "the session keeps its pages"
    n_before = sum(b.rows for b in r.batches)
    eng.submit(GenerateRequest("t2", [40, 41], max_new_tokens=2, session_id="s", retain_session=True))
    ev2 = run(eng)
    # only the last generated token of turn one (not yet in the cache) and the new tokens are executed
    rows2 = sum(b.rows for b in r.batches) - n_before
    assert rows2 <= 1 + 2 + 2
    hist = [1, 2, 3, 4, 5] + first + [40, 41]
    assert toks(ev2, "t2") == expected(r, hist, 2)
    assert eng.reset_session("s") is True and eng.reset_session("s") is False
    assert eng.kv.stats().used_pages == 0
    eng.submit(GenerateRequest("t3", [1, 2, 3, 4, 5], max_new_tokens=3, session_id="s"))
    assert toks(run(eng), "t3") == first
    assert eng.kv.stats().used_pages == 0


def test_cancel_reports_waiting_running_and_unknown():
    eng, r = make(max_active=1)
    eng.submit(GenerateRequest("run", list(range(1, 40)), max_new_tokens=50))
    eng.submit(GenerateRequest("wait", [1, 2, 3], max_new_tokens=5))
    ev = []
    eng.step(ev.append)
    assert eng.cancel_request("nobody") is False
    assert eng.cancel_request("wait") is True
    assert eng.cancel_request("run") is True
    while eng.has_work():
        eng.step(ev.append)
    assert fin(ev, "wait").reason == FinishReason.CANCELLED and fin(ev, "run").reason == FinishReason.CANCELLED
    assert toks(ev, "wait") == []
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0
    # cancelling a finished request is unknown again
    assert eng.cancel_request("run") is False


def test_cancelling_an_unrelated_request_does_not_disturb_a_parked_transaction():
    eng, r = make()
    eng.submit(GenerateRequest("parked", [1, 2, 3, 4], max_new_tokens=3))
    eng.submit(GenerateRequest("other", [9, 8, 7], max_new_tokens=30))
    ev = []
    eng.step(ev.append)
    assert eng.cancel_request("other")
    ev += run(eng)
    assert toks(ev, "parked") == expected(r, [1, 2, 3, 4], 3) and fin(ev, "other").reason == FinishReason.CANCELLED
    assert eng.kv.stats().used_pages == 0


def test_exact_fork_executes_only_the_suffix():
    eng, r = make(Recording())
    base = list(range(1, 33))                 # two full pages
    eng.submit(GenerateRequest("src", base, max_new_tokens=1, session_id="src", retain_session=True))
    run(eng)
    n_before = sum(b.rows for b in r.batches)
    eng.fork_session_exact("src", GenerateRequest("f", [77, 78], max_new_tokens=2))
    ev = run(eng)
    assert len(toks(ev, "f")) == 2
    assert sum(b.rows for b in r.batches) - n_before <= 1 + 2 + 2, "the shared prefix was not executed again"
    assert eng.kv.stats().forks == 1
    eng.reset_session("src")
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0


def test_exact_fork_of_an_unknown_or_busy_session_changes_nothing():
    eng, r = make()
    with pytest.raises((KeyError, ValueError)):
        eng.fork_session_exact("nope", GenerateRequest("x", [1], max_new_tokens=1))
    eng.submit(GenerateRequest("busy", list(range(1, 20)), max_new_tokens=20, session_id="s", retain_session=True))
    ev = []
    eng.step(ev.append)
    before = eng.kv.stats()
    with pytest.raises((KeyError, ValueError, RuntimeError)):
        # the source is not a retained session yet (its request is still running under another id)
        eng.fork_session_exact("s", GenerateRequest("x", [1], max_new_tokens=1))
    after = eng.kv.stats()
    assert (before.used_pages, before.forks) == (after.used_pages, after.forks)
    ev += run(eng)
    assert len(toks(ev, "busy")) == 20


def test_idle_retained_sessions_give_their_pages_to_running_requests():
    """Four retained sessions fill the pool.  A new request does not end with an out-of-pages error: the sessions
    retained longest are dropped until it fits; the younger ones stay and still continue."""
    eng, r = make(pages=8, page=16, max_active=4)
    for i in range(4):
        eng.submit(GenerateRequest(f"s{i}", list(range(1, 30)), max_new_tokens=2, session_id=f"sess{i}", retain_session=True))
    run(eng)
    assert eng.kv.free_pages == 0 and len(eng._sessions) == 4
    prompt = list(range(1, 40))
    eng.submit(GenerateRequest("new", prompt, max_new_tokens=3))
    ev = run(eng)
    assert toks(ev, "new") == expected(r, prompt, 3) and fin(ev, "new").reason == FinishReason.MAX_TOKENS
    assert eng.stats.page_deadlocks == 0 and eng.stats.session_evictions >= 1
    kept = sorted(eng._sessions)
    assert kept and kept[-1] == "sess3" and "sess0" not in kept
    eng.submit(GenerateRequest("c", [5], max_new_tokens=1, session_id="sess3", retain_session=True))
    ev2 = run(eng)
    assert len(toks(ev2, "c")) == 1 and fin(ev2, "c").prompt_tokens > 29, "the kept session continued from its history"
    eng.kv.check_invariants()


def test_a_session_takes_one_request_at_a_time():
    eng, r = make()
    eng.submit(GenerateRequest("a", list(range(1, 20)), max_new_tokens=2, session_id="s", retain_session=True))
    with pytest.raises(ValueError):
        eng.submit(GenerateRequest("b", list(range(1, 10)), max_new_tokens=2, session_id="s", retain_session=True))
    run(eng)
    eng.submit(GenerateRequest("b", [3, 4], max_new_tokens=2, session_id="s", retain_session=True))     # free again
    ev = run(eng)
    assert fin(ev, "b").prompt_tokens > 19
    # a cancelled request frees the session name as well (its state is dropped)
    eng.submit(GenerateRequest("c", [3, 4], max_new_tokens=50, session_id="s", retain_session=True))
    eng.step(lambda e: None)
    assert eng.cancel_request("c")
    run(eng)
    eng.submit(GenerateRequest("d", [9, 9, 9], max_new_tokens=1, session_id="s"))
    ev = run(eng)
    assert fin(ev, "d").prompt_tokens == 3
    assert eng.reset_session("s") is False
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0


def test_a_parked_transaction_whose_completion_never_comes_times_out():
    """The provider loses a completion: the load stays in flight (its credit cannot be revoked), but the request
    does not wait for ever - after `materialization_timeout_s` the transaction is rolled back with an error and
    the engine serves the next request."""
    import time
    from ferrule_b200.runtime.io_protocol import MaterializationKey, ResourceId, ResourceKind
    from ferrule_b200.runtime.provider import FakeMaterializationProvider
    from ferrule_b200.runtime.registry import LoadRegistry
    key = lambda e: MaterializationKey("m", b"s", bytes([e]), ResourceId(ResourceKind.ROUTED_EXPERT, 1, e), 1, "cuda", 0, 0, 0)
    r = MockRunner()
    prov = FakeMaterializationProvider(auto=True)
    sched = SchedulerConfig(max_active_sequences=4, max_decode_batch=4, max_batch_tokens=64, prefill_chunk_size=16, ctx_size=256)
    eng = Engine(r, EngineConfig(scheduler=sched, kv_pages=32, page_size=16, materialization_timeout_s=0.05),
                 registry=LoadRegistry(prov))
    r.wait_next = [[key(1)]]
    prov.lose_next()
    eng.submit(GenerateRequest("lost", [5, 6, 7], max_new_tokens=3))
    ev = []
    t0 = time.perf_counter()
    eng.run_until_idle(ev.append, max_steps=10 ** 7)
    assert 0.04 < time.perf_counter() - t0 < 5.0
    assert fin(ev, "lost").reason == FinishReason.ERROR and eng.stats.materialization_timeouts == 1
    assert not eng._waiting and eng.registry.residual().get("continuations", 0) == 0
    assert eng.registry.residual()["in_flight"] == 1, "the owed completion is still owed"
    eng.submit(GenerateRequest("next", [1, 2], max_new_tokens=2))
    ev2 = run(eng)
    assert toks(ev2, "next") == expected(r, [1, 2], 2)
    # a dependency list the registry refuses fails the transaction instead of the engine
    r.wait_next = [[key(3), key(3)]]
    eng.submit(GenerateRequest("dup", [1, 2], max_new_tokens=2))
    ev3 = run(eng)
    assert fin(ev3, "dup").reason == FinishReason.ERROR
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0


def test_a_publish_that_the_backend_refuses_becomes_a_rollback():
    """`end_transaction(PUBLISH)` raises: nothing of the step is published, the prepared commit is withdrawn, the
    transaction is ended as an abort (a failing abort has nothing more to undo), the request ends with an error and
    every page and credit is back; the engine serves the next request."""
    r = MockRunner()
    eng, _ = make(r)
    orig, state = r.end_transaction, {"left": 2}

    def flaky(txn_id, intent):
        if state["left"]:
            state["left"] -= 1
            raise RuntimeError("cleanup failed")
        return orig(txn_id, intent)

    r.end_transaction = flaky
    eng.submit(GenerateRequest("a", [1, 2, 3], max_new_tokens=3))
    ev = run(eng)
    assert toks(ev, "a") == [] and fin(ev, "a").reason == FinishReason.ERROR
    assert "cleanup failed" in str(eng.last_error) and eng.stats.aborted_transactions == 1
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0 and eng.broker.outstanding() == 0 and not eng._ending
    eng.submit(GenerateRequest("b", [1, 2, 3], max_new_tokens=3))
    ev2 = run(eng)
    assert toks(ev2, "b") == expected(r, [1, 2, 3], 3)


def test_text_held_by_the_detokeniser_is_flushed_with_the_finish_event():
    """A token that ends inside a multi-byte character holds its whole text back; when the stream ends there, the
    complete part still reaches the client (on the finish event) and the total text."""
    from ferrule_b200.runtime.engine import Engine, EngineConfig, FinishEvent, TokenEvent
    from ferrule_b200.runtime.runner import MockRunner
    from ferrule_b200.runtime.scheduler import SchedulerConfig
    from ferrule_b200.runtime.session import GenerateRequest
    table = {1: b"hi", 2: b"A\xe6", 3: b"\xbc\xa2"}

    def decode(ids):
        return b"".join(table.get(i, b"?") for i in ids).decode("utf-8", errors="replace")
    for n_out, want_text, want_tail in ((2, "hiA", "A"), (3, "hiA\u6f22", "")):
        runner = MockRunner(vocab=16, eos=15, next_token_fn=lambda t, p: {7: 1, 1: 2, 2: 3}.get(t, 1))
        eng = Engine(runner, EngineConfig(scheduler=SchedulerConfig(max_active_sequences=2, max_decode_batch=2,
                                                                    max_batch_tokens=32, prefill_chunk_size=16,
                                                                    ctx_size=64), kv_pages=16, page_size=8))
        eng.detokenize = decode
        eng.submit(GenerateRequest("r", [7], max_new_tokens=n_out, ignore_eos=True))
        events = []
        for _ in range(50):
            eng.step(events.append)
            if any(isinstance(e, FinishEvent) for e in events):
                break
        fin = [e for e in events if isinstance(e, FinishEvent)][0]
        streamed = "".join(e.text for e in events if isinstance(e, TokenEvent)) + fin.tail
        assert fin.text == want_text and fin.tail == want_tail and streamed == want_text
        eng.shutdown()
