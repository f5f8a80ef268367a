"""Owner state machine against the deterministic mock runner (CPU)."""
import pytest

from ferrule_b200.runtime.engine import Engine, EngineConfig, FinishEvent, TokenEvent
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


def expected_tokens(r, prompt, n):
    out, tok, pos = [], prompt[-1], len(prompt) - 1
    for _ in range(n):
        tok = r.next_token_fn(tok, pos)
        pos += 1
        out.append(tok)
    return out


def run(engine):
    events = []
    engine.run_until_idle(events.append, max_steps=10000)
    return events


def tokens_of(events, rid):
    return [e.token for e in events if isinstance(e, TokenEvent) and e.request_id == rid]


def finish_of(events, rid):
    return [e for e in events if isinstance(e, FinishEvent) and e.request_id == rid][0]


def test_single_request_greedy_and_chunked_prefill():
    eng, r = make()
    prompt = list(range(5, 45))               # 40 tokens -> 3 prefill chunks of 16
    eng.submit(GenerateRequest("a", prompt, max_new_tokens=6))
    ev = run(eng)
    assert tokens_of(ev, "a") == expected_tokens(r, prompt, 6)
    f = finish_of(ev, "a")
    assert f.reason == FinishReason.MAX_TOKENS and f.generated_tokens == 6 and f.prompt_tokens == 40
    assert eng.stats.prefill_chunks == 3 and eng.stats.prefill_tokens == 40
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0 and eng.kv.stats().quarantined_pages == 0


def test_many_requests_mixed_batches_match_isolated_runs():
    eng, r = make(max_batch_tokens=40)
    prompts = {f"r{i}": [(i * 13 + j) % 900 + 1 for j in range(7 + 9 * i)] for i in range(6)}
    for rid, p in prompts.items():
        eng.submit(GenerateRequest(rid, p, max_new_tokens=5 + len(p) % 4))
    ev = run(eng)
    for rid, p in prompts.items():
        n = 5 + len(p) % 4
        assert tokens_of(ev, rid) == expected_tokens(r, p, n), rid
    assert eng.stats.finished == 6
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0


def test_eos_stops_without_emitting_eos():
    r = MockRunner(eos=77, next_token_fn=lambda t, p: 77 if p >= 12 else (t + 1) % 50)
    eng, _ = make(r)
    eng.submit(GenerateRequest("e", list(range(10)), max_new_tokens=20))
    ev = run(eng)
    toks = tokens_of(ev, "e")
    assert 77 not in toks and len(toks) == 3          # positions 10, 11, 12 hold generated tokens
    assert finish_of(ev, "e").reason == FinishReason.EOS
    eng2, _ = make(MockRunner(eos=77, next_token_fn=lambda t, p: 77))
    eng2.submit(GenerateRequest("i", [1, 2, 3], max_new_tokens=4, ignore_eos=True))
    ev2 = run(eng2)
    assert tokens_of(ev2, "i") == [77] * 4


def test_context_limit_and_no_candidate():
    eng, r = make(ctx=20)
    eng.submit(GenerateRequest("c", list(range(1, 17)), max_new_tokens=50))
    ev = run(eng)
    assert finish_of(ev, "c").reason == FinishReason.CONTEXT
    assert len(tokens_of(ev, "c")) == 4               # positions 16..19
    r2 = MockRunner()
    r2.no_candidate_rows = {2}
    eng2, _ = make(r2)
    eng2.submit(GenerateRequest("n", [1, 2, 3], max_new_tokens=5))
    assert finish_of(run(eng2), "n").reason == FinishReason.NO_CANDIDATE


def test_stop_string_uses_detokenized_text():
    eng, r = make()
    eng.detokenize = lambda toks: "".join(chr(97 + t % 26) for t in toks)
    prompt = [3, 4, 5]
    exp = expected_tokens(r, prompt, 10)
    text = "".join(chr(97 + t % 26) for t in exp)
    stop = text[3:5]
    eng.submit(GenerateRequest("s", prompt, max_new_tokens=10, stop=[stop]))
    ev = run(eng)
    f = finish_of(ev, "s")
    assert f.reason == FinishReason.STOP_STRING and f.text.endswith(stop)
    assert len(tokens_of(ev, "s")) == text.index(stop) + 2


def test_cancel_waiting_idle_and_running():
    eng, r = make(max_active=1)
    eng.submit(GenerateRequest("a", list(range(1, 30)), max_new_tokens=50))
    eng.submit(GenerateRequest("b", [1, 2, 3], max_new_tokens=5))
    assert eng.cancel_request("b")                     # still waiting
    events = []
    for _ in range(4):
        eng.step(events.append)
    assert eng.cancel_request("a")
    eng.run_until_idle(events.append)
    assert finish_of(events, "a").reason == FinishReason.CANCELLED
    assert finish_of(events, "b").reason == FinishReason.CANCELLED
    assert not eng.cancel_request("zzz")
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0


def test_execute_failure_aborts_and_returns_custody():
    r = MockRunner()
    eng, _ = make(r)
    r.fail_next_execute = 1
    r.pending_ends = 2                                  # backend takes three calls to finish the abort
    eng.submit(GenerateRequest("f", list(range(1, 10)), max_new_tokens=3))
    events = []
    eng.step(events.append)
    st = eng.kv.stats()
    assert st.open_reservations == 1 and eng.broker.outstanding() == 1      # custody retained while PENDING
    eng.run_until_idle(events.append)
    assert finish_of(events, "f").reason == FinishReason.ERROR
    assert eng.stats.aborted_transactions == 1
    assert eng.broker.outstanding() == 0
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0 and eng.kv.stats().open_reservations == 0
    assert [c for c in r.calls if c[0] == "end_abort"] == [("end_abort", 0)] * 3


def test_publish_pending_delays_token_visibility():
    r = MockRunner()
    r.pending_ends = 1
    eng, _ = make(r)
    eng.submit(GenerateRequest("p", [1, 2, 3], max_new_tokens=2))
    events = []
    eng.step(events.append)            # prefill executed, publish pending
    assert eng.kv.sequence(0).committed_tokens == 0
    eng.step(events.append)            # publish completes; next txn starts
    assert eng.kv.sequence(0).committed_tokens >= 3
    eng.run_until_idle(events.append)
    assert len(tokens_of(events, "p")) == 2


def test_kv_exhaustion_stalls_then_proceeds():
    eng, r = make(pages=6, page=16, max_batch_tokens=64, chunk=64)
    eng.submit(GenerateRequest("a", list(range(1, 60)), max_new_tokens=8))     # 4 pages
    eng.submit(GenerateRequest("b", list(range(1, 50)), max_new_tokens=8))     # 4 pages: must wait
    ev = run(eng)
    assert len(tokens_of(ev, "a")) == 8 and len(tokens_of(ev, "b")) == 8
    assert eng.stats.kv_stalls > 0
    assert eng.broker.usage[list(eng.broker.usage)[10]].high_water <= 6


def test_fork_exact_shares_pages_and_copies_on_write():
    eng, r = make(page=16)
    base = list(range(1, 41))                           # 40 tokens: pages 0,1 full, page 2 half
    eng.submit(GenerateRequest("base", base, max_new_tokens=3, retain_session=True, session_id="s"))
    ev = run(eng)
    base_out = tokens_of(ev, "base")
    used_before = eng.kv.stats().used_pages
    child = eng.fork_session_exact("s", GenerateRequest("child", [500, 501], max_new_tokens=4))
    assert eng.kv.stats().shared_pages == used_before
    ev2 = run(eng)
    cont = base[:] + base_out                           # committed tokens of the session (position 43)
    committed = cont[:43]
    assert tokens_of(ev2, "child") == expected_tokens(r, committed + [500, 501], 4)
    assert len(r.copied_pages) == 1                     # the shared partial tail page was copied once
    assert eng.kv.stats().cow_copies == 1
    # the retained session still continues correctly from its own pages
    eng.submit(GenerateRequest("again", [9], max_new_tokens=2, session_id="s"))
    ev3 = run(eng)
    assert tokens_of(ev3, "again") == expected_tokens(r, committed + [9], 2)
    eng.kv.check_invariants()


def test_preempt_restore_roundtrip():
    eng, r = make()
    eng.submit(GenerateRequest("a", list(range(1, 25)), max_new_tokens=10))
    events = []
    for _ in range(4):
        eng.step(events.append)
    used = eng.kv.stats().used_pages
    eng.preempt_session("a")
    eng.step(events.append)
    assert eng.kv.stats().used_pages == 0 and used > 0
    eng.restore_session("a")
    eng.run_until_idle(events.append)
    assert tokens_of(events, "a") == expected_tokens(r, list(range(1, 25)), 10)
    eng.kv.check_invariants()


def test_shutdown_drains():
    r = MockRunner()
    r.pending_ends = 1
    eng, _ = make(r)
    eng.submit(GenerateRequest("a", [1, 2, 3], max_new_tokens=100))
    eng.step(lambda e: None)
    done = False
    for _ in range(10):
        done = eng.shutdown()
        if done:
            break
    assert done
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0 and eng.broker.outstanding() == 0
    with pytest.raises(RuntimeError):
        eng.submit(GenerateRequest("b", [1], max_new_tokens=1))


def test_waiting_transaction_resumes_after_materialization():
    from ferrule_b200.runtime.io_protocol import MaterializationKey, ResourceId, ResourceKind
    from ferrule_b200.runtime.provider import FakeMaterializationProvider
    from ferrule_b200.runtime.registry import LoadRegistry
    key = lambda e: MaterializationKey("m", b"s", bytes([e]), ResourceId(ResourceKind.ROUTED_EXPERT, 1, e), 1, "cuda", 0, 0, 0)
    r = MockRunner()
    prov = FakeMaterializationProvider(auto=True)
    sched = SchedulerConfig(max_active_sequences=4, max_decode_batch=4, max_batch_tokens=64, prefill_chunk_size=16, ctx_size=256)
    eng = Engine(r, EngineConfig(scheduler=sched, kv_pages=32, page_size=16), registry=LoadRegistry(prov))
    r.wait_next = [[key(1), key(2)], [key(3)]]            # the first batch suspends twice
    eng.submit(GenerateRequest("w", [5, 6, 7], max_new_tokens=3))
    ev = run(eng)
    assert tokens_of(ev, "w") == expected_tokens(r, [5, 6, 7], 3)
    assert eng.stats.waits == 2 and eng.stats.resumes == 2
    assert eng.registry.stats.published == 3
    assert [c[0] for c in r.calls if c[1] == 0][:4] == ["prepare", "execute", "resume", "resume"]
    # a failed dependency aborts the transaction and fails the request, custody returned
    r.wait_next = [[key(9)]]
    prov.script_next("fail")
    eng.submit(GenerateRequest("x", [1, 2], max_new_tokens=2))
    ev = run(eng)
    assert finish_of(ev, "x").reason == FinishReason.ERROR
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0 and eng.broker.outstanding() == 0


def test_decode_lookahead_prediction_is_never_wrong_and_mostly_available():
    """The engine tells the runner which batch it will lower next; a runner that launches that batch early
    must never be handed a different one without noticing, and in steady decode the prediction must exist."""
    r = MockRunner(page_size=16, eos=999)
    eng, _ = make(r, pages=256, max_batch_tokens=64, ctx=256)
    # different lengths: sequences leave the cohort at different steps; one stops at EOS, one has a stop string
    r.next_token_fn = lambda t, p: 999 if (t % 7 == 3 and p > 40) else (7 * t + 3 * p + 1) % 900
    for i in range(6):
        eng.submit(GenerateRequest(f"r{i}", [(i * 11 + j) % 800 + 1 for j in range(20 + i)],
                                   max_new_tokens=20 + 5 * i, ignore_eos=(i % 2 == 0)))
    ev = run(eng)
    assert eng.stats.finished == 6
    assert r.prediction_misses == 0
    assert r.prediction_hits >= eng.stats.decode_steps // 2      # most decode steps were predicted
    # page-boundary steps and steps after a sequence left are not predicted; nothing may be predicted wrongly
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0


def test_decode_lookahead_declines_when_the_next_action_is_not_a_pure_decode():
    r = MockRunner(page_size=16)
    eng, _ = make(r, pages=256, max_batch_tokens=64)
    eng.submit(GenerateRequest("a", list(range(1, 30)), max_new_tokens=30))
    ev = []
    for _ in range(6):
        eng.step(ev.append)
    hits = r.prediction_hits
    assert hits > 0
    # an arrival cannot be foreseen: the step predicted before it is handed a different (mixed) batch, which the
    # runner notices by comparing; while the newcomer prefills nothing is predicted
    eng.submit(GenerateRequest("b", list(range(1, 40)), max_new_tokens=5))
    eng.step(ev.append)
    assert r.prediction_misses == 1 and r.predicted is None
    eng.run_until_idle(ev.append)
    assert r.prediction_misses == 1 and r.prediction_hits > hits


def _prefix_engine(cache_tokens, kv_pages=96, block=32):
    import torch
    from ferrule_b200.models import config as C, weights as W
    from ferrule_b200.models.runner import DeepSeekRunner
    from ferrule_b200.runtime.engine import Engine, EngineConfig
    from ferrule_b200.runtime.scheduler import SchedulerConfig
    cfg = C.tiny_fixture().with_(n_mtp_layers=0)
    w = W.random_weights(cfg, device="cpu", seed=0, dtype=torch.float32)
    runner = DeepSeekRunner(w, n_pages=kv_pages, page_size=16, max_rows=128, max_seqs=4, max_seq_len=512, device="cpu")
    sched = SchedulerConfig(max_active_sequences=4, max_decode_batch=4, max_batch_tokens=96, prefill_chunk_size=48,
                            ctx_size=512)
    return cfg, Engine(runner, EngineConfig(scheduler=sched, kv_pages=kv_pages, page_size=16,
                                            prefix_cache_tokens=cache_tokens, prefix_block=block))


def _run_all(eng, reqs):
    from ferrule_b200.runtime.engine import TokenEvent
    from ferrule_b200.runtime.session import GenerateRequest
    for rid, toks in reqs:
        eng.submit(GenerateRequest(rid, toks, max_new_tokens=5, ignore_eos=True))
    ev = []
    eng.run_until_idle(ev.append, max_steps=4000)
    assert eng.last_error is None, eng.last_error
    return {rid: [e.token for e in ev if isinstance(e, TokenEvent) and e.request_id == rid] for rid, _ in reqs}


def test_prompt_prefix_cache_forks_cached_pages_and_streams_the_same_tokens():
    """Requests that start with the tokens of an earlier prompt fork its KV pages (whole prefix blocks) instead of
    recomputing them: same greedy tokens as without the cache, fewer prefill tokens, shared pages while they run,
    and the cache gives its pages back at shutdown."""
    import torch
    g = torch.Generator().manual_seed(9)
    shared = torch.randint(0, 1000, (100,), generator=g).tolist()
    tails = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (7, 30, 1)]
    waves = [[("a", shared + tails[0])], [("b", shared + tails[1]), ("c", shared + tails[2])],
             [("d", shared[:64] + tails[1])], [("e", shared[:96])]]
    _, plain = _prefix_engine(0)
    want = {}
    for wv in waves:
        want.update(_run_all(plain, wv))
    _, eng = _prefix_engine(4096)
    got = {}
    for wv in waves:
        got.update(_run_all(eng, wv))
        eng.kv.check_invariants()
    assert got == want and all(len(v) == 5 for v in got.values())
    st = eng.stats
    # a: miss (and becomes the entry for blocks 32/64/96); b, c: 96 tokens each; d: 64; e: 96 tokens are the whole
    # prompt, one token must stay for the request itself -> 64
    assert st.prefix_hits == 4 and st.prefix_tokens_reused == 96 + 96 + 64 + 64
    assert st.prefill_tokens == plain.stats.prefill_tokens - st.prefix_tokens_reused
    assert eng.kv.stats().forks == 4 and st.prefix_entries >= 1
    assert eng.kv.stats().used_pages > 0                     # the cache still holds the prefix
    while not eng.shutdown():
        pass
    assert eng.kv.stats().used_pages == 0 and eng.kv.stats().free_pages == eng.kv.stats().total_pages


def test_prompt_prefix_cache_gives_way_under_page_pressure_and_budget():
    """Entries leave oldest-first when the token budget is exceeded, and a stalled reservation evicts cached
    prefixes before anything else is tried; evicted prefixes are simply recomputed."""
    import torch
    g = torch.Generator().manual_seed(10)
    prompts = [torch.randint(0, 1000, (70,), generator=g).tolist() for _ in range(4)]
    _, eng = _prefix_engine(128, kv_pages=24)              # 128 cached tokens = two 64-token entries at most
    for i, p_ in enumerate(prompts):
        _run_all(eng, [(f"r{i}", p_)])
        eng.kv.check_invariants()
    assert eng.stats.prefix_entries == 4 and eng.stats.prefix_evictions >= 2 and len(eng._prefix_lru) <= 2
    # three long prompts at once need more pages than the cache leaves free: the cache yields, nothing fails
    long = [torch.randint(0, 1000, (120,), generator=g).tolist() for _ in range(3)]
    out = _run_all(eng, [(f"l{i}", p_) for i, p_ in enumerate(long)])
    assert all(len(v) == 5 for v in out.values()) and eng.stats.kv_stalls >= 0
    eng.kv.check_invariants()
    # an evicted prefix is a miss, a kept one a hit
    hits0 = eng.stats.prefix_hits
    _run_all(eng, [("again", prompts[0] + [5, 6])])
    assert eng.stats.prefix_hits in (hits0, hits0 + 1)
    while not eng.shutdown():
        pass
    assert eng.kv.stats().used_pages == 0
