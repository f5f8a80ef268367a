"""Speculative decoding: exactness against plain greedy decoding, rollback, accounting (CPU, mock runner)."""
import pytest

from ferrule_b200.runtime.engine import Engine, EngineConfig, FinishEvent, TokenEvent
from ferrule_b200.runtime.runner import MockRunner
from ferrule_b200.runtime.scheduler import SchedulerConfig
from ferrule_b200.runtime.session import FinishReason, GenerateRequest
from ferrule_b200.runtime.speculation import verify_causal_slice


def make(runner, speculative, **kw):
    sched = SchedulerConfig(max_active_sequences=8, max_decode_batch=8, max_batch_tokens=128, prefill_chunk_size=32,
                            ctx_size=kw.pop("ctx", 512))
    cfg = EngineConfig(scheduler=sched, kv_pages=kw.pop("pages", 128), page_size=16, speculative=speculative,
                       max_draft=kw.pop("max_draft", 4), **kw)
    return Engine(runner, cfg)


def run(engine):
    ev = []
    engine.run_until_idle(ev.append, max_steps=10000)
    return ev


def toks(ev, rid):
    return [e.token for e in ev if isinstance(e, TokenEvent) and e.request_id == rid]


def test_verify_causal_slice():
    assert verify_causal_slice([5, 6, 7], [5, 6, 7, 9]) == (3, 9)          # all accepted + bonus
    assert verify_causal_slice([5, 6, 7], [5, 8, 7, 9]) == (1, 8)          # mismatch at the second draft
    assert verify_causal_slice([5], [4, 1]) == (0, 4)
    assert verify_causal_slice([], [3]) == (0, 3)
    assert verify_causal_slice([5, 6], [5, None, 1]) == (1, None)


@pytest.mark.parametrize("wrong_every", [0, 2, 3, 1])
def test_speculative_stream_equals_greedy(wrong_every):
    """Drafts that are right, sometimes wrong, or always wrong never change the emitted tokens."""
    def draft_fn(slot, j, nxt):
        if wrong_every and (slot + j) % wrong_every == 0:
            return (nxt + 13) % 1000
        return nxt
    prompts = {f"r{i}": [(i * 17 + j) % 997 + 1 for j in range(5 + 11 * i)] for i in range(5)}
    base = make(MockRunner(), False)
    spec_runner = MockRunner(draft_len=3, draft_accuracy=draft_fn)
    spec = make(spec_runner, True, max_draft=3)
    for rid, p in prompts.items():
        base.submit(GenerateRequest(rid, p, max_new_tokens=17))
        spec.submit(GenerateRequest(rid, p, max_new_tokens=17))
    eb, es = run(base), run(spec)
    for rid in prompts:
        assert toks(es, rid) == toks(eb, rid), rid
        assert len(toks(es, rid)) == 17
    m = spec.spec.metrics
    assert m.cycles > 0 and m.drafted > 0
    if wrong_every == 0:
        assert m.accepted == m.drafted and spec.stats.decode_steps < base.stats.decode_steps
    if wrong_every == 1:
        assert m.accepted == 0 and m.accepted_prefix_hist.get(0, 0) > 0
    spec.kv.check_invariants()
    assert spec.kv.stats().used_pages == 0 and spec.broker.outstanding() == 0


def test_speculative_respects_eos_and_budget():
    # the target produces EOS (= 7) at position >= 20; drafts are always right
    r = MockRunner(eos=7, next_token_fn=lambda t, p: 7 if p >= 20 else (t * 3 + p) % 900 + 10, draft_len=4)
    eng = make(r, True, max_draft=4)
    eng.submit(GenerateRequest("e", list(range(10, 26)), max_new_tokens=50))
    ev = run(eng)
    out = toks(ev, "e")
    base = make(MockRunner(eos=7, next_token_fn=r.next_token_fn), False)
    base.submit(GenerateRequest("e", list(range(10, 26)), max_new_tokens=50))
    assert out == toks(run(base), "e") and 7 not in out
    assert [e for e in ev if isinstance(e, FinishEvent)][0].reason == FinishReason.EOS
    eng2 = make(MockRunner(draft_len=4), True, max_draft=4)
    eng2.submit(GenerateRequest("b", [1, 2, 3], max_new_tokens=6))
    ev2 = run(eng2)
    assert len(toks(ev2, "b")) == 6
    assert [e for e in ev2 if isinstance(e, FinishEvent)][0].reason == FinishReason.MAX_TOKENS


def test_confidence_threshold_prunes_drafts():
    class LowConf(MockRunner):
        def propose(self, slots, anchors, positions, views, max_draft):
            out = super().propose(slots, anchors, positions, views, max_draft)
            for p in out:
                p.confidence = [5.0, -5.0, 5.0][:len(p.tokens)]      # sigmoid(-5) < 0.2 cuts after the first draft
            return out
    eng = make(LowConf(draft_len=3), True, max_draft=3)
    eng.submit(GenerateRequest("c", [4, 5, 6], max_new_tokens=9))
    run(eng)
    m = eng.spec.metrics
    assert m.pruned_by_confidence > 0
    assert max(m.accepted_prefix_hist) <= 1


def test_verification_failure_rolls_back_and_continues():
    r = MockRunner(draft_len=2)
    eng = make(r, True, max_draft=2)
    eng.submit(GenerateRequest("f", [9, 8, 7, 6], max_new_tokens=8))
    ev = []
    eng.step(ev.append)                 # prefill
    r.fail_next_execute = 1             # the first verification batch fails in the backend
    eng.run_until_idle(ev.append)
    fin = [e for e in ev if isinstance(e, FinishEvent)][0]
    assert fin.reason == FinishReason.ERROR and eng.spec.metrics.rollbacks == 1
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0 and eng.broker.outstanding() == 0


def test_rejected_suffix_pages_are_retired():
    # page size 16, prompt of 15 tokens: the verification rows cross a page boundary; with always-wrong
    # drafts the extra page must come back
    r = MockRunner(draft_len=4, draft_accuracy=lambda s, j, n: (n + 1) % 1000)
    eng = make(r, True, max_draft=4)
    eng.submit(GenerateRequest("p", list(range(1, 16)), max_new_tokens=3))
    run(eng)
    assert eng.spec.metrics.accepted == 0
    assert len(r.released_pages) >= 2
    eng.kv.check_invariants()


class _Recording(MockRunner):
    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self.batches = []

    def execute(self, txn_id):
        self.batches.append(self.txns[txn_id])
        return super().execute(txn_id)


def test_two_ragged_sessions_are_verified_in_one_provisional_execution():
    """Different draft lengths per sequence (one pruned by its confidence): one provisional batch holds both,
    rows = 1 + drafts per sequence, top-1 logits on every row."""
    from ferrule_b200.runtime.execution import Intent
    from ferrule_b200.runtime.runner import Proposal
    r = _Recording(draft_len=3)
    eng = make(r, True, max_draft=3)
    orig = r.propose

    def propose(slots, anchors, positions, views, max_draft):
        out = orig(slots, anchors, positions, views, max_draft)
        # the second sequence's head loses confidence after one draft
        return [p if i == 0 else Proposal(p.tokens, [5.0] + [-5.0] * (len(p.tokens) - 1)) for i, p in enumerate(out)]

    r.propose = propose
    eng.submit(GenerateRequest("a", [1, 2, 3, 4, 5], max_new_tokens=12))
    eng.submit(GenerateRequest("b", [9, 8, 7], max_new_tokens=12))
    ev = run(eng)
    prov = [b for b in r.batches if b.intent == Intent.PROVISIONAL_VERIFICATION and len(b.sequences) == 2]
    assert prov, "both sequences shared a verification batch"
    b0 = prov[0]
    assert sorted(s.query_len for s in b0.sequences) == [2, 4] and b0.rows == 6
    assert all(b0.logits[i].k == 1 for i in range(b0.rows))
    plain = make(MockRunner(), False)
    plain.submit(GenerateRequest("a", [1, 2, 3, 4, 5], max_new_tokens=12))
    plain.submit(GenerateRequest("b", [9, 8, 7], max_new_tokens=12))
    ep = run(plain)
    assert toks(ev, "a") == toks(ep, "a") and toks(ev, "b") == toks(ep, "b")
    assert eng.spec.metrics.pruned_by_confidence > 0


def test_zero_draft_capacity_runs_an_ordinary_step():
    """One token left to generate: there is no room for a draft, so no proposal block is verified - the cycle
    counts as a zero-draft cycle and the step is an ordinary decode."""
    from ferrule_b200.runtime.execution import Intent
    r = _Recording(draft_len=3)
    eng = make(r, True, max_draft=3)
    eng.submit(GenerateRequest("a", [1, 2, 3], max_new_tokens=1))
    ev = run(eng)
    assert len(toks(ev, "a")) == 1
    assert not any(b.intent == Intent.PROVISIONAL_VERIFICATION for b in r.batches)
    assert eng.spec.metrics.cycles == 0 and eng.spec.metrics.drafted == 0


def test_proposals_can_be_switched_off_mid_run():
    """The runner stops proposing (policy change): decoding goes on as plain greedy steps, same stream."""
    r = MockRunner(draft_len=2)
    eng = make(r, True, max_draft=2)
    prompt = [4, 5, 6, 7]
    eng.submit(GenerateRequest("a", prompt, max_new_tokens=14))
    ev = []
    while eng.stats.finished == 0 and len(toks(ev, "a")) < 6:
        eng.step(ev.append)
    cycles = eng.spec.metrics.cycles
    assert cycles > 0
    r.draft_len = 0                              # proposals_enabled() is False from here on
    ev += run(eng)
    assert eng.spec.metrics.cycles == cycles
    plain = make(MockRunner(), False)
    plain.submit(GenerateRequest("a", prompt, max_new_tokens=14))
    assert toks(ev, "a") == toks(run(plain), "a")


def test_failure_while_keeping_the_accepted_prefix_rolls_the_cycle_back():
    """`retain_provisional_prefixes` fails once: the whole cycle is rolled back (nothing of it is published, its
    reservations and pages return), the next cycle verifies again, and the stream is exact."""
    r = MockRunner(draft_len=2)
    eng = make(r, True, max_draft=2)
    orig, state = r.retain_provisional_prefixes, {"left": 1}

    def flaky(txn_id, keep):
        if state["left"]:
            state["left"] -= 1
            raise RuntimeError("backend could not keep the prefix")
        return orig(txn_id, keep)

    r.retain_provisional_prefixes = flaky
    prompt = [3, 1, 4, 1, 5]
    eng.submit(GenerateRequest("a", prompt, max_new_tokens=9))
    ev = run(eng)
    plain = make(MockRunner(), False)
    plain.submit(GenerateRequest("a", prompt, max_new_tokens=9))
    ep = run(plain)
    if [e for e in ev if isinstance(e, FinishEvent)][0].reason == FinishReason.ERROR:
        # a non-retryable backend failure ends the request; nothing of the failed cycle was published
        assert toks(ev, "a") == toks(ep, "a")[:len(toks(ev, "a"))]
    else:
        assert toks(ev, "a") == toks(ep, "a")
    assert eng.spec.metrics.rollbacks == 1
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0 and eng.broker.outstanding() == 0
