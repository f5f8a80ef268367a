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
