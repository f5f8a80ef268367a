"""Regression tests for state-machine faults found in review (CPU, mock runner)."""
import pytest
import torch

from ferrule_b200.runtime.engine import Engine, EngineConfig, FinishEvent, TokenEvent
from ferrule_b200.runtime.kv_pages import KvError, KvPageManager
from ferrule_b200.runtime.runner import MockRunner
from ferrule_b200.runtime.scheduler import SchedulerConfig
from ferrule_b200.runtime.session import FinishReason, GenerateRequest


def make(runner=None, speculative=False, **kw):
    sched = SchedulerConfig(max_active_sequences=8, max_decode_batch=8, max_batch_tokens=64, prefill_chunk_size=16,
                            ctx_size=kw.pop("ctx", 256))
    cfg = EngineConfig(scheduler=sched, kv_pages=kw.pop("pages", 16), page_size=16, speculative=speculative, **kw)
    r = runner or MockRunner(page_size=16)
    return Engine(r, cfg), r


def test_free_after_preempt_release_keeps_last_page_intact():
    """A preempted sequence's released pages are marked -1; freeing it must not touch page n-1."""
    kv = KvPageManager(4, 16)
    a, b = kv.alloc_sequence(), kv.alloc_sequence()
    ra = kv.reserve(a, 20)                       # pages 0, 1
    kv.publish_commit(kv.prepare_commit([(ra.res_id, 20)]))
    rb = kv.reserve(b, 30)                       # pages 2, 3: b owns the last page of the pool
    kv.publish_commit(kv.prepare_commit([(rb.res_id, 30)]))
    assert 3 in kv.sequence(b).pages
    kv.preempt_sequence(a)
    ret = kv.release_preempted_pages(a)
    kv.confirm_page_retirement(ret.pages)
    ret = kv.free_sequence_pages(a)
    assert ret.pages == []
    kv.check_invariants()
    assert kv.sequence(b).pages == [2, 3]
    with pytest.raises(KvError):
        kv._decref(-1, ret)
    kv.free_sequence_pages(b)


def test_truncate_after_preempt_release_skips_released_pages():
    kv = KvPageManager(4, 16)
    a = kv.alloc_sequence()
    r = kv.reserve(a, 40)
    kv.publish_commit(kv.prepare_commit([(r.res_id, 40)]))
    kv.preempt_sequence(a)
    kv.confirm_page_retirement(kv.release_preempted_pages(a).pages)
    assert kv.truncate_sequence(a, 0).pages == []
    kv.check_invariants()


def test_cancel_of_a_suspended_request_releases_everything():
    eng, r = make(pages=4)
    ev = []
    eng.submit(GenerateRequest("a", list(range(1, 21)), max_new_tokens=50))
    eng.submit(GenerateRequest("b", list(range(1, 31)), max_new_tokens=50))
    for _ in range(6):
        eng.step(ev.append)
    eng.preempt_session("a")
    assert "a" in eng._snapshots and "a" in eng.scheduler.suspended
    assert eng.cancel_request("a")
    eng.step(ev.append)
    assert "a" not in eng._snapshots and "a" not in eng.scheduler.suspended
    eng.kv.check_invariants()
    eng.cancel_request("b")
    eng.run_until_idle(ev.append)
    eng.kv.check_invariants()
    st = eng.kv.stats()
    assert st.used_pages == 0 and st.quarantined_pages == 0
    fins = {e.request_id: e.reason for e in ev if isinstance(e, FinishEvent)}
    assert fins["a"] == FinishReason.CANCELLED


def test_rejected_continuation_keeps_the_session_and_leaks_no_page():
    eng, r = make(ctx=64)
    ev = []
    eng.submit(GenerateRequest("s1", list(range(1, 31)), max_new_tokens=4, session_id="sess", retain_session=True))
    eng.run_until_idle(ev.append)
    used = eng.kv.stats().used_pages
    assert "sess" in eng._sessions and used > 0
    with pytest.raises(ValueError):
        eng.submit(GenerateRequest("s2", list(range(1, 60)), max_new_tokens=4, session_id="sess",
                                   retain_session=True))
    st = eng.kv.stats()
    assert "sess" in eng._sessions and st.used_pages == used and st.quarantined_pages == 0
    # the session still works
    eng.submit(GenerateRequest("s3", [5, 6], max_new_tokens=3, session_id="sess", retain_session=True))
    eng.run_until_idle(ev.append)
    assert len([e for e in ev if isinstance(e, TokenEvent) and e.request_id == "s3"]) == 3
    eng.kv.check_invariants()


def test_stop_string_inside_a_speculative_cycle_keeps_kv_and_position_in_step():
    """Speculation + stop string + session continuation: the retained KV must end where the tokens end."""
    r = MockRunner(page_size=16, draft_len=3)
    text_of = lambda toks: "".join(chr(ord("a") + t % 26) for t in toks)      # noqa: E731
    sched = SchedulerConfig(max_active_sequences=4, max_decode_batch=4, max_batch_tokens=64, prefill_chunk_size=16,
                            ctx_size=256)
    eng = Engine(r, EngineConfig(scheduler=sched, kv_pages=32, page_size=16, speculative=True, max_draft=3),
                 detokenize=text_of)
    prompt = list(range(3, 12))
    # plain greedy run to learn the stream, then stop on the text of its 2nd token (inside the first cycle)
    base = Engine(MockRunner(page_size=16), EngineConfig(scheduler=sched, kv_pages=32, page_size=16),
                  detokenize=text_of)
    base.submit(GenerateRequest("b", prompt, max_new_tokens=8))
    bev = []
    base.run_until_idle(bev.append)
    stream = [e.token for e in bev if isinstance(e, TokenEvent)]
    stop = text_of(stream[:2])
    ev = []
    eng.submit(GenerateRequest("a", prompt, max_new_tokens=8, stop=[stop], session_id="s", retain_session=True))
    eng.run_until_idle(ev.append)
    fin = [e for e in ev if isinstance(e, FinishEvent)][0]
    assert fin.reason == FinishReason.STOP_STRING
    seq = eng._sessions["s"]
    assert eng.kv.sequence(seq.kv_seq).committed_tokens == seq.position
    # the continuation runs and matches a fresh greedy run over the same token history
    more = [7, 8, 9]
    eng.submit(GenerateRequest("c", more, max_new_tokens=4, session_id="s", retain_session=True))
    eng.run_until_idle(ev.append)
    got = [e.token for e in ev if isinstance(e, TokenEvent) and e.request_id == "c"]
    hist = seq.tokens[:seq.position] + more
    ref = Engine(MockRunner(page_size=16), EngineConfig(scheduler=sched, kv_pages=32, page_size=16))
    ref.submit(GenerateRequest("r", hist, max_new_tokens=4))
    rev = []
    ref.run_until_idle(rev.append)
    assert got == [e.token for e in rev if isinstance(e, TokenEvent)]
    eng.kv.check_invariants()


def test_mtp_eh_proj_column_order_is_embedding_then_hidden():
    """Hand-built eh_proj: identity on the embedding half, zero on the hidden half -> the stage's layer input
    equals the normalised embedding, whatever the previous hidden state is."""
    from ferrule_b200.models import config as C
    from ferrule_b200.models import weights as W
    from ferrule_b200.models.deepseek import DeviceBatch, KvPool, ReferenceForward
    from ferrule_b200.ops import reference as ref
    cfg = C.tiny_fixture()
    w = W.random_weights(cfg, device="cpu", seed=0, dtype=torch.float32)
    assert w.mtp, "the fixture has an MTP stage"
    H = cfg.hidden
    m = w.mtp[0]
    m.eh_proj = torch.cat([torch.eye(H), torch.zeros(H, H)], dim=1)
    pool = KvPool(cfg, 8, 16, "cpu", dtype=torch.float32)
    fwd = ReferenceForward(w, pool)
    T = 3
    b = DeviceBatch(torch.tensor([5, 6, 7], dtype=torch.int32), torch.arange(T, dtype=torch.int32),
                    torch.arange(T, dtype=torch.int64), torch.zeros(T, dtype=torch.int32),
                    torch.arange(T, dtype=torch.int32), torch.zeros(1, 2, dtype=torch.int32),
                    torch.arange(T, dtype=torch.int32), T, T)
    seen = {}
    orig = fwd.layer

    def spy(lw, layer, h, bb, allreduce=None):
        seen["h"] = h.clone()
        return orig(lw, layer, h, bb, allreduce)
    fwd.layer = spy
    fwd.mtp_forward(0, torch.randn(T, H), b)
    want = ref.rmsnorm(w.embed[b.token_ids.long()].float(), m.enorm, cfg.rms_eps)
    assert torch.allclose(seen["h"], want, atol=1e-5)


def test_worker_answers_500_on_unexpected_submit_failure():
    import asyncio

    from ferrule_b200.server.worker import ModelWorker, WorkerError
    from ferrule_b200.utils.tokenizer import ByteTokenizer

    class Boom(ByteTokenizer):
        def encode(self, text):
            raise KeyError("tokenizer table is broken")

    async def go():
        sched = SchedulerConfig(max_active_sequences=2, max_decode_batch=2, max_batch_tokens=32,
                                prefill_chunk_size=16, ctx_size=128)
        worker = ModelWorker(lambda: Engine(MockRunner(vocab=300, page_size=16),
                                            EngineConfig(scheduler=sched, kv_pages=16, page_size=16)), Boom())
        worker.start()
        try:
            with pytest.raises(WorkerError) as ei:
                await worker.submit(text="hi", token_ids=None, max_tokens=2, stop=[])
            assert ei.value.status == 500
            assert worker.healthy
        finally:
            worker.stop()
    asyncio.run(go())
